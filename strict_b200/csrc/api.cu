// Context, memory and op-level C entry points of libstrictb200.so.
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <thread>
#include <vector>

#include "common.cuh"

static thread_local std::string g_last_error;

void sb_set_error(const std::string& msg) { g_last_error = msg; }
int sb_fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

namespace {
struct OptionName { const char* name; int SbOptions::*field; };
const OptionName kOptions[] = {
    {"pdl", &SbOptions::pdl},
    {"attn_tc", &SbOptions::attn_tc},
    {"gemm_pair", &SbOptions::gemm_pair},
    {"prefetch", &SbOptions::prefetch},
    {"deep_ring", &SbOptions::deep_ring},
    {"attn_blocks_per_sm", &SbOptions::attn_blocks_per_sm},
    {"split_target", &SbOptions::split_target},
    {"tp_two_shot", &SbOptions::tp_two_shot},
    {"wait_limit", &SbOptions::wait_limit},
    {"prefill_chunk", &SbOptions::prefill_chunk},
    {"row_cluster", &SbOptions::row_cluster},
    {"attn_prefetch", &SbOptions::attn_prefetch},
    {"blur_rows", &SbOptions::blur_rows},
    {"host_timeout_ms", &SbOptions::host_timeout_ms},
    {"fuse_rope", &SbOptions::fuse_rope},
};
// STRICTB200_<NAME> of every option, read once, here
void options_from_environment(SbOptions* o) {
  for (const OptionName& n : kOptions) {
    std::string env = "STRICTB200_";
    for (const char* c = n.name; *c; c++) env += (char)toupper((unsigned char)*c);
    if (const char* v = getenv(env.c_str())) o->*(n.field) = atoi(v);
  }
}
}  // namespace

int sb_sync(strictb200_ctx* ctx, const char* what) {
  if (!ctx->tp || ctx->tp_world == 1) {
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
    return STRICTB200_OK;
  }
  if (ctx->opt.host_timeout_ms <= 0) {
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
  } else {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(ctx->opt.host_timeout_ms);
    for (int polls = 0;; polls++) {
      cudaError_t e = cudaStreamQuery(ctx->stream);
      if (e == cudaSuccess) break;
      if (e != cudaErrorNotReady) return sb_fail(STRICTB200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
      if (int rc = sb_tp_async_error(ctx)) {
        sb_tp_abort(ctx);
        return sb_fail(STRICTB200_ERR_NCCL, std::string(what) + ": NCCL reported an asynchronous error (code " + std::to_string(rc) + "); the communicator was aborted");
      }
      if (std::chrono::steady_clock::now() > deadline) {
        sb_tp_abort(ctx);
        return sb_fail(STRICTB200_ERR_TIMEOUT, std::string(what) + ": the stream did not finish within " + std::to_string(ctx->opt.host_timeout_ms) +
                                                   " ms; the NCCL communicator was aborted");
      }
      if (polls > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));  // spin first: a decode step lasts a few ms
    }
  }
  if (int rc = sb_tp_async_error(ctx)) {
    sb_tp_abort(ctx);
    return sb_fail(STRICTB200_ERR_NCCL, std::string(what) + ": NCCL reported an asynchronous error (code " + std::to_string(rc) + "); the communicator was aborted");
  }
  return STRICTB200_OK;
}

// Reads and clears the error word the kernels of this context set when a bounded wait expired.
// The stream must have been synchronised by the caller.
int sb_check_status(strictb200_ctx* ctx, const char* what) {
  const int code = *(volatile int*)ctx->h_status;
  if (!code) return STRICTB200_OK;
  *(volatile int*)ctx->h_status = 0;
  // a GEMM block that gave up may have left its stream-K tile counters mid-count
  if (ctx->gemm_ws && ctx->gemm_count_bytes) cudaMemsetAsync(ctx->gemm_ws, 0, ctx->gemm_count_bytes, ctx->stream);
  return sb_fail(STRICTB200_ERR_TIMEOUT, std::string(what) + ": a bounded device-side wait expired (code " + std::to_string(code) +
                                             "); the results of this call are not valid");
}

int sb_ws(strictb200_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->ws_bytes) {
    ctx->ws_generation++;
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->ws) SB_CUDA(cudaFree(ctx->ws));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    size_t want = bytes + (bytes >> 2) + (1 << 20);
    SB_CUDA(cudaMalloc(&ctx->ws, want));
    ctx->ws_bytes = want;
  }
  *out = ctx->ws;
  return STRICTB200_OK;
}

int sb_ws2(strictb200_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->ws2_bytes) {
    ctx->ws_generation++;
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->ws2) SB_CUDA(cudaFree(ctx->ws2));
    ctx->ws2 = nullptr;
    ctx->ws2_bytes = 0;
    size_t want = bytes + (bytes >> 2) + (1 << 20);
    SB_CUDA(cudaMalloc(&ctx->ws2, want));
    ctx->ws2_bytes = want;
  }
  *out = ctx->ws2;
  return STRICTB200_OK;
}

__global__ void flush_kernel(uint4* p, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) p[i] = make_uint4((uint32_t)i, 0u, 0u, 0u);
}

int sb_trace_set_gemm_split(const SbTraceDev&);  // one per instrumented translation unit
int sb_trace_set_norm(const SbTraceDev&);
int sb_trace_set_rope(const SbTraceDev&);
int sb_trace_set_attention(const SbTraceDev&);
static int trace_set_all(const SbTraceDev& t) {
  return sb_trace_set_gemm_split(t) | sb_trace_set_norm(t) | sb_trace_set_rope(t) | sb_trace_set_attention(t);
}

extern "C" {

int strictb200_trace_begin(strictb200_ctx* ctx, int capacity) {
  SB_ENTER(ctx);
  SB_REQUIRE(capacity > 0 && capacity <= (1 << 24), "capacity must be between 1 and 2^24 records");
  SB_REQUIRE(!ctx->trace_rec, "a trace is already armed on this context");
  SB_TRY(sb_sync(ctx, "trace_begin"));
  SB_CUDA(cudaMalloc(&ctx->trace_rec, (size_t)capacity * 64));
  SB_CUDA(cudaMalloc(&ctx->trace_count, 256));
  SB_CUDA(cudaMemset(ctx->trace_count, 0, 256));
  ctx->trace_capacity = (unsigned)capacity;
  if (trace_set_all(SbTraceDev{ctx->trace_rec, ctx->trace_count, ctx->trace_capacity})) return sb_fail(STRICTB200_ERR_CUDA, "trace: cannot set the device variables");
  return STRICTB200_OK;
}

int strictb200_trace_end(strictb200_ctx* ctx, uint64_t* out_records, int max_records, int* out_count) {
  SB_ENTER(ctx);
  SB_REQUIRE(ctx->trace_rec, "no trace is armed on this context");
  SB_REQUIRE(out_count && (out_records || max_records == 0), "null pointer");
  int st = sb_sync(ctx, "trace_end");
  trace_set_all(SbTraceDev{nullptr, nullptr, 0});
  unsigned n = 0;
  cudaMemcpy(&n, ctx->trace_count, 4, cudaMemcpyDeviceToHost);
  *out_count = (int)n;  // blocks that reported, also beyond the capacity
  unsigned take = n < ctx->trace_capacity ? n : ctx->trace_capacity;
  if ((int)take > max_records) take = (unsigned)max_records;
  if (take) cudaMemcpy(out_records, ctx->trace_rec, (size_t)take * 64, cudaMemcpyDeviceToHost);
  cudaFree(ctx->trace_rec);
  cudaFree(ctx->trace_count);
  ctx->trace_rec = nullptr; ctx->trace_count = nullptr; ctx->trace_capacity = 0;
  return st;
}

int strictb200_version(void) { return STRICTB200_VERSION; }
const char* strictb200_last_error(void) { return g_last_error.c_str(); }

int strictb200_create(int device, strictb200_ctx** out) {
  if (!out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null out pointer");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return sb_fail(STRICTB200_ERR_CUDA, std::string("no CUDA device: ") + cudaGetErrorString(e) +
                                            " (this library has no CPU path)");
  if (device < 0 || device >= n) return sb_fail(STRICTB200_ERR_INVALID_ARG, "device index out of range");
  cudaDeviceProp prop;
  SB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return sb_fail(STRICTB200_ERR_UNSUPPORTED, std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) +
                                                   std::to_string(prop.minor) + "; kernels are built for sm_100a only");
  SB_CUDA(cudaSetDevice(device));
  strictb200_ctx* c = new strictb200_ctx;
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  options_from_environment(&c->opt);
  SB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  SB_CUDA(cudaEventCreate(&c->ev0));
  SB_CUDA(cudaEventCreate(&c->ev1));
  SB_CUDA(cudaHostAlloc((void**)&c->h_status, sizeof(int), cudaHostAllocMapped));
  *c->h_status = 0;
  SB_CUDA(cudaHostGetDevicePointer((void**)&c->d_status, c->h_status, 0));
  *out = c;
  return STRICTB200_OK;
}

int strictb200_destroy(strictb200_ctx* ctx) {
  if (!ctx) return STRICTB200_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  sb_tp_destroy(ctx);
  if (ctx->ws) cudaFree(ctx->ws);
  if (ctx->flush_buf) cudaFree(ctx->flush_buf);
  if (ctx->gemm_ws) cudaFree(ctx->gemm_ws);
  if (ctx->ws2) cudaFree(ctx->ws2);
  if (ctx->prefill_ws) cudaFree(ctx->prefill_ws);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  cudaEventDestroy(ctx->ev0);
  cudaEventDestroy(ctx->ev1);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return STRICTB200_OK;
}

// ---------------------------------------------------------------- recorded call sequences
struct strictb200_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t launches = 0;  // kernels in the recorded sequence
  uint64_t ws_generation = 0;  // the context's scratch generation the recorded pointers belong to
};
int strictb200_graph_begin(strictb200_ctx* ctx) {
  SB_ENTER(ctx);
  SB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->rec_launches0 = ctx->launches;
  return STRICTB200_OK;
}
int strictb200_graph_end(strictb200_ctx* ctx, strictb200_graph** out) {
  SB_ENTER(ctx);
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
  const uint64_t recorded = ctx->launches - ctx->rec_launches0;
  ctx->launches = ctx->rec_launches0;  // recorded kernels have not run
  if (e != cudaSuccess || !g) {
    cudaGetLastError();
    return sb_fail(STRICTB200_ERR_CUDA, std::string("recording failed (a recorded call synchronised, copied or allocated?): ") + cudaGetErrorString(e));
  }
  SB_REQUIRE(out, "null output pointer");
  strictb200_graph* r = new strictb200_graph;
  r->graph = g;
  r->launches = recorded;
  r->ws_generation = ctx->ws_generation;
  e = cudaGraphInstantiate(&r->exec, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    delete r;
    return sb_fail(STRICTB200_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
  }
  *out = r;
  return STRICTB200_OK;
}
int strictb200_graph_launch(strictb200_ctx* ctx, strictb200_graph* g, int times) {
  SB_ENTER(ctx);
  SB_REQUIRE(g && g->exec && times >= 0, "bad graph or repeat count");
  if (g->ws_generation != ctx->ws_generation)
    return sb_fail(STRICTB200_ERR_INVALID_ARG,
                   "the context's scratch memory was re-allocated by a larger call after this sequence was recorded; record it again");
  for (int i = 0; i < times; i++) SB_CUDA(cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->launches * (uint64_t)times;
  return STRICTB200_OK;
}
int strictb200_graph_destroy(strictb200_graph* g) {
  if (!g) return STRICTB200_OK;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return STRICTB200_OK;
}

int strictb200_synchronize(strictb200_ctx* ctx) {
  SB_ENTER(ctx);
  return sb_sync(ctx, "synchronize");
}

int strictb200_malloc(strictb200_ctx* ctx, size_t bytes, void** d_out) {
  SB_ENTER(ctx);
  SB_REQUIRE(d_out, "null out pointer");
  *d_out = nullptr;
  if (bytes == 0) return STRICTB200_OK;
  SB_CUDA(cudaMalloc(d_out, bytes));
  return STRICTB200_OK;
}
int strictb200_free(strictb200_ctx* ctx, void* d_ptr) {
  SB_ENTER(ctx);
  if (!d_ptr) return STRICTB200_OK;
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  SB_CUDA(cudaFree(d_ptr));
  return STRICTB200_OK;
}
int strictb200_memset(strictb200_ctx* ctx, void* d_ptr, int byte, size_t bytes) {
  SB_ENTER(ctx);
  if (bytes == 0) return STRICTB200_OK;
  SB_REQUIRE(d_ptr, "null pointer");
  SB_CUDA(cudaMemsetAsync(d_ptr, byte, bytes, ctx->stream));
  return STRICTB200_OK;
}
int strictb200_upload(strictb200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
  SB_ENTER(ctx);
  if (bytes == 0) return STRICTB200_OK;
  SB_REQUIRE(d_dst && h_src, "null pointer");
  SB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}
int strictb200_download(strictb200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
  SB_ENTER(ctx);
  if (bytes == 0) return STRICTB200_OK;
  SB_REQUIRE(h_dst && d_src, "null pointer");
  SB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}
int strictb200_upload_async(strictb200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
  SB_ENTER(ctx);
  if (bytes == 0) return STRICTB200_OK;
  SB_REQUIRE(d_dst && h_src, "null pointer");
  SB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return STRICTB200_OK;
}
int strictb200_download_async(strictb200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
  SB_ENTER(ctx);
  if (bytes == 0) return STRICTB200_OK;
  SB_REQUIRE(h_dst && d_src, "null pointer");
  SB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return STRICTB200_OK;
}
int strictb200_host_alloc(strictb200_ctx* ctx, size_t bytes, void** h_out) {
  SB_ENTER(ctx);
  SB_REQUIRE(h_out, "null out pointer");
  SB_CUDA(cudaHostAlloc(h_out, bytes ? bytes : 1, cudaHostAllocDefault));
  return STRICTB200_OK;
}
int strictb200_host_free(strictb200_ctx* ctx, void* h_ptr) {
  SB_ENTER(ctx);
  if (h_ptr) SB_CUDA(cudaFreeHost(h_ptr));
  return STRICTB200_OK;
}
int strictb200_timer_begin(strictb200_ctx* ctx) {
  SB_ENTER(ctx);
  SB_CUDA(cudaEventRecord(ctx->ev0, ctx->stream));
  return STRICTB200_OK;
}
int strictb200_timer_end(strictb200_ctx* ctx, float* ms_out) {
  SB_ENTER(ctx);
  SB_REQUIRE(ms_out, "null out pointer");
  SB_CUDA(cudaEventRecord(ctx->ev1, ctx->stream));
  SB_CUDA(cudaEventSynchronize(ctx->ev1));
  SB_CUDA(cudaEventElapsedTime(ms_out, ctx->ev0, ctx->ev1));
  return STRICTB200_OK;
}
int strictb200_launch_count(strictb200_ctx* ctx, uint64_t* out) {
  if (!ctx || !out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  *out = ctx->launches;
  return STRICTB200_OK;
}
int strictb200_device_status(strictb200_ctx* ctx, int* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(out, "null out pointer");
  SB_TRY(sb_sync(ctx, "device_status"));
  *out = *(volatile int*)ctx->h_status;
  return sb_check_status(ctx, "device_status");
}
int strictb200_set_option(strictb200_ctx* ctx, const char* name, int value) {
  if (!ctx || !name) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  for (const OptionName& n : kOptions)
    if (!strcmp(n.name, name)) {
      ctx->opt.*(n.field) = value;
      return STRICTB200_OK;
    }
  return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("unknown option ") + name);
}
int strictb200_get_option(strictb200_ctx* ctx, const char* name, int* out) {
  if (!ctx || !name || !out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  for (const OptionName& n : kOptions)
    if (!strcmp(n.name, name)) {
      *out = ctx->opt.*(n.field);
      return STRICTB200_OK;
    }
  return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("unknown option ") + name);
}
int strictb200_flush_l2(strictb200_ctx* ctx) {
  SB_ENTER(ctx);
  if (!ctx->flush_buf) {
    ctx->flush_bytes = (size_t)256 << 20;  // 2x the 126 MB L2
    SB_CUDA(cudaMalloc(&ctx->flush_buf, ctx->flush_bytes));
  }
  flush_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>((uint4*)ctx->flush_buf, ctx->flush_bytes / 16);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

// ---------------------------------------------------------------- element-wise
int strictb200_ew_binary(strictb200_ctx* ctx, int op, const float* a, const float* b, float* out, int64_t count) {
  SB_ENTER(ctx);
  if (op < 0 || op > 3) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "unsupported instruction " + std::to_string(op));
  SB_REQUIRE(count >= 0, "negative count");
  if (count == 0) return STRICTB200_OK;
  SB_REQUIRE(a && b && out, "null pointer");
  return k_ew_binary(ctx, op, a, b, out, count);
}
int strictb200_ew_program(strictb200_ctx* ctx, const int32_t* code, int n_instr, const float* const* arrays, int n_arrays,
                          const float* scalars, int n_scalars, const float* consts, int n_consts, float* out, int64_t count) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0 && n_instr >= 0 && n_arrays >= 0 && n_scalars >= 0 && n_consts >= 0, "negative size");
  SB_REQUIRE(n_instr <= 64 && n_arrays <= 8 && n_scalars <= 8 && n_consts <= 16, "program too large");
  if (count == 0) return STRICTB200_OK;
  SB_REQUIRE(out && (n_instr == 0 || code), "null pointer");
  return k_ew_program(ctx, code, n_instr, arrays, n_arrays, scalars, n_scalars, consts, n_consts, out, count);
}

int strictb200_ew_program2(strictb200_ctx* ctx, const int32_t* code, int n_instr, const float* const* arrays, int n_arrays,
                           const float* scalars, int n_scalars, const float* consts, int n_consts, float* out, int64_t count) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0 && n_instr >= 0 && n_arrays >= 0 && n_scalars >= 0 && n_consts >= 0, "negative size");
  SB_REQUIRE(n_instr <= 256 && n_arrays <= 8 && n_scalars <= 8 && n_consts <= 16, "program too large");
  if (count == 0) return STRICTB200_OK;
  SB_REQUIRE(out && (n_instr == 0 || code), "null pointer");
  return k_ew_program2(ctx, code, n_instr, arrays, n_arrays, scalars, n_scalars, consts, n_consts, out, count);
}

// ---------------------------------------------------------------- generator
int strictb200_gen_normal_f32(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t first, int64_t count, float std_, float* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0 && first >= 0, "negative size");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(out, "null pointer");
  return k_gen_normal_f32(ctx, sb_stream_key(seed, tensor), first, count, std_, out);
}
int strictb200_gen_normal_bf16(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t first, int64_t count, float std_, uint16_t* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0 && first >= 0, "negative size");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(out, "null pointer");
  return k_gen_normal_bf16(ctx, sb_stream_key(seed, tensor), first, count, std_, (bf16*)out);
}
int strictb200_gen_tokens(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t count, uint32_t range, int32_t* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0, "negative size");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(out && range > 0, "null pointer or empty range");
  return k_gen_tokens(ctx, sb_stream_key(seed, tensor), count, range, out);
}
int strictb200_gen_weight_e4m3(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t row0, int64_t rows, int64_t K, int64_t col0,
                               int64_t cols, float std_, uint8_t* q, float* scale) {
  SB_ENTER(ctx);
  SB_REQUIRE(rows >= 0 && row0 >= 0 && K > 0 && col0 >= 0 && cols > 0 && col0 + cols <= K, "bad shape");
  if (!rows) return STRICTB200_OK;
  SB_REQUIRE(q && scale, "null pointer");
  return k_gen_weight_e4m3(ctx, sb_stream_key(seed, tensor), row0, rows, K, col0, cols, std_, q, cols, scale);
}

// ---------------------------------------------------------------- quantisation / GEMM
int strictb200_quantize_rows(strictb200_ctx* ctx, const uint16_t* x, int64_t M, int64_t K, uint8_t* q, float* scale) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && K > 0 && K % 16 == 0, "bad shape (K must be a multiple of 16)");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && q && scale, "null pointer");
  return k_quantize_rows(ctx, (const bf16*)x, M, K, K, q, scale);
}

static int gemm_entry(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint8_t* xq, const float* sx, const uint8_t* wq,
                      const float* sw, void* out, int out_dtype, int kernel) {
  SB_REQUIRE(M >= 0 && N > 0 && K > 0, "bad shape");
  SB_REQUIRE(K % 64 == 0 && N % 16 == 0, "K must be a multiple of 64 and N of 16");
  SB_REQUIRE(out_dtype == 0 || out_dtype == 1, "out_dtype must be 0 (bf16) or 1 (fp32)");
  if (kernel < 0 || kernel > 3) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "unknown kernel selector");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(xq && sx && wq && sw && out, "null pointer");
  GemmArgs g;
  g.M = M; g.N = N; g.K = K;
  g.xq = xq; g.ldx = K; g.sx = sx; g.wq = wq; g.ldw = K; g.sw = sw;
  g.out = out; g.out_f32 = out_dtype; g.kernel = kernel;
  g.splits = 1;
  // few tokens, automatic kernel choice: the job is a stream of weights, so K is split until the
  // grid covers the GPU and a second kernel sums the partial results
  const int splits = (kernel == 0 || kernel == 3) && N % 4 == 0 ? sb_gemm_pick_splits(ctx, M, N, K) : 1;
  if (splits > 1) {
    void* ws;
    SB_TRY(sb_ws2(ctx, (size_t)splits * M * N * sizeof(float), &ws));
    g.out = nullptr; g.part = (float*)ws; g.splits = splits; g.raw = 1;
    SB_TRY(k_gemm_fp8(ctx, g));
    return k_reduce_scale(ctx, (const float*)ws, splits, sx, sw, M, N, out_dtype ? (float*)out : nullptr, out_dtype ? nullptr : (bf16*)out);
  }
  return k_gemm_fp8(ctx, g);
}
int strictb200_gemm_fp8(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint8_t* xq, const float* sx, const uint8_t* wq,
                        const float* sw, void* out, int out_dtype, int kernel) {
  SB_ENTER(ctx);
  return gemm_entry(ctx, M, N, K, xq, sx, wq, sw, out, out_dtype, kernel);
}
int strictb200_gemm_fp8w(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* x, const uint8_t* wq, const float* sw,
                         uint16_t* y, int kernel) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 64 == 0, "bad shape");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && wq && sw && y, "null pointer");
  void* ws;
  size_t qbytes = ((size_t)sb_qrows(M) * K + 255) & ~(size_t)255;
  SB_TRY(sb_ws(ctx, qbytes + (size_t)M * 4, &ws));
  uint8_t* xq = (uint8_t*)ws;
  float* sx = (float*)((char*)ws + qbytes);
  SB_TRY(k_quantize_rows(ctx, (const bf16*)x, M, K, K, xq, sx));
  return gemm_entry(ctx, M, N, K, xq, sx, wq, sw, y, 0, kernel);
}
int strictb200_gemm_f32(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const float* x, const float* w, const float* bias, float* y) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 4 == 0, "bad shape (K must be a multiple of 4)");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && w && y, "null pointer");
  return k_gemm_f32(ctx, M, N, K, x, w, bias, y, 0);
}

// ---------------------------------------------------------------- norms / activations
int strictb200_rmsnorm(strictb200_ctx* ctx, const uint16_t* x, uint16_t* residual, const float* gain, float eps, int64_t M, int64_t d,
                       uint16_t* y) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && d > 0 && d % 8 == 0 && d <= 16384, "bad shape (d must be a multiple of 8, at most 16384)");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && gain && y, "null pointer");
  RowNormArgs a;
  a.x_in = (const bf16*)x; a.residual = (bf16*)residual; a.gain = gain; a.eps = eps; a.y = (bf16*)y;
  return k_rownorm(ctx, a, M, d);
}
int strictb200_layernorm(strictb200_ctx* ctx, const float* x, const float* gain, const float* bias, float eps, int64_t M, int64_t d, float* y) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && d > 0, "bad shape");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && gain && bias && y, "null pointer");
  return k_layernorm(ctx, x, gain, bias, eps, M, d, y);
}
int strictb200_swiglu(strictb200_ctx* ctx, const uint16_t* gate_up, int64_t M, int64_t I, uint16_t* y) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && I > 0 && I % 8 == 0, "bad shape (I must be a multiple of 8)");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(gate_up && y, "null pointer");
  return k_swiglu(ctx, (const bf16*)gate_up, nullptr, M, I, (bf16*)y, nullptr, nullptr);
}
int strictb200_gelu_tanh(strictb200_ctx* ctx, const float* x, int64_t count, float* y) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0, "negative size");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(x && y, "null pointer");
  return k_gelu_tanh(ctx, x, count, y);
}
int strictb200_rope_qknorm_kvappend(strictb200_ctx* ctx, const uint16_t* qkv, const int32_t* seq, const int32_t* pos, int64_t T, int Hq,
                                    int Hkv, int D, const float* qgain, const float* kgain, float eps, float theta, int max_pos,
                                    uint16_t* q_out, uint16_t* kcache, uint16_t* vcache, int maxlen) {
  SB_ENTER(ctx);
  if (D != 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "head_dim must be 128");
  SB_REQUIRE(T >= 0 && Hq > 0 && Hkv > 0 && max_pos > 0 && maxlen > 0, "bad shape");
  if (!T) return STRICTB200_OK;
  SB_REQUIRE(qkv && seq && pos && qgain && kgain && q_out && kcache && vcache, "null pointer");
  float *c, *s;
  SB_TRY(sb_rope_table(ctx, max_pos, D, theta, &c, &s));
  RopeArgs a;
  a.qkv = (const bf16*)qkv; a.seq = seq; a.pos = pos; a.cos_t = c; a.sin_t = s; a.qgain = qgain; a.kgain = kgain;
  a.eps = eps; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.maxlen = maxlen; a.max_pos = max_pos;
  a.q_out = (bf16*)q_out; a.kcache = (bf16*)kcache; a.vcache = (bf16*)vcache;
  int st = k_rope_qknorm_kvappend(ctx, a, T);
  cudaStreamSynchronize(ctx->stream);
  cudaFree(c);
  cudaFree(s);
  return st;
}

// ---------------------------------------------------------------- attention
int strictb200_attn_prefill(strictb200_ctx* ctx, const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const int32_t* lens,
                            const int32_t* past, int B, int S, int Hq, int Hkv, int D, int maxlen, float scale, uint16_t* out) {
  SB_ENTER(ctx);
  if (D != 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "head_dim must be 128");
  SB_REQUIRE(B >= 0 && S >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && maxlen > 0, "bad shape");
  if (!B || !S) return STRICTB200_OK;
  SB_REQUIRE(q && kc && vc && lens && out, "null pointer");
  return k_attn_prefill(ctx, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, lens, past, nullptr, B, S, (int64_t)B * S, Hq, Hkv, D, maxlen, scale, (bf16*)out);
}
int strictb200_attn_decode(strictb200_ctx* ctx, const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const int32_t* lens, int B,
                           int Hq, int Hkv, int D, int maxlen, float scale, uint16_t* out) {
  SB_ENTER(ctx);
  if (D != 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "head_dim must be 128");
  SB_REQUIRE(B >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16 && maxlen > 0, "bad shape");
  if (!B) return STRICTB200_OK;
  SB_REQUIRE(q && kc && vc && lens && out, "null pointer");
  int nsplit = sb_attn_decode_splits(ctx, B, Hkv, maxlen);
  void* ws;
  SB_TRY(sb_ws(ctx, sb_attn_decode_scratch(B, Hq, D, nsplit), &ws));
  return k_attn_decode(ctx, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, lens, 0, B, Hq, Hkv, D, maxlen, scale, nsplit, (float*)ws,
                       (bf16*)out, nullptr, nullptr, nullptr);
}

// ---------------------------------------------------------------- embedding / sampling
int strictb200_embedding_bf16(strictb200_ctx* ctx, const uint16_t* table, const int32_t* ids, int64_t T, int64_t d, int64_t vocab,
                              uint16_t* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(T >= 0 && d > 0 && d % 8 == 0 && vocab > 0, "bad shape");
  if (!T) return STRICTB200_OK;
  SB_REQUIRE(table && ids && out, "null pointer");
  return k_embedding_bf16(ctx, (const bf16*)table, ids, T, d, vocab, (bf16*)out);
}
int strictb200_argmax(strictb200_ctx* ctx, const float* x, int64_t M, int64_t N, int32_t* out) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && N > 0, "bad shape");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(x && out, "null pointer");
  void* ws;
  SB_TRY(sb_ws(ctx, sb_argmax_scratch(M, N), &ws));
  return k_argmax(ctx, x, M, N, N, out, nullptr, ws);
}

}  // extern "C"
