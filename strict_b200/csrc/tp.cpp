// Tensor-parallel plumbing: NCCL over NVLink, bound at run time with dlopen so the library
// loads (and the single-GPU path runs) on machines without NCCL, and so that it shares the
// NCCL already loaded by the host process when there is one.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
enum { NCCL_INT8 = 0, NCCL_FLOAT32 = 7, NCCL_SUM = 0 };
struct Nccl {
  void* lib = nullptr;
  int (*GetUniqueId)(nccl_uid*) = nullptr;
  int (*CommInitRank)(nccl_comm*, int, nccl_uid, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
  int (*CommDestroy)(nccl_comm) = nullptr;
  int (*CommAbort)(nccl_comm) = nullptr;
  int (*CommGetAsyncError)(nccl_comm, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
Nccl g_nccl;

int load_nccl() {
  if (g_nccl.lib) return STRICTB200_OK;
  // STRICTB200_NCCL_LIB names another library with NCCL's entry points (failure-injection tests load a stand-in)
  void* h = nullptr;
  if (const char* other = getenv("STRICTB200_NCCL_LIB")) h = dlopen(other, RTLD_NOW | RTLD_LOCAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return sb_fail(STRICTB200_ERR_NCCL, std::string("cannot load libnccl.so.2: ") + dlerror());
#define SYM(field, name)                                                                       \
  *(void**)(&g_nccl.field) = dlsym(h, name);                                                   \
  if (!g_nccl.field) return sb_fail(STRICTB200_ERR_NCCL, std::string("libnccl lacks ") + name);
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(AllReduce, "ncclAllReduce")
  SYM(AllGather, "ncclAllGather")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(GetErrorString, "ncclGetErrorString")
  SYM(CommAbort, "ncclCommAbort")
  SYM(CommGetAsyncError, "ncclCommGetAsyncError")
#undef SYM
  g_nccl.lib = h;
  return STRICTB200_OK;
}
int nccl_fail(const char* what, int rc) {
  return sb_fail(STRICTB200_ERR_NCCL, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"));
}
}  // namespace

constexpr long long COMM_MAX_ELEMS = 1 << 20;  // floats per epoch parity (4 MiB): 64 tokens x 16384 channels
constexpr size_t COMM_FLAG_BYTES = 256;        // 2 parities x 8 source ranks, padded
constexpr int COMM_ROWS = 64;                  // rows of the row-granular exchange
constexpr long long COMM_ROW_ELEMS = (long long)COMM_ROWS * 4096;  // values per (parity, source rank) of the row area
// row area: [parity][source rank] areas of 2 x COMM_ROW_ELEMS words; a value travels as one word that carries the row's epoch modulo 4 in
// its two lowest mantissa bits (the first half of an area is used)
constexpr size_t COMM_ROW_OFFSET = COMM_FLAG_BYTES + 2 * COMM_MAX_ELEMS * sizeof(float);
// [2 parities][8 source ranks] areas of partial sums, then [2 parities] areas of finished sums (two-shot exchange)
constexpr size_t COMM_BYTES = COMM_ROW_OFFSET + (size_t)(2 * 8 + 2) * COMM_ROW_ELEMS * 2 * sizeof(float);

struct TpState {
  nccl_comm comm = nullptr;
  // peer-memory all-reduce
  void* comm_buf = nullptr;       // this rank's buffer: [flags | data parity 0 | data parity 1 | row packets]
  void* peer_buf[8] = {nullptr};  // every rank's buffer as mapped into this process
  int* local = nullptr;           // [epoch, done, ... | per-row epochs at int 64]
  bool opened = false;
  bool absent_peers = false;      // failure-injection set-up: the "peers" are local areas nobody writes
  long long row_d = 0;            // row width the row-granular exchange is tied to (0: not used yet)
  int row_two_shot = -1;          // and its one- or two-shot form (-1: not used yet)
  TpCommDev dev{};
};

// Publish kernel: scaled split-K sum of this rank's partial projection -> own peer buffer, then the
// last block to finish raises the epoch flag in every rank's buffer.
__global__ void tp_publish_kernel(const float* __restrict__ part, int splits, const float* __restrict__ sx, const float* __restrict__ sw,
                                  int64_t M, int64_t N, TpCommDev c) {
  pdl_trigger();
  pdl_wait();
  const int e = *(volatile int*)c.epoch + 1;  // stable during the kernel: only its last block advances it
  float* out = c.data[c.rank] + (size_t)(e & 1) * c.max_elems;
  int64_t total = M * N / 4, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t m = (i * 4) / N, n = (i * 4) - m * N;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; s++) {
      float4 p = *(const float4*)(part + ((int64_t)s * M + m) * N + n);
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    float a = sx[m];
    float4 w = *(const float4*)(sw + n);
    float4 r;
    r.x = __fmul_rn(__fmul_rn(acc.x, a), w.x); r.y = __fmul_rn(__fmul_rn(acc.y, a), w.y);
    r.z = __fmul_rn(__fmul_rn(acc.z, a), w.z); r.w = __fmul_rn(__fmul_rn(acc.w, a), w.w);
    *(float4*)(out + m * N + n) = r;
  }
  // Device-scope fence per thread; the block that takes the last ticket has observed every other
  // block's writes through the counter and makes all of them visible system-wide with one fence
  // before it raises the flags in the peers' buffers.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned ticket = atomicAdd(c.done, 1u);
    if (ticket == gridDim.x - 1) {
      *c.done = 0;
      *(volatile int*)c.epoch = e;
      __threadfence_system();
      for (int r = 0; r < c.world; r++) *(volatile int*)(c.flags[r] + (e & 1) * 8 + c.rank) = e;
      __threadfence_system();
    }
  }
}

int sb_tp_allreduce_f32(strictb200_ctx* ctx, float* buf, int64_t count) {
  if (ctx->tp_world == 1) return STRICTB200_OK;
  if (!ctx->tp || !ctx->tp->comm) return sb_fail(STRICTB200_ERR_NCCL, "this context has no NCCL communicator (never initialised, or aborted after an error)");
  int rc = g_nccl.AllReduce(buf, buf, (size_t)count, NCCL_FLOAT32, NCCL_SUM, ctx->tp->comm, ctx->stream);
  if (rc) return nccl_fail("ncclAllReduce", rc);
  return STRICTB200_OK;
}
int sb_tp_allgather(strictb200_ctx* ctx, const void* send, void* recv, int64_t bytes_per_rank) {
  if (ctx->tp_world == 1) {
    if (send != recv) SB_CUDA(cudaMemcpyAsync(recv, send, (size_t)bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return STRICTB200_OK;
  }
  if (!ctx->tp || !ctx->tp->comm) return sb_fail(STRICTB200_ERR_NCCL, "this context has no NCCL communicator (never initialised, or aborted after an error)");
  int rc = g_nccl.AllGather(send, recv, (size_t)bytes_per_rank, NCCL_INT8, ctx->tp->comm, ctx->stream);
  if (rc) return nccl_fail("ncclAllGather", rc);
  return STRICTB200_OK;
}
const TpCommDev* sb_tp_comm(strictb200_ctx* ctx) { return ctx->tp && ctx->tp->opened ? &ctx->tp->dev : nullptr; }
bool sb_tp_comm_fits(strictb200_ctx* ctx, int64_t M, int64_t d) {
  return ctx->tp && ctx->tp->opened && d % 4 == 0 && M * d <= COMM_MAX_ELEMS;
}
// The packet area is addressed by row * d + column and validated by a two-bit tag of the row's
// epoch, which tells a fresh word from the one its slot held before (epoch - 2) as long as every
// call writes the same slots: two row widths, or the one- and the two-shot form, on one context
// could take each other's stale words for fresh ones. The first width and form that use the
// exchange own it; others go through the publish kernel and its flags.
bool sb_tp_row_exchange_ok(strictb200_ctx* ctx, int64_t M, int64_t d, int two_shot) {
  if (!ctx->tp || !ctx->tp->opened || M > COMM_ROWS || M * d > COMM_ROW_ELEMS) return false;
  if (!ctx->tp->row_d) { ctx->tp->row_d = d; ctx->tp->row_two_shot = two_shot; }
  return ctx->tp->row_d == d && ctx->tp->row_two_shot == two_shot;
}

int k_tp_publish(strictb200_ctx* ctx, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t N) {
  if (!ctx->tp || !ctx->tp->opened) return sb_fail(STRICTB200_ERR_INVALID_ARG, "peer buffers are not open");
  if (N % 4 || M * N > COMM_MAX_ELEMS) return sb_fail(STRICTB200_ERR_INVALID_ARG, "tp_publish: result does not fit the peer buffer");
  int64_t blocks = (M * N / 4 + 255) / 256;
  int grid = (int)(blocks < 1 ? 1 : (blocks > ctx->sm_count ? ctx->sm_count : blocks));
  SB_CUDA(sb_launch(ctx, tp_publish_kernel, dim3(grid), dim3(256), 0, part, splits, sx, sw, M, N, ctx->tp->dev));
  ctx->launches++;
  return STRICTB200_OK;
}

int sb_tp_async_error(strictb200_ctx* ctx) {
  if (!ctx->tp || !ctx->tp->comm || !g_nccl.CommGetAsyncError) return 0;
  int async = 0;
  int rc = g_nccl.CommGetAsyncError(ctx->tp->comm, &async);
  return rc ? rc : async;
}
void sb_tp_abort(strictb200_ctx* ctx) {
  if (!ctx->tp || !ctx->tp->comm || !g_nccl.CommAbort) return;
  g_nccl.CommAbort(ctx->tp->comm);
  ctx->tp->comm = nullptr;  // aborted communicators are freed by ncclCommAbort; collectives on this context now fail
}

void sb_tp_destroy(strictb200_ctx* ctx) {
  if (ctx->tp) {
    for (int r = 0; r < 8; r++)
      if (ctx->tp->peer_buf[r] && ctx->tp->peer_buf[r] != ctx->tp->comm_buf) {
        if (ctx->tp->absent_peers) cudaFree(ctx->tp->peer_buf[r]);
        else cudaIpcCloseMemHandle(ctx->tp->peer_buf[r]);
      }
    if (ctx->tp->comm_buf) cudaFree(ctx->tp->comm_buf);
    if (ctx->tp->local) cudaFree(ctx->tp->local);
    if (ctx->tp->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->tp->comm);
    delete ctx->tp;
    ctx->tp = nullptr;
  }
}

extern "C" {
int strictb200_tp_unique_id(void* h_id128) {
  if (!h_id128) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null id buffer");
  SB_TRY(load_nccl());
  nccl_uid id;
  int rc = g_nccl.GetUniqueId(&id);
  if (rc) return nccl_fail("ncclGetUniqueId", rc);
  memcpy(h_id128, &id, 128);
  return STRICTB200_OK;
}
int strictb200_tp_init(strictb200_ctx* ctx, int world, int rank, const void* h_id128) {
  SB_ENTER(ctx);
  SB_REQUIRE(world == 1 || world == 2 || world == 4 || world == 8, "world must be 1, 2, 4 or 8");
  SB_REQUIRE(rank >= 0 && rank < world, "rank out of range");
  SB_REQUIRE(!ctx->tp, "tensor parallelism already initialised on this context");
  if (world == 1) return STRICTB200_OK;
  SB_REQUIRE(h_id128, "null id buffer");
  SB_TRY(load_nccl());
  nccl_uid id;
  memcpy(&id, h_id128, 128);
  TpState* tp = new TpState;
  int rc = g_nccl.CommInitRank(&tp->comm, world, id, rank);
  if (rc) {
    delete tp;
    return nccl_fail("ncclCommInitRank", rc);
  }
  ctx->tp = tp;
  ctx->tp_world = world;
  ctx->tp_rank = rank;
  return STRICTB200_OK;
}
int strictb200_tp_comm_handle(strictb200_ctx* ctx, void* h_handle64) {
  SB_ENTER(ctx);
  SB_REQUIRE(h_handle64, "null handle buffer");
  SB_REQUIRE(ctx->tp && ctx->tp_world > 1, "tensor parallelism is not initialised on this context");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  TpState* tp = ctx->tp;
  if (!tp->comm_buf) {
    SB_CUDA(cudaMalloc(&tp->comm_buf, COMM_BYTES));
    SB_CUDA(cudaMemset(tp->comm_buf, 0, COMM_BYTES));
    SB_CUDA(cudaMalloc((void**)&tp->local, 256 + COMM_ROWS * sizeof(int)));
    SB_CUDA(cudaMemset(tp->local, 0, 256 + COMM_ROWS * sizeof(int)));
  }
  cudaIpcMemHandle_t h;
  SB_CUDA(cudaIpcGetMemHandle(&h, tp->comm_buf));
  memcpy(h_handle64, &h, 64);
  return STRICTB200_OK;
}
static void fill_comm_dev(strictb200_ctx* ctx);
int strictb200_tp_comm_open(strictb200_ctx* ctx, const void* h_handles) {
  SB_ENTER(ctx);
  SB_REQUIRE(h_handles, "null handle buffer");
  SB_REQUIRE(ctx->tp && ctx->tp->comm_buf, "call strictb200_tp_comm_handle first");
  TpState* tp = ctx->tp;
  SB_REQUIRE(!tp->opened, "peer buffers already open");
  for (int r = 0; r < ctx->tp_world; r++) {
    if (r == ctx->tp_rank) { tp->peer_buf[r] = tp->comm_buf; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)h_handles + 64 * r, 64);
    SB_CUDA(cudaIpcOpenMemHandle(&tp->peer_buf[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  fill_comm_dev(ctx);
  return STRICTB200_OK;
}
int strictb200_tp_comm_open_absent_peers(strictb200_ctx* ctx, int world) {
  SB_ENTER(ctx);
  SB_REQUIRE(world == 2 || world == 4 || world == 8, "world must be 2, 4 or 8");
  SB_REQUIRE(!ctx->tp, "tensor parallelism already initialised on this context");
  TpState* tp = new TpState;
  tp->absent_peers = true;
  ctx->tp = tp;
  ctx->tp_world = world;
  ctx->tp_rank = 0;
  for (int r = 0; r < world; r++) {
    SB_CUDA(cudaMalloc(&tp->peer_buf[r], COMM_BYTES));
    SB_CUDA(cudaMemset(tp->peer_buf[r], 0, COMM_BYTES));
  }
  tp->comm_buf = tp->peer_buf[0];
  SB_CUDA(cudaMalloc((void**)&tp->local, 256 + COMM_ROWS * sizeof(int)));
  SB_CUDA(cudaMemset(tp->local, 0, 256 + COMM_ROWS * sizeof(int)));
  fill_comm_dev(ctx);
  return STRICTB200_OK;
}
static void fill_comm_dev(strictb200_ctx* ctx) {
  TpState* tp = ctx->tp;
  TpCommDev& d = tp->dev;
  for (int r = 0; r < ctx->tp_world; r++) {
    d.flags[r] = (int*)tp->peer_buf[r];
    d.data[r] = (float*)((char*)tp->peer_buf[r] + COMM_FLAG_BYTES);
    d.row_data[r] = (float*)((char*)tp->peer_buf[r] + COMM_ROW_OFFSET);
  }
  d.row_epoch = tp->local + 64;
  d.row_elems = COMM_ROW_ELEMS;
  d.max_rows = COMM_ROWS;
  d.epoch = tp->local;
  d.done = (unsigned*)(tp->local + 1);
  d.status = ctx->d_status;
  d.world = ctx->tp_world;
  d.rank = ctx->tp_rank;
  d.max_elems = COMM_MAX_ELEMS;
  d.wait_limit = 1u << 22;
  tp->opened = true;
}
int strictb200_tp_allreduce_rownorm(strictb200_ctx* ctx, const float* d_part, int splits, const float* d_sx, const float* d_sw,
                                    float* d_residual_f32, const float* d_gain, float eps, int64_t M, int64_t d, uint16_t* d_y,
                                    uint8_t* d_split, float* d_split_scale) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && d > 0 && d % 8 == 0 && d <= 16384 && splits >= 1, "bad shape");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(d_part && d_sx && d_sw && d_gain, "null pointer");
  SB_REQUIRE((d_split == nullptr) == (d_split_scale == nullptr), "the split output needs both its buffers");
  SB_REQUIRE(ctx->tp_world > 1, "tensor parallelism is not initialised on this context");
  if (!sb_tp_comm_fits(ctx, M, d)) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "tp_allreduce_rownorm needs open peer buffers and M*d <= 1M values");
  RowNormArgs a;
  a.comm = sb_tp_comm(ctx);
  a.part = d_part; a.splits = splits; a.sx = d_sx; a.sw = d_sw;
  a.residual_f32 = d_residual_f32; a.gain = d_gain; a.eps = eps;
  a.y = (bf16*)d_y; a.q = d_split; a.qscale = d_split_scale;
  return k_rownorm(ctx, a, M, d);
}
int strictb200_tp_info(strictb200_ctx* ctx, int* world, int* rank) {
  if (!ctx) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null context");
  if (world) *world = ctx->tp_world;
  if (rank) *rank = ctx->tp_rank;
  return STRICTB200_OK;
}
int strictb200_tp_allreduce_f32(strictb200_ctx* ctx, float* d_buf, int64_t count) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0, "negative count");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(d_buf, "null pointer");
  return sb_tp_allreduce_f32(ctx, d_buf, count);
}
}
