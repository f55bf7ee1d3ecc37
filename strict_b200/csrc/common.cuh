// Internal declarations shared by the translation units of libstrictb200.so.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <utility>

#include "../../include/strictb200.h"

struct TpState;     // tp.cpp

// All-reduce over peer memory (tp.cpp): every rank owns a buffer that all ranks of the box map
// (CUDA IPC). Passed to kernels by value. Two exchanges use it:
//   row-granular (the decode step's default): the row kernel that consumes the sum pushes each of
//     its values into the peers' buffers as one word whose two lowest mantissa bits carry the row's
//     epoch modulo 4, and polls its own buffer until the words of every peer carry the current tag
//     (row_data, row_epoch); sums are taken over the values with those two bits cleared;
//   whole-result (shapes the row exchange does not take): a publish kernel writes the rank's fp32
//     partial result into its own buffer and raises an epoch flag in every peer's buffer; the
//     consumer waits for all flags and adds the ranks' data in rank order with plain peer loads
//     (data, flags, epoch, done).
// Every wait is bounded by wait_limit polls; on expiry the kernel sets *status and goes on.
struct TpCommDev {
  float* data[8];   // rank r's data area, two epoch parities of max_elems floats each
  int* flags[8];    // rank r's flag area: flags[parity * 8 + source rank] = last epoch published
  int* epoch;       // this rank's epoch counter (device memory, advanced by the publish kernel)
  unsigned* done;   // this rank's block counter of the publish kernel
  int* status;      // host-visible error word
  int world, rank;
  long long max_elems;
  // Row-granular variant (the row kernel itself exchanges the sums): every value is pushed into
  // the peers' buffers as a word that carries its epoch tag, so a word validates itself and
  // neither fences nor separate flags are needed.
  float* row_data[8];   // rank r's packet area: [parity][source rank] areas of 2 * row_elems words (the first row_elems in use)
  int* row_epoch;       // this rank's per-row epoch counters (device memory, one writer per row)
  long long row_elems;  // values per (parity, source rank)
  int max_rows;
  unsigned wait_limit;  // polls before a wait gives up (the context's wait_limit option, copied at launch)
};
struct SbProfiler;  // model.cu
void sb_prof_split(strictb200_ctx*, int cls);  // model.cu: inside a profiled call, the following launches count for class `cls`

// Switches of a context. Each is read once from the environment (STRICTB200_<NAME IN CAPITALS>)
// when the context is created and can be changed afterwards with strictb200_set_option; no
// launch path reads the environment. -1 stands for the library's own choice.
struct SbOptions {
  int pdl = 1;                 // launch the decode-path kernels with programmatic dependent launch
  int attn_tc = -1;            // prefill attention: 0 mma.sync, 1 tcgen05 one query tile per block, 2 two tiles per block
  int gemm_pair = 1;           // many-token GEMM on SM pairs (0: the one-SM persistent kernel)
  int prefetch = 1;            // GEMMs request their first ring of weight tiles before the dependency wait
  int deep_ring = 1;           // few-token GEMM: a ring that fills the SM when the grid is one block per SM
  int attn_blocks_per_sm = 0;  // >0: size decode-attention key chunks for that many blocks per SM
  int split_target = 0;        // >0: blocks a few-token GEMM's K splits aim at
  int tp_two_shot = -1;        // fused all-reduce: 0 one shot, 1 two shots
  int wait_limit = 1 << 22;    // polls of a cross-rank wait before the kernel gives up and sets the error word
  int prefill_chunk = 16384;   // token rows per prefill chunk
  int fuse_rope = 0;           // decode step: QK-norm, RoPE and the cache append inside the attention kernel (bit-identical; measured no faster)
  int row_cluster = 4;         // blocks (one cluster) per row of the decode row kernels, where the row has 1024 columns per block; 0 or 1 = one block per row
  int attn_prefetch = 1;       // decode attention starts to load its first key/value tiles before the dependency wait
  int blur_rows = 0;           // rows of the image per block of the blur kernel; 0 = chosen from the image and the grid
  int host_timeout_ms = 0;     // >0: a synchronising call gives up after this long, aborts the NCCL communicator and returns ERR_TIMEOUT
};

// One-time set-up that belongs to a device (function attributes are set per device): run(device, f)
// calls f the first time it is reached for that device, under a lock, and again on a later call
// if it failed. Contexts on different devices, driven from different threads, each get their turn.
struct SbDeviceOnce {
  std::mutex mu;
  bool done[64] = {};
  template <typename F>
  cudaError_t run(int device, F&& f) {
    if (device < 0 || device >= 64) return f();
    std::lock_guard<std::mutex> lock(mu);
    if (done[device]) return cudaSuccess;
    cudaError_t e = f();
    if (e == cudaSuccess) done[device] = true;
    return e;
  }
};

struct strictb200_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  uint64_t launches = 0;
  // scratch for op-level entry points (quantised activations, split partials)
  void* ws = nullptr;
  size_t ws_bytes = 0;
  uint64_t rec_launches0 = 0;  // launch counter when a recording began
  void* ws2 = nullptr;  // second scratch (split-K partial results of the stand-alone GEMM entry)
  size_t ws2_bytes = 0;
  void* flush_buf = nullptr;
  size_t flush_bytes = 0;
  int tp_world = 1, tp_rank = 0;
  TpState* tp = nullptr;
  SbProfiler* prof = nullptr;
  int* h_status = nullptr;  // pinned, device-visible error word written by kernels whose bounded waits expired
  int* d_status = nullptr;
  void* gemm_ws = nullptr;  // stream-K tile counters + partial tiles of the tensor-memory GEMM
  size_t gemm_count_bytes = 0, gemm_part_bytes = 0;
  SbOptions opt;
  unsigned long long* trace_rec = nullptr;  // armed trace (strictb200_trace_begin): records, counter, capacity
  unsigned int* trace_count = nullptr;
  unsigned int trace_capacity = 0;
  // scratch of the prefill chunks (activations of up to opt.prefill_chunk token rows), grow-only
  void* prefill_ws = nullptr;
  size_t prefill_ws_bytes = 0;
  uint64_t ws_generation = 0;  // advanced whenever a scratch buffer is re-allocated (recorded sequences check it)
};

void sb_set_error(const std::string& msg);
int sb_fail(int code, const std::string& msg);
// Waits for the context's stream. Under tensor parallelism it also polls NCCL's asynchronous error
// state (a failed peer or link) and, with the host_timeout_ms option, gives up after that long; in
// both cases the communicator is aborted so that its kernels leave the GPU, and the call returns
// ERR_NCCL / ERR_TIMEOUT instead of hanging.
int sb_sync(strictb200_ctx* ctx, const char* what);
int sb_check_status(strictb200_ctx* ctx, const char* what);  // after a stream synchronise: ERR_TIMEOUT if a kernel's wait expired
int sb_ws(strictb200_ctx* ctx, size_t bytes, void** out);  // grow-only context scratch
int sb_ws2(strictb200_ctx* ctx, size_t bytes, void** out);  // a second one, for calls that already hold the first

#define SB_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return sb_fail(_e == cudaErrorMemoryAllocation ? STRICTB200_ERR_OOM : STRICTB200_ERR_CUDA, \
                     std::string(#expr) + ": " + cudaGetErrorString(_e));                      \
  } while (0)
#define SB_TRY(expr)            \
  do {                          \
    int _s = (expr);            \
    if (_s != STRICTB200_OK) return _s; \
  } while (0)
#define SB_REQUIRE(cond, msg) \
  do {                        \
    if (!(cond)) return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string(msg) + " (" #cond ")"); \
  } while (0)
#define SB_ENTER(ctx)                                                  \
  do {                                                                 \
    if (!(ctx)) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null context"); \
    SB_CUDA(cudaSetDevice((ctx)->device));                             \
  } while (0)
// after a kernel launch
#define SB_LAUNCHED(ctx)          \
  do {                            \
    (ctx)->launches++;            \
    SB_CUDA(cudaGetLastError());  \
  } while (0)

// ------------------------------------------------------------------ launchers (internal API)
// Every launcher enqueues on ctx->stream and returns a status.
typedef __nv_bfloat16 bf16;

// elementwise.cu
int k_ew_binary(strictb200_ctx*, int op, const float* a, const float* b, float* out, int64_t n);
int k_ew_program(strictb200_ctx*, const int32_t* h_code, int n_instr, const float* const* h_arrays, int n_arrays,
                 const float* h_scalars, int n_scalars, const float* h_consts, int n_consts, float* out, int64_t n);
int k_ew_program2(strictb200_ctx*, const int32_t* h_code, int n_instr, const float* const* h_arrays, int n_arrays,
                  const float* h_scalars, int n_scalars, const float* h_consts, int n_consts, float* out, int64_t n);
// gen.cu
int k_gen_normal_f32(strictb200_ctx*, uint64_t key, int64_t first, int64_t count, float std_, float* out);
int k_gen_normal_bf16(strictb200_ctx*, uint64_t key, int64_t first, int64_t count, float std_, bf16* out);
int k_gen_tokens(strictb200_ctx*, uint64_t key, int64_t count, uint32_t range, int32_t* out);
int k_gen_weight_e4m3(strictb200_ctx*, uint64_t key, int64_t row0, int64_t rows, int64_t K, int64_t col0, int64_t cols,
                      float std_, uint8_t* q, int64_t ldq, float* scale);
uint64_t sb_stream_key(uint64_t seed, uint64_t tensor);
// norm.cu
// Activations enter the FP8 GEMMs as two E4M3 terms, x = s*(hi + lo/16) with s a power of two.
// Row layout of the split buffer: tokens in groups of 8; group g occupies rows [16g, 16g+16):
// 8 hi rows then 8 lo rows, so that the hi and lo accumulators of a token land in the same
// thread (mma.sync n-tile pairs) / adjacent accumulator columns (tensor memory).
inline int64_t sb_qrows(int64_t M) { return 16 * ((M + 7) / 8); }
int k_quantize_rows(strictb200_ctx*, const bf16* x, int64_t M, int64_t K, int64_t ldx, uint8_t* q, float* scale);
// Single-term absmax/448 quantisation of weight rows (the tied LM head).
int k_quantize_weight_rows(strictb200_ctx*, const bf16* x, int64_t M, int64_t K, int64_t ldx, uint8_t* q, float* scale);
// Row op of the residual stream. For every token row:
//   y_in  = part ? sum over groups g of (sum over splits s of part[g][s][row]) * sx[g][row] * sw[col]   (fp32)
//         : x_f32 ? x_f32 : x_in (bf16)
//   resid = residual_f32 ? residual_f32 + y_in (fp32, stored back)
//         : residual ? bf16(residual + y_in) (stored back) : y_in
//   n     = bf16((resid * r) * gain) ; written as bf16 (y) and/or as the two-term E4M3 split (q, qscale)
struct RowNormArgs {
  const float* x_f32 = nullptr;      // [M,d] fp32 input (e.g. after an all-reduce)
  const bf16* x_in = nullptr;        // [M,d] (used when part and x_f32 are null)
  const float* part = nullptr;       // [groups][splits][M,d] fp32 raw accumulators
  int groups = 1, splits = 1;
  const float* sx = nullptr;         // [groups][M]
  const float* sw = nullptr;         // [d]
  const TpCommDev* comm = nullptr;   // input = sum over ranks of the published partial results (fused all-reduce)
  float* residual_f32 = nullptr;     // [M,d] fp32 residual stream, in/out, may be null
  bf16* residual = nullptr;          // [M,d] bf16 residual, in/out, may be null
  const float* gain = nullptr;       // [d]; null: only the residual update is done
  float eps = 1e-6f;
  bf16* y = nullptr;                 // [M,d] normalised bf16 output, may be null
  uint8_t* q = nullptr;              // split output [sb_qrows(M), d], may be null
  float* qscale = nullptr;           // [M]
};
int k_rownorm(strictb200_ctx*, const RowNormArgs& a, int64_t M, int64_t d);
int k_reduce_scale(strictb200_ctx*, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t N, float* out,
                   bf16* out_bf16 = nullptr);
int k_layernorm(strictb200_ctx*, const float* x, const float* g, const float* b, float eps, int64_t M, int64_t d, float* y);
int k_add_f32(strictb200_ctx*, float* x, const float* y, int64_t n);
int k_swiglu(strictb200_ctx*, const bf16* gate_up, const float* gate_up_f32, int64_t M, int64_t I, bf16* y, uint8_t* q, float* qscale);
// gate_up as split-K partials [splits][M][2I] + scales -> two-term split of silu(gate)*up
int k_swiglu_part(strictb200_ctx*, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t I, uint8_t* q,
                  float* qscale);
int k_gelu_tanh(strictb200_ctx*, const float* x, int64_t n, float* y);
#ifdef __CUDACC__
// tanh-approximated GELU in fp32 with the operation order of the element-wise kernel
__device__ __forceinline__ float sb_gelu_tanh(float v) {
  const float u = __fmul_rn(0.797884583f, __fadd_rn(v, __fmul_rn(0.044715f, __fmul_rn(__fmul_rn(v, v), v))));
  return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(u)));
}
#endif
// rope.cu
struct RopeArgs {
  const bf16* qkv = nullptr;      // [T, nqkv] bf16 (used when part and qkv_f32 are null)
  const float* qkv_f32 = nullptr; // [T, nqkv] fp32 projection result
  const float* part = nullptr;    // [splits][T, nqkv] raw accumulators
  int splits = 1;
  const float* sx = nullptr;      // [T]
  const float* sw = nullptr;      // [nqkv]
  const int32_t* seq = nullptr;   // [T] sequence of each row (null: row t is sequence t)
  const int32_t* pos = nullptr;   // [T] position of each row (null: pos = lens[seq])
  const int32_t* lens = nullptr;  // [B] current lengths (decode)
  const float* cos_t = nullptr;   // [max_pos, D/2]
  const float* sin_t = nullptr;
  const float* qgain = nullptr;
  const float* kgain = nullptr;
  float eps = 1e-6f;
  int Hq = 0, Hkv = 0, D = 128, maxlen = 0, max_pos = 0;
  bf16* q_out = nullptr;          // [T,Hq,D]
  bf16* kcache = nullptr;         // [B,Hkv,maxlen,D]
  bf16* vcache = nullptr;
};
int k_rope_qknorm_kvappend(strictb200_ctx*, const RopeArgs& a, int64_t T);
int sb_rope_table(strictb200_ctx*, int max_pos, int D, float theta, float** d_cos, float** d_sin);
// gemm_fp8.cu
struct GemmArgs {
  int64_t M = 0, N = 0, K = 0;
  const uint8_t* xq = nullptr;  // split activations [sb_qrows(M), K], row stride ldx
  int64_t ldx = 0;
  const float* sx = nullptr;    // [M]
  const uint8_t* wq = nullptr;  // [N,K], row stride ldw
  int64_t ldw = 0;
  const float* sw = nullptr;    // [N]
  void* out = nullptr;          // [M,N] bf16 or fp32 (when splits == 1)
  int out_f32 = 0;
  float* part = nullptr;        // [splits][M,N] raw accumulators (when splits > 1 or raw)
  int splits = 1;
  int raw = 0;                  // 1: always write raw accumulators to part, even for splits == 1
  int kernel = 0;               // 0 auto, 1 skinny, 2 mma.sync tiles, 3 tcgen05
  int i8 = 0;                   // 1: int8 weights and two int8 activation terms (gemm_int8.cu); part then holds int32 sums [splits][2][M,N]
};
int k_gemm_fp8(strictb200_ctx*, const GemmArgs& a);
int sb_gemm_pick_splits(strictb200_ctx*, int64_t M, int64_t N, int64_t K);
// gemm_f32.cu
int k_gemm_f32(strictb200_ctx*, int64_t M, int64_t N, int64_t K, const float* x, const float* w, const float* bias, float* y,
               int accumulate);
// attention.cu
int k_attn_prefill(strictb200_ctx*, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, const int32_t* past,
                   const int32_t* qstart, int B, int S, int64_t q_rows, int Hq, int Hkv, int D, int maxlen, float scale, bf16* out);
size_t sb_attn_decode_scratch(int B, int Hq, int D, int nsplit);
int sb_attn_decode_splits(strictb200_ctx*, int B, int Hkv, int maxlen);
int sb_attn_decode_chunk(strictb200_ctx*, int B, int Hkv, int maxlen, int len_plan);  // keys per block for sequences of about len_plan keys (at most 8 chunks cover maxlen)
// rope != null: the queries and the new token's key/value rows are computed inside the attention kernel from the qkv
// projection's partial results (what k_rope_qknorm_kvappend would do in a kernel of its own); q is then unused
int k_attn_decode(strictb200_ctx*, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, int len_add, int B, int Hq,
                  int Hkv, int D, int maxlen, float scale, int nsplit, float* scratch, bf16* out, uint8_t* q_out, float* qscale_out,
                  const RopeArgs* rope = nullptr, int chunk = 0);
int k_attn_f32(strictb200_ctx*, const float* qkv, float* kc, float* vc, const int32_t* seq, const int32_t* pos, const int32_t* lens,
               int64_t T, int H, int D, int maxlen, float scale, float* out);
// sampling.cu
int k_embedding_bf16(strictb200_ctx*, const bf16* table, const int32_t* ids, int64_t T, int64_t d, int64_t vocab, bf16* out);
int k_embedding_bf16_f32(strictb200_ctx*, const bf16* table, const int32_t* ids, int64_t T, int64_t d, int64_t vocab, float* out);
int k_embedding_f32(strictb200_ctx*, const float* wte, const float* wpe, const int32_t* ids, const int32_t* pos, const int32_t* lens,
                    int64_t T, int64_t d, int64_t vocab, int max_pos, float* out);
int k_argmax(strictb200_ctx*, const float* x, int64_t M, int64_t N, int64_t ldx, int32_t* out, float* val_out, void* scratch);
size_t sb_argmax_scratch(int64_t M, int64_t N);  // bytes of chunk winners for the two-stage pick
int k_gather_rows(strictb200_ctx*, const void* src, const int32_t* rows, int64_t n_rows, int64_t row_bytes, void* dst);
int k_add_i32(strictb200_ctx*, int32_t* x, const int32_t* inc, int32_t c, int64_t n);
int k_f32_to_bf16(strictb200_ctx*, const float* x, int64_t n, bf16* y);
int k_bf16_to_f32(strictb200_ctx*, const bf16* x, int64_t n, float* y);
// tp.cpp
const TpCommDev* sb_tp_comm(strictb200_ctx*);  // null unless the peer buffers were opened
bool sb_tp_comm_fits(strictb200_ctx*, int64_t M, int64_t d);  // the peer-memory all-reduce takes an [M,d] result
bool sb_tp_row_exchange_ok(strictb200_ctx*, int64_t M, int64_t d, int two_shot);  // ... with the row-granular exchange (one row width per context)
// out[m,n] = (sum_s part[s][m,n]) * sx[m] * sw[n] written to this rank's peer buffer, then published
int k_tp_publish(strictb200_ctx*, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t N);
int sb_tp_allreduce_f32(strictb200_ctx*, float* buf, int64_t count);
int sb_tp_allgather(strictb200_ctx*, const void* send, void* recv, int64_t bytes_per_rank);
void sb_tp_destroy(strictb200_ctx*);
int sb_tp_async_error(strictb200_ctx*);  // 0 = none; else the NCCL result code of the communicator's asynchronous error
void sb_tp_abort(strictb200_ctx*);       // ncclCommAbort: stops the communicator's kernels; the communicator is unusable afterwards

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__
// Programmatic dependent launch. A kernel launched through sb_launch may begin while its
// predecessor in the stream is still running: pdl_trigger() lets the successor start launching,
// pdl_wait() blocks until the predecessor has completed and its writes are visible. Every such
// kernel calls pdl_wait() before it reads or writes anything another kernel touches (so the
// ordering stays transitive along the stream); only reads of constants (weights) may precede it.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Diagnostics: per-block time stamps of the decode step's kernels. While a trace is armed
// (strictb200_trace_begin) thread 0 of every block of an instrumented kernel records the global
// timer at block start, after the dependency wait and at block end, with the SM it ran on; the
// host reads the records back (strictb200_trace_end). The pointer lives in a device variable of
// each translation unit (read at run time, so a recorded CUDA graph can be traced as it is); when
// it is null a block pays one cached load.
struct SbTraceDev {
  unsigned long long* rec;  // [capacity][8]: start, after the wait, end, kernel id | tag << 8 | SM << 48, three optional marks inside the kernel, 0
  unsigned int* count;
  unsigned int capacity;
};
static __device__ SbTraceDev sb_trace_dev;
#define SB_TRACE_TU(name) \
  int sb_trace_set_##name(const SbTraceDev& t) { return cudaMemcpyToSymbol(sb_trace_dev, &t, sizeof t) == cudaSuccess ? 0 : 1; }
enum { SB_K_GEMM = 1, SB_K_ROWNORM = 2, SB_K_ROPE = 3, SB_K_ATTN = 4, SB_K_COMBINE = 5, SB_K_SWIGLU = 6, SB_K_ROWNORM_TP = 7 };
__device__ __forceinline__ unsigned long long sb_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void sb_trace_emit(int kid, uint32_t tag, const unsigned long long* marks) {
  if (!marks[0]) return;
  const unsigned long long t2 = sb_globaltimer();
  unsigned int smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  const unsigned int i = atomicAdd(sb_trace_dev.count, 1u);
  if (i < sb_trace_dev.capacity) {
    unsigned long long* r = sb_trace_dev.rec + (size_t)i * 8;
    r[0] = marks[0]; r[1] = marks[1]; r[2] = t2;
    r[3] = (unsigned long long)kid | ((unsigned long long)tag << 8) | ((unsigned long long)smid << 48);
    r[4] = marks[2]; r[5] = marks[3]; r[6] = marks[4]; r[7] = 0;
  }
}
// In a kernel: SB_TRACE_BEGIN() first, SB_TRACE_WAITED() by thread 0 right after its pdl_wait(), SB_TRACE_END(id, tag) last;
// SB_TRACE_MARK(0..2) stamps a point in between (as thread 0 reaches it).
#define SB_TRACE_BEGIN()                                 \
  __shared__ unsigned long long sb_tr_[5];               \
  if (threadIdx.x == 0) {                                \
    sb_tr_[0] = sb_trace_dev.rec ? sb_globaltimer() : 0; \
    sb_tr_[1] = sb_tr_[2] = sb_tr_[3] = sb_tr_[4] = 0;   \
  }
#define SB_TRACE_WAITED() \
  if (threadIdx.x == 0 && sb_tr_[0]) sb_tr_[1] = sb_globaltimer();
#define SB_TRACE_MARK(i) \
  if (threadIdx.x == 0 && sb_tr_[0]) sb_tr_[2 + (i)] = sb_globaltimer();
#define SB_TRACE_END(kid, tag) \
  if (threadIdx.x == 0) sb_trace_emit(kid, (uint32_t)(tag), sb_tr_);
// L2 eviction policy for data that is read exactly once per step (weights, the KV cache): such
// lines are the first to be replaced, so the 126 MB L2 keeps the small tensors the kernels hand
// to each other, the scale/gain vectors and the kernels' own instructions resident.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
template <typename... KArgs, typename... Args>
inline cudaError_t sb_launch(strictb200_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// Same, as thread-block clusters of `cluster` blocks (the grid must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t sb_launch_cluster(strictb200_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt.pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// One-value-per-block exchange inside a thread-block cluster of at most 8 blocks: every block
// pushes its value into the others' shared memory with st.async, which also completes bytes on
// the receiver's mbarrier, so a block waits only for the values it needs and nobody reads a
// block that may already have left (measured about 0.4 us, against 0.9 us for a cluster
// barrier plus remote reads plus a second barrier before exit).
struct ClusterExchange {
  float slot[2][8];
  unsigned long long bar[2];  // one barrier per exchange: a fast block's second value must not count for a slow block's first wait
};
// All threads of all blocks call this once at kernel start (before any long wait).
__device__ __forceinline__ void cluster_exchange_init(ClusterExchange* x) {
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&x->bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&x->bar[1])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
// All threads of all blocks call this with a block-uniform value, at most once per `which` (0,
// then 1); returns false if the other blocks' values did not arrive within the spin limit
// (slot[which][] is then incomplete). Afterwards slot[which][r] holds block r's value in every block.
__device__ __forceinline__ bool cluster_exchange(ClusterExchange* x, float v, uint32_t nblocks, uint32_t rank, int which = 0) {
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&x->bar[which]);
  if (threadIdx.x == 0) {
    x->slot[which][rank] = v;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(4u * (nblocks - 1)) : "memory");
  }
  if (which == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every block's barriers are initialised
  if (threadIdx.x < nblocks && threadIdx.x != rank) {
    uint32_t rslot, rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rslot) : "r"((uint32_t)__cvta_generic_to_shared(&x->slot[which][rank])), "r"(threadIdx.x));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar), "r"(threadIdx.x));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(rslot), "r"(__float_as_uint(v)), "r"(rbar) : "memory");
  }
  uint32_t done = 0;
  for (uint32_t spins = 0; !done && spins < (1u << 20); spins++)
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(0u) : "memory");
  return done != 0;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions over blockDim.x threads (multiple of 32, <= 1024). `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : -INFINITY;
  return warp_max(t);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
// E4M3 encode, round-to-nearest-even, saturating to +-448 (cvt.rn.satfinite.e4m3x2.f32).
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
  return (uint32_t)r;
}
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  return f32x2_to_e4m3x2(a, b) | (f32x2_to_e4m3x2(c, d) << 16);
}
// E4M3 pair -> two floats (exact; through f16x2).
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t pair) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)pair));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// Exponent e of the power-of-two row scale: the smallest 2^e with amax/2^e <= 448.
__device__ __forceinline__ int sb_scale_exponent(float amax) {
  if (!(amax >= 7.888609e-31f)) return 0;
  uint32_t b = __float_as_uint(amax);
  int E = (int)((b >> 23) & 255) - 126;
  return (b & 0x7FFFFFu) <= 0x600000u ? E - 9 : E - 8;
}
__device__ __forceinline__ float sb_pow2(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }
// Two-term split of 8 values already divided by the row scale: hi = e4m3(v), lo = e4m3(16*(v-hi)).
__device__ __forceinline__ void sb_split8(const float* v, uint2* hi, uint2* lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    h[i] = f32x2_to_e4m3x2(v[2 * i], v[2 * i + 1]);
    float2 hv = e4m3x2_to_f32x2(h[i]);
    l[i] = f32x2_to_e4m3x2(__fmul_rn(16.0f, __fsub_rn(v[2 * i], hv.x)), __fmul_rn(16.0f, __fsub_rn(v[2 * i + 1], hv.y)));
  }
  *hi = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
  *lo = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
}
// Store the split of 8 consecutive columns of token row m into the split buffer q [*, K].
__device__ __forceinline__ void sb_store_split8(uint8_t* q, int64_t K, int64_t m, int64_t k, const float* v, float inv) {
  float t[8];
#pragma unroll
  for (int i = 0; i < 8; i++) t[i] = __fmul_rn(v[i], inv);
  uint2 hi, lo;
  sb_split8(t, &hi, &lo);
  int64_t row = 16 * (m >> 3) + (m & 7);
  *(uint2*)(q + row * K + k) = hi;
  *(uint2*)(q + (row + 8) * K + k) = lo;
}
// The same for 4 consecutive columns.
__device__ __forceinline__ void sb_store_split4(uint8_t* q, int64_t K, int64_t m, int64_t k, const float* v, float inv) {
  uint32_t h[2], l[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    float a = __fmul_rn(v[2 * i], inv), b = __fmul_rn(v[2 * i + 1], inv);
    h[i] = f32x2_to_e4m3x2(a, b);
    float2 hv = e4m3x2_to_f32x2(h[i]);
    l[i] = f32x2_to_e4m3x2(__fmul_rn(16.0f, __fsub_rn(a, hv.x)), __fmul_rn(16.0f, __fsub_rn(b, hv.y)));
  }
  int64_t row = 16 * (m >> 3) + (m & 7);
  *(uint32_t*)(q + row * K + k) = h[0] | (h[1] << 16);
  *(uint32_t*)(q + (row + 8) * K + k) = l[0] | (l[1] << 16);
}
#endif
