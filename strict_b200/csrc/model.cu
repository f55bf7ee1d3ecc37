// Model and KV-cache objects: weights resident in HBM, the prefill and decode schedules of
// the GPT-2 (fp32) and Qwen3 (E4M3 weights, bf16 activations) stacks, tensor-parallel shards,
// and the CUDA-graph replay of the decode step.
//
// Data layout in HBM (per rank):
//   Qwen3 linear weights   E4M3 [N_local, K_local] row-major (K contiguous) + fp32 scale[N_local]
//     wqkv  = [q heads | k heads | v heads] of this rank, K = d_model
//     wo    = all d_model rows, K = this rank's slice of Hq*D (column shard)
//     wgu   = [gate rows | up rows] of this rank, K = d_model
//     wdown = all d_model rows, K = this rank's slice of d_ff
//     head  = this rank's slice of the vocabulary rows
//   embedding bf16 [V, d] (replicated); norm gains fp32; RoPE cos/sin fp32 [max_pos, D/2]
//   KV cache bf16 [L][B][Hkv_local][maxlen][D] for K and for V (fp32 for GPT-2)
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

enum { T_NORM1 = 0, T_Q = 1, T_K = 2, T_V = 3, T_QN = 4, T_KN = 5, T_O = 6, T_NORM2 = 7, T_GATE = 8, T_UP = 9, T_DOWN = 10 };
enum { G_EMBED = 1, G_WPE = 2, G_HEAD = 3, G_NORMF = 4 };
inline uint64_t layer_tensor(int l, int kind) { return 16ull * (uint64_t)(l + 1) + (uint64_t)kind; }

struct QW {
  uint8_t* q = nullptr;
  float* s = nullptr;
  int64_t N = 0, K = 0;
};
struct FW {
  float* w = nullptr;
  float* b = nullptr;
  int64_t N = 0, K = 0;
};
struct LayerW {
  float *norm1_g = nullptr, *norm1_b = nullptr, *norm2_g = nullptr, *norm2_b = nullptr, *qn_g = nullptr, *kn_g = nullptr;
  QW wqkv, wo, wgu, wdown;
  FW fqkv, fo, ffc, fproj;
};

}  // namespace

struct strictb200_model {
  strictb200_ctx* ctx = nullptr;
  strictb200_model_config c;
  int world = 1, rank = 0;
  int Hq_l = 0, Hkv_l = 0;
  int64_t I_l = 0, V_l = 0;
  std::vector<LayerW> L;
  bf16* embed = nullptr;   // Qwen3
  float* wte = nullptr;    // GPT-2
  float* wpe = nullptr;
  float *normf_g = nullptr, *normf_b = nullptr;
  QW head;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  std::vector<void*> allocs;
  uint64_t weight_bytes = 0;  // bytes of the tensors a decode step streams (linears + head)
  int use_graph = 1;
};

struct strictb200_kv {
  strictb200_model* m = nullptr;
  int B = 0, maxlen = 0;
  void *k = nullptr, *v = nullptr;
  size_t layer_stride = 0;  // elements per layer
  int32_t* d_lens = nullptr;
  std::vector<int32_t> h_lens;
  // decode state
  int32_t *d_ids = nullptr, *d_next = nullptr, *d_hist = nullptr;
  int hist_cap = 0;
  void* dec = nullptr;  // one allocation carved into the decode buffers
  size_t dec_bytes = 0;
  cudaGraphExec_t graph = nullptr;
  uint64_t graph_kernels = 0;
  bool warmed = false;
  int nsplit = 1;        // key chunks per sequence of the decode attention, and
  int chunk = 0;         // keys per chunk: planned for the lengths the cache holds now (plan_attention), 0 = not planned yet
  int plan_until = 0;    // the plan is kept until a sequence grows beyond this length
  std::vector<void*> allocs;
};

namespace {

template <typename T>
int dalloc(strictb200_model* m, T** p, size_t count) {
  *p = nullptr;
  if (!count) return STRICTB200_OK;
  void* v;
  SB_CUDA(cudaMalloc(&v, count * sizeof(T)));
  m->allocs.push_back(v);
  *p = (T*)v;
  return STRICTB200_OK;
}
int fill_f32(strictb200_ctx* ctx, float* p, size_t n, float v) {
  std::vector<float> h(n, v);
  SB_CUDA(cudaMemcpyAsync(p, h.data(), n * 4, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}
int alloc_qw(strictb200_model* m, QW& w, int64_t N, int64_t K) {
  w.N = N; w.K = K;
  SB_TRY(dalloc(m, &w.q, (size_t)N * K));
  SB_TRY(dalloc(m, &w.s, (size_t)N));
  m->weight_bytes += (uint64_t)N * K + (uint64_t)N * 4;
  return STRICTB200_OK;
}
int alloc_fw(strictb200_model* m, FW& w, int64_t N, int64_t K) {
  w.N = N; w.K = K;
  SB_TRY(dalloc(m, &w.w, (size_t)N * K));
  SB_TRY(dalloc(m, &w.b, (size_t)N));
  SB_TRY(fill_f32(m->ctx, w.b, N, 0.f));
  m->weight_bytes += (uint64_t)N * K * 4 + (uint64_t)N * 4;
  return STRICTB200_OK;
}

// ------------------------------------------------------------------ decode buffers
struct DecBuf {
  float* x;        // [B,d] fp32 residual stream
  uint8_t* aq;     // [B, max(d, Hq_l*D, I_l)] quantised GEMM input
  float* sa;       // [B]
  float* part;     // split-K partials, max over the layer's GEMMs
  bf16* qb;        // [B,Hq_l,D]
  bf16* att;       // [B,Hq_l*D]
  float* gu;       // [B,2*I_l] fp32 gate/up projection
  float* attn_ws;  // split-KV partials
  float* red;      // [B,d] fp32 all-reduce buffer (TP)
  float* logits;   // [B,V_l] (+ [world][B,V_l] gathered when TP)
  float* logits_all;
  float* xf;       // GPT-2: [B,d] fp32 residual
  float* af;       // GPT-2: [B,max(3d, d_ff)]
  float* bf;       // GPT-2: second scratch
  float* best_val; // [world][B]
  int32_t* best_idx;
  void* am_ws;     // chunk winners of the two-stage argmax
};

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct Carver {
  char* base;
  size_t off = 0;
  template <typename T>
  T* take(size_t count) {
    T* p = base ? (T*)(base + off) : nullptr;
    off += align256(count * sizeof(T));
    return p;
  }
};

struct GemmPlan { int splits; };

int plan_splits(strictb200_model* m, int64_t M, int64_t N, int64_t K) { return sb_gemm_pick_splits(m->ctx, M, N, K); }
// K splits of the decode gate/up projection: 1 (the GEMM writes the scaled fp32 result) unless the
// shard is so narrow that its tiles leave most SMs idle; the SwiGLU kernel sums at most 4 partials.
int plan_gate_up_splits(strictb200_model* m, int64_t M) {
  const int64_t tiles = (2 * (int64_t)m->I_l + 127) / 128;
  if (M > 32 || m->I_l % 128 || tiles >= m->ctx->sm_count) return 1;
  int s = sb_gemm_pick_splits(m->ctx, M, 2 * (int64_t)m->I_l, m->c.d_model);
  return s > 4 ? 4 : s;
}

void carve_decode(strictb200_kv* kv, char* base, DecBuf* out, size_t* total) {
  strictb200_model* m = kv->m;
  const auto& c = m->c;
  int64_t B = kv->B, d = c.d_model, D = c.head_dim;
  Carver cv{base};
  DecBuf b{};
  if (c.arch == STRICTB200_QWEN3) {
    int64_t nq = (int64_t)m->Hq_l * D, nqkv = nq + 2 * (int64_t)m->Hkv_l * D;
    int64_t amax = std::max<int64_t>(d, std::max<int64_t>(nq, m->I_l));
    b.x = cv.take<float>(B * d);
    b.aq = cv.take<uint8_t>(sb_qrows(B) * amax);
    b.sa = cv.take<float>(B);
    size_t p1 = (size_t)plan_splits(m, B, nqkv, d) * B * nqkv;
    size_t p2 = (size_t)plan_splits(m, B, d, nq) * B * d;
    size_t p3 = (size_t)plan_splits(m, B, d, m->I_l) * B * d;
    size_t p4 = (size_t)plan_gate_up_splits(m, B) * B * 2 * m->I_l;
    b.part = cv.take<float>(std::max(std::max(p1, p2), std::max(p3, p4)));
    b.qb = cv.take<bf16>(B * nq);
    b.att = cv.take<bf16>(B * nq);
    b.gu = cv.take<float>(B * 2 * m->I_l);
    // room for the most chunks any plan uses (8, or one per 64-key tile of a short cache)
    b.attn_ws = cv.take<float>(sb_attn_decode_scratch((int)B, m->Hq_l, (int)D, std::min(8, (kv->maxlen + 63) / 64)) / sizeof(float));
    b.red = cv.take<float>(B * d);
  } else {
    int64_t w = std::max<int64_t>(3 * d, c.d_ff);
    b.xf = cv.take<float>(B * d);
    b.af = cv.take<float>(B * w);
    b.bf = cv.take<float>(B * w);
  }
  b.logits = cv.take<float>(B * m->V_l);
  b.logits_all = cv.take<float>(m->world > 1 ? (size_t)m->world * B * m->V_l : 1);
  b.best_val = cv.take<float>((size_t)m->world * B);
  b.best_idx = cv.take<int32_t>((size_t)m->world * B);
  b.am_ws = cv.take<uint8_t>(sb_argmax_scratch(B, m->V_l));
  *out = b;
  *total = cv.off;
}

// Pick the global argmax from per-rank (value, index) pairs; rank r's indices are offset by r*V_l.
__global__ void merge_argmax_kernel(const float* __restrict__ vals, const int32_t* __restrict__ idx, int world, int B, int V_l,
                                    int32_t* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float best = -INFINITY;
  int bi = 0;
  for (int r = 0; r < world; r++) {
    float v = vals[r * B + b];
    int i = idx[r * B + b] + r * V_l;
    if (v > best) { best = v; bi = i; }  // ranks ascend, so ties keep the lowest index
  }
  out[b] = bi;
}
// logits_all [world][B,V_l] -> [B, world*V_l]
__global__ void interleave_logits_kernel(const float* __restrict__ in, int world, int B, int64_t V_l, float* __restrict__ out) {
  int64_t total = (int64_t)world * B * V_l, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t r = i / (B * V_l), rem = i - r * B * V_l, b = rem / V_l, v = rem - b * V_l;
    out[b * world * V_l + r * V_l + v] = in[i];
  }
}

// ------------------------------------------------------------------ shared pieces
int run_gemm(strictb200_model* m, int64_t M, const QW& w, const uint8_t* aq, const float* sa, void* out, int out_f32, float* part,
             int splits, int raw) {
  GemmArgs g;
  g.M = M; g.N = w.N; g.K = w.K;
  g.xq = aq; g.ldx = w.K; g.sx = sa; g.wq = w.q; g.ldw = w.K; g.sw = w.s;
  g.out = out; g.out_f32 = out_f32; g.part = part; g.splits = splits; g.raw = raw;
  return k_gemm_fp8(m->ctx, g);
}

// Head + greedy pick for M rows whose quantised final-norm output is in (aq, sa).
int head_and_pick(strictb200_model* m, int64_t M, const uint8_t* aq, const float* sa, DecBuf& b, int32_t* d_next, float* h_logits,
                  int stride_B /* rows the logits buffers were carved for */) {
  strictb200_ctx* ctx = m->ctx;
  SB_TRY(run_gemm(m, M, m->head, aq, sa, b.logits, 1, nullptr, 1, 0));
  if (m->world == 1) {
    SB_TRY(k_argmax(ctx, b.logits, M, m->V_l, m->V_l, d_next, nullptr, b.am_ws));
    if (h_logits) SB_CUDA(cudaMemcpyAsync(h_logits, b.logits, (size_t)M * m->V_l * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return STRICTB200_OK;
  }
  (void)stride_B;
  float* my_val = b.best_val + (size_t)m->rank * M;
  int32_t* my_idx = b.best_idx + (size_t)m->rank * M;
  SB_TRY(k_argmax(ctx, b.logits, M, m->V_l, m->V_l, my_idx, my_val, b.am_ws));
  SB_TRY(sb_tp_allgather(ctx, my_val, b.best_val, M * 4));
  SB_TRY(sb_tp_allgather(ctx, my_idx, b.best_idx, M * 4));
  merge_argmax_kernel<<<(unsigned)((M + 127) / 128), 128, 0, ctx->stream>>>(b.best_val, b.best_idx, m->world, (int)M, (int)m->V_l, d_next);
  SB_LAUNCHED(ctx);
  if (h_logits) {
    SB_TRY(sb_tp_allgather(ctx, b.logits, b.logits_all, M * m->V_l * 4));
    void* tmp;  // grow-only context scratch: no allocation once it has reached this size
    SB_TRY(sb_ws2(ctx, (size_t)m->world * M * m->V_l * 4, &tmp));
    interleave_logits_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(b.logits_all, m->world, (int)M, m->V_l, (float*)tmp);
    SB_LAUNCHED(ctx);
    SB_CUDA(cudaMemcpyAsync(h_logits, tmp, (size_t)m->world * M * m->V_l * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return STRICTB200_OK;
}

bf16* kv_k(strictb200_kv* kv, int l) { return (bf16*)kv->k + (size_t)l * kv->layer_stride; }
bf16* kv_v(strictb200_kv* kv, int l) { return (bf16*)kv->v + (size_t)l * kv->layer_stride; }
float* kv_kf(strictb200_kv* kv, int l) { return (float*)kv->k + (size_t)l * kv->layer_stride; }
float* kv_vf(strictb200_kv* kv, int l) { return (float*)kv->v + (size_t)l * kv->layer_stride; }

// ------------------------------------------------------------------ per-class device timing
// When ctx->prof is set, every call of the decode body is bracketed by a pair of CUDA events
// tagged with its kernel class; strictb200_profile_decode sums them up afterwards.
struct ProfSpan { int cls; cudaEvent_t a, b; };
}  // namespace
struct SbProfiler {
  std::vector<ProfSpan> spans;
  std::vector<cudaEvent_t> pool;
  size_t used = 0;
  ProfSpan* open = nullptr;  // the span of the call that is being made
  cudaEvent_t get() {
    if (used == pool.size()) { cudaEvent_t e; cudaEventCreate(&e); pool.push_back(e); }
    return pool[used++];
  }
};
// Inside a bracketed call: what is launched from here on belongs to class `cls` (a call that
// launches kernels of two classes, e.g. the attention kernel and the merge of its key chunks).
void sb_prof_split(strictb200_ctx* ctx, int cls) {
  SbProfiler* p = ctx->prof;
  if (!p || !p->open) return;
  cudaEvent_t e = p->get();
  cudaEventRecord(e, ctx->stream);
  p->spans.push_back(ProfSpan{p->open->cls, p->open->a, e});
  p->open->cls = cls;
  p->open->a = e;
}
namespace {
template <typename F>
int prof(strictb200_ctx* ctx, int cls, F&& f) {
  SbProfiler* p = ctx->prof;
  if (!p) return f();
  ProfSpan sp{cls, p->get(), p->get()};
  cudaEventRecord(sp.a, ctx->stream);
  p->open = &sp;
  int st = f();
  p->open = nullptr;
  cudaEventRecord(sp.b, ctx->stream);
  p->spans.push_back(sp);
  return st;
}
#define PROF(cls, expr) SB_TRY(prof(ctx, cls, [&]() -> int { return (expr); }))

// ------------------------------------------------------------------ Qwen3 decode step body
// Everything below is enqueued on the stream with device-resident state only, so the whole
// body can be captured into a CUDA graph.
int qwen_decode_body(strictb200_model* m, strictb200_kv* kv, DecBuf& b) {
  strictb200_ctx* ctx = m->ctx;
  const auto& c = m->c;
  const int64_t B = kv->B, d = c.d_model, D = c.head_dim;
  const int64_t nq = (int64_t)m->Hq_l * D, nqkv = nq + 2 * (int64_t)m->Hkv_l * D;
  const float scale = 1.0f / sqrtf((float)D);
  const bool tp = m->world > 1;
  PROF(STRICTB200_K_EMBED, k_embedding_bf16_f32(ctx, m->embed, kv->d_ids, B, d, c.vocab, b.x));
  {
    RowNormArgs a;
    a.x_f32 = b.x; a.gain = m->L[0].norm1_g; a.eps = c.eps; a.q = b.aq; a.qscale = b.sa;
    PROF(STRICTB200_K_ROWNORM, k_rownorm(ctx, a, B, d));
  }
  for (int l = 0; l < c.n_layers; l++) {
    LayerW& w = m->L[l];
    // qkv projection -> raw split-K partials, consumed by the rope kernel
    int s1 = plan_splits(m, B, nqkv, d);
    PROF(STRICTB200_K_GEMM_QKV, run_gemm(m, B, w.wqkv, b.aq, b.sa, nullptr, 0, b.part, s1, 1));
    RopeArgs r;
    r.part = b.part; r.splits = s1; r.sx = b.sa; r.sw = w.wqkv.s; r.lens = kv->d_lens;
    r.cos_t = m->rope_cos; r.sin_t = m->rope_sin; r.qgain = w.qn_g; r.kgain = w.kn_g; r.eps = c.eps;
    r.Hq = m->Hq_l; r.Hkv = m->Hkv_l; r.D = (int)D; r.maxlen = kv->maxlen; r.max_pos = c.max_pos;
    r.q_out = b.qb; r.kcache = kv_k(kv, l); r.vcache = kv_v(kv, l);
    // QK-norm, RoPE and the cache append inside the attention kernel (one kernel less per layer), or as a kernel of their own.
    // The merge kernel overwrites b.sa (the o_proj operand's scales) only after every attention block has read it.
    const bool fuse_rope = ctx->opt.fuse_rope && s1 <= 8 && m->Hq_l / m->Hkv_l <= 16;
    if (!fuse_rope) PROF(STRICTB200_K_ROPE, k_rope_qknorm_kvappend(ctx, r, B));
    // split-KV attention over len+1 keys; the combine emits the quantised o_proj input
    PROF(STRICTB200_K_ATTN, k_attn_decode(ctx, b.qb, kv_k(kv, l), kv_v(kv, l), kv->d_lens, 1, (int)B, m->Hq_l, m->Hkv_l, (int)D, kv->maxlen,
                                          scale, kv->nsplit, b.attn_ws, b.att, b.aq, b.sa, fuse_rope ? &r : nullptr, kv->chunk));
    // o_proj -> partials -> (all-reduce) -> residual + norm2 + quantise
    int s2 = plan_splits(m, B, d, nq);
    PROF(STRICTB200_K_GEMM_O, run_gemm(m, B, w.wo, b.aq, b.sa, nullptr, 0, b.part, s2, 1));
    {
      RowNormArgs a;
      if (tp && sb_tp_comm_fits(ctx, B, d)) {
        // all-reduce over peer memory inside the row kernel that consumes it (NCCL below when the batch does not fit the peer buffers)
        a.comm = sb_tp_comm(ctx);
        a.part = b.part; a.splits = s2; a.sx = b.sa; a.sw = w.wo.s;
      } else if (tp) {
        PROF(STRICTB200_K_ROWNORM, k_reduce_scale(ctx, b.part, s2, b.sa, w.wo.s, B, d, b.red));
        PROF(STRICTB200_K_ALLREDUCE, sb_tp_allreduce_f32(ctx, b.red, B * d));
        a.x_f32 = b.red;
      } else {
        a.part = b.part; a.splits = s2; a.sx = b.sa; a.sw = w.wo.s;
      }
      a.residual_f32 = b.x; a.gain = w.norm2_g; a.eps = c.eps; a.q = b.aq; a.qscale = b.sa;
      PROF(STRICTB200_K_ROWNORM, k_rownorm(ctx, a, B, d));
    }
    // gate/up -> bf16, SwiGLU + quantise, down -> partials -> residual + next norm + quantise
    const int s3 = plan_gate_up_splits(m, B);
    if (s3 > 1) {
      // narrow shard: K splits so that the grid covers the GPU; SwiGLU sums the partials (every
      // block of a row has read the row's input scale before the row's new scale is written)
      PROF(STRICTB200_K_GEMM_GU, run_gemm(m, B, w.wgu, b.aq, b.sa, nullptr, 0, b.part, s3, 1));
      PROF(STRICTB200_K_SWIGLU, k_swiglu_part(ctx, b.part, s3, b.sa, w.wgu.s, B, m->I_l, b.aq, b.sa));
    } else {
      PROF(STRICTB200_K_GEMM_GU, run_gemm(m, B, w.wgu, b.aq, b.sa, b.gu, 1, nullptr, 1, 0));
      PROF(STRICTB200_K_SWIGLU, k_swiglu(ctx, nullptr, b.gu, B, m->I_l, nullptr, b.aq, b.sa));
    }
    int s4 = plan_splits(m, B, d, m->I_l);
    PROF(STRICTB200_K_GEMM_DOWN, run_gemm(m, B, w.wdown, b.aq, b.sa, nullptr, 0, b.part, s4, 1));
    {
      RowNormArgs a;
      if (tp && sb_tp_comm_fits(ctx, B, d)) {
        a.comm = sb_tp_comm(ctx);
        a.part = b.part; a.splits = s4; a.sx = b.sa; a.sw = w.wdown.s;
      } else if (tp) {
        PROF(STRICTB200_K_ROWNORM, k_reduce_scale(ctx, b.part, s4, b.sa, w.wdown.s, B, d, b.red));
        PROF(STRICTB200_K_ALLREDUCE, sb_tp_allreduce_f32(ctx, b.red, B * d));
        a.x_f32 = b.red;
      } else {
        a.part = b.part; a.splits = s4; a.sx = b.sa; a.sw = w.wdown.s;
      }
      a.residual_f32 = b.x;
      a.gain = l + 1 < c.n_layers ? m->L[l + 1].norm1_g : m->normf_g;
      a.eps = c.eps; a.q = b.aq; a.qscale = b.sa;
      PROF(STRICTB200_K_ROWNORM, k_rownorm(ctx, a, B, d));
    }
  }
  PROF(STRICTB200_K_HEAD, head_and_pick(m, B, b.aq, b.sa, b, kv->d_next, nullptr, (int)B));
  PROF(STRICTB200_K_EMBED, k_add_i32(ctx, kv->d_lens, nullptr, 1, B));
  return STRICTB200_OK;
}

// ------------------------------------------------------------------ GPT-2 rows (prefill chunk or decode)
// xf [T,d] must already hold wte[id]+wpe[pos]. seq/pos may be null for decode (row t = sequence
// t at position lens[t]).
int gpt2_layers(strictb200_model* m, strictb200_kv* kv, int64_t T, float* xf, float* af, float* bf_, const int32_t* seq,
                const int32_t* pos) {
  strictb200_ctx* ctx = m->ctx;
  const auto& c = m->c;
  const int64_t d = c.d_model;
  const float scale = 1.0f / sqrtf((float)c.head_dim);
  for (int l = 0; l < c.n_layers; l++) {
    LayerW& w = m->L[l];
    SB_TRY(k_layernorm(ctx, xf, w.norm1_g, w.norm1_b, c.eps, T, d, af));
    SB_TRY(k_gemm_f32(ctx, T, 3 * d, d, af, w.fqkv.w, w.fqkv.b, bf_, 0));
    SB_TRY(k_attn_f32(ctx, bf_, kv_kf(kv, l), kv_vf(kv, l), seq, pos, kv->d_lens, T, c.n_q_heads, c.head_dim, kv->maxlen, scale, af));
    SB_TRY(k_gemm_f32(ctx, T, d, d, af, w.fo.w, w.fo.b, xf, 1));
    SB_TRY(k_layernorm(ctx, xf, w.norm2_g, w.norm2_b, c.eps, T, d, af));
    SB_TRY(k_gemm_f32(ctx, T, c.d_ff, d, af, w.ffc.w, w.ffc.b, bf_, 2));  // GELU in the epilogue
    SB_TRY(k_gemm_f32(ctx, T, d, c.d_ff, bf_, w.fproj.w, w.fproj.b, xf, 1));
  }
  return STRICTB200_OK;
}

int gpt2_decode_body(strictb200_model* m, strictb200_kv* kv, DecBuf& b) {
  strictb200_ctx* ctx = m->ctx;
  const auto& c = m->c;
  const int64_t B = kv->B, d = c.d_model;
  SB_TRY(k_embedding_f32(ctx, m->wte, m->wpe, kv->d_ids, nullptr, kv->d_lens, B, d, c.vocab, c.max_pos, b.xf));
  SB_TRY(gpt2_layers(m, kv, B, b.xf, b.af, b.bf, nullptr, nullptr));
  SB_TRY(k_layernorm(ctx, b.xf, m->normf_g, m->normf_b, c.eps, B, d, b.af));
  SB_TRY(k_gemm_f32(ctx, B, c.vocab, d, b.af, m->wte, nullptr, b.logits, 0));
  SB_TRY(k_argmax(ctx, b.logits, B, c.vocab, c.vocab, kv->d_next, nullptr, b.am_ws));
  SB_TRY(k_add_i32(ctx, kv->d_lens, nullptr, 1, B));
  return STRICTB200_OK;
}

int decode_body(strictb200_model* m, strictb200_kv* kv) {
  DecBuf b;
  size_t total;
  carve_decode(kv, (char*)kv->dec, &b, &total);
  return m->c.arch == STRICTB200_QWEN3 ? qwen_decode_body(m, kv, b) : gpt2_decode_body(m, kv, b);
}

// Enqueue one decode step (ids already in kv->d_ids; result in kv->d_next).
int decode_enqueue(strictb200_model* m, strictb200_kv* kv) {
  strictb200_ctx* ctx = m->ctx;
  for (int b = 0; b < kv->B; b++)
    if (kv->h_lens[b] + 1 > kv->maxlen || kv->h_lens[b] + 1 > m->c.max_pos)
      return sb_fail(STRICTB200_ERR_INVALID_ARG, "decode: sequence " + std::to_string(b) + " has no room left in the cache");
  if (m->c.arch == STRICTB200_QWEN3) {
    // The key chunks of the decode attention are planned for the lengths the cache holds, not for a full cache, and planned
    // again when the longest sequence has grown by 256 keys; a new plan needs a new recording of the step.
    int longest = 0;
    for (int b = 0; b < kv->B; b++) longest = std::max(longest, kv->h_lens[b] + 1);
    if (!kv->chunk || longest > kv->plan_until) {
      const int chunk = sb_attn_decode_chunk(ctx, kv->B, m->Hkv_l, kv->maxlen, std::min(kv->maxlen, longest + 128));
      if (chunk != kv->chunk) {
        kv->chunk = chunk;
        kv->nsplit = (kv->maxlen + chunk - 1) / chunk;
        if (kv->graph) { cudaGraphExecDestroy(kv->graph); kv->graph = nullptr; }
      }
      kv->plan_until = std::min(kv->maxlen, longest + 256);
    }
  }
  if (!m->use_graph || !kv->warmed) {
    // the first step runs as plain launches: it also performs the one-time kernel attribute set-up
    SB_TRY(decode_body(m, kv));
    kv->warmed = true;
  } else {
    if (!kv->graph) {
      cudaGraph_t g;
      uint64_t before = ctx->launches;
      SB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
      int st = decode_body(m, kv);
      cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
      if (st != STRICTB200_OK) { if (e == cudaSuccess && g) cudaGraphDestroy(g); return st; }
      if (e != cudaSuccess) return sb_fail(STRICTB200_ERR_CUDA, std::string("graph capture: ") + cudaGetErrorString(e));
      kv->graph_kernels = ctx->launches - before;
      ctx->launches = before;
      e = cudaGraphInstantiate(&kv->graph, g, 0);
      cudaGraphDestroy(g);
      if (e != cudaSuccess) return sb_fail(STRICTB200_ERR_CUDA, std::string("graph instantiate: ") + cudaGetErrorString(e));
    }
    SB_CUDA(cudaGraphLaunch(kv->graph, ctx->stream));
    ctx->launches += kv->graph_kernels;
  }
  for (int b = 0; b < kv->B; b++) kv->h_lens[b] += 1;
  return STRICTB200_OK;
}

// ------------------------------------------------------------------ prefill
// Activations and index arrays of a prefill chunk are carved out of one grow-only scratch
// buffer of the context: after the first prompt of a given size no prefill allocates.
int prefill_scratch(strictb200_ctx* ctx, size_t bytes, char** out) {
  if (bytes > ctx->prefill_ws_bytes) {
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->prefill_ws) SB_CUDA(cudaFree(ctx->prefill_ws));
    ctx->prefill_ws = nullptr;
    ctx->prefill_ws_bytes = 0;
    SB_CUDA(cudaMalloc(&ctx->prefill_ws, bytes));
    ctx->prefill_ws_bytes = bytes;
  }
  *out = (char*)ctx->prefill_ws;
  return STRICTB200_OK;
}
struct ChunkIdx {
  int32_t *tok, *seq, *pos, *la, *past, *qs, *last;
};
void carve_idx(Carver& cv, int64_t T, int nb, ChunkIdx* o) {
  o->tok = cv.take<int32_t>(T); o->seq = cv.take<int32_t>(T); o->pos = cv.take<int32_t>(T);
  o->la = cv.take<int32_t>(nb); o->past = cv.take<int32_t>(nb); o->qs = cv.take<int32_t>(nb); o->last = cv.take<int32_t>(nb);
}
struct QwenChunk {
  float *x, *qkv, *gu, *y, *sa, *last;
  bf16 *qb, *att;
  uint8_t* aq;
  DecBuf hb;
};
void carve_qwen_chunk(strictb200_model* m, Carver& cv, int64_t T, int nb, QwenChunk* o) {
  const int64_t d = m->c.d_model, D = m->c.head_dim;
  const int64_t nq = (int64_t)m->Hq_l * D, nqkv = nq + 2 * (int64_t)m->Hkv_l * D;
  const int64_t amax = std::max<int64_t>(d, std::max<int64_t>(nq, m->I_l));
  o->x = cv.take<float>(T * d);
  o->qkv = cv.take<float>(T * nqkv);
  o->qb = cv.take<bf16>(T * nq);
  o->att = cv.take<bf16>(T * nq);
  o->gu = cv.take<float>(T * 2 * m->I_l);
  o->y = cv.take<float>(T * d);
  o->aq = cv.take<uint8_t>(sb_qrows(T) * amax);
  o->sa = cv.take<float>(T);
  o->last = cv.take<float>((size_t)nb * d);
  o->hb = DecBuf{};
  o->hb.logits = cv.take<float>((size_t)nb * m->V_l);
  o->hb.logits_all = cv.take<float>(m->world > 1 ? (size_t)m->world * nb * m->V_l : 1);
  o->hb.best_val = cv.take<float>((size_t)m->world * nb);
  o->hb.best_idx = cv.take<int32_t>((size_t)m->world * nb);
  o->hb.am_ws = cv.take<uint8_t>(sb_argmax_scratch(nb, m->V_l));
}
struct Gpt2Chunk {
  float *xf, *af, *bf_, *last, *lastn, *logits;
  void* am_ws;
};
void carve_gpt2_chunk(strictb200_model* m, Carver& cv, int64_t T, int nb, Gpt2Chunk* o) {
  const int64_t d = m->c.d_model, wd = std::max<int64_t>(3 * d, m->c.d_ff);
  o->xf = cv.take<float>(T * d);
  o->af = cv.take<float>(T * wd);
  o->bf_ = cv.take<float>(T * wd);
  o->last = cv.take<float>((size_t)nb * d);
  o->lastn = cv.take<float>((size_t)nb * d);
  o->logits = cv.take<float>((size_t)nb * m->c.vocab);
  o->am_ws = cv.take<uint8_t>(sb_argmax_scratch(nb, m->c.vocab));
}

int qwen_prefill_chunk(strictb200_model* m, strictb200_kv* kv, int64_t T, int nb, const int32_t* d_tok, const int32_t* d_seq,
                       const int32_t* d_pos, const int32_t* d_lens_after, const int32_t* d_past, const int32_t* d_qstart,
                       const int32_t* d_last_rows, int b0, int32_t* d_next, float* h_logits, int max_new, QwenChunk& cb) {
  strictb200_ctx* ctx = m->ctx;
  const auto& c = m->c;
  const int64_t d = c.d_model, D = c.head_dim;
  const int64_t nq = (int64_t)m->Hq_l * D;
  const float scale = 1.0f / sqrtf((float)D);
  const bool tp = m->world > 1;
  bf16 *qb = cb.qb, *att = cb.att;
  uint8_t* aq = cb.aq;
  float *x = cb.x, *y = cb.y, *sa = cb.sa, *qkv = cb.qkv, *gu = cb.gu;
  SB_TRY(k_embedding_bf16_f32(ctx, m->embed, d_tok, T, d, c.vocab, x));
  {
    RowNormArgs a;
    a.x_f32 = x; a.gain = m->L[0].norm1_g; a.eps = c.eps; a.q = aq; a.qscale = sa;
    SB_TRY(k_rownorm(ctx, a, T, d));
  }
  // caches of this chunk's sequences start at sequence b0
  const size_t seq_stride = (size_t)m->Hkv_l * kv->maxlen * D;
  for (int l = 0; l < c.n_layers; l++) {
    LayerW& w = m->L[l];
    bf16* kc = kv_k(kv, l) + (size_t)b0 * seq_stride;
    bf16* vc = kv_v(kv, l) + (size_t)b0 * seq_stride;
    SB_TRY(run_gemm(m, T, w.wqkv, aq, sa, qkv, 1, nullptr, 1, 0));
    {
      RopeArgs r;
      r.qkv_f32 = qkv; r.seq = d_seq; r.pos = d_pos;
      r.cos_t = m->rope_cos; r.sin_t = m->rope_sin; r.qgain = w.qn_g; r.kgain = w.kn_g; r.eps = c.eps;
      r.Hq = m->Hq_l; r.Hkv = m->Hkv_l; r.D = (int)D; r.maxlen = kv->maxlen; r.max_pos = c.max_pos;
      r.q_out = qb; r.kcache = kc; r.vcache = vc;
      SB_TRY(k_rope_qknorm_kvappend(ctx, r, T));
    }
    SB_TRY(k_attn_prefill(ctx, qb, kc, vc, d_lens_after, d_past, d_qstart, nb, max_new, T, m->Hq_l, m->Hkv_l, (int)D, kv->maxlen, scale, att));
    SB_TRY(k_quantize_rows(ctx, att, T, nq, nq, aq, sa));
    {
      RowNormArgs a;
      SB_TRY(run_gemm(m, T, w.wo, aq, sa, y, 1, nullptr, 1, 0));
      if (tp) SB_TRY(sb_tp_allreduce_f32(ctx, y, T * d));
      a.x_f32 = y; a.residual_f32 = x; a.gain = w.norm2_g; a.eps = c.eps; a.q = aq; a.qscale = sa;
      SB_TRY(k_rownorm(ctx, a, T, d));
    }
    SB_TRY(run_gemm(m, T, w.wgu, aq, sa, gu, 1, nullptr, 1, 0));
    SB_TRY(k_swiglu(ctx, nullptr, gu, T, m->I_l, nullptr, aq, sa));
    {
      RowNormArgs a;
      SB_TRY(run_gemm(m, T, w.wdown, aq, sa, y, 1, nullptr, 1, 0));
      if (tp) SB_TRY(sb_tp_allreduce_f32(ctx, y, T * d));
      a.x_f32 = y; a.residual_f32 = x;
      if (l + 1 < c.n_layers) { a.gain = m->L[l + 1].norm1_g; a.q = aq; a.qscale = sa; }
      a.eps = c.eps;
      SB_TRY(k_rownorm(ctx, a, T, d));
    }
  }
  // last real row of every sequence -> final norm -> head -> greedy pick
  float* last = cb.last;
  SB_TRY(k_gather_rows(ctx, x, d_last_rows, nb, d * 4, last));
  {
    RowNormArgs a;
    a.x_f32 = last; a.gain = m->normf_g; a.eps = c.eps; a.q = aq; a.qscale = sa;
    SB_TRY(k_rownorm(ctx, a, nb, d));
  }
  SB_TRY(head_and_pick(m, nb, aq, sa, cb.hb, d_next, h_logits, nb));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}

int gpt2_prefill_chunk(strictb200_model* m, strictb200_kv* kv, int64_t T, int nb, const int32_t* d_tok, const int32_t* d_seq,
                       const int32_t* d_pos, const int32_t* d_last_rows, int32_t* d_next, float* h_logits, Gpt2Chunk& cb) {
  strictb200_ctx* ctx = m->ctx;
  const auto& c = m->c;
  const int64_t d = c.d_model;
  float *xf = cb.xf, *af = cb.af, *bf_ = cb.bf_, *last = cb.last, *lastn = cb.lastn, *logits = cb.logits;
  SB_TRY(k_embedding_f32(ctx, m->wte, m->wpe, d_tok, d_pos, nullptr, T, d, c.vocab, c.max_pos, xf));
  SB_TRY(gpt2_layers(m, kv, T, xf, af, bf_, d_seq, d_pos));
  SB_TRY(k_gather_rows(ctx, xf, d_last_rows, nb, d * 4, last));
  SB_TRY(k_layernorm(ctx, last, m->normf_g, m->normf_b, c.eps, nb, d, lastn));
  SB_TRY(k_gemm_f32(ctx, nb, c.vocab, d, lastn, m->wte, nullptr, logits, 0));
  SB_TRY(k_argmax(ctx, logits, nb, c.vocab, c.vocab, d_next, nullptr, cb.am_ws));
  if (h_logits) SB_CUDA(cudaMemcpyAsync(h_logits, logits, (size_t)nb * c.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}

// ------------------------------------------------------------------ named tensors
struct Slice {
  void* dev = nullptr;       // device pointer of the local shard
  size_t elem = 0;           // bytes per element on the device
  int host_f32 = 0;          // host side is fp32 even though the device holds bf16
  int64_t rows = 0, cols = 0;          // full tensor shape
  // up to three row ranges of the full tensor (src row, count, dst row) and one column window
  int nr = 0;
  int64_t src_row[3], n_rows[3], dst_row[3];
  int64_t col0 = 0, ncols = 0;
};

bool find_slice(strictb200_model* m, const std::string& name, Slice* s) {
  const auto& c = m->c;
  const int64_t d = c.d_model, D = c.head_dim, I = c.d_ff;
  const int64_t nq = (int64_t)c.n_q_heads * D, nkv = (int64_t)c.n_kv_heads * D;
  const int64_t nq_l = (int64_t)m->Hq_l * D, nkv_l = (int64_t)m->Hkv_l * D;
  const int r = m->rank;
  auto full = [&](void* p, size_t elem, int64_t rows, int64_t cols) {
    s->dev = p; s->elem = elem; s->rows = rows; s->cols = cols;
    s->nr = 1; s->src_row[0] = 0; s->n_rows[0] = rows; s->dst_row[0] = 0; s->col0 = 0; s->ncols = cols;
    return p != nullptr;
  };
  const bool qwen = c.arch == STRICTB200_QWEN3;
  if (name == "embed") {
    if (qwen) { bool ok = full(m->embed, 2, c.vocab, d); s->host_f32 = 1; return ok; }
    return full(m->wte, 4, c.vocab, d);
  }
  if (name == "wpe") return full(m->wpe, 4, c.max_pos, d);
  if (name == "normf.g") return full(m->normf_g, 4, 1, d);
  if (name == "normf.b") return full(m->normf_b, 4, 1, d);
  if (name == "head.q" || name == "head.s") {
    bool isq = name == "head.q";
    if (!m->head.q) return false;
    s->dev = isq ? (void*)m->head.q : (void*)m->head.s; s->elem = isq ? 1 : 4;
    s->rows = c.vocab; s->cols = isq ? d : 1;
    s->nr = 1; s->src_row[0] = (int64_t)r * m->V_l; s->n_rows[0] = m->V_l; s->dst_row[0] = 0; s->col0 = 0; s->ncols = s->cols;
    return true;
  }
  if (name.rfind("layers.", 0) != 0) return false;
  size_t dot = name.find('.', 7);
  if (dot == std::string::npos) return false;
  int l = atoi(name.substr(7, dot - 7).c_str());
  if (l < 0 || l >= c.n_layers) return false;
  LayerW& w = m->L[l];
  std::string k = name.substr(dot + 1);
  if (k == "norm1.g") return full(w.norm1_g, 4, 1, d);
  if (k == "norm1.b") return full(w.norm1_b, 4, 1, d);
  if (k == "norm2.g") return full(w.norm2_g, 4, 1, d);
  if (k == "norm2.b") return full(w.norm2_b, 4, 1, d);
  if (k == "qnorm.g") return full(w.qn_g, 4, 1, D);
  if (k == "knorm.g") return full(w.kn_g, 4, 1, D);
  if (qwen) {
    bool isq = k.size() > 2 && k.substr(k.size() - 2) == ".q";
    bool iss = k.size() > 2 && k.substr(k.size() - 2) == ".s";
    if (!isq && !iss) return false;
    std::string base = k.substr(0, k.size() - 2);
    s->elem = isq ? 1 : 4;
    if (base == "wqkv") {
      s->dev = isq ? (void*)w.wqkv.q : (void*)w.wqkv.s;
      s->rows = nq + 2 * nkv; s->cols = isq ? d : 1; s->col0 = 0; s->ncols = s->cols;
      s->nr = 3;
      s->src_row[0] = r * nq_l; s->n_rows[0] = nq_l; s->dst_row[0] = 0;
      s->src_row[1] = nq + r * nkv_l; s->n_rows[1] = nkv_l; s->dst_row[1] = nq_l;
      s->src_row[2] = nq + nkv + r * nkv_l; s->n_rows[2] = nkv_l; s->dst_row[2] = nq_l + nkv_l;
      return true;
    }
    if (base == "wgu") {
      s->dev = isq ? (void*)w.wgu.q : (void*)w.wgu.s;
      s->rows = 2 * I; s->cols = isq ? d : 1; s->col0 = 0; s->ncols = s->cols;
      s->nr = 2;
      s->src_row[0] = r * m->I_l; s->n_rows[0] = m->I_l; s->dst_row[0] = 0;
      s->src_row[1] = I + r * m->I_l; s->n_rows[1] = m->I_l; s->dst_row[1] = m->I_l;
      return true;
    }
    if (base == "wo" || base == "wdown") {
      QW& q = base == "wo" ? w.wo : w.wdown;
      int64_t Kfull = base == "wo" ? nq : I, Kl = base == "wo" ? nq_l : m->I_l;
      s->dev = isq ? (void*)q.q : (void*)q.s;
      s->rows = d; s->cols = isq ? Kfull : 1;
      s->nr = 1; s->src_row[0] = 0; s->n_rows[0] = d; s->dst_row[0] = 0;
      s->col0 = isq ? r * Kl : 0; s->ncols = isq ? Kl : 1;
      return true;
    }
    return false;
  }
  bool isw = k.size() > 2 && k.substr(k.size() - 2) == ".w";
  bool isb = k.size() > 2 && k.substr(k.size() - 2) == ".b";
  if (!isw && !isb) return false;
  std::string base = k.substr(0, k.size() - 2);
  FW* f = base == "wqkv" ? &w.fqkv : base == "wo" ? &w.fo : base == "wfc" ? &w.ffc : base == "wproj" ? &w.fproj : nullptr;
  if (!f) return false;
  return isw ? full(f->w, 4, f->N, f->K) : full(f->b, 4, 1, f->N);
}

}  // namespace

extern "C" {

int strictb200_model_create(strictb200_ctx* ctx, const strictb200_model_config* cfg, strictb200_model** out) {
  SB_ENTER(ctx);
  SB_REQUIRE(cfg && out, "null argument");
  *out = nullptr;
  const strictb200_model_config& c = *cfg;
  SB_REQUIRE(c.arch == STRICTB200_GPT2 || c.arch == STRICTB200_QWEN3, "unknown architecture");
  SB_REQUIRE(c.n_layers > 0 && c.d_model > 0 && c.n_q_heads > 0 && c.n_kv_heads > 0 && c.head_dim > 0 && c.d_ff > 0 && c.vocab > 0 &&
                 c.max_pos > 0,
             "non-positive dimension");
  SB_REQUIRE(c.n_q_heads % c.n_kv_heads == 0, "query heads must be a multiple of KV heads");
  const int world = ctx->tp_world;
  if (c.arch == STRICTB200_GPT2) {
    if (world != 1) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "the GPT-2 path is single-GPU");
    SB_REQUIRE(c.n_q_heads == c.n_kv_heads && c.n_q_heads * c.head_dim == c.d_model, "GPT-2 needs heads*head_dim == d_model");
    SB_REQUIRE(c.d_model % 4 == 0 && c.d_ff % 4 == 0 && c.head_dim % 4 == 0, "dimensions must be multiples of 4");
  } else {
    if (c.head_dim != 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "Qwen3 path: head_dim must be 128");
    SB_REQUIRE(c.d_model % 64 == 0 && c.d_model <= 16384, "d_model must be a multiple of 64, at most 16384");
    SB_REQUIRE(c.n_kv_heads % world == 0 && c.d_ff % (world * 64) == 0 && c.vocab % (world * 16) == 0,
               "heads, d_ff/64 and vocab/16 must divide by the tensor-parallel world size");
    SB_REQUIRE(c.n_q_heads / c.n_kv_heads <= 16, "at most 16 query heads per KV head");
  }
  strictb200_model* m = new strictb200_model;
  m->ctx = ctx; m->c = c; m->world = world; m->rank = ctx->tp_rank;
  m->Hq_l = c.n_q_heads / world; m->Hkv_l = c.n_kv_heads / world;
  m->I_l = c.d_ff / world; m->V_l = c.vocab / world;
  m->L.resize(c.n_layers);
  const int64_t d = c.d_model, D = c.head_dim;
  int st = STRICTB200_OK;
  auto fail = [&](int s) { strictb200_model_destroy(m); return s; };
#define M_TRY(e) do { st = (e); if (st != STRICTB200_OK) return fail(st); } while (0)
  M_TRY(dalloc(m, &m->normf_g, d)); M_TRY(fill_f32(ctx, m->normf_g, d, 1.f));
  M_TRY(dalloc(m, &m->normf_b, d)); M_TRY(fill_f32(ctx, m->normf_b, d, 0.f));
  if (c.arch == STRICTB200_GPT2) {
    M_TRY(dalloc(m, &m->wte, (size_t)c.vocab * d));
    M_TRY(dalloc(m, &m->wpe, (size_t)c.max_pos * d));
    m->weight_bytes += (uint64_t)c.vocab * d * 4;
  } else {
    M_TRY(dalloc(m, &m->embed, (size_t)c.vocab * d));
    M_TRY(alloc_qw(m, m->head, m->V_l, d));
    M_TRY(sb_rope_table(ctx, c.max_pos, (int)D, c.rope_theta, &m->rope_cos, &m->rope_sin));
    m->allocs.push_back(m->rope_cos);
    m->allocs.push_back(m->rope_sin);
  }
  for (int l = 0; l < c.n_layers; l++) {
    LayerW& w = m->L[l];
    M_TRY(dalloc(m, &w.norm1_g, d)); M_TRY(fill_f32(ctx, w.norm1_g, d, 1.f));
    M_TRY(dalloc(m, &w.norm1_b, d)); M_TRY(fill_f32(ctx, w.norm1_b, d, 0.f));
    M_TRY(dalloc(m, &w.norm2_g, d)); M_TRY(fill_f32(ctx, w.norm2_g, d, 1.f));
    M_TRY(dalloc(m, &w.norm2_b, d)); M_TRY(fill_f32(ctx, w.norm2_b, d, 0.f));
    if (c.arch == STRICTB200_GPT2) {
      M_TRY(alloc_fw(m, w.fqkv, 3 * d, d));
      M_TRY(alloc_fw(m, w.fo, d, d));
      M_TRY(alloc_fw(m, w.ffc, c.d_ff, d));
      M_TRY(alloc_fw(m, w.fproj, d, c.d_ff));
    } else {
      M_TRY(dalloc(m, &w.qn_g, D)); M_TRY(fill_f32(ctx, w.qn_g, D, 1.f));
      M_TRY(dalloc(m, &w.kn_g, D)); M_TRY(fill_f32(ctx, w.kn_g, D, 1.f));
      M_TRY(alloc_qw(m, w.wqkv, (int64_t)(m->Hq_l + 2 * m->Hkv_l) * D, d));
      M_TRY(alloc_qw(m, w.wo, d, (int64_t)m->Hq_l * D));
      M_TRY(alloc_qw(m, w.wgu, 2 * m->I_l, d));
      M_TRY(alloc_qw(m, w.wdown, d, m->I_l));
    }
  }
#undef M_TRY
  *out = m;
  return STRICTB200_OK;
}

int strictb200_model_destroy(strictb200_model* m) {
  if (!m) return STRICTB200_OK;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  for (void* p : m->allocs) cudaFree(p);
  delete m;
  return STRICTB200_OK;
}

int strictb200_model_init_random(strictb200_model* m, uint64_t seed) {
  if (!m) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null model");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  const auto& c = m->c;
  const float SD = 0.02f;
  const int64_t d = c.d_model, D = c.head_dim, I = c.d_ff;
  const int64_t nq = (int64_t)c.n_q_heads * D;
  const int64_t nq_l = (int64_t)m->Hq_l * D, nkv_l = (int64_t)m->Hkv_l * D;
  const int r = m->rank;
  auto key = [&](uint64_t t) { return sb_stream_key(seed, t); };
  if (c.arch == STRICTB200_GPT2) {
    SB_TRY(k_gen_normal_f32(ctx, key(G_EMBED), 0, (int64_t)c.vocab * d, SD, m->wte));
    SB_TRY(k_gen_normal_f32(ctx, key(G_WPE), 0, (int64_t)c.max_pos * d, SD, m->wpe));
    for (int l = 0; l < c.n_layers; l++) {
      LayerW& w = m->L[l];
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_Q)), 0, d * d, SD, w.fqkv.w));
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_K)), 0, d * d, SD, w.fqkv.w + d * d));
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_V)), 0, d * d, SD, w.fqkv.w + 2 * d * d));
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_O)), 0, d * d, SD, w.fo.w));
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_GATE)), 0, I * d, SD, w.ffc.w));
      SB_TRY(k_gen_normal_f32(ctx, key(layer_tensor(l, T_DOWN)), 0, d * I, SD, w.fproj.w));
    }
  } else {
    SB_TRY(k_gen_normal_bf16(ctx, key(G_EMBED), 0, (int64_t)c.vocab * d, SD, m->embed));
    if (c.tied) {
      SB_TRY(k_quantize_weight_rows(ctx, m->embed + (int64_t)r * m->V_l * d, m->V_l, d, d, m->head.q, m->head.s));
    } else {
      SB_TRY(k_gen_weight_e4m3(ctx, key(G_HEAD), (int64_t)r * m->V_l, m->V_l, d, 0, d, SD, m->head.q, d, m->head.s));
    }
    for (int l = 0; l < c.n_layers; l++) {
      LayerW& w = m->L[l];
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_Q)), r * nq_l, nq_l, d, 0, d, SD, w.wqkv.q, d, w.wqkv.s));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_K)), r * nkv_l, nkv_l, d, 0, d, SD, w.wqkv.q + nq_l * d, d, w.wqkv.s + nq_l));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_V)), r * nkv_l, nkv_l, d, 0, d, SD, w.wqkv.q + (nq_l + nkv_l) * d, d,
                               w.wqkv.s + nq_l + nkv_l));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_O)), 0, d, nq, r * nq_l, nq_l, SD, w.wo.q, nq_l, w.wo.s));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_GATE)), r * m->I_l, m->I_l, d, 0, d, SD, w.wgu.q, d, w.wgu.s));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_UP)), r * m->I_l, m->I_l, d, 0, d, SD, w.wgu.q + m->I_l * d, d, w.wgu.s + m->I_l));
      SB_TRY(k_gen_weight_e4m3(ctx, key(layer_tensor(l, T_DOWN)), 0, d, I, r * m->I_l, m->I_l, SD, w.wdown.q, m->I_l, w.wdown.s));
    }
  }
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}

int strictb200_model_set_tensor(strictb200_model* m, const char* name, const void* h_data, size_t bytes) {
  if (!m || !name || !h_data) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  Slice s;
  if (!find_slice(m, name, &s)) return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("unknown tensor ") + name);
  size_t helem = s.host_f32 ? 4 : s.elem;
  if (bytes != (size_t)s.rows * s.cols * helem)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("tensor ") + name + " expects " + std::to_string((size_t)s.rows * s.cols * helem) + " bytes");
  for (int i = 0; i < s.nr; i++) {
    if (s.host_f32) {
      // fp32 host rows -> bf16 device rows through a staging buffer
      float* tmp;
      size_t n = (size_t)s.n_rows[i] * s.ncols;
      SB_CUDA(cudaMalloc((void**)&tmp, n * 4));
      cudaError_t e = cudaMemcpy2DAsync(tmp, s.ncols * 4, (const char*)h_data + ((size_t)s.src_row[i] * s.cols + s.col0) * 4, s.cols * 4,
                                        s.ncols * 4, s.n_rows[i], cudaMemcpyHostToDevice, ctx->stream);
      int st = e == cudaSuccess ? k_f32_to_bf16(ctx, tmp, n, (bf16*)s.dev + (size_t)s.dst_row[i] * s.ncols) : STRICTB200_ERR_CUDA;
      cudaStreamSynchronize(ctx->stream);
      cudaFree(tmp);
      if (e != cudaSuccess) return sb_fail(STRICTB200_ERR_CUDA, cudaGetErrorString(e));
      SB_TRY(st);
    } else {
      SB_CUDA(cudaMemcpy2DAsync((char*)s.dev + (size_t)s.dst_row[i] * s.ncols * s.elem, s.ncols * s.elem,
                                (const char*)h_data + ((size_t)s.src_row[i] * s.cols + s.col0) * s.elem, s.cols * s.elem, s.ncols * s.elem,
                                s.n_rows[i], cudaMemcpyHostToDevice, ctx->stream));
    }
  }
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  if (std::string(name) == "embed" && m->c.arch == STRICTB200_QWEN3 && m->c.tied) {
    SB_TRY(k_quantize_weight_rows(ctx, m->embed + (int64_t)m->rank * m->V_l * m->c.d_model, m->V_l, m->c.d_model, m->c.d_model, m->head.q, m->head.s));
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return STRICTB200_OK;
}

int strictb200_model_get_tensor(strictb200_model* m, const char* name, void* h_data, size_t bytes) {
  if (!m || !name || !h_data) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  if (m->world != 1) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "get_tensor reads whole tensors and needs a single-rank model");
  Slice s;
  if (!find_slice(m, name, &s)) return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("unknown tensor ") + name);
  size_t helem = s.host_f32 ? 4 : s.elem;
  size_t n = (size_t)s.rows * s.cols;
  if (bytes != n * helem) return sb_fail(STRICTB200_ERR_INVALID_ARG, std::string("tensor ") + name + " holds " + std::to_string(n * helem) + " bytes");
  if (s.host_f32) {
    float* tmp;
    SB_CUDA(cudaMalloc((void**)&tmp, n * 4));
    int st = k_bf16_to_f32(ctx, (const bf16*)s.dev, n, tmp);
    cudaError_t e = cudaMemcpyAsync(h_data, tmp, n * 4, cudaMemcpyDeviceToHost, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    SB_TRY(st);
    if (e != cudaSuccess) return sb_fail(STRICTB200_ERR_CUDA, cudaGetErrorString(e));
    return STRICTB200_OK;
  }
  SB_CUDA(cudaMemcpyAsync(h_data, s.dev, n * s.elem, cudaMemcpyDeviceToHost, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}

int strictb200_model_weight_bytes(strictb200_model* m, uint64_t* out) {
  if (!m || !out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  *out = m->weight_bytes;
  return STRICTB200_OK;
}
int strictb200_model_set_graph(strictb200_model* m, int enabled) {
  if (!m) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null model");
  m->use_graph = enabled ? 1 : 0;
  return STRICTB200_OK;
}

// ---------------------------------------------------------------- KV cache
int strictb200_kv_create(strictb200_model* m, int batch, int maxlen, strictb200_kv** out) {
  if (!m || !out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  *out = nullptr;
  SB_REQUIRE(batch > 0 && maxlen > 0, "batch and maxlen must be positive");
  SB_REQUIRE(maxlen <= m->c.max_pos, "maxlen exceeds the model's max_pos");
  strictb200_kv* kv = new strictb200_kv;
  kv->m = m; kv->B = batch;
  kv->maxlen = (maxlen + 63) / 64 * 64;  // whole 64-key tiles
  const bool qwen = m->c.arch == STRICTB200_QWEN3;
  const size_t esz = qwen ? 2 : 4;
  kv->layer_stride = (size_t)batch * (qwen ? m->Hkv_l : m->c.n_kv_heads) * kv->maxlen * m->c.head_dim;
  size_t bytes = kv->layer_stride * m->c.n_layers * esz;
  auto fail = [&](int s) { strictb200_kv_destroy(kv); return s; };
  auto alloc = [&](void** p, size_t n) -> int {
    SB_CUDA(cudaMalloc(p, n ? n : 1));
    kv->allocs.push_back(*p);
    return STRICTB200_OK;
  };
  int st;
#define K_TRY(e) do { st = (e); if (st != STRICTB200_OK) return fail(st); } while (0)
  K_TRY(alloc(&kv->k, bytes));
  K_TRY(alloc(&kv->v, bytes));
  // zero so that the padding rows of a partly filled 64-key tile are finite
  if (cudaMemsetAsync(kv->k, 0, bytes, ctx->stream) != cudaSuccess || cudaMemsetAsync(kv->v, 0, bytes, ctx->stream) != cudaSuccess)
    return fail(sb_fail(STRICTB200_ERR_CUDA, "memset of the cache failed"));
  K_TRY(alloc((void**)&kv->d_lens, (size_t)batch * 4));
  K_TRY(alloc((void**)&kv->d_ids, (size_t)batch * 4));
  K_TRY(alloc((void**)&kv->d_next, (size_t)batch * 4));
  cudaMemsetAsync(kv->d_lens, 0, (size_t)batch * 4, ctx->stream);
  cudaMemsetAsync(kv->d_ids, 0, (size_t)batch * 4, ctx->stream);
  kv->h_lens.assign(batch, 0);
  kv->nsplit = qwen ? sb_attn_decode_splits(ctx, batch, m->Hkv_l, kv->maxlen) : 1;
  DecBuf tmp;
  carve_decode(kv, nullptr, &tmp, &kv->dec_bytes);
  K_TRY(alloc(&kv->dec, kv->dec_bytes));
#undef K_TRY
  if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return fail(sb_fail(STRICTB200_ERR_CUDA, "cache set-up failed"));
  *out = kv;
  return STRICTB200_OK;
}

int strictb200_kv_destroy(strictb200_kv* kv) {
  if (!kv) return STRICTB200_OK;
  cudaSetDevice(kv->m->ctx->device);
  cudaStreamSynchronize(kv->m->ctx->stream);
  if (kv->graph) cudaGraphExecDestroy(kv->graph);
  for (void* p : kv->allocs) cudaFree(p);
  delete kv;
  return STRICTB200_OK;
}

int strictb200_kv_reset(strictb200_kv* kv) {
  if (!kv) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null cache");
  strictb200_ctx* ctx = kv->m->ctx;
  SB_ENTER(ctx);
  SB_CUDA(cudaMemsetAsync(kv->d_lens, 0, (size_t)kv->B * 4, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  std::fill(kv->h_lens.begin(), kv->h_lens.end(), 0);
  kv->plan_until = 0;  // the next decode step plans the attention's key chunks for the new lengths
  return STRICTB200_OK;
}

int strictb200_kv_lens(strictb200_kv* kv, int32_t* h_lens) {
  if (!kv || !h_lens) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = kv->m->ctx;
  SB_ENTER(ctx);
  SB_CUDA(cudaMemcpyAsync(h_lens, kv->d_lens, (size_t)kv->B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}

int strictb200_kv_fill_synthetic(strictb200_kv* kv, uint64_t seed, int len) {
  if (!kv) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null cache");
  strictb200_model* m = kv->m;
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(len >= 0 && len <= kv->maxlen && len < m->c.max_pos, "len outside the cache");
  size_t n = kv->layer_stride * m->c.n_layers;
  if (m->c.arch == STRICTB200_QWEN3) {
    SB_TRY(k_gen_normal_bf16(ctx, sb_stream_key(seed, 0x4B00 + m->rank), 0, (int64_t)n, 1.0f, (bf16*)kv->k));
    SB_TRY(k_gen_normal_bf16(ctx, sb_stream_key(seed, 0x5600 + m->rank), 0, (int64_t)n, 1.0f, (bf16*)kv->v));
  } else {
    SB_TRY(k_gen_normal_f32(ctx, sb_stream_key(seed, 0x4B00), 0, (int64_t)n, 1.0f, (float*)kv->k));
    SB_TRY(k_gen_normal_f32(ctx, sb_stream_key(seed, 0x5600), 0, (int64_t)n, 1.0f, (float*)kv->v));
  }
  std::vector<int32_t> h(kv->B, len);
  SB_CUDA(cudaMemcpyAsync(kv->d_lens, h.data(), (size_t)kv->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  kv->h_lens = h;
  kv->plan_until = 0;
  return STRICTB200_OK;
}

// ---------------------------------------------------------------- prefill / decode
int strictb200_prefill(strictb200_model* m, strictb200_kv* kv, const int32_t* h_tokens, const int32_t* h_lens, int B, int S,
                       int32_t* h_next, float* h_logits) {
  if (!m || !kv || !h_tokens || !h_lens || !h_next) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(kv->m == m, "cache belongs to another model");
  SB_REQUIRE(B == kv->B && S > 0, "batch must match the cache and S must be positive");
  const auto& c = m->c;
  for (int b = 0; b < B; b++) {
    SB_REQUIRE(h_lens[b] > 0 && h_lens[b] <= S, "every sequence needs between 1 and S tokens");
    SB_REQUIRE(kv->h_lens[b] + h_lens[b] <= kv->maxlen && kv->h_lens[b] + h_lens[b] <= c.max_pos, "prompt does not fit the cache");
    for (int i = 0; i < h_lens[b]; i++)
      SB_REQUIRE(h_tokens[(size_t)b * S + i] >= 0 && h_tokens[(size_t)b * S + i] < c.vocab, "token id outside the vocabulary");
  }
  const int64_t MAX_T = ctx->opt.prefill_chunk > 0 ? ctx->opt.prefill_chunk : 16384;  // token rows per chunk (bounds the activation scratch)
  int b0 = 0;
  int32_t* d_next = kv->d_next;  // the decode step's own buffer: nothing else uses it during a prefill
  while (b0 < B) {
    int nb = 0;
    int64_t T = 0;
    while (b0 + nb < B && (nb == 0 || T + h_lens[b0 + nb] <= MAX_T)) { T += h_lens[b0 + nb]; nb++; }
    std::vector<int32_t> tok(T), seq(T), pos(T), la(nb), past(nb), qstart(nb), last(nb);
    int64_t t = 0;
    int max_new = 0;
    for (int j = 0; j < nb; j++) {
      int b = b0 + j;
      qstart[j] = (int32_t)t;
      past[j] = kv->h_lens[b];
      la[j] = kv->h_lens[b] + h_lens[b];
      max_new = std::max(max_new, h_lens[b]);
      for (int i = 0; i < h_lens[b]; i++, t++) {
        tok[t] = h_tokens[(size_t)b * S + i];
        seq[t] = c.arch == STRICTB200_QWEN3 ? j : b;  // the fp32 path addresses the cache by absolute sequence index
        pos[t] = kv->h_lens[b] + i;
      }
      last[j] = (int32_t)t - 1;
    }
    // one carve pass to size the scratch, one to place the buffers
    ChunkIdx ix;
    QwenChunk qc;
    Gpt2Chunk gc;
    char* base = nullptr;
    for (int pass = 0; pass < 2; pass++) {
      Carver cv{base};
      carve_idx(cv, T, nb, &ix);
      if (c.arch == STRICTB200_QWEN3) carve_qwen_chunk(m, cv, T, nb, &qc);
      else carve_gpt2_chunk(m, cv, T, nb, &gc);
      if (pass == 0) SB_TRY(prefill_scratch(ctx, cv.off, &base));
    }
    SB_CUDA(cudaMemcpyAsync(ix.tok, tok.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.seq, seq.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.pos, pos.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.la, la.data(), nb * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.past, past.data(), nb * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.qs, qstart.data(), nb * 4, cudaMemcpyHostToDevice, ctx->stream));
    SB_CUDA(cudaMemcpyAsync(ix.last, last.data(), nb * 4, cudaMemcpyHostToDevice, ctx->stream));
    float* hl = h_logits ? h_logits + (size_t)b0 * c.vocab : nullptr;
    // both chunk functions end with a stream synchronise, so the host vectors above outlive their copies
    if (c.arch == STRICTB200_QWEN3) {
      SB_TRY(qwen_prefill_chunk(m, kv, T, nb, ix.tok, ix.seq, ix.pos, ix.la, ix.past, ix.qs, ix.last, b0, d_next + b0, hl, max_new, qc));
    } else {
      SB_TRY(gpt2_prefill_chunk(m, kv, T, nb, ix.tok, ix.seq, ix.pos, ix.last, d_next + b0, hl, gc));
    }
    SB_TRY(sb_check_status(ctx, "prefill"));
    for (int j = 0; j < nb; j++) kv->h_lens[b0 + j] += h_lens[b0 + j];
    b0 += nb;
  }
  kv->plan_until = 0;  // the lengths jumped: the next decode step plans the attention's key chunks for them
  SB_CUDA(cudaMemcpyAsync(kv->d_lens, kv->h_lens.data(), (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaMemcpyAsync(h_next, d_next, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  SB_TRY(sb_sync(ctx, "prefill"));
  return sb_check_status(ctx, "prefill");
}

int strictb200_decode_step(strictb200_model* m, strictb200_kv* kv, const int32_t* h_ids, int32_t* h_next, float* h_logits) {
  if (!m || !kv || !h_ids || !h_next) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(kv->m == m, "cache belongs to another model");
  for (int b = 0; b < kv->B; b++) SB_REQUIRE(h_ids[b] >= 0 && h_ids[b] < m->c.vocab, "token id outside the vocabulary");
  SB_CUDA(cudaMemcpyAsync(kv->d_ids, h_ids, (size_t)kv->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  SB_TRY(decode_enqueue(m, kv));
  SB_CUDA(cudaMemcpyAsync(h_next, kv->d_next, (size_t)kv->B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (h_logits) {
    DecBuf b;
    size_t total;
    carve_decode(kv, (char*)kv->dec, &b, &total);
    if (m->world == 1) {
      SB_CUDA(cudaMemcpyAsync(h_logits, b.logits, (size_t)kv->B * m->V_l * 4, cudaMemcpyDeviceToHost, ctx->stream));
    } else {
      SB_TRY(sb_tp_allgather(ctx, b.logits, b.logits_all, (int64_t)kv->B * m->V_l * 4));
      void* tmp;  // grow-only context scratch
      SB_TRY(sb_ws2(ctx, (size_t)m->world * kv->B * m->V_l * 4, &tmp));
      interleave_logits_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(b.logits_all, m->world, kv->B, m->V_l, (float*)tmp);
      SB_LAUNCHED(ctx);
      SB_CUDA(cudaMemcpyAsync(h_logits, tmp, (size_t)m->world * kv->B * m->V_l * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
  }
  SB_TRY(sb_sync(ctx, "decode_step"));
  return sb_check_status(ctx, "decode_step");
}

int strictb200_decode_steps_device(strictb200_model* m, strictb200_kv* kv, int32_t* d_ids, int n_steps) {
  if (!m || !kv) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(kv->m == m && n_steps >= 0, "bad arguments");
  if (d_ids && d_ids != kv->d_ids) SB_CUDA(cudaMemcpyAsync(kv->d_ids, d_ids, (size_t)kv->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  for (int s = 0; s < n_steps; s++) {
    SB_TRY(decode_enqueue(m, kv));
    SB_CUDA(cudaMemcpyAsync(kv->d_ids, kv->d_next, (size_t)kv->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (kv->d_hist && s < kv->hist_cap)
      SB_CUDA(cudaMemcpyAsync(kv->d_hist + (size_t)s * kv->B, kv->d_next, (size_t)kv->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  }
  if (d_ids && d_ids != kv->d_ids) SB_CUDA(cudaMemcpyAsync(d_ids, kv->d_ids, (size_t)kv->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  return STRICTB200_OK;
}

int strictb200_kv_device_ids(strictb200_kv* kv, int32_t** d_ids_out) {
  if (!kv || !d_ids_out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  *d_ids_out = kv->d_ids;
  return STRICTB200_OK;
}

int strictb200_generate(strictb200_model* m, strictb200_kv* kv, const int32_t* h_ids, int n_steps, int32_t* h_out) {
  if (!m || !kv || !h_ids || !h_out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(kv->m == m && n_steps >= 0, "bad arguments");
  if (!n_steps) return STRICTB200_OK;
  for (int b = 0; b < kv->B; b++) SB_REQUIRE(h_ids[b] >= 0 && h_ids[b] < m->c.vocab, "token id outside the vocabulary");
  if (kv->hist_cap < n_steps) {
    void* p;
    SB_CUDA(cudaMalloc(&p, (size_t)n_steps * kv->B * 4));
    kv->allocs.push_back(p);
    kv->d_hist = (int32_t*)p;
    kv->hist_cap = n_steps;
  }
  SB_CUDA(cudaMemcpyAsync(kv->d_ids, h_ids, (size_t)kv->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  SB_TRY(strictb200_decode_steps_device(m, kv, nullptr, n_steps));
  SB_CUDA(cudaMemcpyAsync(h_out, kv->d_hist, (size_t)n_steps * kv->B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  SB_TRY(sb_sync(ctx, "generate"));
  return sb_check_status(ctx, "generate");
}

int strictb200_profile_decode(strictb200_model* m, strictb200_kv* kv, int n_steps, float* ms_out, uint64_t* calls_out, int n_classes) {
  if (!m || !kv || !ms_out || !calls_out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  strictb200_ctx* ctx = m->ctx;
  SB_ENTER(ctx);
  SB_REQUIRE(kv->m == m && n_steps > 0 && n_classes >= STRICTB200_K_COUNT, "bad arguments");
  if (m->c.arch != STRICTB200_QWEN3) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "per-class timing covers the Qwen3 decode step");
  for (int i = 0; i < n_classes; i++) { ms_out[i] = 0.f; calls_out[i] = 0; }
  SbProfiler prof;
  int saved = m->use_graph;
  m->use_graph = 0;
  ctx->prof = &prof;
  int st = STRICTB200_OK;
  for (int s = 0; s < n_steps && st == STRICTB200_OK; s++) {
    st = decode_enqueue(m, kv);
    if (st == STRICTB200_OK && cudaMemcpyAsync(kv->d_ids, kv->d_next, (size_t)kv->B * 4, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
      st = sb_fail(STRICTB200_ERR_CUDA, "copy of the next ids failed");
  }
  ctx->prof = nullptr;
  m->use_graph = saved;
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (st == STRICTB200_OK && e == cudaSuccess) {
    for (const ProfSpan& sp : prof.spans) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) { ms_out[sp.cls] += ms; calls_out[sp.cls]++; }
    }
  }
  for (cudaEvent_t ev : prof.pool) cudaEventDestroy(ev);
  if (st != STRICTB200_OK) return st;
  if (e != cudaSuccess) return sb_fail(STRICTB200_ERR_CUDA, cudaGetErrorString(e));
  return STRICTB200_OK;
}

int strictb200_decode_bytes(strictb200_model* m, strictb200_kv* kv, uint64_t* out) {
  if (!m || !kv || !out) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  const auto& c = m->c;
  uint64_t kvb = 0;
  const uint64_t esz = c.arch == STRICTB200_QWEN3 ? 2 : 4;
  const uint64_t heads = c.arch == STRICTB200_QWEN3 ? m->Hkv_l : c.n_kv_heads;
  for (int b = 0; b < kv->B; b++) kvb += (uint64_t)(kv->h_lens[b] + 1) * heads * c.head_dim * 2 * esz * c.n_layers;
  *out = m->weight_bytes + kvb;
  return STRICTB200_OK;
}

}  // extern "C"
