// TEST INFRASTRUCTURE — CPU oracle for the LLM forward path (GPT-2 fp32, Qwen3 FP8).
//
// Only tests, the smoke check and the benchmark's cpu_baseline / reference arm may
// build or call this file; the product library never links it.
//
// PARITY UNPINNED: strict-lang/Strict has no LLM forward pass (its only device code is
// the element-wise emitter, Strict.Compiler.Cuda/InstructionsToCuda.cs:25-74), so no
// reference test pins these functions. They restate the architecture constants of the
// benchmark configurations under the numerics contract written next to each function.
// The element-wise ops (or_ew_binary / or_ew_program) follow
// Strict.Compiler.Cuda/InstructionsToCuda.cs:31-53,101-109 and are pinned by the four
// known answers of Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:46-57.
//
// Numerics contract of the FP8 (Qwen3) path, which the device kernels also follow:
//  * the residual stream is fp32 (a linear layer's fp32 result is added to it unrounded); the
//    qkv and gate/up projections hand their fp32 results to the fused consumers (QK-norm+RoPE,
//    SwiGLU) unrounded; norm outputs, q, k, v (the cache), the attention output and the SwiGLU
//    output are bf16;
//  * a linear layer computes y = (sum_k x_k * w_k) * s_w with bf16 inputs x, E4M3 weights w and
//    one fp32 scale per output channel: every product is exact, the sum is fp32 or better, the
//    output is rounded to bf16 (logits stay fp32). So that the FP8 tensor cores can take the
//    activations directly, a bf16 row is carried as TWO E4M3 terms with a power-of-two scale,
//    x = s * (hi + lo/16): s = 2^e is the smallest power of two with absmax/s <= 448,
//    hi = e4m3(x/s), lo = e4m3(16*(x/s - hi)). The split is exact for every element at or above
//    absmax/14336 (|x/s| >= 2^-6) and deterministic below; this file applies the same split
//    (or_split_rows);
//  * tensor parallelism changes only the order of the fp32 sums, so it has no oracle mode;
//  * RMSNorm: r = 1/sqrt(mean(x^2)+eps); y = bf16((x*r)*g), statistics in fp32 or better;
//  * RoPE pairs (i, i+D/2), angle = pos * theta^(-2i/D), cos/sin evaluated in double and
//    rounded to fp32; q/k are RMS-normalised per head first; results rounded to bf16;
//  * softmax in fp32 or better, scale 1/sqrt(D) applied to the fp32 score;
//  * logits are fp32 (not rounded to bf16); argmax ties go to the lowest index.
#include <omp.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <memory>
#include <vector>

#include "oracle_num.h"

using namespace oracle;

namespace {

// Allocator for the multi-gigabyte buffers (weights, embedding, KV cache): resize() leaves the
// elements untouched, so the first touch of every page is the parallel loop that fills it
// instead of a serial zero-fill that a second pass then overwrites.
template <class T>
struct NoInit : std::allocator<T> {
  template <class U> struct rebind { using other = NoInit<U>; };
  template <class U, class... A>
  void construct(U* p, A&&... a) {
    if constexpr (sizeof...(A) == 0) ::new ((void*)p) U;
    else ::new ((void*)p) U(std::forward<A>(a)...);
  }
};
using BigF = std::vector<float, NoInit<float>>;
using BigB = std::vector<uint8_t, NoInit<uint8_t>>;

struct Config {
  int arch;  // 0 = GPT-2 (fp32 weights), 1 = Qwen3 (E4M3 weights)
  int n_layers, d_model, n_q_heads, n_kv_heads, head_dim, d_ff, vocab, max_pos;
  float eps, rope_theta;
  int tied;
};

float E4M3_LUT[256];
struct LutInit {
  LutInit() {
    for (int i = 0; i < 256; i++) E4M3_LUT[i] = e4m3_to_f32((uint8_t)i);
  }
} lut_init;

// ---------------------------------------------------------------- primitives

// Power-of-two row scale: the smallest 2^e with absmax/2^e <= 448 (e = 0 for an all-zero row).
int scale_exponent(float amax) {
  if (!(amax >= 7.888609e-31f)) return 0;  // below 2^-100: treated as zero
  uint32_t b = f_bits(amax);
  int E = (int)((b >> 23) & 255) - 126;    // amax = f * 2^E, f in [0.5, 1)
  return (b & 0x7FFFFFu) <= 0x600000u ? E - 9 : E - 8;  // f <= 0.875 = 448 / 2^9
}

// Two-term E4M3 split of bf16-valued rows: x = s*(hi + lo/16). Writes hi/lo code bytes (may be
// null) and the dequantised value hi + lo/16 (may be null).
void split_rows(const float* x, int64_t M, int64_t K, int64_t ldx, uint8_t* hi, uint8_t* lo, float* eff, float* scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    const float* r = x + m * ldx;
    float amax = 0.f;
    for (int64_t k = 0; k < K; k++) amax = std::max(amax, std::fabs(r[k]));
    int e = scale_exponent(amax);
    float inv = std::ldexp(1.0f, -e);
    scale[m] = std::ldexp(1.0f, e);
    for (int64_t k = 0; k < K; k++) {
      float v = r[k] * inv;
      uint8_t h = f32_to_e4m3(v);
      float hv = E4M3_LUT[h];
      uint8_t l = f32_to_e4m3(16.0f * (v - hv));
      if (hi) hi[m * K + k] = h;
      if (lo) lo[m * K + k] = l;
      if (eff) eff[m * K + k] = hv + 0.0625f * E4M3_LUT[l];
    }
  }
}

// out[m,n] = (float(sum_k a[m,k]*w[n,k]) * sa[m]) * sw[n]; a = dequantised split activations
// (exact in fp32), w = E4M3 codes; products exact, sum in double.
void gemm_q(const float* af, const float* sa, const uint8_t* wq, int64_t ldw, const float* sw,
            int64_t M, int64_t N, int64_t K, float* out, int64_t ldo) {
#pragma omp parallel
  {
    std::vector<float> wf(K);
#pragma omp for schedule(dynamic, 16)
    for (int64_t n = 0; n < N; n++) {
      const uint8_t* wr = wq + n * ldw;
      for (int64_t k = 0; k < K; k++) wf[k] = E4M3_LUT[wr[k]];
      for (int64_t m = 0; m < M; m++) {
        const float* a = af + m * K;
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int64_t k = 0;
        for (; k + 8 <= K; k += 8)
          for (int j = 0; j < 8; j++) acc[j] += (double)a[k + j] * (double)wf[k + j];
        for (; k < K; k++) acc[0] += (double)a[k] * (double)wf[k];
        double t = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        out[m * ldo + n] = ((float)t * sa[m]) * sw[n];
      }
    }
  }
}

// y[m,n] = sum_k x[m,k]*w[n,k] + b[n], fp32 inputs, double accumulation.
void gemm_f32(const float* x, const float* w, const float* b, int64_t M, int64_t N, int64_t K,
              float* out) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t n = 0; n < N; n++) {
    const float* wr = w + n * K;
    for (int64_t m = 0; m < M; m++) {
      const float* a = x + m * K;
      double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int64_t k = 0;
      for (; k + 8 <= K; k += 8)
        for (int j = 0; j < 8; j++) acc[j] += (double)a[k + j] * (double)wr[k + j];
      for (; k < K; k++) acc[0] += (double)a[k] * (double)wr[k];
      double t = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      out[m * N + n] = (float)t + (b ? b[n] : 0.f);
    }
  }
}

void rmsnorm_row(const float* x, const float* g, int64_t d, float eps, float* y) {
  double ss = 0;
  for (int64_t i = 0; i < d; i++) ss += (double)x[i] * x[i];
  float ms = (float)(ss / (double)d);
  float r = 1.0f / std::sqrt(ms + eps);
  for (int64_t i = 0; i < d; i++) y[i] = (x[i] * r) * g[i];
}

void layernorm_row(const float* x, const float* g, const float* b, int64_t d, float eps, float* y) {
  double s = 0;
  for (int64_t i = 0; i < d; i++) s += x[i];
  float mean = (float)(s / (double)d);
  double v = 0;
  for (int64_t i = 0; i < d; i++) { double t = (double)x[i] - (double)mean; v += t * t; }
  float var = (float)(v / (double)d);
  float r = 1.0f / std::sqrt(var + eps);
  for (int64_t i = 0; i < d; i++) y[i] = ((x[i] - mean) * r) * g[i] + b[i];
}

float gelu_tanh(float x) {
  float u = 0.797884583f * (x + 0.044715f * ((x * x) * x));
  return (0.5f * x) * (1.0f + std::tanh(u));
}
float silu_mul(float g, float u) { return (g / (1.0f + std::exp(-g))) * u; }

// cos/sin table entry for position p and pair index i of D/2.
void rope_cs(int p, int i, int D, float theta, float* c, float* s) {
  double inv = std::pow((double)theta, -2.0 * (double)i / (double)D);
  double a = (double)p * inv;
  *c = (float)std::cos(a);
  *s = (float)std::sin(a);
}

// Per-head RMS norm (gain g[D]) then rotary embedding; in/out fp32 holding bf16 values.
void qknorm_rope_head(const float* x, const float* g, int D, float eps, int pos, float theta,
                      float* out) {
  std::vector<float> n(D);
  rmsnorm_row(x, g, D, eps, n.data());
  int h = D / 2;
  for (int i = 0; i < h; i++) {
    float c, s;
    rope_cs(pos, i, D, theta, &c, &s);
    out[i] = round_bf16(n[i] * c - n[i + h] * s);
    out[i + h] = round_bf16(n[i + h] * c + n[i] * s);
  }
}

// One query vector against keys/values [len, D] (row stride D). fp32 in, fp32 out (unrounded).
void attend_one(const float* q, const float* k, const float* v, int len, int D, float scale,
                float* out) {
  std::vector<float> s(len);
  float m = -INFINITY;
  for (int j = 0; j < len; j++) {
    double acc = 0;
    const float* kr = k + (int64_t)j * D;
    for (int i = 0; i < D; i++) acc += (double)q[i] * (double)kr[i];
    s[j] = (float)acc * scale;
    m = std::max(m, s[j]);
  }
  double l = 0;
  std::vector<double> o(D, 0.0);
  for (int j = 0; j < len; j++) {
    double p = std::exp((double)s[j] - (double)m);
    l += p;
    const float* vr = v + (int64_t)j * D;
    for (int i = 0; i < D; i++) o[i] += p * (double)vr[i];
  }
  for (int i = 0; i < D; i++) out[i] = (float)(o[i] / l);
}

// ---------------------------------------------------------------- model

struct QLinear {  // E4M3 weight [N,K] with per-row scale
  int64_t N = 0, K = 0;
  BigB q;
  std::vector<float> s;
};
struct FLinear {  // fp32 weight [N,K] with bias
  int64_t N = 0, K = 0;
  std::vector<float> w, b;
};

struct Layer {
  std::vector<float> norm1_g, norm1_b, norm2_g, norm2_b, qn_g, kn_g;
  QLinear wqkv, wo, wgu, wdown;  // Qwen
  FLinear fqkv, fo, ffc, fproj;  // GPT-2
};

struct Model {
  Config c;
  std::vector<Layer> L;
  BigF embed;  // Qwen: bf16 values held as fp32; GPT-2: fp32  [V,d]
  std::vector<float> wpe;    // GPT-2 [max_pos,d]
  std::vector<float> normf_g, normf_b;
  QLinear head;  // Qwen LM head (untied: own tensor; tied: quantised embedding)
};

struct State {
  int B, maxlen;
  std::vector<int> len;
  BigF k, v;  // [L][B][Hkv][maxlen][D]
};

void gen_normal_rows(uint64_t key, int64_t rows, int64_t K, float std_, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int64_t k = 0; k < K; k++) out[r * K + k] = std_ * normal_at(key, (uint64_t)(r * K + k));
}

// Generate rows [row0,row0+rows) of an E4M3 weight whose fp32 source is std*N(0,1).
void gen_qlinear_rows(uint64_t key, int64_t rows, int64_t K, float std_, uint8_t* q, float* s) {
#pragma omp parallel
  {
    std::vector<float> w(K);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      float amax = 0.f;
      for (int64_t k = 0; k < K; k++) {
        w[k] = std_ * normal_at(key, (uint64_t)(r * K + k));
        amax = std::max(amax, std::fabs(w[k]));
      }
      float inv = 1.0f, sc = 1.0f;
      if (amax > 0.f) { inv = 448.0f / amax; sc = amax / 448.0f; }
      for (int64_t k = 0; k < K; k++) q[r * K + k] = f32_to_e4m3(w[k] * inv);
      s[r] = sc;
    }
  }
}

enum { T_NORM1 = 0, T_Q = 1, T_K = 2, T_V = 3, T_QN = 4, T_KN = 5, T_O = 6, T_NORM2 = 7,
       T_GATE = 8, T_UP = 9, T_DOWN = 10 };
enum { G_EMBED = 1, G_WPE = 2, G_HEAD = 3, G_NORMF = 4 };
uint64_t layer_tensor(int l, int kind) { return 16ull * (uint64_t)(l + 1) + (uint64_t)kind; }

// Per-row absmax quantisation of a weight matrix given as fp32 values (the tied LM head).
void quant_weight_rows(const float* x, int64_t M, int64_t K, uint8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    const float* r = x + m * K;
    float amax = 0.f;
    for (int64_t k = 0; k < K; k++) amax = std::max(amax, std::fabs(r[k]));
    float inv = 1.0f, sc = 1.0f;
    if (amax > 0.f) { inv = 448.0f / amax; sc = amax / 448.0f; }
    for (int64_t k = 0; k < K; k++) q[m * K + k] = f32_to_e4m3(r[k] * inv);
    scale[m] = sc;
  }
}
void quant_head_from_embed(Model* m) {
  const Config& c = m->c;
  m->head.N = c.vocab; m->head.K = c.d_model;
  m->head.q.resize((size_t)c.vocab * c.d_model);
  m->head.s.resize(c.vocab);
  quant_weight_rows(m->embed.data(), c.vocab, c.d_model, m->head.q.data(), m->head.s.data());
}

Model* model_create(const Config& c, uint64_t seed) {
  Model* m = new Model;
  m->c = c;
  const float SD = 0.02f;
  int64_t d = c.d_model, D = c.head_dim, I = c.d_ff;
  int64_t nq = (int64_t)c.n_q_heads * D, nkv = (int64_t)c.n_kv_heads * D;
  m->L.resize(c.n_layers);
  m->embed.resize((size_t)c.vocab * d);
  gen_normal_rows(stream_key(seed, G_EMBED), c.vocab, d, SD, m->embed.data());
  m->normf_g.assign(d, 1.0f); m->normf_b.assign(d, 0.0f);
  if (c.arch == 0) {
    m->wpe.resize((size_t)c.max_pos * d);
    gen_normal_rows(stream_key(seed, G_WPE), c.max_pos, d, SD, m->wpe.data());
  } else {
    {
      float* e = m->embed.data();
      const int64_t n = (int64_t)m->embed.size();
#pragma omp parallel for schedule(static)
      for (int64_t i = 0; i < n; i++) e[i] = round_bf16(e[i]);
    }
    if (c.tied) quant_head_from_embed(m);
    else {
      m->head.N = c.vocab; m->head.K = d;
      m->head.q.resize((size_t)c.vocab * d); m->head.s.resize(c.vocab);
      gen_qlinear_rows(stream_key(seed, G_HEAD), c.vocab, d, SD, m->head.q.data(), m->head.s.data());
    }
  }
  for (int l = 0; l < c.n_layers; l++) {
    Layer& y = m->L[l];
    y.norm1_g.assign(d, 1.0f); y.norm1_b.assign(d, 0.0f);
    y.norm2_g.assign(d, 1.0f); y.norm2_b.assign(d, 0.0f);
    if (c.arch == 0) {
      auto mk = [&](FLinear& f, int64_t N, int64_t K) { f.N = N; f.K = K; f.w.resize((size_t)N * K); f.b.assign(N, 0.f); };
      mk(y.fqkv, 3 * d, d);
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_Q)), d, d, SD, y.fqkv.w.data());
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_K)), d, d, SD, y.fqkv.w.data() + d * d);
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_V)), d, d, SD, y.fqkv.w.data() + 2 * d * d);
      mk(y.fo, d, d);
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_O)), d, d, SD, y.fo.w.data());
      mk(y.ffc, I, d);
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_GATE)), I, d, SD, y.ffc.w.data());
      mk(y.fproj, d, I);
      gen_normal_rows(stream_key(seed, layer_tensor(l, T_DOWN)), d, I, SD, y.fproj.w.data());
    } else {
      y.qn_g.assign(D, 1.0f); y.kn_g.assign(D, 1.0f);
      auto mk = [&](QLinear& f, int64_t N, int64_t K) { f.N = N; f.K = K; f.q.resize((size_t)N * K); f.s.resize(N); };
      mk(y.wqkv, nq + 2 * nkv, d);
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_Q)), nq, d, SD, y.wqkv.q.data(), y.wqkv.s.data());
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_K)), nkv, d, SD, y.wqkv.q.data() + nq * d, y.wqkv.s.data() + nq);
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_V)), nkv, d, SD, y.wqkv.q.data() + (nq + nkv) * d, y.wqkv.s.data() + nq + nkv);
      mk(y.wo, d, nq);
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_O)), d, nq, SD, y.wo.q.data(), y.wo.s.data());
      mk(y.wgu, 2 * I, d);
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_GATE)), I, d, SD, y.wgu.q.data(), y.wgu.s.data());
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_UP)), I, d, SD, y.wgu.q.data() + I * d, y.wgu.s.data() + I);
      mk(y.wdown, d, I);
      gen_qlinear_rows(stream_key(seed, layer_tensor(l, T_DOWN)), d, I, SD, y.wdown.q.data(), y.wdown.s.data());
    }
  }
  return m;
}

// Linear layer on bf16-valued rows x[T, K]: exact products with the E4M3 weights.
void qlinear(const QLinear& w, const float* x, int64_t T, float* out) {
  std::vector<float> eff((size_t)T * w.K), sa(T);
  split_rows(x, T, w.K, w.K, nullptr, nullptr, eff.data(), sa.data());
  gemm_q(eff.data(), sa.data(), w.q.data(), w.K, w.s.data(), T, w.N, w.K, out, w.N);
}

float* kv_at(BigF& buf, const Model* m, const State* st, int l, int b, int h) {
  const Config& c = m->c;
  return buf.data() + ((((int64_t)l * st->B + b) * c.n_kv_heads + h) * st->maxlen) * c.head_dim;
}

// Run `S` new tokens per sequence (row-major tokens[B,S]; only the first n_new[b] are real)
// through the model, append to the cache, return fp32 logits [B,V] of each sequence's last
// real token.
void forward(Model* m, State* st, const int* tokens, const int* n_new, int B, int S, float* logits) {
  const Config& c = m->c;
  int64_t d = c.d_model, D = c.head_dim, I = c.d_ff;
  int Hq = c.n_q_heads, Hkv = c.n_kv_heads, G = Hq / Hkv;
  int64_t nq = (int64_t)Hq * D, nkv = (int64_t)Hkv * D, nqkv = nq + 2 * nkv;
  // Pack real tokens: row t <-> (b, i)
  std::vector<int> rb, rpos, rtok;
  for (int b = 0; b < B; b++)
    for (int i = 0; i < n_new[b]; i++) { rb.push_back(b); rpos.push_back(st->len[b] + i); rtok.push_back(tokens[b * S + i]); }
  int64_t T = (int64_t)rb.size();
  std::vector<float> x((size_t)T * d), a((size_t)T * d), qkv((size_t)T * nqkv), att((size_t)T * nq),
      y((size_t)T * d), gu, hact((size_t)T * I);
  const bool qw = c.arch == 1;
  for (int64_t t = 0; t < T; t++)
    for (int64_t i = 0; i < d; i++) {
      float e = m->embed[(size_t)rtok[t] * d + i];
      x[t * d + i] = qw ? e : e + m->wpe[(size_t)rpos[t] * d + i];
    }
  float scale = 1.0f / std::sqrt((float)D);
  for (int l = 0; l < c.n_layers; l++) {
    Layer& ly = m->L[l];
    // --- attention block
#pragma omp parallel for
    for (int64_t t = 0; t < T; t++) {
      if (qw) { rmsnorm_row(&x[t * d], ly.norm1_g.data(), d, c.eps, &a[t * d]); for (int64_t i = 0; i < d; i++) a[t * d + i] = round_bf16(a[t * d + i]); }
      else layernorm_row(&x[t * d], ly.norm1_g.data(), ly.norm1_b.data(), d, c.eps, &a[t * d]);
    }
    if (qw) {
      qlinear(ly.wqkv, a.data(), T, qkv.data());
    } else gemm_f32(a.data(), ly.fqkv.w.data(), ly.fqkv.b.data(), T, nqkv, d, qkv.data());
    // q/k post-processing + cache append
#pragma omp parallel for
    for (int64_t t = 0; t < T; t++) {
      float* row = &qkv[t * nqkv];
      int b = rb[t], p = rpos[t];
      if (qw) {
        std::vector<float> tmp(D);
        for (int h = 0; h < Hq; h++) {
          qknorm_rope_head(row + h * D, ly.qn_g.data(), (int)D, c.eps, p, c.rope_theta, tmp.data());
          std::copy(tmp.begin(), tmp.end(), row + h * D);
        }
        for (int h = 0; h < Hkv; h++) {
          qknorm_rope_head(row + nq + h * D, ly.kn_g.data(), (int)D, c.eps, p, c.rope_theta, tmp.data());
          std::copy(tmp.begin(), tmp.end(), row + nq + h * D);
        }
      }
      for (int h = 0; h < Hkv; h++) {
        std::copy(row + nq + h * D, row + nq + (h + 1) * D, kv_at(st->k, m, st, l, b, h) + (int64_t)p * D);
        float* vdst = kv_at(st->v, m, st, l, b, h) + (int64_t)p * D;
        for (int i = 0; i < D; i++) vdst[i] = qw ? round_bf16(row[nq + nkv + h * D + i]) : row[nq + nkv + h * D + i];
      }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t t = 0; t < T; t++) {
      int b = rb[t], p = rpos[t];
      for (int h = 0; h < Hq; h++) {
        float* o = &att[t * nq + h * D];
        attend_one(&qkv[t * nqkv + h * D], kv_at(st->k, m, st, l, b, h / G), kv_at(st->v, m, st, l, b, h / G),
                   p + 1, (int)D, scale, o);
        if (qw) for (int i = 0; i < D; i++) o[i] = round_bf16(o[i]);
      }
    }
    if (qw) {
      qlinear(ly.wo, att.data(), T, y.data());
      for (int64_t i = 0; i < T * d; i++) x[i] = x[i] + y[i];
    } else {
      gemm_f32(att.data(), ly.fo.w.data(), ly.fo.b.data(), T, d, nq, y.data());
      for (int64_t i = 0; i < T * d; i++) x[i] = x[i] + y[i];
    }
    // --- MLP block
#pragma omp parallel for
    for (int64_t t = 0; t < T; t++) {
      if (qw) { rmsnorm_row(&x[t * d], ly.norm2_g.data(), d, c.eps, &a[t * d]); for (int64_t i = 0; i < d; i++) a[t * d + i] = round_bf16(a[t * d + i]); }
      else layernorm_row(&x[t * d], ly.norm2_g.data(), ly.norm2_b.data(), d, c.eps, &a[t * d]);
    }
    if (qw) {
      gu.resize((size_t)T * 2 * I);
      qlinear(ly.wgu, a.data(), T, gu.data());
#pragma omp parallel for
      for (int64_t t = 0; t < T; t++)
        for (int64_t i = 0; i < I; i++)
          hact[t * I + i] = round_bf16(silu_mul(gu[t * 2 * I + i], gu[t * 2 * I + I + i]));
      qlinear(ly.wdown, hact.data(), T, y.data());
      for (int64_t i = 0; i < T * d; i++) x[i] = x[i] + y[i];
    } else {
      gu.resize((size_t)T * I);
      gemm_f32(a.data(), ly.ffc.w.data(), ly.ffc.b.data(), T, I, d, gu.data());
      for (int64_t i = 0; i < T * I; i++) hact[i] = gelu_tanh(gu[i]);
      gemm_f32(hact.data(), ly.fproj.w.data(), ly.fproj.b.data(), T, d, I, y.data());
      for (int64_t i = 0; i < T * d; i++) x[i] = x[i] + y[i];
    }
  }
  // --- last real token of each sequence -> final norm -> head
  std::vector<float> last((size_t)B * d, 0.f);
  {
    int64_t t = 0;
    for (int b = 0; b < B; b++) {
      if (n_new[b] > 0) {
        const float* src = &x[(t + n_new[b] - 1) * d];
        if (qw) { rmsnorm_row(src, m->normf_g.data(), d, c.eps, &last[b * d]); for (int64_t i = 0; i < d; i++) last[b * d + i] = round_bf16(last[b * d + i]); }
        else layernorm_row(src, m->normf_g.data(), m->normf_b.data(), d, c.eps, &last[b * d]);
      }
      t += n_new[b];
      st->len[b] += n_new[b];
    }
  }
  if (logits) {
    if (qw) qlinear(m->head, last.data(), B, logits);
    else gemm_f32(last.data(), m->embed.data(), nullptr, B, c.vocab, d, logits);
  }
}

struct NamedTensor { void* ptr; int64_t bytes; };

NamedTensor find_tensor(Model* m, const std::string& name) {
  auto F = [](auto& v) { return NamedTensor{v.data(), (int64_t)v.size() * 4}; };
  auto U = [](auto& v) { return NamedTensor{v.data(), (int64_t)v.size()}; };
  if (name == "embed") return F(m->embed);
  if (name == "wpe") return F(m->wpe);
  if (name == "normf.g") return F(m->normf_g);
  if (name == "normf.b") return F(m->normf_b);
  if (name == "head.q") return U(m->head.q);
  if (name == "head.s") return F(m->head.s);
  if (name.rfind("layers.", 0) == 0) {
    size_t dot = name.find('.', 7);
    int l = std::atoi(name.substr(7, dot - 7).c_str());
    if (l < 0 || l >= (int)m->L.size()) return {nullptr, 0};
    Layer& y = m->L[l];
    std::string k = name.substr(dot + 1);
    if (k == "norm1.g") return F(y.norm1_g);
    if (k == "norm1.b") return F(y.norm1_b);
    if (k == "norm2.g") return F(y.norm2_g);
    if (k == "norm2.b") return F(y.norm2_b);
    if (k == "qnorm.g") return F(y.qn_g);
    if (k == "knorm.g") return F(y.kn_g);
    if (k == "wqkv.q") return U(y.wqkv.q);
    if (k == "wqkv.s") return F(y.wqkv.s);
    if (k == "wo.q") return U(y.wo.q);
    if (k == "wo.s") return F(y.wo.s);
    if (k == "wgu.q") return U(y.wgu.q);
    if (k == "wgu.s") return F(y.wgu.s);
    if (k == "wdown.q") return U(y.wdown.q);
    if (k == "wdown.s") return F(y.wdown.s);
    if (k == "wqkv.w") return F(y.fqkv.w);
    if (k == "wqkv.b") return F(y.fqkv.b);
    if (k == "wo.w") return F(y.fo.w);
    if (k == "wo.b") return F(y.fo.b);
    if (k == "wfc.w") return F(y.ffc.w);
    if (k == "wfc.b") return F(y.ffc.b);
    if (k == "wproj.w") return F(y.fproj.w);
    if (k == "wproj.b") return F(y.fproj.b);
  }
  return {nullptr, 0};
}

}  // namespace

// ================================================================== C interface (ctypes)
extern "C" {

int or_num_threads(void) { return omp_get_max_threads(); }
void or_set_threads(int n) { omp_set_num_threads(n); }

// ---- generator / formats
uint64_t or_stream_key(uint64_t seed, uint64_t tensor) { return stream_key(seed, tensor); }
void or_gen_normal(uint64_t seed, uint64_t tensor, int64_t first, int64_t count, float std_, float* out) {
  uint64_t key = stream_key(seed, tensor);
#pragma omp parallel for
  for (int64_t i = 0; i < count; i++) out[i] = std_ * normal_at(key, (uint64_t)(first + i));
}
void or_gen_tokens(uint64_t seed, uint64_t tensor, int64_t count, uint32_t range, int32_t* out) {
  uint64_t key = stream_key(seed, tensor);
  for (int64_t i = 0; i < count; i++) out[i] = (int32_t)uniform_int(key, (uint64_t)i, range);
}
void or_gen_qlinear(uint64_t seed, uint64_t tensor, int64_t rows, int64_t K, float std_, uint8_t* q, float* s) {
  gen_qlinear_rows(stream_key(seed, tensor), rows, K, std_, q, s);
}
void or_f32_to_bf16(const float* x, int64_t n, uint16_t* out) { for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16(x[i]); }
void or_bf16_to_f32(const uint16_t* x, int64_t n, float* out) { for (int64_t i = 0; i < n; i++) out[i] = bf16_to_f32(x[i]); }
void or_f32_to_e4m3(const float* x, int64_t n, uint8_t* out) { for (int64_t i = 0; i < n; i++) out[i] = f32_to_e4m3(x[i]); }
void or_e4m3_to_f32(const uint8_t* x, int64_t n, float* out) { for (int64_t i = 0; i < n; i++) out[i] = e4m3_to_f32(x[i]); }

// ---- element-wise surface (Strict.Compiler.Cuda/InstructionsToCuda.cs:101-109)
// op: 0 add, 1 subtract, 2 multiply, 3 divide. C float semantics.
int or_ew_binary(int op, const float* a, const float* b, float* out, int64_t n) {
  if (op < 0 || op > 3) return 1;
  for (int64_t i = 0; i < n; i++) {
    float x = a[i], y = b[i];
    out[i] = op == 0 ? x + y : op == 1 ? x - y : op == 2 ? x * y : x / y;
  }
  return 0;
}
// Register program of (opcode, a, b, c) int32 quadruples, the instruction subset the
// emitter handles (InstructionsToCuda.cs:31-53): 0 LOAD_ARRAY r[c]=arrays[a][idx];
// 1 LOAD_SCALAR r[c]=scalars[a]; 2 LOAD_CONST r[c]=consts[a]; 3..6 ADD/SUB/MUL/DIV
// r[c]=r[a] op r[b]; 7 RETURN r[a]. Without a RETURN the output is 0.0f (cs:30).
int or_ew_program(const int32_t* code, int n_instr, const float* const* arrays, const float* scalars,
                  const float* consts, float* out, int64_t n) {
  for (int64_t idx = 0; idx < n; idx++) {
    float r[16] = {0};
    float res = 0.0f;
    for (int i = 0; i < n_instr; i++) {
      const int32_t* q = code + 4 * i;
      switch (q[0]) {
        case 0: r[q[3]] = arrays[q[1]][idx]; break;
        case 1: r[q[3]] = scalars[q[1]]; break;
        case 2: r[q[3]] = consts[q[1]]; break;
        case 3: r[q[3]] = r[q[1]] + r[q[2]]; break;
        case 4: r[q[3]] = r[q[1]] - r[q[2]]; break;
        case 5: r[q[3]] = r[q[1]] * r[q[2]]; break;
        case 6: r[q[3]] = r[q[1]] / r[q[2]]; break;
        case 7: res = r[q[1]]; break;
        default: return 1;
      }
    }
    out[idx] = res;
  }
  return 0;
}

// ---- primitives (fp32 buffers hold the values; callers round to bf16 where the contract says)
void or_split_rows(const float* x, int64_t M, int64_t K, uint8_t* hi, uint8_t* lo, float* eff, float* scale) {
  split_rows(x, M, K, K, hi, lo, eff, scale);
}
void or_quant_weight_rows(const float* x, int64_t M, int64_t K, uint8_t* q, float* scale) { quant_weight_rows(x, M, K, q, scale); }
// y = (x . W^T) * sw for bf16-valued x [M,K] and E4M3 W [N,K]; fp32 result (unrounded)
void or_linear_fp8w(const float* x, const uint8_t* wq, const float* sw, int64_t M, int64_t N, int64_t K, float* out) {
  std::vector<float> eff((size_t)M * K), sa(M);
  split_rows(x, M, K, K, nullptr, nullptr, eff.data(), sa.data());
  gemm_q(eff.data(), sa.data(), wq, K, sw, M, N, K, out, N);
}
void or_gemm_f32(const float* x, const float* w, const float* b, int64_t M, int64_t N, int64_t K, float* out) { gemm_f32(x, w, b, M, N, K, out); }
void or_rmsnorm(const float* x, const float* g, int64_t M, int64_t d, float eps, float* y) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; m++) rmsnorm_row(x + m * d, g, d, eps, y + m * d);
}
void or_layernorm(const float* x, const float* g, const float* b, int64_t M, int64_t d, float eps, float* y) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; m++) layernorm_row(x + m * d, g, b, d, eps, y + m * d);
}
void or_gelu_tanh(const float* x, int64_t n, float* y) { for (int64_t i = 0; i < n; i++) y[i] = gelu_tanh(x[i]); }
void or_swiglu(const float* gate, const float* up, int64_t n, float* y) { for (int64_t i = 0; i < n; i++) y[i] = silu_mul(gate[i], up[i]); }
void or_rope_table(int n_pos, int D, float theta, float* cos_out, float* sin_out) {
  for (int p = 0; p < n_pos; p++)
    for (int i = 0; i < D / 2; i++) rope_cs(p, i, D, theta, &cos_out[p * (D / 2) + i], &sin_out[p * (D / 2) + i]);
}
// x [T, H, D] fp32 (bf16 values), positions [T]; out rounded to bf16 values.
void or_qknorm_rope(const float* x, const float* g, const int* pos, int64_t T, int H, int D, float eps,
                    float theta, float* out) {
#pragma omp parallel for
  for (int64_t t = 0; t < T; t++)
    for (int h = 0; h < H; h++)
      qknorm_rope_head(x + (t * H + h) * D, g, D, eps, pos[t], theta, out + (t * H + h) * D);
}
// Causal GQA attention over packed sequences. q [B,S,Hq,D], k/v [B,S,Hkv,D]; out [B,S,Hq,D] fp32
// (unrounded). Only rows < lens[b] are computed.
void or_attn_prefill(const float* q, const float* k, const float* v, const int* lens, int B, int S,
                     int Hq, int Hkv, int D, float scale, float* out) {
  int G = Hq / Hkv;
#pragma omp parallel
  {
    std::vector<float> kk, vv;
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; b++)
      for (int h = 0; h < Hq; h++) {
        int len = lens[b];
        kk.resize((size_t)len * D); vv.resize((size_t)len * D);
        for (int j = 0; j < len; j++) {
          const float* kr = k + (((int64_t)b * S + j) * Hkv + h / G) * D;
          const float* vr = v + (((int64_t)b * S + j) * Hkv + h / G) * D;
          std::copy(kr, kr + D, &kk[(size_t)j * D]);
          std::copy(vr, vr + D, &vv[(size_t)j * D]);
        }
        for (int i = 0; i < len; i++)
          attend_one(q + (((int64_t)b * S + i) * Hq + h) * D, kk.data(), vv.data(), i + 1, D, scale,
                     out + (((int64_t)b * S + i) * Hq + h) * D);
      }
  }
}
// Decode attention: q [B,Hq,D]; caches [B,Hkv,maxlen,D]; lens[b] keys are attended.
void or_attn_decode(const float* q, const float* kc, const float* vc, const int* lens, int B, int Hq,
                    int Hkv, int maxlen, int D, float scale, float* out) {
  int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; b++)
    for (int h = 0; h < Hq; h++) {
      int64_t off = (((int64_t)b * Hkv + h / G) * maxlen) * D;
      attend_one(q + ((int64_t)b * Hq + h) * D, kc + off, vc + off, lens[b], D, scale,
                 out + ((int64_t)b * Hq + h) * D);
    }
}
void or_argmax(const float* x, int64_t M, int64_t N, int32_t* out) {
  for (int64_t m = 0; m < M; m++) {
    int64_t best = 0;
    for (int64_t n = 1; n < N; n++) if (x[m * N + n] > x[m * N + best]) best = n;
    out[m] = (int32_t)best;
  }
}

// ---- model
void* or_model_create(const int32_t* icfg, float eps, float rope_theta, uint64_t seed) {
  Config c;
  c.arch = icfg[0]; c.n_layers = icfg[1]; c.d_model = icfg[2]; c.n_q_heads = icfg[3];
  c.n_kv_heads = icfg[4]; c.head_dim = icfg[5]; c.d_ff = icfg[6]; c.vocab = icfg[7];
  c.max_pos = icfg[8]; c.tied = icfg[9]; c.eps = eps; c.rope_theta = rope_theta;
  return model_create(c, seed);
}
void or_model_free(void* m) { delete (Model*)m; }
// Returns a pointer into the model's storage (fp32 or E4M3 bytes); the caller may read or
// overwrite it in place. After overwriting "embed" of a tied Qwen model call or_model_retie.
int64_t or_model_tensor(void* m, const char* name, void** ptr) {
  NamedTensor t = find_tensor((Model*)m, name);
  *ptr = t.ptr;
  return t.bytes;
}
void or_model_retie(void* m) { Model* mm = (Model*)m; if (mm->c.arch == 1 && mm->c.tied) quant_head_from_embed(mm); }
void* or_state_create(void* mv, int B, int maxlen) {
  Model* m = (Model*)mv;
  State* s = new State;
  s->B = B; s->maxlen = maxlen; s->len.assign(B, 0);
  size_t n = (size_t)m->c.n_layers * B * m->c.n_kv_heads * maxlen * m->c.head_dim;
  s->k.resize(n); s->v.resize(n);
  float *kp = s->k.data(), *vp = s->v.data();
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; i++) { kp[i] = 0.f; vp[i] = 0.f; }
  return s;
}
void or_state_free(void* s) { delete (State*)s; }
void or_state_reset(void* s) { State* st = (State*)s; std::fill(st->len.begin(), st->len.end(), 0); }
void or_state_lens(void* s, int32_t* out) { State* st = (State*)s; for (int b = 0; b < st->B; b++) out[b] = st->len[b]; }
// The larger instruction set of the element-wise surface (conditionals, loops, variables, loads
// at computed indices): CPU meaning of the same quadruples the device interpreter runs. The
// arithmetic is C float as in the emitted CUDA C (InstructionsToCuda.cs:101-109); the condition
// flag, jumps and loops follow the reference VM's instruction set (Strict.Bytecode/InstructionType.cs:
// 9-47: Modulo, Equal..GreaterThan, Jump*, LoopBegin/LoopEnd, ListCall). Returns 2 if an element
// ran past the step budget.
int or_ew_program2(const int32_t* code, int n_instr, const float* const* arrays, const float* scalars,
                   const float* consts, float* out, int64_t n) {
  int rc = 0;
  for (int64_t idx = 0; idx < n; idx++) {
    float r[32] = {0};
    int loop_begin[4], loop_count[4], loop_i[4], depth = 0;
    bool flag = false;
    float res = 0.0f;
    int pc = 0, steps = 0;
    while (pc < n_instr) {
      if (++steps > (1 << 16)) { res = 0.0f; rc = 2; break; }
      const int32_t* q = code + 4 * pc;
      const int op = q[0], a = q[1], b = q[2], c = q[3];
      int next = pc + 1;
      switch (op) {
        case 0: r[c] = arrays[a][idx]; break;
        case 1: r[c] = scalars[a]; break;
        case 2: r[c] = consts[a]; break;
        case 3: r[c] = r[a] + r[b]; break;
        case 4: r[c] = r[a] - r[b]; break;
        case 5: r[c] = r[a] * r[b]; break;
        case 6: r[c] = r[a] / r[b]; break;
        case 7: res = r[a]; next = n_instr; break;
        case 8: r[c] = std::fmod(r[a], r[b]); break;
        case 9: flag = r[a] == r[b]; break;
        case 10: flag = r[a] != r[b]; break;
        case 11: flag = r[a] < r[b]; break;
        case 12: flag = r[a] > r[b]; break;
        case 13: next = a; break;
        case 14: if (flag) next = a; break;
        case 15: if (!flag) next = a; break;
        case 16: {
          const float cf = r[a];
          const int count = cf >= 1.0f ? (cf < 1048576.0f ? (int)cf : 1048576) : 0;
          if (count <= 0 || depth >= 4) { next = b; break; }
          loop_begin[depth] = pc; loop_count[depth] = count; loop_i[depth] = 0; depth++;
          r[c] = 0.0f;
          break;
        }
        case 17:
          if (depth > 0 && loop_begin[depth - 1] == a) {
            if (++loop_i[depth - 1] < loop_count[depth - 1]) { r[code[4 * a + 3]] = (float)loop_i[depth - 1]; next = a + 1; }
            else depth--;
          }
          break;
        case 18: { const float f = r[b]; r[c] = (f >= 0.0f && f < (float)n) ? arrays[a][(int64_t)f] : 0.0f; break; }
        case 19: r[c] = r[a]; break;
        case 20: r[c] = (float)idx; break;
        default: return 1;
      }
      pc = next;
    }
    out[idx] = res;
  }
  return rc;
}

// 5x5 box blur over interleaved RGB bytes, restating
// Strict.Compiler.Assembly.Tests/BlurPerformanceTests.cs:52-141: a pixel with all 25 neighbours
// inside the image (row and column in [2, size-2)) gets sum / 25 per channel (BlurInteriorPixel,
// :85-120), any other pixel the sum of the neighbours that exist divided by their count
// (BlurEdgePixel, :122-141); integer division, result written to a second buffer.
void or_blur5x5_rgb8(const uint8_t* src, uint8_t* dst, int width, int height) {
  const int64_t stride = (int64_t)width * 3;
#pragma omp parallel for schedule(static)
  for (int row = 0; row < height; row++)
    for (int column = 0; column < width; column++) {
      const int64_t base = row * stride + (int64_t)column * 3;
      const bool interior = row >= 2 && row < height - 2 && column >= 2 && column < width - 2;
      for (int channel = 0; channel < 3; channel++) {
        if (interior) {
          int sum = 0;
          for (int ky = -2; ky <= 2; ky++)
            for (int kx = -2; kx <= 2; kx++) sum += src[base + ky * stride + kx * 3 + channel];
          dst[base + channel] = (uint8_t)(sum / 25);
        } else {
          int sum = 0, count = 0;
          for (int ky = -2; ky <= 2; ky++)
            for (int kx = -2; kx <= 2; kx++) {
              const int nx = column + kx, ny = row + ky;
              if ((unsigned)nx >= (unsigned)width || (unsigned)ny >= (unsigned)height) continue;
              sum += src[ny * stride + (int64_t)nx * 3 + channel];
              count++;
            }
          dst[base + channel] = (uint8_t)(sum / count);
        }
      }
    }
}
// The reference's harness blurs in place, iteration after iteration (ApplyBlurSingleThread copies
// its output over the input, :66): `iterations` passes, result in `pixels`.
void or_blur5x5_rgb8_inplace(uint8_t* pixels, int width, int height, int iterations) {
  std::vector<uint8_t> out((size_t)width * height * 3);
  for (int it = 0; it < iterations; it++) {
    or_blur5x5_rgb8(pixels, out.data(), width, height);
    std::copy(out.begin(), out.end(), pixels);
  }
}
// AdjustBrightness over the flat number layout of ValueArrayInstance (element i, member m at
// offset + i*flat_width + m, fp32; Strict.Expressions/ValueArrayInstance.cs:128,339): the first
// `channels` members of every element get `brightness` added
// (ImageProcessing/AdjustBrightness.strict:16), in double as the VM computes
// (Strict/VirtualMachine.Loops.cs:312-327), stored back as float
// (ValueArrayInstance.cs:105). clamp01 keeps the result inside [0,1], the range Color.strict
// allows; the .strict code itself does not clamp.
void or_adjust_brightness(float* flat, int64_t offset, int64_t count, int flat_width, int channels, double brightness, int clamp01) {
  for (int64_t i = 0; i < count; i++)
    for (int m = 0; m < channels; m++) {
      double s = (double)flat[offset + i * flat_width + m] + brightness;
      if (clamp01) s = s < 0.0 ? 0.0 : (s > 1.0 ? 1.0 : s);
      flat[offset + i * flat_width + m] = (float)s;
    }
}

// int8-weight linear layer (numerics contract of the integer path; no reference counterpart, so
// unpinned like the FP8 path, but every intermediate is an exact integer and the device result
// must equal this one bit for bit):
//  * weights: one fp32 scale per output channel, sw = absmax / 127 (1 for a row of zeros),
//    q = round-to-nearest-even(w / sw) clamped to [-127, 127];
//  * activations: per token, s = the smallest power of two with absmax / s <= 16256 (1 for a row of
//    zeros), v = round-to-nearest-even(x / s) (exact scaling), carried as v = 128 * hi + lo with
//    hi = floor((v + 64) / 128) in [-127, 127] and lo in [-64, 63];
//  * y = bf16(((float)(128 * sum_k hi*q + sum_k lo*q) * s) * sw): integer sums, one conversion to
//    fp32 (round to nearest even), two fp32 products, one rounding to bf16.
void or_quantize_weights_int8(const float* w, int64_t N, int64_t K, int8_t* q, float* sw) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    float amax = 0.f;
    for (int64_t k = 0; k < K; k++) amax = std::max(amax, std::fabs(w[n * K + k]));
    const float s = amax > 0.f ? amax / 127.f : 1.f;
    sw[n] = s;
    for (int64_t k = 0; k < K; k++) {
      int v = (int)std::nearbyint(w[n * K + k] / s);
      q[n * K + k] = (int8_t)std::min(127, std::max(-127, v));
    }
  }
}
// x: bf16-valued fp32 rows. hi, lo: [M, K]; scale: [M].
void or_quantize_rows_int8(const float* x, int64_t M, int64_t K, int8_t* hi, int8_t* lo, float* scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    float amax = 0.f;
    for (int64_t k = 0; k < K; k++) amax = std::max(amax, std::fabs(x[m * K + k]));
    float s = 1.f;
    if (amax > 0.f) {
      int e;
      const float mant = std::frexp(amax, &e);
      s = std::ldexp(1.f, mant <= 0.9921875f ? e - 14 : e - 13);
    }
    scale[m] = s;
    const float inv = 1.f / s;
    for (int64_t k = 0; k < K; k++) {
      const int v = (int)std::nearbyint(x[m * K + k] * inv);
      const int h = (v + 64) >> 7;
      hi[m * K + k] = (int8_t)h;
      lo[m * K + k] = (int8_t)(v - h * 128);
    }
  }
}
// out: bf16 bit patterns [M, N].
void or_gemm_int8w(const float* x, const int8_t* wq, const float* sw, int64_t M, int64_t N, int64_t K, uint16_t* out) {
  std::vector<int8_t> hi((size_t)M * K), lo((size_t)M * K);
  std::vector<float> sx((size_t)M);
  or_quantize_rows_int8(x, M, K, hi.data(), lo.data(), sx.data());
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++)
    for (int64_t m = 0; m < M; m++) {
      int64_t sh = 0, sl = 0;
      const int8_t *h = &hi[(size_t)m * K], *l = &lo[(size_t)m * K], *w = wq + n * K;
      for (int64_t k = 0; k < K; k++) { sh += (int)h[k] * (int)w[k]; sl += (int)l[k] * (int)w[k]; }
      const float v = (float)(sh * 128 + sl);
      out[m * N + n] = f32_to_bf16((v * sx[m]) * sw[n]);
    }
}

// Benchmark set-up only: positions [0,len) of every sequence get cheap pseudo-random values in
// [-1,1) (a multiplicative hash of the element index; the values do not matter for timing) and
// the lengths are set to len, so that a decode step at a long context can be timed without the
// hours a CPU prefill of that context would take.
int or_state_fill_synthetic(void* mv, void* sv, uint64_t seed, int len) {
  Model* m = (Model*)mv;
  State* st = (State*)sv;
  if (len < 0 || len > st->maxlen) return 1;
  const int64_t D = m->c.head_dim, rows = (int64_t)m->c.n_layers * st->B * m->c.n_kv_heads;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    for (int which = 0; which < 2; which++) {
      float* base = (which ? st->v.data() : st->k.data()) + r * st->maxlen * D;
      uint64_t x = (seed + 1) * 0x9E3779B97F4A7C15ull + (uint64_t)(2 * r + which) * 0xD1B54A32D192ED03ull;
      for (int64_t i = 0; i < (int64_t)len * D; i++) {
        x = x * 6364136223846793005ull + 1442695040888963407ull;
        base[i] = (float)(int32_t)(x >> 32) * (1.0f / 2147483648.0f);
      }
    }
  }
  std::fill(st->len.begin(), st->len.end(), len);
  return 0;
}
int or_prefill(void* m, void* s, const int32_t* tokens, const int32_t* lens, int B, int S, float* logits) {
  State* st = (State*)s;
  for (int b = 0; b < B; b++) if (st->len[b] + lens[b] > st->maxlen || lens[b] > S) return 1;
  forward((Model*)m, st, tokens, lens, B, S, logits);
  return 0;
}
int or_decode(void* m, void* s, const int32_t* ids, int B, float* logits) {
  State* st = (State*)s;
  std::vector<int> one(B, 1);
  for (int b = 0; b < B; b++) if (st->len[b] + 1 > st->maxlen) return 1;
  forward((Model*)m, st, ids, one.data(), B, 1, logits);
  return 0;
}

}  // extern "C"
