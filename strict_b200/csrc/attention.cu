// GQA attention over the bf16 KV cache (head_dim 128) and the fp32 attention of the GPT-2 path.
//
//  * prefill: flash-style causal kernel; one block = 64 query positions of one query head,
//    KV tiles of 64 keys double-buffered in shared memory by cp.async, bf16 mma.sync
//    m16n8k16 with fp32 online softmax; keys come straight from the cache, so a chunked
//    prefill (past > 0) is the same kernel.
//  * decode: split-KV. One block = one KV head of one sequence over one chunk of keys; the
//    G = Hq/Hkv query heads that share the KV head are the rows of the MMA tile, so every
//    K/V byte is read from HBM once. Each block writes (m, l, o) partials; a combine kernel
//    merges the chunks and can emit the two-term E4M3 split of the token row the next GEMM consumes.
//
// Shared-memory tiles hold rows of 128 bf16 (256 B = 16 chunks of 16 B); chunk c of row r
// lives at chunk c ^ (r & 7), which makes every ldmatrix phase conflict-free.
#include <cstdlib>
#include <mutex>

#include <cmath>

#include "common.cuh"

namespace {

constexpr int D = 128;
constexpr int KT = 64;  // keys per tile
constexpr int DEC_STAGES = 2;  // K/V tile ring of the decode kernel; 3 stages (2 blocks/SM) measured 4 % slower than 2 (3 blocks/SM)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t s, const void* g, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(g), "r"(sz));
}
__device__ __forceinline__ void cp_async16_hint(uint32_t s, const void* g, bool valid, uint64_t policy) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(s), "l"(g), "r"(sz), "l"(policy));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}
// The softmax weights enter the P.V product as two bf16 terms, p = hi + lo (16 mantissa bits):
// a single bf16 P is off by up to 2^-9, which is enough to move the bf16-rounded attention
// output by an ulp on a few percent of its elements, and the E4M3 quantisation that follows
// turns each such ulp into a 6-12 % step. V is exact in bf16, so two MMAs recover the product.
__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
  float ah = round_bf16(a), bh = round_bf16(b);
  hi = pack_bf16(ah, bh);
  lo = pack_bf16(a - ah, b - bh);
}
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4)); }

// Copy `rows` rows of 128 bf16 (global row stride 128 elements) into a swizzled tile; rows at
// or beyond `valid_rows` are zero-filled.
__device__ __forceinline__ void load_tile(uint32_t tile, const bf16* src, int rows, int valid_rows, int nthreads) {
  for (int c = threadIdx.x; c < rows * 16; c += nthreads) {
    int r = c >> 4, cc = c & 15;
    bool v = r < valid_rows;
    cp_async16(tile + tile_off(r, cc), src + (int64_t)(v ? r : 0) * D + cc * 8, v);
  }
}

// Same, with an L2 eviction policy on the global reads (the decode kernel reads every key and
// value exactly once).
__device__ __forceinline__ void load_tile_hint(uint32_t tile, const bf16* src, int rows, int valid_rows, int nthreads, uint64_t policy) {
  for (int c = threadIdx.x; c < rows * 16; c += nthreads) {
    int r = c >> 4, cc = c & 15;
    bool v = r < valid_rows;
    cp_async16_hint(tile + tile_off(r, cc), src + (int64_t)(v ? r : 0) * D + cc * 8, v, policy);
  }
}

// ------------------------------------------------------------------ prefill
// grid (ceil(S/64), Hq, B), 128 threads.
__global__ void __launch_bounds__(128) attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                                           const int32_t* __restrict__ lens, const int32_t* __restrict__ past,
                                                           const int32_t* __restrict__ qstart, int S, int Hq, int Hkv, int maxlen,
                                                           float scale_log2, bf16* __restrict__ out) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * 64;
  const int len = lens[b], pst = past ? past[b] : 0;
  const int n_new = len - pst;
  if (q0 >= n_new) return;
  const int64_t row0 = qstart ? qstart[b] : (int64_t)b * S;  // first row of this sequence in q / out
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int hk = h / (Hq / Hkv);
  const uint32_t sQ = smem_u32(smem), sK = sQ + 64 * 256, sV = sK + 2 * KT * 256;
  const bf16* kbase = kc + ((int64_t)b * Hkv + hk) * maxlen * D;
  const bf16* vbase = vc + ((int64_t)b * Hkv + hk) * maxlen * D;
  // last key any row of this block may see
  const int kv_end = min(len, pst + q0 + 64);
  const int ntiles = (kv_end + KT - 1) / KT;

  // Q tile: rows q0..q0+63 of head h; global row stride Hq*D
  for (int c = threadIdx.x; c < 64 * 16; c += 128) {
    int r = c >> 4, cc = c & 15;
    bool v = q0 + r < n_new;
    cp_async16(sQ + tile_off(r, cc), q + ((row0 + (v ? q0 + r : 0)) * Hq + h) * D + cc * 8, v);
  }
  load_tile(sK, kbase, KT, min(KT, len), 128);
  load_tile(sV, vbase, KT, min(KT, len), 128);
  cp_async_commit();

  uint32_t qf[8][4];
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[j][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int qpos0 = pst + q0 + warp * 16 + g;  // position of row g; row g+8 is qpos0+8
  const int mi = lane >> 3, r8 = lane & 7;

  for (int t = 0; t < ntiles; t++) {
    if (t + 1 < ntiles) {
      int k0 = (t + 1) * KT;
      load_tile(sK + ((t + 1) & 1) * KT * 256, kbase + (int64_t)k0 * D, KT, min(KT, len - k0), 128);
      load_tile(sV + ((t + 1) & 1) * KT * 256, vbase + (int64_t)k0 * D, KT, min(KT, len - k0), 128);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ks++) ldsm_x4(sQ + tile_off(warp * 16 + (mi & 1) * 8 + r8, 2 * ks + (mi >> 1)), qf[ks]);
    }
    const uint32_t tK = sK + (t & 1) * KT * 256, tV = sV + (t & 1) * KT * 256;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) s[j][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
#pragma unroll
      for (int jp = 0; jp < 4; jp++) {
        uint32_t kb[4];
        ldsm_x4(tK + tile_off(jp * 16 + (mi >> 1) * 8 + r8, 2 * ks + (mi & 1)), kb);
        mma_bf16(s[2 * jp], qf[ks], kb[0], kb[1]);
        mma_bf16(s[2 * jp + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // scale, mask, online softmax
    const int kbase_pos = t * KT;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int kpos = kbase_pos + 8 * j + 2 * tig + (i & 1);
        int qpos = qpos0 + ((i >> 1) << 3);
        float v = s[j][i] * scale_log2;
        v = (kpos > qpos || kpos >= len) ? -INFINITY : v;
        s[j][i] = v;
        mx[i >> 1] = fmaxf(mx[i >> 1], v);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    float ls[2] = {0.f, 0.f};
    uint32_t pf[4][4], pl[4][4];  // P = hi + lo, two bf16 terms (see split_bf16)
#pragma unroll
    for (int j = 0; j < 8; j++) {
      float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
      float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
      ls[0] += p0 + p1;
      ls[1] += p2 + p3;
      split_bf16(p0, p1, pf[j >> 1][(j & 1) * 2], pl[j >> 1][(j & 1) * 2]);
      split_bf16(p2, p3, pf[j >> 1][(j & 1) * 2 + 1], pl[j >> 1][(j & 1) * 2 + 1]);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) l_run[r] = l_run[r] * corr[r] + ls[r];
#pragma unroll
    for (int j = 0; j < 16; j++) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
#pragma unroll
      for (int jj = 0; jj < 8; jj++) {
        uint32_t vb[4];
        ldsm_x4_t(tV + tile_off(kk * 16 + (mi & 1) * 8 + r8, 2 * jj + (mi >> 1)), vb);
        mma_bf16(o[2 * jj], pf[kk], vb[0], vb[1]);
        mma_bf16(o[2 * jj + 1], pf[kk], vb[2], vb[3]);
        mma_bf16(o[2 * jj], pl[kk], vb[0], vb[1]);
        mma_bf16(o[2 * jj + 1], pl[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    int row = q0 + warp * 16 + g + r * 8;
    if (row < n_new) {
      float inv = 1.0f / l_run[r];
      bf16* dst = out + ((row0 + row) * Hq + h) * D;
#pragma unroll
      for (int j = 0; j < 16; j++) *(uint32_t*)(dst + 8 * j + 2 * tig) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------ decode (split-KV)
// What the decode step's RoPE kernel does for one head (rope.cu, operation for operation): sum of
// the qkv projection's split-K partials, the two scales, per-head RMS norm, rotary embedding at
// position p, rounded to bf16. One warp per head, four dimensions per lane. is_v: the value head is
// only summed, scaled and rounded.
struct RopeFuseArgs {
  const float* part;   // [splits][B][nqkv] raw accumulators of the qkv projection (null: q is read from memory)
  int splits;
  const float* sx;     // [B]
  const float* sw;     // [nqkv]
  const float* cos_t;  // [max_pos][64]
  const float* sin_t;
  const float* qgain;
  const float* kgain;
  float eps;
  int max_pos;
  bf16* kcache;        // the caches again, writable: the new token's key and value rows are appended here
  bf16* vcache;
};
__device__ __forceinline__ uint2 rope_head_bf16(const RopeFuseArgs& r, int B, int b, int64_t nqkv, int64_t col0, const float* gain, int p, bool is_v,
                                                int lane) {
  const int64_t col = col0 + lane * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float4 v[8];
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (s < r.splits) v[s] = *(const float4*)(r.part + ((int64_t)s * B + b) * nqkv + col);
  const float4 w = *(const float4*)(r.sw + col);
  const float sxr = r.sx[b];
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (s < r.splits) { acc[0] += v[s].x; acc[1] += v[s].y; acc[2] += v[s].z; acc[3] += v[s].w; }
  float x[4] = {__fmul_rn(__fmul_rn(acc[0], sxr), w.x), __fmul_rn(__fmul_rn(acc[1], sxr), w.y), __fmul_rn(__fmul_rn(acc[2], sxr), w.z),
                __fmul_rn(__fmul_rn(acc[3], sxr), w.w)};
  float o[4];
  if (!is_v) {
    const float4 gv = *(const float4*)(gain + lane * 4);
    const int i0 = (lane & 15) * 4;
    const float4 c = *(const float4*)(r.cos_t + (int64_t)p * (D / 2) + i0), sn4 = *(const float4*)(r.sin_t + (int64_t)p * (D / 2) + i0);
    const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float rr = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)D), r.eps)));
    const float n[4] = {__fmul_rn(__fmul_rn(x[0], rr), gv.x), __fmul_rn(__fmul_rn(x[1], rr), gv.y), __fmul_rn(__fmul_rn(x[2], rr), gv.z),
                        __fmul_rn(__fmul_rn(x[3], rr), gv.w)};
    const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {sn4.x, sn4.y, sn4.z, sn4.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float other = __shfl_xor_sync(0xffffffffu, n[j], 16);
      o[j] = lane < 16 ? __fsub_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j])) : __fadd_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) o[j] = x[j];
  }
  return make_uint2(f32_to_bf16_bits(o[0]) | (f32_to_bf16_bits(o[1]) << 16), f32_to_bf16_bits(o[2]) | (f32_to_bf16_bits(o[3]) << 16));
}

// A length that the previous step's last kernel writes: read around every cache, before and after the dependency wait.
__device__ __forceinline__ int ld_volatile_i32(const int32_t* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// grid (nsplit, Hkv, B), 128 threads. Warp w owns keys [16w,16w+16) of every 64-key tile.
// scratch: o_part [B][Hq][nsplit][128] then ml_part [B][Hq][nsplit][2].
// FUSED: the queries do not come from memory; every block computes the (at most 16) query heads of
// its KV head from the qkv projection's partial results (sum, scales, QK-norm, RoPE), and the block
// whose key chunk holds the new token's position also computes that token's key and value rows,
// appends them to the cache and patches them into its own shared-memory tile (its tile load may
// have read that row before the append). One kernel less per layer of the decode step.
template <bool FUSED>
__global__ void __launch_bounds__(128) attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                                          const int32_t* __restrict__ lens, int len_add, int B, int Hq, int Hkv, int maxlen,
                                                          int chunk, int nsplit, float scale_log2, float* __restrict__ o_part,
                                                          float* __restrict__ ml_part, RopeFuseArgs rf, int prefetch) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(16) bf16 q_s[FUSED ? 16 * D : 8];    // the query heads of this KV head
  __shared__ __align__(16) bf16 kv_new[FUSED ? 2 * D : 8];  // the new token's key row, then its value row
  SB_TRACE_BEGIN();
  pdl_trigger();
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int k_begin = split * chunk;
  const uint32_t sK = smem_u32(smem), sV = sK + DEC_STAGES * KT * 256;
  const bf16* kbase = kc + ((int64_t)b * Hkv + hk) * maxlen * D;
  const bf16* vbase = vc + ((int64_t)b * Hkv + hk) * maxlen * D;
  const uint64_t kv_policy = l2_evict_first_policy();
  // Before the dependency wait: the first tiles of this block's keys and values start to stream
  // while the preceding kernels (the qkv projection's tail, RoPE) still run. Only rows that were
  // written in earlier steps are touched, never the block's last tile (it may hold the row the
  // preceding kernel appends), and the length they are derived from is read again after the wait:
  // if it changed, the tiles are loaded again from scratch.
  const int len_early = min(ld_volatile_i32(lens + b) + len_add, maxlen);
  int npre = 0;
  if (prefetch && k_begin < len_early) {
    const int nt = (min(len_early, k_begin + chunk) - k_begin + KT - 1) / KT;
    npre = min(DEC_STAGES - 1, nt - 1);
    for (int t = 0; t < npre; t++) {
      const int k0 = k_begin + t * KT;
      load_tile_hint(sK + t * KT * 256, kbase + (int64_t)k0 * D, KT, KT, 128, kv_policy);
      load_tile_hint(sV + t * KT * 256, vbase + (int64_t)k0 * D, KT, KT, 128, kv_policy);
      cp_async_commit();
    }
  }
  pdl_wait();
  SB_TRACE_WAITED();
  const int len = min(ld_volatile_i32(lens + b) + len_add, maxlen);
  if (len != len_early && npre) {  // not expected: the length belongs to the previous step
    cp_async_wait<0>();
    __syncthreads();
    npre = 0;
  }
  if (k_begin >= len) return;
  const int k_end = min(len, k_begin + chunk);
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  // FUSED: position of the new token = the sequence's length before this step; its row is the last key
  const int p_new = FUSED ? len - 1 : -1;
  const bool owns_new = FUSED && p_new >= k_begin && p_new < k_end && p_new < rf.max_pos;
  const int ntiles = (k_end - k_begin + KT - 1) / KT;

  // prologue: the first DEC_STAGES-1 tiles are in flight before any is consumed (one group per tile)
  for (int t = npre; t < DEC_STAGES - 1; t++) {
    if (t < ntiles) {
      int k0 = k_begin + t * KT;
      load_tile_hint(sK + t * KT * 256, kbase + (int64_t)k0 * D, KT, min(KT, k_end - k0), 128, kv_policy);
      load_tile_hint(sV + t * KT * 256, vbase + (int64_t)k0 * D, KT, min(KT, k_end - k0), 128, kv_policy);
    }
    cp_async_commit();
  }

  if (FUSED) {
    const int64_t nqkv = (int64_t)(Hq + 2 * Hkv) * D;
    const int pos = min(p_new, rf.max_pos - 1);
    // items 0..G-1: the query heads; for the owner of the new position also G: the key head, G+1: the value head
    for (int i = warp; i < G + (owns_new ? 2 : 0); i += 4) {
      if (i < G) {
        const uint2 w = rope_head_bf16(rf, B, b, nqkv, (int64_t)(hk * G + i) * D, rf.qgain, pos, false, lane);
        *(uint2*)(q_s + i * D + lane * 4) = w;
      } else {
        const bool is_v = i == G + 1;
        const uint2 w = rope_head_bf16(rf, B, b, nqkv, (int64_t)(Hq + (is_v ? Hkv : 0) + hk) * D, rf.kgain, pos, is_v, lane);
        *(uint2*)(kv_new + (is_v ? D : 0) + lane * 4) = w;
        bf16* cache = is_v ? rf.vcache : rf.kcache;
        *(uint2*)(cache + (((int64_t)b * Hkv + hk) * maxlen + p_new) * D + lane * 4) = w;
      }
    }
    __syncthreads();
  }
  // Q fragments: rows = the G query heads of this KV head (zero beyond), from memory or from the prologue above
  uint32_t qf[8][4];
  {
    const bf16* q0 = FUSED ? q_s : q + ((int64_t)b * Hq + hk * G) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      int d0 = ks * 16 + 2 * tig;
      qf[ks][0] = g < G ? *(const uint32_t*)(q0 + g * D + d0) : 0u;
      qf[ks][1] = g + 8 < G ? *(const uint32_t*)(q0 + (g + 8) * D + d0) : 0u;
      qf[ks][2] = g < G ? *(const uint32_t*)(q0 + g * D + d0 + 8) : 0u;
      qf[ks][3] = g + 8 < G ? *(const uint32_t*)(q0 + (g + 8) * D + d0 + 8) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[j][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int mi = lane >> 3, r8 = lane & 7;

  for (int t = 0; t < ntiles; t++) {
    {
      const int tn = t + DEC_STAGES - 1;  // refill the stage consumed in the previous iteration
      if (tn < ntiles) {
        int k0 = k_begin + tn * KT;
        load_tile_hint(sK + (tn % DEC_STAGES) * KT * 256, kbase + (int64_t)k0 * D, KT, min(KT, k_end - k0), 128, kv_policy);
        load_tile_hint(sV + (tn % DEC_STAGES) * KT * 256, vbase + (int64_t)k0 * D, KT, min(KT, k_end - k0), 128, kv_policy);
      }
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();  // all but the newest DEC_STAGES-1 groups: tile t has landed
    }
    __syncthreads();
    const uint32_t tK = sK + (t % DEC_STAGES) * KT * 256, tV = sV + (t % DEC_STAGES) * KT * 256;
    if (FUSED && owns_new && p_new >= k_begin + t * KT && p_new < k_begin + (t + 1) * KT) {
      // the tile copy may have read the new token's row before it was appended: put the rows computed above in its place
      if (warp == 0) {
        const int row = p_new - (k_begin + t * KT), cc = lane & 15;
        const uint4 w = *(const uint4*)(kv_new + (lane < 16 ? 0 : D) + cc * 8);
        *(uint4*)(smem + ((lane < 16 ? tK : tV) - sK) + tile_off(row, cc)) = w;
      }
      __syncthreads();
    }
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      uint32_t kb[4];
      ldsm_x4(tK + tile_off(warp * 16 + (mi >> 1) * 8 + r8, 2 * ks + (mi & 1)), kb);
      mma_bf16(s[0], qf[ks], kb[0], kb[1]);
      mma_bf16(s[1], qf[ks], kb[2], kb[3]);
    }
    const int kpos0 = k_begin + t * KT + warp * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int kpos = kpos0 + 8 * j + 2 * tig + (i & 1);
        float v = kpos >= k_end ? -INFINITY : s[j][i] * scale_log2;
        s[j][i] = v;
        mx[i >> 1] = fmaxf(mx[i >> 1], v);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    uint32_t pf[4], pl[4];
    {
      float p[2][4];
#pragma unroll
      for (int j = 0; j < 2; j++) {
        p[j][0] = exp2f(s[j][0] - m_use[0]); p[j][1] = exp2f(s[j][1] - m_use[0]);
        p[j][2] = exp2f(s[j][2] - m_use[1]); p[j][3] = exp2f(s[j][3] - m_use[1]);
      }
      l_run[0] = l_run[0] * corr[0] + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
      l_run[1] = l_run[1] * corr[1] + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
      split_bf16(p[0][0], p[0][1], pf[0], pl[0]); split_bf16(p[0][2], p[0][3], pf[1], pl[1]);
      split_bf16(p[1][0], p[1][1], pf[2], pl[2]); split_bf16(p[1][2], p[1][3], pf[3], pl[3]);
    }
#pragma unroll
    for (int j = 0; j < 16; j++) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
      uint32_t vb[4];
      ldsm_x4_t(tV + tile_off(warp * 16 + (mi & 1) * 8 + r8, 2 * jj + (mi >> 1)), vb);
      mma_bf16(o[2 * jj], pf, vb[0], vb[1]);
      mma_bf16(o[2 * jj + 1], pf, vb[2], vb[3]);
      mma_bf16(o[2 * jj], pl, vb[0], vb[1]);
      mma_bf16(o[2 * jj + 1], pl, vb[2], vb[3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  // merge the four warps through shared memory (tiles are free after the last barrier)
  float* so = (float*)smem;                       // [4 warps][16 rows][128]
  float* sml = so + 4 * 16 * D;                   // [4 warps][16 rows][2]
#pragma unroll
  for (int r = 0; r < 2; r++) {
    int row = g + 8 * r;
    if (row < G) {
#pragma unroll
      for (int j = 0; j < 16; j++) {
        so[(warp * 16 + row) * D + 8 * j + 2 * tig] = o[j][2 * r];
        so[(warp * 16 + row) * D + 8 * j + 2 * tig + 1] = o[j][2 * r + 1];
      }
      if (tig == 0) { sml[(warp * 16 + row) * 2] = m_run[r]; sml[(warp * 16 + row) * 2 + 1] = l_run[r]; }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * D; e += 128) {
    int row = e / D, d = e - row * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) M = fmaxf(M, sml[(w * 16 + row) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      float mw = sml[(w * 16 + row) * 2];
      float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += sml[(w * 16 + row) * 2 + 1] * f;
      O += so[(w * 16 + row) * D + d] * f;
    }
    int64_t idx = ((int64_t)b * Hq + hk * G + row) * nsplit + split;
    o_part[idx * D + d] = O;
    if (d == 0) { ml_part[idx * 2] = M; ml_part[idx * 2 + 1] = L; }
  }
  SB_TRACE_END(SB_K_ATTN, 0);
}

// grid B, 512 threads: merge the key chunks of every head of one token. A thread owns 8
// consecutive dims of one head (two when Hq > 32) and keeps them in registers for the optional
// two-term E4M3 split of the whole token row [Hq*128] (the o_proj input).
constexpr int CB_THREADS = 512, CB_ITEMS = 2;
__global__ void __launch_bounds__(CB_THREADS) attn_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                                                  const int32_t* __restrict__ lens, int len_add, int Hq, int maxlen, int chunk,
                                                                  int nsplit, bf16* __restrict__ out, uint8_t* __restrict__ q_out,
                                                                  float* __restrict__ qscale) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const int len = min(lens[b] + len_add, maxlen);
  const int ns = (len + chunk - 1) / chunk;
  float v[CB_ITEMS][8];
  float amax = 0.f;
#pragma unroll
  for (int it = 0; it < CB_ITEMS; it++) {
    int e8 = threadIdx.x + it * CB_THREADS;  // index of an 8-dim group of the row
    if (e8 < Hq * (D / 8)) {
      int h = e8 / (D / 8), d = (e8 - h * (D / 8)) * 8;
      int64_t base = ((int64_t)b * Hq + h) * nsplit;
      float M = -INFINITY;
      for (int s = 0; s < ns; s++) M = fmaxf(M, ml_part[(base + s) * 2]);
      float L = 0.f, O[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < ns; s++) {
        float f = exp2f(ml_part[(base + s) * 2] - M);
        L += ml_part[(base + s) * 2 + 1] * f;
        const float4* op = (const float4*)(o_part + (base + s) * D + d);
        float4 o0 = op[0], o1 = op[1];
        O[0] += o0.x * f; O[1] += o0.y * f; O[2] += o0.z * f; O[3] += o0.w * f;
        O[4] += o1.x * f; O[5] += o1.y * f; O[6] += o1.z * f; O[7] += o1.w * f;
      }
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        v[it][i] = ns > 0 ? round_bf16(O[i] / L) : 0.f;
        amax = fmaxf(amax, fabsf(v[it][i]));
      }
#pragma unroll
      for (int i = 0; i < 4; i++) w[i] = pack_bf16(v[it][2 * i], v[it][2 * i + 1]);
      *(uint4*)(out + ((int64_t)b * Hq + h) * D + d) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (!q_out) return;
  amax = block_max(amax, red);
  int ex = sb_scale_exponent(amax);
  float inv = sb_pow2(-ex);
  if (threadIdx.x == 0) qscale[b] = sb_pow2(ex);
#pragma unroll
  for (int it = 0; it < CB_ITEMS; it++) {
    int e8 = threadIdx.x + it * CB_THREADS;
    if (e8 < Hq * (D / 8)) sb_store_split8(q_out, (int64_t)Hq * D, b, (int64_t)e8 * 8, v[it], inv);
  }
}

// The decode-step shape of the merge: one thread per 4-dim group of the token's attention row
// (blockDim.x == Hq * 32 <= 1024), at most 8 key chunks, so a thread has at most 16 small loads
// in flight. Every partial is loaded in one batch together with the sequence length (slots of
// chunks beyond the length hold stale data and are masked out of the arithmetic, which is that
// of the kernel above).
__global__ void __launch_bounds__(1024) attn_combine_decode_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                                                   const int32_t* __restrict__ lens, int len_add, int Hq, int maxlen, int chunk,
                                                                   int nsplit, bf16* __restrict__ out, uint8_t* __restrict__ q_out,
                                                                   float* __restrict__ qscale, int* __restrict__ status) {
  __shared__ float red[32];
  __shared__ __align__(8) ClusterExchange xch;
  SB_TRACE_BEGIN();
  if (gridDim.y > 1) cluster_exchange_init(&xch);  // the blocks of one cluster share a token (some of its heads each)
  pdl_trigger();
  pdl_wait();
  SB_TRACE_WAITED();
  const int b = blockIdx.x;
  const int e4 = blockIdx.y * blockDim.x + threadIdx.x, h = e4 >> 5, d = (e4 & 31) * 4;
  const int64_t base = ((int64_t)b * Hq + h) * nsplit;
  const int len_raw = lens[b];
  float2 ml[8];
  float4 o[8];
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (s < nsplit) {
      ml[s] = *(const float2*)(ml_part + (base + s) * 2);
      o[s] = *(const float4*)(o_part + (base + s) * D + d);
    }
  const int len = min(len_raw + len_add, maxlen);
  const int ns = (len + chunk - 1) / chunk;
  float M = -INFINITY;
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (s < ns) M = fmaxf(M, ml[s].x);
  float L = 0.f, O[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (s < ns) {
      float f = exp2f(ml[s].x - M);
      L += ml[s].y * f;
      O[0] += o[s].x * f; O[1] += o[s].y * f; O[2] += o[s].z * f; O[3] += o[s].w * f;
    }
  float v[4], amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    v[i] = ns > 0 ? round_bf16(O[i] / L) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  *(uint2*)(out + ((int64_t)b * Hq + h) * D + d) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  if (q_out) {
    amax = block_max(amax, red);
    if (gridDim.y > 1) {
      if (!cluster_exchange(&xch, amax, gridDim.y, blockIdx.y, 0) && threadIdx.x == 0) { *(volatile int*)status = 6; __threadfence_system(); }
      for (uint32_t r = 0; r < gridDim.y; r++) amax = fmaxf(amax, ((volatile float*)xch.slot[0])[r]);
    }
    const int ex = sb_scale_exponent(amax);
    if (blockIdx.y == 0 && threadIdx.x == 0) qscale[b] = sb_pow2(ex);
    sb_store_split4(q_out, (int64_t)Hq * D, b, (int64_t)e4 * 4, v, sb_pow2(-ex));
  }
  SB_TRACE_END(SB_K_COMBINE, 0);
}

// ------------------------------------------------------------------ fp32 attention (GPT-2 path)
__global__ void kv_append_f32_kernel(const float* __restrict__ qkv, float* __restrict__ kc, float* __restrict__ vc,
                                     const int32_t* __restrict__ seq, const int32_t* __restrict__ pos, const int32_t* __restrict__ lens, int H,
                                     int Dh, int maxlen) {
  pdl_trigger();
  pdl_wait();
  int64_t t = blockIdx.x;
  int b = seq ? seq[t] : (int)t;
  int p = pos ? pos[t] : lens[b];
  if (p < 0 || p >= maxlen) return;
  int hd = H * Dh;
  for (int e = threadIdx.x; e < hd; e += blockDim.x) {
    int h = e / Dh, d = e - h * Dh;
    int64_t dst = (((int64_t)b * H + h) * maxlen + p) * Dh + d;
    kc[dst] = qkv[t * 3 * hd + hd + e];
    vc[dst] = qkv[t * 3 * hd + 2 * hd + e];
  }
}
// grid (H, T), 256 threads; scores of one (token, head) live in shared memory.
__global__ void __launch_bounds__(256) attn_f32_kernel(const float* __restrict__ qkv, const float* __restrict__ kc, const float* __restrict__ vc,
                                                       const int32_t* __restrict__ seq, const int32_t* __restrict__ pos,
                                                       const int32_t* __restrict__ lens, int H, int Dh, int maxlen, float scale,
                                                       float* __restrict__ out, float* kc_new, float* vc_new) {
  // kc_new/vc_new (decode: every row is its own sequence) make this block also append its head's
  // new key and value; it then takes position p from the projection output, not from the cache.
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float sc[];  // [maxlen rounded up to 4] scores, [Dh] query, [blockDim.x] float4 partial rows
  __shared__ float red[32];
  int h = blockIdx.x;
  int64_t t = blockIdx.y;
  int b = seq ? seq[t] : (int)t;
  int p = pos ? pos[t] : lens[b];
  if (p < 0 || p >= maxlen) return;
  int n = p + 1;
  float* qs = sc + ((maxlen + 3) & ~3);
  int hd = H * Dh;
  for (int d = threadIdx.x; d < Dh; d += blockDim.x) qs[d] = qkv[t * 3 * hd + h * Dh + d];
  __syncthreads();
  const float* kb = kc + ((int64_t)b * H + h) * maxlen * Dh;
  const float* vb = vc + ((int64_t)b * H + h) * maxlen * Dh;
  const float* k_own = qkv + t * 3 * hd + hd + h * Dh;
  const float* v_own = k_own + hd;
  const int own = kc_new ? p : -1;
  if (kc_new)
    for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
      const int64_t dst = (((int64_t)b * H + h) * maxlen + p) * Dh + d;
      kc_new[dst] = k_own[d];
      vc_new[dst] = v_own[d];
    }
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float4* kr = (const float4*)(j == own ? k_own : kb + (int64_t)j * Dh);
    float acc = 0.f;
    for (int d4 = 0; d4 < Dh / 4; d4++) {
      float4 kv = kr[d4];
      acc += kv.x * qs[4 * d4] + kv.y * qs[4 * d4 + 1] + kv.z * qs[4 * d4 + 2] + kv.w * qs[4 * d4 + 3];
    }
    acc *= scale;
    sc[j] = acc;
    mx = fmaxf(mx, acc);
  }
  mx = block_max(mx, red);
  float l = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float e = expf(sc[j] - mx);
    sc[j] = e;
    l += e;
  }
  l = block_sum(l, red);
  __syncthreads();
  float inv = 1.0f / l;
  // P.V: the block's threads form groups of Dh/4 lanes; group g adds the keys g, g+G, ... with one
  // float4 of the value row per lane (a single query row would otherwise walk all keys on Dh
  // threads, one dependent step per key), then the groups' partial rows are added in group order.
  const int dl = Dh / 4, G = (int)blockDim.x / dl;
  float* part = qs + Dh;  // [blockDim.x] float4
  if (G >= 1) {
    const int g = (int)threadIdx.x / dl, c = (int)threadIdx.x % dl;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (g < G) {
#pragma unroll 8
      for (int j = g; j < n; j += G) {
        const float4 v = *(const float4*)((j == own ? v_own : vb + (int64_t)j * Dh) + 4 * c);
        const float pj = sc[j];
        acc.x += pj * v.x; acc.y += pj * v.y; acc.z += pj * v.z; acc.w += pj * v.w;
      }
    }
    *(float4*)(part + 4 * threadIdx.x) = acc;
    __syncthreads();
    for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
      float o = 0.f;
      for (int gg = 0; gg < G; gg++) o += part[(gg * dl + d / 4) * 4 + (d & 3)];
      out[t * hd + h * Dh + d] = o * inv;
    }
  } else {  // head wider than four times the block: one thread per output column
    for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
      float acc = 0.f;
      for (int j = 0; j < n; j++) acc += sc[j] * (j == own ? v_own[d] : vb[(int64_t)j * Dh + d]);
      out[t * hd + h * Dh + d] = acc * inv;
    }
  }
}

}  // namespace

int k_attn_prefill_tc(strictb200_ctx* ctx, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, const int32_t* past,
                      const int32_t* qstart, int B, int S, int64_t q_rows, int Hq, int Hkv, int maxlen, float scale, bf16* out);  // attention_tc.cu

int k_attn_prefill(strictb200_ctx* ctx, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, const int32_t* past,
                   const int32_t* qstart, int B, int S, int64_t q_rows, int Hq, int Hkv, int Dh, int maxlen, float scale, bf16* out) {
  if (Dh != D) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: head_dim must be 128");
  // tcgen05 kernel first; the mma.sync kernel below takes what it declines
  if (ctx->opt.attn_tc != 0) {
    int st = k_attn_prefill_tc(ctx, q, kc, vc, lens, past, qstart, B, S, q_rows, Hq, Hkv, maxlen, scale, out);
    if (st != STRICTB200_ERR_UNSUPPORTED) return st;
  }
  static SbDeviceOnce once;
  size_t smem = 64 * 256 + 4 * KT * 256;
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  if (Hq > 65535 || B > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: too many heads or sequences");
  dim3 grid((S + 63) / 64, Hq, B);
  attn_prefill_kernel<<<grid, 128, smem, ctx->stream>>>(q, kc, vc, lens, past, qstart, S, Hq, Hkv, maxlen, scale * LOG2E, out);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

SB_TRACE_TU(attention)

// Keys per block. All blocks of a launch take about the same time, so the grid runs in waves of
// (blocks resident per SM) x (SM count): the chunk is the multiple of the tile size that
// minimises waves x (tiles per chunk + per-block overhead) among the chunk sizes that leave at
// most 8 chunks for a full cache. The waves are counted for sequences of `len_plan` keys (0: a
// full cache): a cache that holds 2100 of 2432 keys in chunks of 512 runs four full chunks and a
// stub per sequence, chunks of 448 run five even ones (14 % less attention time, measured). The
// attn_blocks_per_sm option restores the plain "that many blocks per SM" rule.
static int decode_chunk(strictb200_ctx* ctx, int B, int Hkv, int maxlen, int len_plan = 0) {
  const int per_sm = ctx->opt.attn_blocks_per_sm;
  const int tiles = (maxlen + KT - 1) / KT;
  const int tiles_plan = len_plan > 0 && len_plan < maxlen ? (len_plan + KT - 1) / KT : tiles;
  if (per_sm > 0) {
    int64_t c = (int64_t)maxlen * B * Hkv / ((int64_t)ctx->sm_count * per_sm);
    c = (c + KT - 1) / KT * KT;
    if (c < 256) c = 256;
    if (c > maxlen) c = (int64_t)tiles * KT;
    return (int)c;
  }
  static SbDeviceOnce once;
  static int resident_of[64] = {};  // blocks of the kernel an SM holds, per device
  const size_t smem_dec = 2 * DEC_STAGES * KT * 256;
  static int resident_fused_of[64] = {};
  once.run(ctx->device, [&] {
    cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dec);
    cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dec);
    int r = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, attn_decode_kernel<false>, 128, smem_dec) != cudaSuccess || r < 1) r = 1;
    resident_of[ctx->device & 63] = r;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, attn_decode_kernel<true>, 128, smem_dec) != cudaSuccess || r < 1) r = 1;
    resident_fused_of[ctx->device & 63] = r;
    return cudaSuccess;
  });
  const int res0 = (ctx->opt.fuse_rope ? resident_fused_of : resident_of)[ctx->device & 63];
  const int resident = res0 > 0 ? res0 : 1;
  const int64_t slots = (int64_t)ctx->sm_count * resident, pairs = (int64_t)B * Hkv;
  int best = tiles;
  double best_cost = 1e30;
  // At most 8 chunks per sequence: that is what the fast merge kernel takes. 16 chunks for the few
  // (sequence, head) pairs of TP=8 shortened the attention kernel but the general merge kernel they
  // need cost more than that (21.9 against 17.0 us per layer for the pair, measured on eight GPUs).
  for (int c = (tiles + 7) / 8; c <= tiles; c++) {
    if (c < 4 && c < tiles) continue;  // at least 256 keys per block
    // (counting a stub as a whole block is deliberate: weighting blocks by their length made the rule pick three long
    // chunks where five short ones measured 47 us against 66)
    const int64_t blocks = pairs * ((tiles_plan + c - 1) / c), waves = (blocks + slots - 1) / slots;
    const double cost = (double)waves * ((double)std::min(c, tiles_plan) + 1.5);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = c; }
  }
  return best * KT;
}
int sb_attn_decode_splits(strictb200_ctx* ctx, int B, int Hkv, int maxlen) {
  int c = decode_chunk(ctx, B, Hkv, maxlen);
  return (maxlen + c - 1) / c;
}
int sb_attn_decode_chunk(strictb200_ctx* ctx, int B, int Hkv, int maxlen, int len_plan) { return decode_chunk(ctx, B, Hkv, maxlen, len_plan); }
size_t sb_attn_decode_scratch(int B, int Hq, int Dh, int nsplit) { return (size_t)B * Hq * nsplit * (Dh + 2) * sizeof(float); }

int k_attn_decode(strictb200_ctx* ctx, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, int len_add, int B, int Hq, int Hkv,
                  int Dh, int maxlen, float scale, int nsplit, float* scratch, bf16* out, uint8_t* q_out, float* qscale_out, const RopeArgs* rope,
                  int chunk) {
  if (Dh != D) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: head_dim must be 128");
  if (Hq / Hkv > 16) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: at most 16 query heads per KV head");
  if (Hq * (D / 8) > CB_THREADS * CB_ITEMS) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: at most 64 query heads per rank");
  if (chunk <= 0) chunk = decode_chunk(ctx, B, Hkv, maxlen);  // else the caller's plan (a multiple of the tile; it has run decode_chunk, which sets the kernel up)
  if (chunk % KT || (maxlen + chunk - 1) / chunk != nsplit) return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: split count does not match the cache size");
  size_t smem = 2 * DEC_STAGES * KT * 256;  // K and V rings; also covers the 34 KB merge area (the attribute is set by decode_chunk above)
  float* o_part = scratch;
  float* ml_part = scratch + (size_t)B * Hq * nsplit * D;
  if (Hkv > 65535 || B > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: too many heads or sequences");
  dim3 grid(nsplit, Hkv, B);
  if (rope) {
    // queries, key and value of the new token come from the qkv projection's partial results (see the kernel)
    if (!rope->part || rope->splits < 1 || rope->splits > 8 || len_add != 1 || Hq / Hkv > 16 || rope->Hq != Hq || rope->Hkv != Hkv ||
        rope->kcache != kc || rope->vcache != vc || rope->lens != lens)
      return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: the fused RoPE prologue needs split-K partials (at most 8), one new token and the same caches");
    RopeFuseArgs rf{rope->part, rope->splits, rope->sx, rope->sw, rope->cos_t, rope->sin_t, rope->qgain, rope->kgain, rope->eps, rope->max_pos,
                    rope->kcache, rope->vcache};
    SB_CUDA(sb_launch(ctx, attn_decode_kernel<true>, grid, dim3(128), smem, (const bf16*)nullptr, kc, vc, lens, len_add, B, Hq, Hkv, maxlen, chunk, nsplit,
                      scale * LOG2E, o_part, ml_part, rf, ctx->opt.attn_prefetch));
  } else {
    SB_CUDA(sb_launch(ctx, attn_decode_kernel<false>, grid, dim3(128), smem, q, kc, vc, lens, len_add, B, Hq, Hkv, maxlen, chunk, nsplit, scale * LOG2E,
                      o_part, ml_part, RopeFuseArgs{}, ctx->opt.attn_prefetch));
  }
  ctx->launches++;
  sb_prof_split(ctx, STRICTB200_K_ATTN_MERGE);
  // The merge stays a kernel of its own: done inside the attention kernel by the last block of every (sequence, head) and
  // of every sequence to finish (fence, counters), it cost 3 us per layer more than this launch (55.0 against 46.8 + 5.1 us).
  if (nsplit <= 8 && Hq <= 32) {
    // blocks per token (one cluster): 8 heads = 256 threads each
    const unsigned per_tok = q_out && ctx->opt.row_cluster > 1 && Hq % 8 == 0 ? (unsigned)std::min(ctx->opt.row_cluster, Hq / 8) : 1u;
    if (per_tok > 1 && Hq % per_tok == 0)
      SB_CUDA(sb_launch_cluster(ctx, attn_combine_decode_kernel, dim3(B, per_tok), dim3((unsigned)(Hq * 32 / per_tok)), 0, dim3(1, per_tok, 1), (const float*)o_part,
                                (const float*)ml_part, lens, len_add, Hq, maxlen, chunk, nsplit, out, q_out, qscale_out, ctx->d_status));
    else
      SB_CUDA(sb_launch(ctx, attn_combine_decode_kernel, dim3(B), dim3((unsigned)(Hq * 32)), 0, (const float*)o_part, (const float*)ml_part, lens, len_add, Hq,
                        maxlen, chunk, nsplit, out, q_out, qscale_out, ctx->d_status));
    ctx->launches++;
    return STRICTB200_OK;
  }
  SB_CUDA(sb_launch(ctx, attn_combine_kernel, dim3(B), dim3(CB_THREADS), 0, o_part, ml_part, lens, len_add, Hq, maxlen, chunk, nsplit, out, q_out, qscale_out));
  ctx->launches++;
  return STRICTB200_OK;
}

int k_attn_f32(strictb200_ctx* ctx, const float* qkv, float* kc, float* vc, const int32_t* seq, const int32_t* pos, const int32_t* lens,
               int64_t T, int H, int Dh, int maxlen, float scale, float* out) {
  if (Dh % 4) return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: head_dim must be a multiple of 4");
  const int threads = 256;
  size_t smem = ((size_t)((maxlen + 3) & ~3) + Dh + 4 * threads) * sizeof(float);
  if (smem > 200 * 1024) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: fp32 path supports at most ~50k positions");
  {
    static std::mutex mu;
    static size_t attr_smem[64] = {};  // largest size this device's kernel has been opened for
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = attr_smem[ctx->device & 63];
    if (have < 48 * 1024) have = 48 * 1024;
    if (smem > have) {
      SB_CUDA(cudaFuncSetAttribute(attn_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      have = smem;
    }
  }
  if (T > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "attention: too many rows for the fp32 path");
  // rows that are sequences of their own (decode) append inside the attention kernel; prompt rows
  // need the keys of other rows of their sequence, so those are appended by a kernel of its own first
  const bool fused_append = seq == nullptr;
  if (!fused_append) {
    SB_CUDA(sb_launch(ctx, kv_append_f32_kernel, dim3((unsigned)T), dim3(256), 0, qkv, kc, vc, seq, pos, lens, H, Dh, maxlen));
    ctx->launches++;
  }
  dim3 grid(H, (unsigned)T);
  SB_CUDA(sb_launch(ctx, attn_f32_kernel, grid, dim3(threads), smem, (const float*)qkv, (const float*)kc, (const float*)vc, seq, pos, lens, H, Dh, maxlen,
                    scale, out, fused_append ? kc : (float*)nullptr, fused_append ? vc : (float*)nullptr));
  ctx->launches++;
  return STRICTB200_OK;
}

// ------------------------------------------------------------------ decode attention without any allocation
// Some hosts of this library must not trigger an allocation while they serve requests: a
// latency-critical decode loop cannot afford the device-wide synchronisation that cudaMalloc and
// cudaFree imply (every stream of the process stalls behind them), and a host that hands out the
// GPU's memory from its own pool at start-up leaves the driver's allocator nothing to give, so a
// late request for scratch would simply fail. For those callers the split-KV partial results live
// in a fixed array that is part of the library image: every GPU that loads the library carries
// these 4 MiB from load to exit, whether or not the entry point is ever called.
namespace {
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)1 << 20;  // 4 MiB of (m, l, o) partials
constexpr int NOALLOC_MAX_DEVICES = 64;
}  // namespace
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
namespace {
// In host code `g_noalloc_scratch` is only a handle for the symbol, never a device address; the
// address a kernel may use is asked for once per device (with that device current) and kept here.
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_mutex;

int noalloc_scratch(strictb200_ctx* ctx, float** out) {
  if (ctx->device < 0 || ctx->device >= NOALLOC_MAX_DEVICES) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "device index beyond the static scratch table");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[ctx->device]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);  // the caller made ctx->device current
    if (e != cudaSuccess || !p) return sb_fail(STRICTB200_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
    g_noalloc_ptr[ctx->device] = p;
  }
  *out = g_noalloc_ptr[ctx->device];
  return STRICTB200_OK;
}
}  // namespace

extern "C" int strictb200_attn_decode_noalloc(strictb200_ctx* ctx, const uint16_t* q, const uint16_t* kc, const uint16_t* vc,
                                              const int32_t* lens, int B, int Hq, int Hkv, int Dh, int maxlen, float scale, uint16_t* out) {
  SB_ENTER(ctx);
  if (Dh != D) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "head_dim must be 128");
  SB_REQUIRE(B >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16 && maxlen > 0, "bad shape");
  if (!B) return STRICTB200_OK;
  SB_REQUIRE(q && kc && vc && lens && out, "null pointer");
  int nsplit = sb_attn_decode_splits(ctx, B, Hkv, maxlen);
  size_t need = sb_attn_decode_scratch(B, Hq, Dh, nsplit) / sizeof(float);
  if (need > NOALLOC_SCRATCH_FLOATS)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "attn_decode_noalloc: batch " + std::to_string(B) + " x " + std::to_string(Hq) + " heads x " +
                                                   std::to_string(nsplit) + " key chunks needs " + std::to_string(need * sizeof(float)) +
                                                   " bytes of partial results; the built-in scratch holds " +
                                                   std::to_string(NOALLOC_SCRATCH_FLOATS * sizeof(float)) + " (use strictb200_attn_decode)");
  float* scratch;
  SB_TRY(noalloc_scratch(ctx, &scratch));
  // Nothing in the scratch has to start at zero: each key chunk a sequence owns is written in full
  // by its block before the combine kernel reads it, and chunks beyond a sequence's length are never read.
  return k_attn_decode(ctx, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, lens, 0, B, Hq, Hkv, Dh, maxlen, scale, nsplit, scratch,
                       (bf16*)out, nullptr, nullptr, nullptr);
}
