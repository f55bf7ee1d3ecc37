// Row-wise kernels of the residual stream: two-term E4M3 split of bf16 rows, fused
// (split-K reduce + dequant) + residual add + RMSNorm + quantise, LayerNorm, SwiGLU, GELU.
// All are HBM/L2 streams: one block per token row, 128-bit loads, warp-shuffle reductions.
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;
constexpr int MAX_CHUNKS = 8;  // 8 values per chunk per thread -> d <= 256*8*8 = 16384

__device__ __forceinline__ void load8_bf16(const bf16* p, float* v) {
  uint4 u = *(const uint4*)p;
  uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8_f32(const float* p, float* v) {
  float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// Peer (or own) buffer read of the fused all-reduce: volatile, so a slot that is rewritten two
// epochs later is never served from a stale cache line.
__device__ __forceinline__ float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void store8_bf16(bf16* p, const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) w[i] = f32_to_bf16_bits(v[2 * i]) | (f32_to_bf16_bits(v[2 * i + 1]) << 16);
  *(uint4*)p = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store8_e4m3(uint8_t* p, const float* v, float inv) {
  uint32_t lo = f32x4_to_e4m3x4(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv), __fmul_rn(v[2], inv), __fmul_rn(v[3], inv));
  uint32_t hi = f32x4_to_e4m3x4(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv), __fmul_rn(v[6], inv), __fmul_rn(v[7], inv));
  *(uint2*)p = make_uint2(lo, hi);
}

// bf16 [M,K] (row stride ldx) -> two-term E4M3 split [sb_qrows(M),K] + power-of-two scale[M]
__global__ void __launch_bounds__(ROW_THREADS) quantize_rows_kernel(const bf16* __restrict__ x, int64_t K, int64_t ldx,
                                                                    uint8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float red[32];
  int64_t row = blockIdx.x;
  const bf16* xr = x + row * ldx;
  float amax = 0.f;
  for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += ROW_THREADS * 8) {
    float v[8];
    load8_bf16(xr + k, v);
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = block_max(amax, red);
  int e = sb_scale_exponent(amax);
  float inv = sb_pow2(-e);
  if (threadIdx.x == 0) scale[row] = sb_pow2(e);
  for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += ROW_THREADS * 8) {
    float v[8];
    load8_bf16(xr + k, v);
    sb_store_split8(q, K, row, k, v, inv);
  }
}

// bf16 weight rows -> single E4M3 term with scale absmax/448 (the tied LM head)
__global__ void __launch_bounds__(ROW_THREADS) quantize_weight_rows_kernel(const bf16* __restrict__ x, int64_t K, int64_t ldx,
                                                                           uint8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float red[32];
  int64_t row = blockIdx.x;
  const bf16* xr = x + row * ldx;
  float amax = 0.f;
  for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += ROW_THREADS * 8) {
    float v[8];
    load8_bf16(xr + k, v);
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = block_max(amax, red);
  float inv = 1.0f, sc = 1.0f;
  if (amax > 0.f) { inv = __fdiv_rn(448.0f, amax); sc = __fdiv_rn(amax, 448.0f); }
  if (threadIdx.x == 0) scale[row] = sc;
  for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += ROW_THREADS * 8) {
    float v[8];
    load8_bf16(xr + k, v);
    store8_e4m3(q + row * K + k, v, inv);
  }
}

struct RowNormDev {
  TpCommDev comm;
  int use_comm;
  const float* x_f32;
  const bf16* x_in;
  const float* part;
  int groups, splits;
  const float* sx;
  const float* sw;
  float* residual_f32;
  bf16* residual;
  const float* gain;
  float eps;
  bf16* y;
  uint8_t* q;
  float* qscale;
  int two_shot;  // fused all-reduce: owner-reduces-and-returns instead of everyone-sends-to-everyone
  int* status;   // host-visible error word of the context
};

__global__ void __launch_bounds__(512) rownorm_kernel(RowNormDev a, int64_t M, int64_t d) {
  const int NT = blockDim.x;
  pdl_trigger();
  pdl_wait();
  int comm_e = 0;
  if (a.use_comm) {
    // Fused all-reduce: wait (bounded) until every rank has published this epoch, then the input
    // row is the sum, in rank order, of the ranks' partial results read over NVLink.
    comm_e = *(volatile int*)a.comm.epoch;
    if ((int)threadIdx.x < a.comm.world) {
      volatile int* f = a.comm.flags[a.comm.rank] + (comm_e & 1) * 8 + threadIdx.x;
      uint32_t spins = 0;
      while (*f - comm_e < 0) {
        if (++spins > a.comm.wait_limit) { *(volatile int*)a.comm.status = 5; __threadfence_system(); break; }
        __nanosleep(64);
      }
    }
    __syncthreads();
  }
  __shared__ float red[32];
  int64_t row = blockIdx.x;
  float v[MAX_CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAX_CHUNKS; c++) {
    int64_t k = ((int64_t)c * NT + threadIdx.x) * 8;
    if (k < d) {
      float* t = v[c];
      if (a.part) {
        float tot[8];
#pragma unroll
        for (int i = 0; i < 8; i++) tot[i] = 0.f;
        float4 w0 = *(const float4*)(a.sw + k), w1 = *(const float4*)(a.sw + k + 4);
        float sw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        for (int g = 0; g < a.groups; g++) {
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; i++) acc[i] = 0.f;
#pragma unroll 4
          for (int s = 0; s < a.splits; s++) {
            const float* p = a.part + (((int64_t)(g * a.splits + s) * M + row) * d + k);
            float4 p0 = *(const float4*)p, p1 = *(const float4*)(p + 4);
            acc[0] += p0.x; acc[1] += p0.y; acc[2] += p0.z; acc[3] += p0.w;
            acc[4] += p1.x; acc[5] += p1.y; acc[6] += p1.z; acc[7] += p1.w;
          }
          float sxr = a.sx[(int64_t)g * M + row];
#pragma unroll
          for (int i = 0; i < 8; i++) tot[i] += __fmul_rn(__fmul_rn(acc[i], sxr), sw[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = tot[i];
      } else if (a.use_comm) {
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = 0.f;
        for (int r = 0; r < a.comm.world; r++) {
          const float* p = a.comm.data[r] + (size_t)(comm_e & 1) * a.comm.max_elems + row * d + k;
          float4 p0 = ld_peer4(p), p1 = ld_peer4(p + 4);
          t[0] += p0.x; t[1] += p0.y; t[2] += p0.z; t[3] += p0.w;
          t[4] += p1.x; t[5] += p1.y; t[6] += p1.z; t[7] += p1.w;
        }
      } else if (a.x_f32) {
        float4 p0 = *(const float4*)(a.x_f32 + row * d + k), p1 = *(const float4*)(a.x_f32 + row * d + k + 4);
        t[0] = p0.x; t[1] = p0.y; t[2] = p0.z; t[3] = p0.w;
        t[4] = p1.x; t[5] = p1.y; t[6] = p1.z; t[7] = p1.w;
      } else {
        load8_bf16(a.x_in + row * d + k, t);
      }
      if (a.residual_f32) {
        float* rp = a.residual_f32 + row * d + k;
        float4 r0 = *(const float4*)rp, r1 = *(const float4*)(rp + 4);
        t[0] = __fadd_rn(r0.x, t[0]); t[1] = __fadd_rn(r0.y, t[1]); t[2] = __fadd_rn(r0.z, t[2]); t[3] = __fadd_rn(r0.w, t[3]);
        t[4] = __fadd_rn(r1.x, t[4]); t[5] = __fadd_rn(r1.y, t[5]); t[6] = __fadd_rn(r1.z, t[6]); t[7] = __fadd_rn(r1.w, t[7]);
        *(float4*)rp = make_float4(t[0], t[1], t[2], t[3]);
        *(float4*)(rp + 4) = make_float4(t[4], t[5], t[6], t[7]);
      } else if (a.residual) {
        float r[8];
        load8_bf16(a.residual + row * d + k, r);
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = round_bf16(__fadd_rn(r[i], t[i]));
        store8_bf16(a.residual + row * d + k, t);
      }
#pragma unroll
      for (int i = 0; i < 8; i++) ss += t[i] * t[i];
    }
  }
  if (!a.gain) return;
  ss = block_sum(ss, red);
  float ms = __fdiv_rn(ss, (float)d);
  float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, a.eps)));
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < MAX_CHUNKS; c++) {
    int64_t k = ((int64_t)c * NT + threadIdx.x) * 8;
    if (k < d) {
      float4 g0 = *(const float4*)(a.gain + k), g1 = *(const float4*)(a.gain + k + 4);
      float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        v[c][i] = round_bf16(__fmul_rn(__fmul_rn(v[c][i], r), g[i]));
        amax = fmaxf(amax, fabsf(v[c][i]));
      }
      if (a.y) store8_bf16(a.y + row * d + k, v[c]);
    }
  }
  if (!a.q) return;
  amax = block_max(amax, red);
  int e = sb_scale_exponent(amax);
  float inv = sb_pow2(-e);
  if (threadIdx.x == 0) a.qscale[row] = sb_pow2(e);
#pragma unroll
  for (int c = 0; c < MAX_CHUNKS; c++) {
    int64_t k = ((int64_t)c * NT + threadIdx.x) * 8;
    if (k < d) sb_store_split8(a.q, d, row, k, v[c], inv);
  }
}

// The same operation for the shapes of a decode step: the row is exactly blockDim.x * 4 wide
// (d <= 4096), the input is one group of at most 8 split-K partials (MODE 0), the published
// partial results of at most 8 ranks (MODE 1) or a finished fp32 row (MODE 2), and the gain is present. A thread owns 4 columns
// so that it never has more than about ten 128-bit loads in flight (beyond that the loads of a
// thread are served in several rounds: 16 loads per thread measured twice the time of 8). The
// constants (weight scales, gain) are fetched before the dependency wait, every load of the row
// is issued in one batch after it, and the arithmetic is that of the kernel above, operation
// for operation.
template <int MODE>
__global__ void __launch_bounds__(1024) rownorm_decode_kernel(RowNormDev a, int64_t M, int64_t d) {
  __shared__ float red[32];
  __shared__ __align__(8) ClusterExchange xch;
  SB_TRACE_BEGIN();
  // gridDim.y blocks of one cluster share a row (a quarter of its columns each at d = 4096): the row's
  // partial results then arrive through four SMs' paths to L2 instead of one, and four SMs issue the
  // arithmetic; the sum of squares and the absolute maximum are exchanged through the cluster.
  if (gridDim.y > 1) cluster_exchange_init(&xch);
  const int64_t row = blockIdx.x, k = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * 4;
  pdl_trigger();
  float4 sw = make_float4(0.f, 0.f, 0.f, 0.f);
  if (MODE == 0 || MODE == 3) sw = *(const float4*)(a.sw + k);
  const float4 g = *(const float4*)(a.gain + k);
  pdl_wait();
  SB_TRACE_WAITED();
  float t[4] = {0.f, 0.f, 0.f, 0.f};
  float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (MODE == 0) {
    float4 p[8];
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) p[s] = *(const float4*)(a.part + (((int64_t)s * M + row) * d + k));
    const float sxr = a.sx[row];
    if (a.residual_f32) r4 = *(const float4*)(a.residual_f32 + row * d + k);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) { acc[0] += p[s].x; acc[1] += p[s].y; acc[2] += p[s].z; acc[3] += p[s].w; }
    t[0] += __fmul_rn(__fmul_rn(acc[0], sxr), sw.x);
    t[1] += __fmul_rn(__fmul_rn(acc[1], sxr), sw.y);
    t[2] += __fmul_rn(__fmul_rn(acc[2], sxr), sw.z);
    t[3] += __fmul_rn(__fmul_rn(acc[3], sxr), sw.w);
    SB_TRACE_MARK(0);
  } else if (MODE == 3) {
    // Fused all-reduce, row-granular: this block sums the rank's own split-K partials of its row
    // and pushes the sums into the peers' buffers as tagged words (below); a receiver polls its own
    // buffer until the words carry the row's current tag. No fence, no other kernel, no grid-wide step.
    float4 p[8];
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) p[s] = *(const float4*)(a.part + (((int64_t)s * M + row) * d + k));
    const float sxr = a.sx[row];
    const int e = *(volatile int*)(a.comm.row_epoch + row) + 1;  // this block is the row's only writer
    if (a.residual_f32) r4 = *(const float4*)(a.residual_f32 + row * d + k);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) { acc[0] += p[s].x; acc[1] += p[s].y; acc[2] += p[s].z; acc[3] += p[s].w; }
    auto clear2f = [](float x) { return __uint_as_float(__float_as_uint(x) & ~3u); };
    const float own[4] = {clear2f(__fmul_rn(__fmul_rn(acc[0], sxr), sw.x)), clear2f(__fmul_rn(__fmul_rn(acc[1], sxr), sw.y)),
                          clear2f(__fmul_rn(__fmul_rn(acc[2], sxr), sw.z)), clear2f(__fmul_rn(__fmul_rn(acc[3], sxr), sw.w))};
    // A value travels as one 32-bit word: its two lowest mantissa bits are replaced by the row's
    // epoch modulo 4 (the two parities of the packet area alternate, so the word that a slot held
    // before always carries epoch - 2, whose tag differs). Every rank adds the values with those
    // two bits cleared, its own included, so all ranks get the same sum. 16 bytes per thread and
    // peer, one store instruction; a warp's store covers four whole 128-byte lines.
    const uint32_t tag = (uint32_t)e & 3u;
    const size_t off = (size_t)(row * d + k);
    const size_t area = (size_t)a.comm.row_elems * 2;
    auto clear2 = [](float x) { return __uint_as_float(__float_as_uint(x) & ~3u); };
    auto push = [&](float* dst, const float* v4) {  // dst: start of a packet area
      asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(dst + off), "r"((__float_as_uint(v4[0]) & ~3u) | tag),
                   "r"((__float_as_uint(v4[1]) & ~3u) | tag), "r"((__float_as_uint(v4[2]) & ~3u) | tag), "r"((__float_as_uint(v4[3]) & ~3u) | tag)
                   : "memory");
    };
    auto poll = [&](const float* src, float* v4) {  // bounded: on expiry the error word is set and the (wrong) values are used
      float4 q0;
      uint32_t spins = 0;
      while (true) {
        q0 = ld_peer4(src + off);
        if (((__float_as_uint(q0.x) ^ tag) & 3u) == 0 && ((__float_as_uint(q0.y) ^ tag) & 3u) == 0 && ((__float_as_uint(q0.z) ^ tag) & 3u) == 0 &&
            ((__float_as_uint(q0.w) ^ tag) & 3u) == 0)
          break;
        if (++spins > a.comm.wait_limit) { *(volatile int*)a.comm.status = 5; __threadfence_system(); break; }
        if ((spins & 4095u) == 0 && *(volatile int*)a.comm.status) break;  // another wait already expired: do not wait it out again
      }
      v4[0] = clear2(q0.x); v4[1] = clear2(q0.y); v4[2] = clear2(q0.z); v4[3] = clear2(q0.w);
    };
    float* mine = a.comm.row_data[a.comm.rank];
    if (!a.two_shot) {
      // one shot: every rank sends its whole row to every peer and sums all of them
#pragma unroll
      for (int r = 0; r < 8; r++)
        if (r < a.comm.world && r != a.comm.rank) push(a.comm.row_data[r] + ((size_t)(e & 1) * 8 + a.comm.rank) * area, own);
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 8; r++)
        if (r < a.comm.world) {
          float v[4] = {own[0], own[1], own[2], own[3]};
          if (r != a.comm.rank) poll(mine + ((size_t)(e & 1) * 8 + r) * area, v);
          sum[0] += v[0]; sum[1] += v[1]; sum[2] += v[2]; sum[3] += v[3];
        }
      // the same value as two shots deliver (there the sum itself travels as a tagged word)
      t[0] += clear2(sum[0]); t[1] += clear2(sum[1]); t[2] += clear2(sum[2]); t[3] += clear2(sum[3]);
    } else {
      // two shots (the one-shot push sends world-1 copies of the row from every rank, 7 MB per
      // rank and sum at 8 ranks): rank j owns the columns [j*d/world, (j+1)*d/world) of every
      // row. Each thread sends its 4 partial sums to the owner of its columns; the owner's
      // threads add the ranks' values in rank order and send the sums back to everyone.
      const int owner = (int)(k / (d / a.comm.world));  // uniform per warp: d/world is a multiple of 128
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      if (owner != a.comm.rank) {
        push(a.comm.row_data[owner] + ((size_t)(e & 1) * 8 + a.comm.rank) * area, own);
        poll(mine + (16 + (size_t)(e & 1)) * area, sum);
      } else {
#pragma unroll
        for (int r = 0; r < 8; r++)
          if (r < a.comm.world) {
            float v[4] = {own[0], own[1], own[2], own[3]};
            if (r != a.comm.rank) poll(mine + ((size_t)(e & 1) * 8 + r) * area, v);
            sum[0] += v[0]; sum[1] += v[1]; sum[2] += v[2]; sum[3] += v[3];
          }
#pragma unroll
        for (int r = 0; r < 8; r++)
          if (r < a.comm.world && r != a.comm.rank) push(a.comm.row_data[r] + (16 + (size_t)(e & 1)) * area, sum);
        sum[0] = clear2(sum[0]); sum[1] = clear2(sum[1]); sum[2] = clear2(sum[2]); sum[3] = clear2(sum[3]);  // what the peers received
      }
      t[0] += sum[0]; t[1] += sum[1]; t[2] += sum[2]; t[3] += sum[3];
    }
    __syncthreads();  // every thread of the row has read the epoch
    if (threadIdx.x == 0) *(volatile int*)(a.comm.row_epoch + row) = e;
  } else if (MODE == 2) {
    const float4 p = *(const float4*)(a.x_f32 + row * d + k);
    if (a.residual_f32) r4 = *(const float4*)(a.residual_f32 + row * d + k);
    t[0] = p.x; t[1] = p.y; t[2] = p.z; t[3] = p.w;
  } else {
    // Fused all-reduce: wait (bounded) until every rank has published this epoch, then the input
    // row is the sum, in rank order, of the ranks' partial results read over NVLink.
    const int comm_e = *(volatile int*)a.comm.epoch;
    if ((int)threadIdx.x < a.comm.world) {
      volatile int* f = a.comm.flags[a.comm.rank] + (comm_e & 1) * 8 + threadIdx.x;
      uint32_t spins = 0;
      while (*f - comm_e < 0) {
        if (++spins > a.comm.wait_limit) { *(volatile int*)a.comm.status = 5; __threadfence_system(); break; }
        __nanosleep(64);
      }
    }
    __syncthreads();
    float4 p[8];
#pragma unroll
    for (int r = 0; r < 8; r++)
      if (r < a.comm.world) p[r] = ld_peer4(a.comm.data[r] + (size_t)(comm_e & 1) * a.comm.max_elems + row * d + k);
    if (a.residual_f32) r4 = *(const float4*)(a.residual_f32 + row * d + k);
#pragma unroll
    for (int r = 0; r < 8; r++)
      if (r < a.comm.world) { t[0] += p[r].x; t[1] += p[r].y; t[2] += p[r].z; t[3] += p[r].w; }
  }
  if (a.residual_f32) {
    t[0] = __fadd_rn(r4.x, t[0]); t[1] = __fadd_rn(r4.y, t[1]); t[2] = __fadd_rn(r4.z, t[2]); t[3] = __fadd_rn(r4.w, t[3]);
    *(float4*)(a.residual_f32 + row * d + k) = make_float4(t[0], t[1], t[2], t[3]);
  }
  float ss = t[0] * t[0] + t[1] * t[1] + t[2] * t[2] + t[3] * t[3];
  ss = block_sum(ss, red);
  if (gridDim.y > 1) {
    if (!cluster_exchange(&xch, ss, gridDim.y, blockIdx.y, 0) && threadIdx.x == 0) { *(volatile int*)a.status = 6; __threadfence_system(); }
    ss = 0.f;
    for (uint32_t r = 0; r < gridDim.y; r++) ss += ((volatile float*)xch.slot[0])[r];  // in block order, the same in every block
  }
  SB_TRACE_MARK(1);
  const float ms = __fdiv_rn(ss, (float)d);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, a.eps)));
  const float gg[4] = {g.x, g.y, g.z, g.w};
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    t[i] = round_bf16(__fmul_rn(__fmul_rn(t[i], r), gg[i]));
    amax = fmaxf(amax, fabsf(t[i]));
  }
  if (a.y) {
    uint2 w;
    w.x = f32_to_bf16_bits(t[0]) | (f32_to_bf16_bits(t[1]) << 16);
    w.y = f32_to_bf16_bits(t[2]) | (f32_to_bf16_bits(t[3]) << 16);
    *(uint2*)(a.y + row * d + k) = w;
  }
  if (a.q) {
    amax = block_max(amax, red);
    if (gridDim.y > 1) {
      if (!cluster_exchange(&xch, amax, gridDim.y, blockIdx.y, 1) && threadIdx.x == 0) { *(volatile int*)a.status = 6; __threadfence_system(); }
      for (uint32_t r = 0; r < gridDim.y; r++) amax = fmaxf(amax, ((volatile float*)xch.slot[1])[r]);
    }
    SB_TRACE_MARK(2);
    const int e = sb_scale_exponent(amax);
    if (blockIdx.y == 0 && threadIdx.x == 0) a.qscale[row] = sb_pow2(e);
    sb_store_split4(a.q, d, row, k, t, sb_pow2(-e));
  }
  SB_TRACE_END(MODE == 3 ? SB_K_ROWNORM_TP : SB_K_ROWNORM, (uint32_t)((uintptr_t)a.gain >> 4));
}


__global__ void __launch_bounds__(ROW_THREADS) layernorm_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                const float* __restrict__ b, float eps, int64_t d, float* __restrict__ y) {
  pdl_trigger();
  __shared__ float red[32];
  int64_t row = blockIdx.x;
  const float* xr = x + row * d;
  if (d <= 4 * ROW_THREADS) {
    // narrow rows: gain and bias are fetched before the dependency wait, the row is read once and
    // stays in registers (same per-thread columns and order of additions as the loops below)
    float gv[4], bv[4], xv[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t k = threadIdx.x + (int64_t)i * ROW_THREADS;
      if (k < d) { gv[i] = g[k]; bv[i] = b[k]; }
    }
    pdl_wait();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t k = threadIdx.x + (int64_t)i * ROW_THREADS;
      if (k < d) { xv[i] = xr[k]; s += xv[i]; }
    }
    const float mean = __fdiv_rn(block_sum(s, red), (float)d);
    float vs = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (threadIdx.x + (int64_t)i * ROW_THREADS < d) { const float t = xv[i] - mean; vs += t * t; }
    const float var = __fdiv_rn(block_sum(vs, red), (float)d);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t k = threadIdx.x + (int64_t)i * ROW_THREADS;
      if (k < d) y[row * d + k] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xv[i], mean), r), gv[i]), bv[i]);
    }
    return;
  }
  pdl_wait();
  float s = 0.f;
  for (int64_t k = threadIdx.x; k < d; k += ROW_THREADS) s += xr[k];
  float mean = __fdiv_rn(block_sum(s, red), (float)d);
  float vs = 0.f;
  for (int64_t k = threadIdx.x; k < d; k += ROW_THREADS) { float t = xr[k] - mean; vs += t * t; }
  float var = __fdiv_rn(block_sum(vs, red), (float)d);
  float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
  for (int64_t k = threadIdx.x; k < d; k += ROW_THREADS)
    y[row * d + k] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xr[k], mean), r), g[k]), b[k]);
}

__global__ void add_f32_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = __fadd_rn(x[i], y[i]);
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

// gate_up [M, 2I] (bf16, or the projection's fp32 result) -> h = bf16(silu(gate)*up); optional
// two-term E4M3 split of h per row. 512 threads; a thread owns up to 4 groups of 8 columns and
// keeps h in registers between the absmax pass and the split (rows wider than 16384 recompute).
constexpr int SW_THREADS = 512, SW_ITEMS = 4;
__global__ void __launch_bounds__(SW_THREADS) swiglu_kernel(const bf16* __restrict__ gu, const float* __restrict__ gu32, int64_t I,
                                                            bf16* __restrict__ y, uint8_t* __restrict__ q, float* __restrict__ qscale) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  int64_t row = blockIdx.x;
  const bool in_regs = I <= (int64_t)SW_THREADS * 8 * SW_ITEMS;
  float hreg[SW_ITEMS][8];
  float amax = 0.f;
  auto compute = [&](int64_t k, float* h) {
    float g[8], u[8];
    if (gu32) { load8_f32(gu32 + row * 2 * I + k, g); load8_f32(gu32 + row * 2 * I + I + k, u); }
    else { load8_bf16(gu + row * 2 * I + k, g); load8_bf16(gu + row * 2 * I + I + k, u); }
#pragma unroll
    for (int i = 0; i < 8; i++) h[i] = round_bf16(silu_mul(g[i], u[i]));
  };
  if (in_regs) {
#pragma unroll
    for (int it = 0; it < SW_ITEMS; it++) {
      int64_t k = ((int64_t)it * SW_THREADS + threadIdx.x) * 8;
      if (k < I) {
        compute(k, hreg[it]);
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(hreg[it][i]));
        if (y) store8_bf16(y + row * I + k, hreg[it]);
      }
    }
  } else {
    for (int64_t k = (int64_t)threadIdx.x * 8; k < I; k += SW_THREADS * 8) {
      float h[8];
      compute(k, h);
#pragma unroll
      for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(h[i]));
      if (y) store8_bf16(y + row * I + k, h);
    }
  }
  if (!q) return;
  amax = block_max(amax, red);
  int e = sb_scale_exponent(amax);
  float inv = sb_pow2(-e);
  if (threadIdx.x == 0) qscale[row] = sb_pow2(e);
  if (in_regs) {
#pragma unroll
    for (int it = 0; it < SW_ITEMS; it++) {
      int64_t k = ((int64_t)it * SW_THREADS + threadIdx.x) * 8;
      if (k < I) sb_store_split8(q, I, row, k, hreg[it], inv);
    }
  } else {
    for (int64_t k = (int64_t)threadIdx.x * 8; k < I; k += SW_THREADS * 8) {
      float h[8];
      compute(k, h);
      sb_store_split8(q, I, row, k, h, inv);
    }
  }
}

// The decode-step shape of the above: a row of I columns is shared by a cluster of gridDim.y
// blocks, one 8-column group per thread (I == gridDim.y * blockDim.x * 8), fp32 input, split
// output. The blocks of a row push their absolute maxima to each other.
__global__ void __launch_bounds__(512) swiglu_decode_kernel(const float* __restrict__ gu32, int64_t I, bf16* __restrict__ y,
                                                            uint8_t* __restrict__ q, float* __restrict__ qscale, int* __restrict__ status) {
  __shared__ float red[32];
  __shared__ __align__(8) ClusterExchange xch;
  if (gridDim.y > 1) cluster_exchange_init(&xch);
  SB_TRACE_BEGIN();
  pdl_trigger();
  pdl_wait();
  SB_TRACE_WAITED();
  const int64_t row = blockIdx.x, k = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * 8;
  float g[8], u[8], h[8];
  load8_f32(gu32 + row * 2 * I + k, g);
  load8_f32(gu32 + row * 2 * I + I + k, u);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    h[i] = round_bf16(silu_mul(g[i], u[i]));
    amax = fmaxf(amax, fabsf(h[i]));
  }
  if (y) store8_bf16(y + row * I + k, h);
  amax = block_max(amax, red);
  if (gridDim.y > 1) {
    if (!cluster_exchange(&xch, amax, gridDim.y, blockIdx.y) && threadIdx.x == 0) { *(volatile int*)status = 6; __threadfence_system(); }
    for (uint32_t r = 0; r < gridDim.y; r++) amax = fmaxf(amax, ((volatile float*)xch.slot[0])[r]);
  }
  const int e = sb_scale_exponent(amax);
  if (blockIdx.y == 0 && threadIdx.x == 0) qscale[row] = sb_pow2(e);
  sb_store_split8(q, I, row, k, h, sb_pow2(-e));
  SB_TRACE_END(SB_K_SWIGLU, 0);
}

// The same for a gate/up projection that arrives as at most 4 raw split-K partials
// [splits][M][2I] with the scales still to apply (the narrow shards of tensor parallelism, whose
// GEMM needs K splits to cover the GPU): 4 columns per thread, so 2 x splits loads in flight.
__global__ void __launch_bounds__(512) swiglu_decode_part_kernel(const float* __restrict__ part, int splits, const float* __restrict__ sx,
                                                                 const float* __restrict__ sw, int64_t M, int64_t I, uint8_t* __restrict__ q,
                                                                 float* __restrict__ qscale, int* __restrict__ status) {
  __shared__ float red[32];
  __shared__ __align__(8) ClusterExchange xch;
  if (gridDim.y > 1) cluster_exchange_init(&xch);
  SB_TRACE_BEGIN();
  pdl_trigger();
  const int64_t row = blockIdx.x, k = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const float4 wg = *(const float4*)(sw + k), wu = *(const float4*)(sw + I + k);
  pdl_wait();
  SB_TRACE_WAITED();
  float4 pg[4], pu[4];
#pragma unroll
  for (int s = 0; s < 4; s++)
    if (s < splits) {
      const float* p = part + ((int64_t)s * M + row) * 2 * I + k;
      pg[s] = *(const float4*)p;
      pu[s] = *(const float4*)(p + I);
    }
  const float sxr = sx[row];
  float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < 4; s++)
    if (s < splits) {
      g[0] += pg[s].x; g[1] += pg[s].y; g[2] += pg[s].z; g[3] += pg[s].w;
      u[0] += pu[s].x; u[1] += pu[s].y; u[2] += pu[s].z; u[3] += pu[s].w;
    }
  const float wgv[4] = {wg.x, wg.y, wg.z, wg.w}, wuv[4] = {wu.x, wu.y, wu.z, wu.w};
  float h[4], amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    h[i] = round_bf16(silu_mul(__fmul_rn(__fmul_rn(g[i], sxr), wgv[i]), __fmul_rn(__fmul_rn(u[i], sxr), wuv[i])));
    amax = fmaxf(amax, fabsf(h[i]));
  }
  amax = block_max(amax, red);
  if (gridDim.y > 1) {
    if (!cluster_exchange(&xch, amax, gridDim.y, blockIdx.y) && threadIdx.x == 0) { *(volatile int*)status = 6; __threadfence_system(); }
    for (uint32_t r = 0; r < gridDim.y; r++) amax = fmaxf(amax, ((volatile float*)xch.slot[0])[r]);
  }
  const int e = sb_scale_exponent(amax);
  if (blockIdx.y == 0 && threadIdx.x == 0) qscale[row] = sb_pow2(e);
  sb_store_split4(q, I, row, k, h, sb_pow2(-e));
  SB_TRACE_END(SB_K_SWIGLU, 0);
}

__global__ void gelu_tanh_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    y[i] = sb_gelu_tanh(x[i]);
  }
}

int stream_grid(strictb200_ctx* ctx, int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads, cap = (int64_t)ctx->sm_count * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

SB_TRACE_TU(norm)

int k_quantize_rows(strictb200_ctx* ctx, const bf16* x, int64_t M, int64_t K, int64_t ldx, uint8_t* q, float* scale) {
  if (K % 8 || ldx % 8) return sb_fail(STRICTB200_ERR_INVALID_ARG, "quantize_rows: K and the row stride must be multiples of 8");
  quantize_rows_kernel<<<(unsigned)M, ROW_THREADS, 0, ctx->stream>>>(x, K, ldx, q, scale);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_quantize_weight_rows(strictb200_ctx* ctx, const bf16* x, int64_t M, int64_t K, int64_t ldx, uint8_t* q, float* scale) {
  if (K % 8 || ldx % 8) return sb_fail(STRICTB200_ERR_INVALID_ARG, "quantize_weight_rows: K and the row stride must be multiples of 8");
  quantize_weight_rows_kernel<<<(unsigned)M, ROW_THREADS, 0, ctx->stream>>>(x, K, ldx, q, scale);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_rownorm(strictb200_ctx* ctx, const RowNormArgs& a, int64_t M, int64_t d) {
  if (d % 8 || d > (int64_t)ROW_THREADS * 8 * MAX_CHUNKS)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "rownorm: d must be a multiple of 8 and at most 16384");
  // one 8-value chunk per thread where the row allows it (more loads in flight per row)
  int threads = (int)((d / 8 + 31) / 32 * 32);
  threads = threads < 128 ? 128 : (threads > 512 ? 512 : threads);
  // many rows (prefill): narrower blocks, two chunks per thread and more blocks per SM keep more bytes in flight
  if (M > 1024 && threads > 256) threads = 256;
  while ((int64_t)threads * 8 * MAX_CHUNKS < d) threads += 32;
  RowNormDev v{a.comm ? *a.comm : TpCommDev{}, a.comm ? 1 : 0, a.x_f32, a.x_in, a.part, a.groups, a.splits, a.sx, a.sw, a.residual_f32, a.residual, a.gain, a.eps, a.y, a.q, a.qscale, 0, ctx->d_status};
  // decode-step shapes: 4 columns per thread, at most 8 partials, no bf16 residual
  const bool narrow = d % 128 == 0 && d <= 4096 && a.gain && !a.residual && M <= 1024;
  // More than four ranks exchange in two shots (one shot sends world-1 copies of every row: at four
  // ranks one shot measured 14730 tokens/s against 14470 for two, at eight 11800 against 14470);
  // the tp_two_shot option (0 / 1) forces either.
  if (a.comm) {
    v.comm.wait_limit = ctx->opt.wait_limit > 0 ? (unsigned)ctx->opt.wait_limit : 1u;
    const int ts = ctx->opt.tp_two_shot;
    v.two_shot = (ts >= 0 ? ts != 0 : a.comm->world > 4) && d % (a.comm->world * 128) == 0;
  }
  if (narrow && a.comm && a.part && a.groups == 1 && a.splits <= 8 && a.comm->world <= 8 && sb_tp_row_exchange_ok(ctx, M, d, v.two_shot)) {
    SB_CUDA(sb_launch(ctx, rownorm_decode_kernel<3>, dim3((unsigned)M), dim3((unsigned)(d / 4)), 0, v, M, d));
    ctx->launches++;
    return STRICTB200_OK;
  }
  if (a.comm && a.part) {
    // shapes the row-granular exchange does not take: publish the scaled sums with a kernel of
    // their own, then the row kernel only gathers
    SB_TRY(k_tp_publish(ctx, a.part, a.splits, a.sx, a.sw, M, d));
    v.part = nullptr;
  }
  if (narrow && a.comm && a.comm->world <= 8) {
    SB_CUDA(sb_launch(ctx, rownorm_decode_kernel<1>, dim3((unsigned)M), dim3((unsigned)(d / 4)), 0, v, M, d));
    ctx->launches++;
    return STRICTB200_OK;
  }
  // blocks per row (one cluster): 256 threads each where the row is wide enough
  const unsigned per_row = ctx->opt.row_cluster > 0 && d % 1024 == 0 ? (unsigned)std::min<int64_t>(ctx->opt.row_cluster, d / 1024) : 1u;
  if (narrow && !a.comm && !a.part && a.x_f32) {
    if (per_row > 1) SB_CUDA(sb_launch_cluster(ctx, rownorm_decode_kernel<2>, dim3((unsigned)M, per_row), dim3((unsigned)(d / 4 / per_row)), 0, dim3(1, per_row, 1), v, M, d));
    else SB_CUDA(sb_launch(ctx, rownorm_decode_kernel<2>, dim3((unsigned)M), dim3((unsigned)(d / 4)), 0, v, M, d));
    ctx->launches++;
    return STRICTB200_OK;
  }
  if (narrow && !a.comm && a.part && a.groups == 1 && a.splits <= 8) {
    if (per_row > 1) SB_CUDA(sb_launch_cluster(ctx, rownorm_decode_kernel<0>, dim3((unsigned)M, per_row), dim3((unsigned)(d / 4 / per_row)), 0, dim3(1, per_row, 1), v, M, d));
    else SB_CUDA(sb_launch(ctx, rownorm_decode_kernel<0>, dim3((unsigned)M), dim3((unsigned)(d / 4)), 0, v, M, d));
    ctx->launches++;
    return STRICTB200_OK;
  }
  SB_CUDA(sb_launch(ctx, rownorm_kernel, dim3((unsigned)M), dim3(threads), 0, v, M, d));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_layernorm(strictb200_ctx* ctx, const float* x, const float* g, const float* b, float eps, int64_t M, int64_t d, float* y) {
  SB_CUDA(sb_launch(ctx, layernorm_kernel, dim3((unsigned)M), dim3(ROW_THREADS), 0, x, g, b, eps, d, y));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_add_f32(strictb200_ctx* ctx, float* x, const float* y, int64_t n) {
  add_f32_kernel<<<stream_grid(ctx, n, 256), 256, 0, ctx->stream>>>(x, y, n);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_swiglu(strictb200_ctx* ctx, const bf16* gate_up, const float* gate_up_f32, int64_t M, int64_t I, bf16* y, uint8_t* q, float* qscale) {
  if (I % 8) return sb_fail(STRICTB200_ERR_INVALID_ARG, "swiglu: I must be a multiple of 8");
  if (gate_up_f32 && q && I % 256 == 0 && M <= 1024) {
    // decode shapes: one 8-column group per thread, a cluster of up to 8 blocks per row
    for (int c = 1; c <= 8; c++) {
      if (I % (8 * c) || (I / (8 * c)) % 32 || I / (8 * c) > 512) continue;
      SB_CUDA(sb_launch_cluster(ctx, swiglu_decode_kernel, dim3((unsigned)M, (unsigned)c), dim3((unsigned)(I / (8 * c))), 0, dim3(1, (unsigned)c, 1),
                                gate_up_f32, I, y, q, qscale, ctx->d_status));
      ctx->launches++;
      return STRICTB200_OK;
    }
  }
  SB_CUDA(sb_launch(ctx, swiglu_kernel, dim3((unsigned)M), dim3(SW_THREADS), 0, gate_up, gate_up_f32, I, y, q, qscale));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_swiglu_part(strictb200_ctx* ctx, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t I, uint8_t* q,
                  float* qscale) {
  if (splits < 1 || splits > 4 || I % 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "swiglu over partials: at most 4 splits, I a multiple of 128");
  for (int c = 1; c <= 8; c++) {
    if (I % (4 * c) || (I / (4 * c)) % 32 || I / (4 * c) > 512) continue;
    SB_CUDA(sb_launch_cluster(ctx, swiglu_decode_part_kernel, dim3((unsigned)M, (unsigned)c), dim3((unsigned)(I / (4 * c))), 0, dim3(1, (unsigned)c, 1), part,
                              splits, sx, sw, M, I, q, qscale, ctx->d_status));
    ctx->launches++;
    return STRICTB200_OK;
  }
  return sb_fail(STRICTB200_ERR_UNSUPPORTED, "swiglu over partials: no block shape for this width");
}
int k_gelu_tanh(strictb200_ctx* ctx, const float* x, int64_t n, float* y) {
  SB_CUDA(sb_launch(ctx, gelu_tanh_kernel, dim3(stream_grid(ctx, n, 256)), dim3(256), 0, x, n, y));
  ctx->launches++;
  return STRICTB200_OK;
}

// out[m,n] = (sum_s part[s][m,n]) * sx[m] * sw[n], fp32 (the input of a cross-rank all-reduce) or bf16
namespace {
__global__ void reduce_scale_kernel(const float* __restrict__ part, int splits, const float* __restrict__ sx, const float* __restrict__ sw,
                                    int64_t M, int64_t N, float* __restrict__ out, bf16* __restrict__ out_bf16) {
  pdl_trigger();
  pdl_wait();
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
    if (out) *(float4*)(out + m * N + n) = r;
    else *(uint2*)(out_bf16 + m * N + n) = make_uint2(f32_to_bf16_bits(r.x) | (f32_to_bf16_bits(r.y) << 16), f32_to_bf16_bits(r.z) | (f32_to_bf16_bits(r.w) << 16));
  }
}
}  // namespace
int k_reduce_scale(strictb200_ctx* ctx, const float* part, int splits, const float* sx, const float* sw, int64_t M, int64_t N, float* out,
                   bf16* out_bf16) {
  if (N % 4) return sb_fail(STRICTB200_ERR_INVALID_ARG, "reduce_scale: N must be a multiple of 4");
  SB_CUDA(sb_launch(ctx, reduce_scale_kernel, dim3(stream_grid(ctx, M * N / 4, 256)), dim3(256), 0, part, splits, sx, sw, M, N, out, out_bf16));
  ctx->launches++;
  return STRICTB200_OK;
}
