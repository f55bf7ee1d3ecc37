// Causal GQA prefill attention on the tcgen05 tensor cores (head_dim 128, bf16).
// One block = 128 query positions of one head, 128 threads: thread r owns query row r, which is
// also lane r of tensor memory, so the softmax needs no shuffles.
// Per 128-key tile:
//   S = Q K^T        tcgen05.mma kind::f16, A = Q tile and B = K tile in shared memory (both
//                    K-major, two 64-dim halves of 128-byte-swizzled rows written by TMA),
//                    fp32 accumulator in tensor memory (128 columns)
//   softmax          every thread reads its row of S with tcgen05.ld (twice: maximum, then
//                    exponentials), keeps running maximum and sum, and writes P as TWO bf16
//                    terms (hi + lo by truncation, so that P.V matches an exact-softmax oracle
//                    to 2^-16)
//                    back to tensor memory with tcgen05.st (2 x 64 columns)
//   O += P V        tcgen05.mma with A = P from tensor memory and B = the V tile in shared
//                    memory, read MN-major (its rows are keys = the K dimension of this product),
//                    accumulating into the running output, which stays in tensor memory (128
//                    columns) for the whole block. P overwrites S in place (32 fp32 columns of a
//                    chunk become 16 columns of P hi and 16 of P lo), so a block needs 256 columns.
//   rescaling        the running output follows the running maximum lazily: a row is rescaled
//                    (read-modify-write of its 128 columns) only when its maximum grew by more
//                    than 2^8; otherwise it keeps the older reference maximum
// The K tile of the next step is requested as soon as S is complete, the V tile as soon as
// the previous P.V is complete, so the copies run under the softmax. Two blocks fit
// an SM (96 KB of shared memory, 256 tensor-memory columns each) and fill each other's gaps.
// Every mbarrier wait is bounded: on expiry the block records an error word in host-visible
// memory, stops, frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int D = 128;
constexpr int BQ = 128;   // query rows per block
constexpr int BKV = 128;  // keys per tile
constexpr int HALF_BYTES = 128 * 128;       // 128 rows x 64 bf16: one TMA box
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 128 x 128 bf16
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void set_status(int* status, int code) {
  *(volatile int*)status = code;
  __threadfence_system();
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand (rows of 128 bytes = 64 bf16 of the reduction dimension, 128-byte swizzle,
// groups of 8 rows 1024 bytes apart): Q and K tiles for S = Q K^T.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: the V tile for O = P V. Its rows are keys (the reduction dimension), each row
// holds 64 contiguous output dims (128 bytes, swizzled); 8-key groups are 1024 bytes apart
// (stride offset), the second 64 dims live in the next 16 KB box (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct TcAttnArgs {
  const int32_t* lens;
  const int32_t* past;
  const int32_t* qstart;
  int S, Hq, Hkv, maxlen;
  float scale_log2;
  bf16* out;
  int* status;
};

__global__ void __launch_bounds__(128) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v, TcAttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_q, bar_k, bar_v, bar_s, bar_o;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
  const int len = a.lens[b], pst = a.past ? a.past[b] : 0;
  const int n_new = len - pst;
  if (q0 >= n_new) return;  // whole block, before anything is allocated
  const int64_t row0 = a.qstart ? a.qstart[b] : (int64_t)b * a.S;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5;
  const int kv_end = min(len, pst + q0 + BQ);  // last key any row of this block may see, exclusive
  const int ntiles = (kv_end + BKV - 1) / BKV;
  const int kv_row0 = (b * a.Hkv + hk) * a.maxlen;

  const uint32_t sQ = smem_u32(smem), sK = sQ + TILE_BYTES, sV = sK + TILE_BYTES;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_q), 1);
    mbar_init(smem_u32(&bar_k), 1);
    mbar_init(smem_u32(&bar_v), 1);
    mbar_init(smem_u32(&bar_s), 1);
    mbar_init(smem_u32(&bar_o), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t tS = tmem, tO = tmem + 128;  // columns: S (then P hi/lo in place) and the running output

  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&bar_q), TILE_BYTES);
    tma_load_2d(sQ, &map_q, h * D, (int)(row0 + q0), smem_u32(&bar_q));
    tma_load_2d(sQ + HALF_BYTES, &map_q, h * D + 64, (int)(row0 + q0), smem_u32(&bar_q));
    mbar_expect_tx(smem_u32(&bar_k), TILE_BYTES);
    tma_load_2d(sK, &map_k, 0, kv_row0, smem_u32(&bar_k));
    tma_load_2d(sK + HALF_BYTES, &map_k, 64, kv_row0, smem_u32(&bar_k));
    mbar_expect_tx(smem_u32(&bar_v), TILE_BYTES);
    tma_load_2d(sV, &map_v, 0, kv_row0, smem_u32(&bar_v));
    tma_load_2d(sV + HALF_BYTES, &map_v, 64, kv_row0, smem_u32(&bar_v));
  }

  // instruction descriptors: D = F32, A = B = BF16, M = 128, N = 128; B of P.V is MN-major
  constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  constexpr uint32_t idesc_pv = idesc_s | (1u << 16);

  float m_run = -INFINITY, l_run = 0.f;
  const int qpos = pst + q0 + (int)threadIdx.x;  // position of this thread's query row
  bool ok = true;

  for (int t = 0; t < ntiles; t++) {
    const uint32_t ph = (uint32_t)(t & 1);
    // ---- S = Q K^T (after the previous P.V has finished reading P and the V tile)
    if (threadIdx.x == 0) {
      bool good = true;
      if (t > 0) {
        good = mbar_wait(smem_u32(&bar_o), ph ^ 1);
        if (good) {
          mbar_expect_tx(smem_u32(&bar_v), TILE_BYTES);
          tma_load_2d(sV, &map_v, 0, kv_row0 + t * BKV, smem_u32(&bar_v));
          tma_load_2d(sV + HALF_BYTES, &map_v, 64, kv_row0 + t * BKV, smem_u32(&bar_v));
        }
      } else {
        good = mbar_wait(smem_u32(&bar_q), 0);
      }
      good = good && mbar_wait(smem_u32(&bar_k), ph);
      if (!good) { set_status(a.status, 7); abort_flag = 1; }
      else {
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; s++) {
          const uint32_t off = (uint32_t)((s >> 2) * HALF_BYTES + (s & 3) * 32);  // 16 dims = 32 bytes inside the 64-dim half
          tc_mma_ss(tS, desc_kmajor(sQ + off), desc_kmajor(sK + off), idesc_s, s ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_s));
      }
    }
    __syncthreads();
    if (*(volatile int*)&abort_flag) { ok = false; break; }
    if (!mbar_wait(smem_u32(&bar_s), ph)) { if (threadIdx.x == 0) set_status(a.status, 8); ok = false; break; }
    tc_fence_after();
    // the K tile is free: request the next one
    if (threadIdx.x == 0 && t + 1 < ntiles) {
      mbar_expect_tx(smem_u32(&bar_k), TILE_BYTES);
      tma_load_2d(sK, &map_k, 0, kv_row0 + (t + 1) * BKV, smem_u32(&bar_k));
      tma_load_2d(sK + HALF_BYTES, &map_k, 64, kv_row0 + (t + 1) * BKV, smem_u32(&bar_k));
    }
    // ---- softmax of this thread's row
    const int k0 = t * BKV;
    const int k_lim = min(len, qpos + 1) - k0;  // keys [0, k_lim) of the tile are visible to this row
    const bool full = k0 + BKV <= min(len, pst + q0 + 1);  // every row of the block sees the whole tile (block-uniform)
    float m_tile = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < 4; c++) {
      uint32_t r[32];
      tc_ld32(tS + lane_base + (uint32_t)(c * 32), r);
      tc_wait_ld();
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j++) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
          if (c * 32 + j < k_lim) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
      }
    }
    m_tile *= a.scale_log2;  // the scale is positive: the maximum commutes with it
    // The running output lives in tensor memory, so following the maximum costs a read-modify-write
    // of the row. It is only done when the maximum grew by more than 2^8 (the exponentials then
    // stay below 256, harmless for the two-term bf16 P and the fp32 sums); otherwise the row keeps
    // its older reference maximum, and the final division by the running sum is unchanged.
    const bool grow = m_tile > m_run + 8.0f;  // also true for the first tile (m_run = -inf)
    const float m_use = grow ? m_tile : m_run;
    const float corr = grow ? exp2f(m_run - m_use) : 1.0f;  // 0 for the first tile
    m_run = m_use;
    if (t > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tc_ld32(tO + lane_base + (uint32_t)(c * 32), r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
        tc_st32(tO + lane_base + (uint32_t)(c * 32), r);
      }
    }
    float row_sum = 0.f;
#pragma unroll 1
    for (int c = 0; c < 4; c++) {
      uint32_t r[32];
      tc_ld32(tS + lane_base + (uint32_t)(c * 32), r);
      tc_wait_ld();
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int kk = c * 32 + 2 * j;
        float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * j]), a.scale_log2, -m_use));
        float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * j + 1]), a.scale_log2, -m_use));
        if (!full) {
          if (kk >= k_lim) p0 = 0.f;
          if (kk + 1 >= k_lim) p1 = 0.f;
        }
        row_sum += p0 + p1;
        // two-term split by truncation: hi = the upper 16 bits of p, lo = the upper 16 bits of the
        // (exact) remainder; p - hi - lo < 2^-16 p, and no conversion instruction is needed
        const uint32_t b0 = __float_as_uint(p0), b1 = __float_as_uint(p1);
        hi[j] = __byte_perm(b0, b1, 0x7632);
        const uint32_t l0 = __float_as_uint(p0 - __uint_as_float(b0 & 0xFFFF0000u)), l1 = __float_as_uint(p1 - __uint_as_float(b1 & 0xFFFF0000u));
        lo[j] = __byte_perm(l0, l1, 0x7632);
      }
      // in place: the 32 fp32 columns of this chunk become 16 columns of P hi and 16 of P lo
      tc_st16(tS + lane_base + (uint32_t)(c * 32), hi);
      tc_st16(tS + lane_base + (uint32_t)(c * 32 + 16), lo);
    }
    tc_wait_st();
    l_run = l_run * corr + row_sum;
    tc_fence_before();
    __syncthreads();  // P of all rows is in tensor memory (and the rescaled O, if any)
    // ---- O += P V
    if (threadIdx.x == 0) {
      if (!mbar_wait(smem_u32(&bar_v), ph)) { set_status(a.status, 9); abort_flag = 1; }
      else {
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; s++) {
          // 16 keys = 16 rows of 128 bytes = 2048 bytes of the V tile = 8 packed columns of P hi (and of P lo)
          const uint64_t dv = desc_mnmajor(sV + (uint32_t)(s * 2048));
          const uint32_t pcol = (uint32_t)((s >> 1) * 32 + (s & 1) * 8);
          tc_mma_ts(tO, tS + pcol, dv, idesc_pv, (t | s) ? 1u : 0u);
          tc_mma_ts(tO, tS + pcol + 16, dv, idesc_pv, 1u);
        }
        tc_commit(smem_u32(&bar_o));
      }
    }
  }

  __syncthreads();
  if (*(volatile int*)&abort_flag) ok = false;
  if (ok && !mbar_wait(smem_u32(&bar_o), (uint32_t)((ntiles - 1) & 1))) { if (threadIdx.x == 0) set_status(a.status, 10); ok = false; }
  tc_fence_after();
  if (ok) {
    const bool live = q0 + (int)threadIdx.x < n_new;
    const float inv = 1.0f / l_run;
    bf16* dst = a.out + ((row0 + q0 + threadIdx.x) * a.Hq + h) * D;
#pragma unroll 1
    for (int c = 0; c < 4; c++) {
      uint32_t r[32];
      tc_ld32(tO + lane_base + (uint32_t)(c * 32), r);
      tc_wait_ld();
      if (live) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 w;
          w.x = f32_to_bf16_bits(__uint_as_float(r[i]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 1]) * inv) << 16);
          w.y = f32_to_bf16_bits(__uint_as_float(r[i + 2]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 3]) * inv) << 16);
          w.z = f32_to_bf16_bits(__uint_as_float(r[i + 4]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 5]) * inv) << 16);
          w.w = f32_to_bf16_bits(__uint_as_float(r[i + 6]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 7]) * inv) << 16);
          *(uint4*)(dst + c * 32 + i) = w;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

// ------------------------------------------------------------------ two query tiles per block
// The kernel above runs S -> softmax -> PV of a block strictly one after the other, so the tensor
// pipe idles during the softmax and the softmax threads idle during the MMAs (two blocks per SM
// hide part of it). Here one block owns TWO tiles of 128 query rows (A and B, 256 consecutive
// positions of one head) that share every K/V tile, with separate roles:
//   warps 0..7   softmax of tile A (its own 256 tensor-memory columns: S/P and O); row r = lane r is
//                served by two threads (warps 0..3 and 4..7) that own 64 of the 128 columns each
//                and exchange only the row maximum, so two warps per scheduler hide each
//                other's tensor-memory and exp2 latencies
//   warps 8..15  softmax of tile B (the other 256 columns), same split
//   warp 16      one lane issues all MMAs in ping-pong order (PV_A(t) S_A(t+1) PV_B(t) S_B(t+1)):
//                while the A threads run their softmax the tensor pipe works on tile B, and so on
//   warp 17      one lane issues the TMA copies into two-stage K and V rings
// The whole tensor memory (512 columns) and 193 KB of shared memory: one block per SM.
constexpr int TC2_THREADS = 576;  // 16 softmax warps + MMA warp + TMA warp

__global__ void __launch_bounds__(TC2_THREADS) attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                      const __grid_constant__ CUtensorMap map_v, TcAttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_q, k_full[2], k_empty[2], v_full[2], v_empty[2], bar_s[2], bar_p[2], bar_o[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float x_max[2][2][BQ], x_sum[2][BQ];  // [tile][column half][row]: exchange between the two threads of a row

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * 2 * BQ;
  const int len = a.lens[b], pst = a.past ? a.past[b] : 0;
  const int n_new = len - pst;
  if (q0 >= n_new) return;  // whole block, before anything is allocated
  const int64_t row0 = a.qstart ? a.qstart[b] : (int64_t)b * a.S;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_row0 = (b * a.Hkv + hk) * a.maxlen;
  // K/V tiles each query tile needs (tile B is empty when the sequence ends inside tile A)
  int nt[2];
  nt[0] = (min(len, pst + q0 + BQ) + BKV - 1) / BKV;
  nt[1] = q0 + BQ < n_new ? (min(len, pst + q0 + 2 * BQ) + BKV - 1) / BKV : 0;
  const int ntiles = max(nt[0], nt[1]);

  const uint32_t sQ = smem_u32(smem), sK = sQ + 2 * TILE_BYTES, sV = sK + 2 * TILE_BYTES;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_q), 1);
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(&k_full[i]), 1); mbar_init(smem_u32(&k_empty[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1); mbar_init(smem_u32(&v_empty[i]), 1);
      mbar_init(smem_u32(&bar_s[i]), 1); mbar_init(smem_u32(&bar_p[i]), 2 * BQ); mbar_init(smem_u32(&bar_o[i]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 16) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  constexpr uint32_t idesc_pv = idesc_s | (1u << 16);

  if (warp == 17) {
    // ---- TMA producer
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&bar_q), (nt[1] ? 2 : 1) * TILE_BYTES);
      for (int w = 0; w < (nt[1] ? 2 : 1); w++) {
        tma_load_2d(sQ + w * TILE_BYTES, &map_q, h * D, (int)(row0 + q0 + w * BQ), smem_u32(&bar_q));
        tma_load_2d(sQ + w * TILE_BYTES + HALF_BYTES, &map_q, h * D + 64, (int)(row0 + q0 + w * BQ), smem_u32(&bar_q));
      }
      for (int t = 0; t < ntiles; t++) {
        const int st = t & 1;
        const uint32_t ph = (uint32_t)((t >> 1) & 1);
        if (t >= 2 && !mbar_wait(smem_u32(&k_empty[st]), ph ^ 1)) { set_status(a.status, 11); break; }
        mbar_expect_tx(smem_u32(&k_full[st]), TILE_BYTES);
        tma_load_2d(sK + st * TILE_BYTES, &map_k, 0, kv_row0 + t * BKV, smem_u32(&k_full[st]));
        tma_load_2d(sK + st * TILE_BYTES + HALF_BYTES, &map_k, 64, kv_row0 + t * BKV, smem_u32(&k_full[st]));
        if (t >= 2 && !mbar_wait(smem_u32(&v_empty[st]), ph ^ 1)) { set_status(a.status, 12); break; }
        mbar_expect_tx(smem_u32(&v_full[st]), TILE_BYTES);
        tma_load_2d(sV + st * TILE_BYTES, &map_v, 0, kv_row0 + t * BKV, smem_u32(&v_full[st]));
        tma_load_2d(sV + st * TILE_BYTES + HALF_BYTES, &map_v, 64, kv_row0 + t * BKV, smem_u32(&v_full[st]));
      }
    }
  } else if (warp == 16) {
    // ---- MMA issue, ping-pong between the two query tiles: S_A(0) S_B(0), then per K/V tile
    // PV_A(t) S_A(t+1) PV_B(t) S_B(t+1). The tensor pipe runs them in program order, so while
    // the A threads are in the softmax of step t+1 the pipe works on tile B, and vice versa.
    if (lane == 0) {
      auto issue_s = [&](int w, int t) {
        const int st = t & 1;
        const uint32_t tS = tmem + (uint32_t)(w * 256);
#pragma unroll
        for (int s = 0; s < 8; s++) {
          const uint32_t off = (uint32_t)((s >> 2) * HALF_BYTES + (s & 3) * 32);
          tc_mma_ss(tS, desc_kmajor(sQ + w * TILE_BYTES + off), desc_kmajor(sK + st * TILE_BYTES + off), idesc_s, s ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_s[w]));
      };
      bool good = mbar_wait(smem_u32(&bar_q), 0) && mbar_wait(smem_u32(&k_full[0]), 0);
      if (good) {
        tc_fence_after();
        for (int w = 0; w < 2; w++)
          if (nt[w] > 0) issue_s(w, 0);
        tc_commit(smem_u32(&k_empty[0]));
      }
      for (int t = 0; t < ntiles && good; t++) {
        const int st = t & 1;
        const uint32_t rph = (uint32_t)((t >> 1) & 1), ph = (uint32_t)(t & 1);
        good = mbar_wait(smem_u32(&v_full[st]), rph);
        bool k_next_ready = false;
        for (int w = 0; w < 2 && good; w++) {
          if (t < nt[w]) {
            good = mbar_wait(smem_u32(&bar_p[w]), ph);  // P (and the rescaled O) of this step are in tensor memory
            if (!good) break;
            tc_fence_after();
            const uint32_t tS = tmem + (uint32_t)(w * 256), tO = tS + 128;
#pragma unroll
            for (int s = 0; s < 8; s++) {
              const uint64_t dv = desc_mnmajor(sV + st * TILE_BYTES + (uint32_t)(s * 2048));
              const uint32_t pcol = (uint32_t)((s >> 1) * 32 + (s & 1) * 8);
              tc_mma_ts(tO, tS + pcol, dv, idesc_pv, (t | s) ? 1u : 0u);
              tc_mma_ts(tO, tS + pcol + 16, dv, idesc_pv, 1u);
            }
            tc_commit(smem_u32(&bar_o[w]));
          }
          if (t + 1 < nt[w]) {
            if (!k_next_ready) {
              good = mbar_wait(smem_u32(&k_full[(t + 1) & 1]), (uint32_t)(((t + 1) >> 1) & 1));
              if (!good) break;
              tc_fence_after();
              k_next_ready = true;
            }
            issue_s(w, t + 1);
          }
        }
        if (!good) break;
        tc_commit(smem_u32(&v_empty[st]));                               // both PV products have read the V tile
        if (t + 1 < ntiles) tc_commit(smem_u32(&k_empty[(t + 1) & 1]));  // both S products of the next step have read its K tile
      }
      if (!good) set_status(a.status, 13);
    }
  } else {
    // ---- softmax warpgroups: w = 0 (tile A) or 1 (tile B)
    const int w = warp >> 3, half = (warp >> 2) & 1, row = (int)threadIdx.x & (BQ - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    auto wg_sync = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(1 + w) : "memory"); };  // the 256 threads of this tile
    const uint32_t tS = tmem + (uint32_t)(w * 256), tO = tS + 128;
    const int qw = q0 + w * BQ;           // first query row of this tile
    const int qpos = pst + qw + row;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < nt[w]; t++) {
      const uint32_t ph = (uint32_t)(t & 1);
      if (!mbar_wait(smem_u32(&bar_s[w]), ph)) { if (row == 0) set_status(a.status, 14); ok = false; break; }
      tc_fence_after();
      const int k0 = t * BKV;
      const int k_lim = min(len, qpos + 1) - k0;
      const bool full = k0 + BKV <= min(len, pst + qw + 1);
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; c++) {
        uint32_t r[32];
        tc_ld32(tS + lane_base + (uint32_t)(c * 32), r);
        tc_wait_ld();
        if (full) {
#pragma unroll
          for (int j = 0; j < 32; j++) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c * 32 + j < k_lim) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        }
      }
      x_max[w][half][row] = m_tile;
      wg_sync();
      m_tile = fmaxf(x_max[w][0][row], x_max[w][1][row]) * a.scale_log2;
      const bool grow = m_tile > m_run + 8.0f;  // lazy rescaling, as in the kernel above
      const float m_use = grow ? m_tile : m_run;
      const float corr = grow ? exp2f(m_run - m_use) : 1.0f;
      m_run = m_use;
      if (t > 0 && __any_sync(0xffffffffu, grow)) {
        // the previous PV of this tile must have finished writing O
        if (!mbar_wait(smem_u32(&bar_o[w]), ph ^ 1)) { if (row == 0) set_status(a.status, 15); ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 2 * half; c < 2 * half + 2; c++) {
          uint32_t r[32];
          tc_ld32(tO + lane_base + (uint32_t)(c * 32), r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
          tc_st32(tO + lane_base + (uint32_t)(c * 32), r);
        }
      }
      float row_sum = 0.f;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; c++) {
        uint32_t r[32];
        tc_ld32(tS + lane_base + (uint32_t)(c * 32), r);
        tc_wait_ld();
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int kk = c * 32 + 2 * j;
          float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * j]), a.scale_log2, -m_use));
          float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * j + 1]), a.scale_log2, -m_use));
          if (!full) {
            if (kk >= k_lim) p0 = 0.f;
            if (kk + 1 >= k_lim) p1 = 0.f;
          }
          row_sum += p0 + p1;
          const uint32_t b0 = __float_as_uint(p0), b1 = __float_as_uint(p1);
          hi[j] = __byte_perm(b0, b1, 0x7632);
          const uint32_t l0 = __float_as_uint(p0 - __uint_as_float(b0 & 0xFFFF0000u)), l1 = __float_as_uint(p1 - __uint_as_float(b1 & 0xFFFF0000u));
          lo[j] = __byte_perm(l0, l1, 0x7632);
        }
        tc_st16(tS + lane_base + (uint32_t)(c * 32), hi);
        tc_st16(tS + lane_base + (uint32_t)(c * 32 + 16), lo);
      }
      tc_wait_st();
      l_run = l_run * corr + row_sum;
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_p[w])) : "memory");
      wg_sync();  // x_max is rewritten in the next step
    }
    if (ok && nt[w] > 0) {
      if (!mbar_wait(smem_u32(&bar_o[w]), (uint32_t)((nt[w] - 1) & 1))) { if (row == 0) set_status(a.status, 16); ok = false; }
      tc_fence_after();
    }
    if (half) x_sum[w][row] = l_run;  // the two threads of a row saw the same maxima: their sums add
    wg_sync();
    if (!half) x_sum[w][row] += l_run;
    wg_sync();
    if (ok && nt[w] > 0) {
      const bool live = qw + row < n_new;
      const float inv = 1.0f / x_sum[w][row];
      bf16* dst = a.out + ((row0 + qw + row) * a.Hq + h) * D;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; c++) {
        uint32_t r[32];
        tc_ld32(tO + lane_base + (uint32_t)(c * 32), r);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 wv;
            wv.x = f32_to_bf16_bits(__uint_as_float(r[i]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 1]) * inv) << 16);
            wv.y = f32_to_bf16_bits(__uint_as_float(r[i + 2]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 3]) * inv) << 16);
            wv.z = f32_to_bf16_bits(__uint_as_float(r[i + 4]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 5]) * inv) << 16);
            wv.w = f32_to_bf16_bits(__uint_as_float(r[i + 6]) * inv) | (f32_to_bf16_bits(__uint_as_float(r[i + 7]) * inv) << 16);
            *(uint4*)(dst + c * 32 + i) = wv;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

int get_encode() {
  if (g_encode) return STRICTB200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  SB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  if (!fn || q != cudaDriverEntryPointSuccess) return sb_fail(STRICTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode = (EncodeFn)fn;
  return STRICTB200_OK;
}

// 2D map of a row-major bf16 matrix [rows, cols] (row stride ld elements), box = 128 rows x 64 columns (128 bytes), 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return sb_fail(STRICTB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return STRICTB200_OK;
}

}  // namespace

// q, out: [q_rows, Hq, 128]; caches [B, Hkv, maxlen, 128]. ERR_UNSUPPORTED for shapes this kernel does not take.
int k_attn_prefill_tc(strictb200_ctx* ctx, const bf16* q, const bf16* kc, const bf16* vc, const int32_t* lens, const int32_t* past,
                      const int32_t* qstart, int B, int S, int64_t q_rows, int Hq, int Hkv, int maxlen, float scale, bf16* out) {
  if (Hq > 65535 || B > 65535 || Hq % Hkv) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: too many heads or sequences");
  if ((int64_t)B * Hkv * maxlen > INT32_MAX || q_rows > INT32_MAX) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: cache too large for 32-bit tile coordinates");
  if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) & 15) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "attention: operands must be 16-byte aligned");
  SB_TRY(get_encode());
  CUtensorMap mq, mk, mv;
  SB_TRY(make_map(&mq, q, q_rows, (int64_t)Hq * D, (int64_t)Hq * D));
  SB_TRY(make_map(&mk, kc, (int64_t)B * Hkv * maxlen, D, D));
  SB_TRY(make_map(&mv, vc, (int64_t)B * Hkv * maxlen, D, D));
  const size_t smem = 3 * TILE_BYTES + 1024;
  static SbDeviceOnce once;
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  TcAttnArgs a{lens, past, qstart, S, Hq, Hkv, maxlen, scale * LOG2E, out, ctx->d_status};
  // two query tiles per block (ping-pong) from 256 new tokens per sequence on; the attn_tc option (1 / 2) forces a kernel
  const int forced = ctx->opt.attn_tc;
  if (forced == 2 || (forced != 1 && S >= 2 * BQ)) {
    const size_t smem2 = 6 * TILE_BYTES + 1024;
    static SbDeviceOnce once2;
    SB_CUDA(once2.run(ctx->device, [&] { return cudaFuncSetAttribute(attn_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2); }));
    dim3 grid2((unsigned)((S + 2 * BQ - 1) / (2 * BQ)), (unsigned)Hq, (unsigned)B);
    attn_prefill_tc2_kernel<<<grid2, TC2_THREADS, smem2, ctx->stream>>>(mq, mk, mv, a);
    SB_LAUNCHED(ctx);
    return STRICTB200_OK;
  }
  dim3 grid((unsigned)((S + BQ - 1) / BQ), (unsigned)Hq, (unsigned)B);
  attn_prefill_tc_kernel<<<grid, 128, smem, ctx->stream>>>(mq, mk, mv, a);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
