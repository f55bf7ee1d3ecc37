// tcgen05 / tensor-memory GEMM, decode flavour: one block = one 128 x BT output tile over one K
// range (grid.z = K splits), two blocks per SM. Used while the whole token batch fits one tile
// (at most 128 tokens = 256 operand rows): the job is then a pure HBM stream of weights, and many
// small independent blocks with the split-K sum left to the row kernel that consumes the result
// measured faster than a persistent schedule with in-kernel fix-up (see gemm_tmem.cu for the
// persistent kernel used for prefill, and for the description of the operand layout).
//   warp 0      TMA producer (first ring of WEIGHT loads issued before the dependency wait)
//   warp 1      TMEM allocation, tcgen05.mma issue, tcgen05.commit
//   warps 2..5  epilogue: tcgen05.ld, acc_hi + acc_lo/16, raw partials or scaled bf16/fp32 output
// No TMA multicast, no clusters; every mbarrier wait is bounded and reports through the
// context's host-visible error word instead of hanging.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int BN = 128;       // output channels per block (UMMA_M)
constexpr int BK = 128;       // bytes of K per stage = one 128-byte swizzle atom
constexpr int UMMA_K = 32;    // bytes (= E4M3 elements) of K per tcgen05.mma
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait attempts before giving up (each blocks up to ~1 us)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. Returns false when the limit expired.
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
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
// The error word lives in pinned host memory: a plain store plus a system-scope fence.
__device__ __forceinline__ void set_status(int* status, int code) {
  *(volatile int*)status = code;
  __threadfence_system();
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Signed 8-bit integer operands, 32-bit integer accumulator (same operand layout and K = 32 per instruction).
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (one swizzle atom
// wide), stored densely with the 128-byte swizzle TMA applies: groups of 8 rows are 1024 bytes
// apart (stride byte offset), layout type 2 = SWIZZLE_128B, descriptor version 1. The tile base
// is 1024-byte aligned; advancing K by 32 bytes inside the atom adds 32 to the start address.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct TmemArgs {
  int M, Mq, N, K;
  const float* sx;
  const float* sw;
  void* out;
  int out_f32;
  float* part;
  int splits;
  int raw;
  int* status;  // host-visible error word
  int prefetch;  // issue the first ring of weight loads before the dependency wait
};

// I8: both operands are signed 8-bit integers (weights int8, activations as two int8 terms
// x = s * (128 * hi + lo), gemm_int8.cu) and the accumulators 32-bit integers; the epilogue joins
// the two terms in 64-bit integers, so the result does not depend on the K split or on any order.
template <int BT, int STAGES, bool I8>
__global__ void __launch_bounds__(192) gemm_tmem_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                        TmemArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024 the swizzle needs
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int STAGE_BYTES = BN * BK + BT * BK;
  constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  SB_TRACE_BEGIN();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, t0 = blockIdx.y * BT;
  // split z owns the k-blocks [z * nkb_all / splits, (z + 1) * nkb_all / splits): sizes differ by at most one
  const int nkb_all = a.K / BK;
  const int kb_first = (int)((int64_t)blockIdx.z * nkb_all / a.splits), kb_last = (int)((int64_t)(blockIdx.z + 1) * nkb_all / a.splits);
  const int k_begin = kb_first * BK, nkb = kb_last - kb_first;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    mbar_init(smem_u32(&bar_acc), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  pdl_trigger();
  if (warp == 0) {
    if (lane == 0) {
      // The weights are constants: their loads for the first ring of stages are issued before the
      // dependency wait, so they stream from HBM while the preceding kernel is still running.
      const int npre = nkb < STAGES ? nkb : STAGES;
      const uint64_t w_policy = l2_evict_first_policy();  // every weight byte is read once per launch
      if (!a.prefetch) pdl_wait();
      for (int kb = 0; kb < npre; kb++) {
        uint32_t full = smem_u32(&bar_full[kb]);
        mbar_expect_tx(full, STAGE_BYTES);
        tma_load_2d_hint(smem_u32(smem + (size_t)kb * STAGE_BYTES), &map_w, k_begin + kb * BK, n0, full, w_policy);
      }
      pdl_wait();
      SB_TRACE_WAITED();
      for (int kb = 0; kb < npre; kb++)
        tma_load_2d(smem_u32(smem + (size_t)kb * STAGE_BYTES) + BN * BK, &map_x, k_begin + kb * BK, t0, smem_u32(&bar_full[kb]));
      for (int kb = npre; kb < nkb; kb++) {
        int s = kb % STAGES;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ((kb / STAGES) & 1) ^ 1)) { set_status(a.status, 1); abort_flag = 1; break; }
        if (*(volatile int*)&abort_flag) break;
        uint32_t full = smem_u32(&bar_full[s]);
        uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        mbar_expect_tx(full, STAGE_BYTES);
        tma_load_2d_hint(dst, &map_w, k_begin + kb * BK, n0, full, w_policy);
        tma_load_2d(dst + BN * BK, &map_x, k_begin + kb * BK, t0, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D = F32 (bits 4-5 = 1), A = B = E4M3 (0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24;
      // integers: D = S32 (bits 4-5 = 2), A (bits 7-9) = B (bits 10-12) = signed 8 bit (1)
      constexpr uint32_t idesc = (I8 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4)) | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
      // The operand tiles cannot arrive before the producer's dependency wait has returned; waiting for the same
      // dependency here keeps the bounded waits below for progress inside this kernel (a predecessor that itself
      // waits for another rank may take longer than any of them).
      pdl_wait();
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; kb++) {
        int s = kb % STAGES;
        if (!mbar_wait(smem_u32(&bar_full[s]), (kb / STAGES) & 1)) { set_status(a.status, 2); abort_flag = 1; ok = false; break; }
        tc_fence_after();
        uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
        uint64_t da = smem_desc(sa), db = smem_desc(sa + BN * BK);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++) {
          // +32 bytes of K inside the swizzle atom = +2 in the (address >> 4) field
          if (I8) tc_mma_i8(tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, (kb | k) ? 1u : 0u);
          else tc_mma_f8(tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, (kb | k) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));  // stage is free once these MMAs have read it
      }
      tc_commit(smem_u32(&bar_acc));  // accumulator complete (arrives after all prior MMAs)
    }
  } else {
    // epilogue: warp w may touch TMEM lanes [32*(w%4), +32)
    const int lg = warp & 3;
    const int n = n0 + lg * 32 + lane;
    pdl_wait();  // the scales and the output buffers belong to the dependency chain
    bool ok = mbar_wait(smem_u32(&bar_acc), 0);
    if (!ok) { if (lane == 0) set_status(a.status, 3); }
    ok = ok && !*(volatile int*)&abort_flag;
    tc_fence_after();
    if (ok) {
      const bool raw = a.raw || a.splits > 1;
      const float swn = (!raw && n < a.N) ? a.sw[n] : 0.f;
#pragma unroll 1
      for (int grp = 0; grp < BT / 16; grp++) {
        uint32_t r[16];
        tc_ld16(tmem + ((uint32_t)(lg * 32) << 16) + (uint32_t)(grp * 16), r);
        tc_wait_ld();
        const int tok0 = ((t0 + grp * 16) >> 1);  // operand rows 16g.. hold tokens 8g..
#pragma unroll
        for (int j = 0; j < 8; j++) {
          int tok = tok0 + j;
          if (I8) {
            if (tok < a.M && n < a.N) {
              if (raw) {  // the two integer sums of this K range, [split][hi, lo][token][channel]
                int32_t* part = (int32_t*)a.part;
                part[(((int64_t)blockIdx.z * 2 + 0) * a.M + tok) * a.N + n] = (int32_t)r[j];
                part[(((int64_t)blockIdx.z * 2 + 1) * a.M + tok) * a.N + n] = (int32_t)r[8 + j];
              } else {
                const float v = __ll2float_rn((int64_t)(int32_t)r[j] * 128 + (int64_t)(int32_t)r[8 + j]);
                const float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), swn);
                if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
                else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
              }
            }
          } else if (tok < a.M && n < a.N) {
            float v = __fadd_rn(__uint_as_float(r[j]), __fmul_rn(0.0625f, __uint_as_float(r[8 + j])));
            if (raw) {
              a.part[((int64_t)blockIdx.z * a.M + tok) * a.N + n] = v;
            } else {
              float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), swn);
              if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
              else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
  }
  SB_TRACE_END(SB_K_GEMM, (uint32_t)a.N ^ ((uint32_t)a.K << 12));
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

// 2D map of a row-major byte matrix [rows, K] (row stride ld bytes), box = box_rows x 128 bytes, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return sb_fail(STRICTB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return STRICTB200_OK;
}

template <int BT, int STAGES, bool I8 = false>
int launch(strictb200_ctx* ctx, const GemmArgs& g, const TmemArgs& ta) {
  constexpr int STAGE_BYTES = BN * BK + BT * BK;
  size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;  // + slack for the 1024-byte round-up
  static SbDeviceOnce once;  // one per instantiation
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(gemm_tmem_kernel<BT, STAGES, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  CUtensorMap mw, mx;
  SB_TRY(make_map(&mw, g.wq, g.N, g.K, g.ldw, BN));
  SB_TRY(make_map(&mx, g.xq, ta.Mq, g.K, g.ldx, BT));
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((ta.Mq + BT - 1) / BT), (unsigned)g.splits);
  if (grid.y > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: M too large for one launch");
  SB_CUDA(sb_launch(ctx, gemm_tmem_kernel<BT, STAGES, I8>, grid, dim3(192), smem, mw, mx, ta));
  ctx->launches++;
  return STRICTB200_OK;
}

}  // namespace

SB_TRACE_TU(gemm_split)

int k_gemm_fp8_tmem_split(strictb200_ctx* ctx, const GemmArgs& g) {
  if (g.K % BK || g.splits < 1 || g.splits > g.K / BK)
    return sb_fail(STRICTB200_ERR_UNSUPPORTED, "tensor-memory GEMM needs K to be a multiple of 128 and at most K/128 splits");
  if (((uintptr_t)g.xq | (uintptr_t)g.wq | (uintptr_t)g.ldx | (uintptr_t)g.ldw) & 15)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: operands and row strides must be 16-byte aligned");
  if ((g.splits > 1 || g.raw) && !g.part) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: split-K needs a partial buffer");
  SB_TRY(get_encode());
  TmemArgs ta{(int)g.M, (int)sb_qrows(g.M), (int)g.N, (int)g.K, g.sx, g.sw, g.out, g.out_f32, g.part, g.splits, g.raw, ctx->d_status, ctx->opt.prefetch};
  // BT = operand rows per block = the whole (split) batch
  // A grid of at most one block per SM gets a ring that fills the SM's shared memory (the whole
  // ring of weight tiles is in flight before the dependency wait); larger grids keep two blocks
  // per SM resident.
  const int64_t blocks = ((g.N + BN - 1) / BN) * g.splits;
  const int deep = ctx->opt.deep_ring;
  if (g.i8) {  // integer operands: the same tiles; token tiles beyond the first go to grid.y
    if (ta.Mq <= 32) return launch<32, 5, true>(ctx, g, ta);
    if (ta.Mq <= 64) return launch<64, 4, true>(ctx, g, ta);
    if (ta.Mq <= 128) return launch<128, 4, true>(ctx, g, ta);
    return launch<256, 4, true>(ctx, g, ta);
  }
  if (ta.Mq <= 32) return deep && blocks <= ctx->sm_count ? launch<32, 10>(ctx, g, ta) : launch<32, 5>(ctx, g, ta);
  if (ta.Mq <= 64) return deep && blocks <= ctx->sm_count ? launch<64, 9>(ctx, g, ta) : launch<64, 4>(ctx, g, ta);
  if (ta.Mq <= 128) return launch<128, 4>(ctx, g, ta);
  if (ta.Mq <= 256) return launch<256, 4>(ctx, g, ta);
  return sb_fail(STRICTB200_ERR_UNSUPPORTED, "the split tensor-memory GEMM takes at most 128 tokens");
}
