// tcgen05 / tensor-memory GEMM for prefill, two SMs per tile: a cluster of two blocks computes one
// 256-channel x 256-operand-row (= 128 tokens) output tile with tcgen05.mma.cta_group::2.
// Each block stages its own 128 weight rows and its own 128 operand rows of every 128-byte K block
// (32 KB per block per K block, against 48 KB for a 128 x 256 tile on one SM), so the tile's
// arithmetic intensity is 1.5 times that of the one-SM kernel in gemm_tmem.cu. That matters
// because the one-SM kernel is bound by the bytes it can keep in flight from L2 to shared memory:
// ncu shows its tensor pipe busy half of the time with 144 KB in flight per SM.
//
// Operand layout, numerics and epilogue are those of gemm_tmem.cu (weights = A operand = TMEM
// lanes, operand rows = B operand = TMEM columns, acc_hi + acc_lo/16, scales, bf16/fp32 stores).
//
// Roles (both blocks of a pair run the same code, 192 threads each; rank 0 is the leader):
//   warp 0      TMA producer of this block's halves; the bytes of both blocks complete on the
//               LEADER's full barrier (the .cta_group::2 form of the tensor copy: each block
//               copies only into its own shared memory)
//   warp 1      TMEM allocation (both blocks, cta_group::2: 512 columns = two accumulators);
//               the leader's lane 0 issues the MMAs for the pair and one tcgen05.commit per
//               block (frees the stage in both blocks, publishes the accumulator to both)
//   warps 2..5  epilogue of this block's 128 channels; hand the accumulator back by arriving on
//               the leader's barrier (remote mbarrier.arrive from the second block)
// Persistent schedule: one pair per two SMs, pair c owns tiles [c*tiles/pairs, (c+1)*tiles/pairs),
// two accumulators so the epilogue of a tile overlaps the MMAs of the next one.
// Every mbarrier wait is bounded: on expiry the block records an error word in host-visible
// memory and stops issuing work; TMEM is freed and the pair leaves together.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int BN = 128;       // channels per block (half of the pair's UMMA_M = 256)
constexpr int BTH = 128;      // operand rows per block (half of the pair's UMMA_N = 256)
constexpr int BK = 128;       // bytes of K per stage = one 128-byte swizzle atom
constexpr int UMMA_K = 32;    // bytes (= E4M3 elements) of K per tcgen05.mma
constexpr int STAGES = 7;
constexpr int STAGE_BYTES = BN * BK + BTH * BK;  // 32 KB per block
constexpr int ACC_COLS = 256, TMEM_COLS = 512;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait attempts before giving up (each blocks up to ~1 us)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Address of the same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Arrive on a barrier given by its cluster address (this block's or the other's).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
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
// Tile load into this block's shared memory whose bytes complete on a barrier of the leader.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(leader_bar)
               : "memory");
}
__device__ __forceinline__ void set_status(int* status, int code) {
  *(volatile int*)status = code;
  __threadfence_system();
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
// Arrive on the barrier at this shared-memory offset in BOTH blocks once all prior MMAs of the pair are
// done: one commit per block, each naming that block's barrier by its cluster address.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(map_to_rank(bar, 0)) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(map_to_rank(bar, 1)) : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
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
// Barrier over the 4 epilogue warps that also ORs a predicate (all 128 leave the tile loop together).
__device__ __forceinline__ bool epi_any(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// K-major tile, 128-byte rows, SWIZZLE_128B (see gemm_tmem.cu).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct PairArgs {
  int M, Mq, N, K;
  const float* sx;
  const float* sw;
  void* out;
  int out_f32;
  int* status;   // host-visible error word
  int tiles_n;   // 256-channel tiles; tile = tt * tiles_n + tn
  int tiles;
};

__global__ void __launch_bounds__(192) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                        PairArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const bool leader = rank == 0;
  const int nkb = a.K / BK;
  const int pairs = gridDim.x / 2, c = blockIdx.x / 2;
  const int tile_begin = (int)((int64_t)c * a.tiles / pairs), tile_end = (int)((int64_t)(c + 1) * a.tiles / pairs);
  const int n_my = (tile_end - tile_begin) * nkb;  // K blocks this pair walks through

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    // accumulator hand-back: the 128 epilogue threads of each block arrive on the leader's barrier
    for (int s = 0; s < 2; s++) { mbar_init(smem_u32(&bar_acc_full[s]), 1); mbar_init(smem_u32(&bar_acc_empty[s]), 256); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync();  // both blocks' barriers exist and both have their tensor memory
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  pdl_trigger();
  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      for (int it = 0; it < n_my; it++) {
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait(smem_u32(&bar_empty[s]), ((it / STAGES) & 1) ^ 1)) { set_status(a.status, 1); abort_flag = 1; break; }
        if (*(volatile int*)&abort_flag) break;
        const int tile = tile_begin + it / nkb, kb = it % nkb;
        const int wy = (tile % a.tiles_n) * 2 * BN + (int)rank * BN, xy = (tile / a.tiles_n) * 2 * BTH + (int)rank * BTH;
        const uint32_t full_leader = map_to_rank(smem_u32(&bar_full[s]), 0);
        if (leader) mbar_expect_tx(smem_u32(&bar_full[s]), 2 * STAGE_BYTES);  // the bytes of both blocks
        const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        tma_load_2d_pair(dst, &map_w, kb * BK, wy, full_leader);
        tma_load_2d_pair(dst + BN * BK, &map_x, kb * BK, xy, full_leader);
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      // instruction descriptor: D = F32, A = B = E4M3, both K-major, N = 256 (>> 3 at bit 17), M = 256 (>> 4 at bit 24)
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      // The operand tiles cannot arrive before the producer's dependency wait has returned; waiting for the same
      // dependency here keeps the bounded waits below for progress inside this kernel (a predecessor that itself
      // waits for another rank may take longer than any of them).
      pdl_wait();
      for (int it = 0; it < n_my; it++) {
        const int kb = it % nkb, seg = it / nkb;
        if (kb == 0) {
          // both blocks' epilogues must have drained this accumulator (it was used two tiles ago)
          if (seg >= 2 && !mbar_wait(smem_u32(&bar_acc_empty[seg & 1]), ((seg >> 1) & 1) ^ 1)) { set_status(a.status, 4); abort_flag = 1; break; }
          tc_fence_after();
        }
        const int s = it % STAGES;
        if (!mbar_wait(smem_u32(&bar_full[s]), (it / STAGES) & 1)) { set_status(a.status, 2); abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t da = smem_desc(sa), db = smem_desc(sa + BN * BK);
        const uint32_t acc = tmem + (uint32_t)((seg & 1) * ACC_COLS);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++)
          tc_mma_f8_pair(acc, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, (kb | k) ? 1u : 0u);
        tc_commit_pair(smem_u32(&bar_empty[s]));                             // the stage is free in both blocks
        if (kb == nkb - 1) tc_commit_pair(smem_u32(&bar_acc_full[seg & 1]));  // accumulator complete, both blocks
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes [32*(w%4), +32) = channels of this block's half
    const int lg = warp & 3;
    const int ch = lg * 32 + lane;
    pdl_wait();  // the scales and the output buffer belong to the dependency chain
    for (int seg = 0; seg < tile_end - tile_begin; seg++) {
      const int tile = tile_begin + seg;
      bool bad = !mbar_wait(smem_u32(&bar_acc_full[seg & 1]), (seg >> 1) & 1);
      if (bad && lane == 0) set_status(a.status, 3);
      if (epi_any(bad)) break;
      tc_fence_after();
      const uint32_t acc = tmem + (uint32_t)((seg & 1) * ACC_COLS) + ((uint32_t)(lg * 32) << 16);
      const int n = (tile % a.tiles_n) * 2 * BN + (int)rank * BN + ch;
      const int tok_base = (tile / a.tiles_n) * BTH;  // 256 operand rows = 128 tokens per tile
      const float swn = n < a.N ? a.sw[n] : 0.f;
#pragma unroll 1
      for (int grp = 0; grp < ACC_COLS / 16; grp++) {
        uint32_t r[16];
        tc_ld16(acc + (uint32_t)(grp * 16), r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int tok = tok_base + grp * 8 + j;  // operand rows 16g.. hold tokens 8g..
          if (tok < a.M && n < a.N) {
            float v = __fadd_rn(__uint_as_float(r[j]), __fmul_rn(0.0625f, __uint_as_float(r[8 + j])));
            float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), swn);
            if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
            else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
          }
        }
      }
      // the accumulator is drained in this block: tell the leader's MMA warp
      tc_fence_before();
      mbar_arrive_cluster(map_to_rank(smem_u32(&bar_acc_empty[seg & 1]), 0));
    }
  }
  // Nobody leaves while the other block may still signal one of its barriers or use its tensor memory.
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
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

// 2D map of a row-major byte matrix [rows, K] (row stride ld bytes), box = 128 rows x 128 bytes, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)BK, 128u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return sb_fail(STRICTB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return STRICTB200_OK;
}

}  // namespace

// Y = ((X . Wq^T) * sx) * sw for many tokens (prefill). ERR_UNSUPPORTED for shapes this kernel does not take.
int k_gemm_fp8_tmem_pair(strictb200_ctx* ctx, const GemmArgs& g) {
  if (g.K % BK || g.splits != 1 || g.raw || !g.out) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "paired tensor-memory GEMM: K % 128, no splits, no raw output");
  if (((uintptr_t)g.xq | (uintptr_t)g.wq | (uintptr_t)g.ldx | (uintptr_t)g.ldw) & 15)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: operands and row strides must be 16-byte aligned");
  SB_TRY(get_encode());
  const int64_t Mq = sb_qrows(g.M);
  const int64_t tiles_n = (g.N + 2 * BN - 1) / (2 * BN), tiles_t = (Mq + 2 * BTH - 1) / (2 * BTH), tiles = tiles_n * tiles_t;
  if (tiles > INT32_MAX / 2) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: too many output tiles");
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;  // + slack for the 1024-byte round-up
  static SbDeviceOnce once;
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  CUtensorMap mw, mx;
  SB_TRY(make_map(&mw, g.wq, g.N, g.K, g.ldw));
  SB_TRY(make_map(&mx, g.xq, Mq, g.K, g.ldx));
  PairArgs pa{(int)g.M, (int)Mq, (int)g.N, (int)g.K, g.sx, g.sw, g.out, g.out_f32, ctx->d_status, (int)tiles_n, (int)tiles};
  int64_t pairs = ctx->sm_count / 2;
  if (pairs > tiles) pairs = tiles;
  SB_CUDA(sb_launch_cluster(ctx, gemm_pair_kernel, dim3((unsigned)(2 * pairs)), dim3(192), smem, dim3(2, 1, 1), mw, mx, pa));
  ctx->launches++;
  return STRICTB200_OK;
}
