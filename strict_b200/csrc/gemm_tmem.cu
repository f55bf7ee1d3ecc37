// tcgen05 / tensor-memory GEMM for sm_100a: Y[M,N] = ((X . Wq^T) * sx) * sw with X carried as
// two E4M3 terms (see gemm_fp8.cu), both operands E4M3, kind::f8f6f4, fp32 accumulator in TMEM.
//
// Orientation: the WEIGHT tile is the A operand (UMMA_M = 128 output channels = 128 TMEM lanes)
// and the activation rows are the B operand (UMMA_N = BT operand rows = BT TMEM columns). The
// same kernel therefore serves decode (BT = 32/64: a pure HBM stream of weights through TMA,
// no thread ever touches a weight byte) and prefill (BT = 256: tensor-bound tiles).
//
// Persistent schedule: the grid is one block per SM. All (output tile, 128-byte K block) pairs
// form one linear list, tile-major, and block c owns a contiguous range of it. By default the
// ranges are cut at tile boundaries (block c owns tiles [c*tiles/G, (c+1)*tiles/G)), so every
// tile goes straight from its accumulator to the epilogue while the MMA warp already fills the
// second accumulator with the next tile. With stream_k set the ranges are [c*total/G,
// (c+1)*total/G) instead and a tile cut by a boundary is finished by whichever of its
// contributors arrives last: each stores its fp32 partial tile to a workspace slot and bumps the
// tile's counter, and the one that sees the final count adds the slots in contributor order (the
// sum order never depends on timing) and runs the epilogue; nobody waits for another block. That
// mode balances bytes per SM exactly but measured slower here (the fix-up is exposed at the end
// of every block), so it is kept for shapes with fewer tiles than SMs only.
//
// Roles inside a block (192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2D loads of the 128x128 B weight tile and the
//               BT x128 B activation tile into a ring of SWIZZLE_128B stages, mbarrier tx counts.
//               The first ring of WEIGHT loads is issued before the programmatic-dependency wait.
//   warp 1      TMEM allocation (two accumulators); one lane issues tcgen05.mma (4 per stage,
//               K = 32 each) and tcgen05.commit to free the stage / publish an accumulator
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (lane = channel, column = operand row),
//               acc_hi + acc_lo/16, scales, bf16/fp32 stores coalesced along the channel; runs
//               while the MMA warp already fills the other accumulator
// No TMA multicast and no clusters are used. Every mbarrier wait is bounded: on expiry the block
// records an error word in host-visible memory, stops issuing work, still frees its TMEM and
// returns, so a lost signal cannot hang the GPU.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int BN = 128;       // output channels per tile (UMMA_M)
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // the 4 epilogue warps
// Barrier over the 4 epilogue warps that also ORs a predicate: every thread learns whether any
// of them wants to give up, so all 128 leave the segment loop together and none is left waiting.
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
  int* status;      // host-visible error word
  int prefetch;     // issue the first ring of weight loads before the dependency wait
  int stream_k;     // 1: cut the linear (tile, K block) list evenly; 0: cut it at tile boundaries
  int tiles_n;      // output tiles along the channels; tile = tt * tiles_n + tn
  int64_t total;    // tiles * (K / 128)
  float* ws_part;   // [2 * gridDim.x][BT/2 tokens][128 channels] partial tiles
  int* ws_count;    // [tiles] contributors that have stored their partial; zero between launches
};

// Block that owns global K-block index g when `total` indices are cut into G ranges
// [floor(c*total/G), floor((c+1)*total/G)).
__device__ __forceinline__ int owner_of(int64_t g, int64_t total, int G) { return (int)(((g + 1) * G + total - 1) / total) - 1; }

template <int BT, int STAGES>
__global__ void __launch_bounds__(192) gemm_tmem_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                        TmemArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024 the swizzle needs
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int STAGE_BYTES = BN * BK + BT * BK;
  constexpr int ACC_COLS = BT < 32 ? 32 : BT;
  constexpr int TMEM_COLS = 2 * ACC_COLS;  // two accumulators; 64..512, a power of two
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag, last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = a.K / BK;
  const int G = gridDim.x, c = blockIdx.x;
  const int64_t ntiles = a.total / nkb;
  const int64_t my_begin = a.stream_k ? (int64_t)c * a.total / G : ((int64_t)c * ntiles / G) * nkb;
  const int64_t my_end = a.stream_k ? (int64_t)(c + 1) * a.total / G : ((int64_t)(c + 1) * ntiles / G) * nkb;
  const int n_my = (int)(my_end - my_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int s = 0; s < 2; s++) { mbar_init(smem_u32(&bar_acc_full[s]), 1); mbar_init(smem_u32(&bar_acc_empty[s]), 128); }
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
      auto coords = [&](int it, int* kx, int* wy, int* xy) {
        int64_t g = my_begin + it;
        int tile = (int)(g / nkb), kb = (int)(g - (int64_t)tile * nkb);
        *kx = kb * BK;
        *wy = (tile % a.tiles_n) * BN;
        *xy = (tile / a.tiles_n) * BT;
      };
      // The weights are constants: their loads for the first ring of stages are issued before the
      // dependency wait, so they stream from HBM while the preceding kernel is still running.
      const int npre = n_my < STAGES ? n_my : STAGES;
      if (!a.prefetch) pdl_wait();
      for (int it = 0; it < npre; it++) {
        int kx, wy, xy;
        coords(it, &kx, &wy, &xy);
        uint32_t full = smem_u32(&bar_full[it]);
        mbar_expect_tx(full, STAGE_BYTES);
        tma_load_2d(smem_u32(smem + (size_t)it * STAGE_BYTES), &map_w, kx, wy, full);
      }
      pdl_wait();
      for (int it = 0; it < npre; it++) {
        int kx, wy, xy;
        coords(it, &kx, &wy, &xy);
        tma_load_2d(smem_u32(smem + (size_t)it * STAGE_BYTES) + BN * BK, &map_x, kx, xy, smem_u32(&bar_full[it]));
      }
      for (int it = npre; it < n_my; it++) {
        int s = it % STAGES;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ((it / STAGES) & 1) ^ 1)) { set_status(a.status, 1); abort_flag = 1; break; }
        if (*(volatile int*)&abort_flag) break;
        int kx, wy, xy;
        coords(it, &kx, &wy, &xy);
        uint32_t full = smem_u32(&bar_full[s]);
        uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        mbar_expect_tx(full, STAGE_BYTES);
        tma_load_2d(dst, &map_w, kx, wy, full);
        tma_load_2d(dst + BN * BK, &map_x, kx, xy, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D = F32 (bits 4-5 = 1), A = B = E4M3 (0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
      // The operand tiles cannot arrive before the producer's dependency wait has returned; waiting for the same
      // dependency here keeps the bounded waits below for progress inside this kernel (a predecessor that itself
      // waits for another rank may take longer than any of them).
      pdl_wait();
      int seg = -1;  // segment = run of K blocks of one tile inside this block's range
      for (int it = 0; it < n_my; it++) {
        const int kb = (int)((my_begin + it) % nkb);
        const bool seg_first = it == 0 || kb == 0;
        const bool seg_last = it == n_my - 1 || kb == nkb - 1;
        if (seg_first) {
          seg++;
          // the epilogue must have drained this accumulator (it was used two segments ago)
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
        for (int k = 0; k < BK / UMMA_K; k++) {
          // +32 bytes of K inside the swizzle atom = +2 in the (address >> 4) field
          tc_mma_f8(acc, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, (!seg_first || k) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));  // stage is free once these MMAs have read it
        if (seg_last) tc_commit(smem_u32(&bar_acc_full[seg & 1]));  // accumulator complete
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes [32*(w%4), +32)
    const int lg = warp & 3;
    const int ch = lg * 32 + lane;  // channel within the tile
    pdl_wait();  // the scales, the workspace and the output buffers belong to the dependency chain
    int seg = -1;
    int it = 0;
    while (it < n_my) {
      const int64_t g0 = my_begin + it;
      const int tile = (int)(g0 / nkb), kb0 = (int)(g0 - (int64_t)tile * nkb);
      const int len = min(nkb - kb0, n_my - it);
      seg++;
      it += len;
      bool bad = !mbar_wait(smem_u32(&bar_acc_full[seg & 1]), (seg >> 1) & 1);
      if (bad && lane == 0) set_status(a.status, 3);
      if (epi_any(bad || *(volatile int*)&abort_flag)) break;
      tc_fence_after();
      const uint32_t acc = tmem + (uint32_t)((seg & 1) * ACC_COLS) + ((uint32_t)(lg * 32) << 16);
      const int n = (tile % a.tiles_n) * BN + ch;
      const int t0 = (tile / a.tiles_n) * BT;
      const bool whole = len == nkb;
      const float swn = n < a.N ? a.sw[n] : 0.f;
      auto finish = [&](int tok, float v) {
        if (tok < a.M && n < a.N) {
          float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), swn);
          if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
          else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
        }
      };
      // a block has at most two cut tiles: its first segment (slot 2c) and its last one (slot 2c+1)
      float* my_part = a.ws_part + (size_t)(2 * c + (seg == 0 ? 0 : 1)) * (BT / 2) * BN;
#pragma unroll 1
      for (int grp = 0; grp < BT / 16; grp++) {
        uint32_t r[16];
        tc_ld16(acc + (uint32_t)(grp * 16), r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float v = __fadd_rn(__uint_as_float(r[j]), __fmul_rn(0.0625f, __uint_as_float(r[8 + j])));
          if (whole) finish(((t0 + grp * 16) >> 1) + j, v);  // operand rows 16g.. hold tokens 8g..
          else my_part[(size_t)(grp * 8 + j) * BN + ch] = v;
        }
      }
      // the accumulator is drained: hand it back to the MMA warp
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_acc_empty[seg & 1]));
      if (!whole) {
        // the last contributor of the tile adds the partial tiles in contributor order and finishes it
        const int64_t tg0 = (int64_t)tile * nkb;
        const int c_first = owner_of(tg0, a.total, G), c_last = owner_of(tg0 + nkb - 1, a.total, G);
        __threadfence();
        epi_bar();
        if (warp == 2 && lane == 0) {
          int old = atomicAdd(&a.ws_count[tile], 1);
          int last = old == c_last - c_first;
          if (last) a.ws_count[tile] = 0;  // ready for the next launch
          last_flag = last;
        }
        epi_bar();
        if (last_flag) {
          __threadfence();
          // 32 tokens at a time: all loads of one contributor are independent and in flight together
          constexpr int TCH = BT / 2 < 32 ? BT / 2 : 32;
#pragma unroll 1
          for (int tk0 = 0; tk0 < BT / 2; tk0 += TCH) {
            float v[TCH];
#pragma unroll
            for (int u = 0; u < TCH; u++) v[u] = 0.f;
            for (int cc = c_first; cc <= c_last; cc++) {
              // contributor cc starts inside this tile -> its first segment (slot 2cc), else its last one
              const int64_t cb = (int64_t)cc * a.total / G;
              const float* p = a.ws_part + (size_t)(2 * cc + (cb >= tg0 ? 0 : 1)) * (BT / 2) * BN + (size_t)tk0 * BN + ch;
#pragma unroll
              for (int u = 0; u < TCH; u++) v[u] += __ldcg(p + (size_t)u * BN);
            }
#pragma unroll
            for (int u = 0; u < TCH; u++) finish((t0 >> 1) + tk0 + u, v[u]);
          }
        }
        epi_bar();  // last_flag is reused by the next segment
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
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

// Stream-K workspace of a context: tile counters (zero between launches) then partial tiles.
int gemm_workspace(strictb200_ctx* ctx, size_t count_bytes, size_t part_bytes, int** count, float** part) {
  count_bytes = (count_bytes + 255) & ~(size_t)255;
  if (count_bytes > ctx->gemm_count_bytes || part_bytes > ctx->gemm_part_bytes) {
    SB_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->ws_generation++;
    if (ctx->gemm_ws) SB_CUDA(cudaFree(ctx->gemm_ws));
    ctx->gemm_ws = nullptr;
    size_t cb = count_bytes > ctx->gemm_count_bytes ? count_bytes * 2 : ctx->gemm_count_bytes;
    size_t pb = part_bytes > ctx->gemm_part_bytes ? part_bytes : ctx->gemm_part_bytes;
    ctx->gemm_count_bytes = ctx->gemm_part_bytes = 0;
    SB_CUDA(cudaMalloc(&ctx->gemm_ws, cb + pb));
    SB_CUDA(cudaMemsetAsync(ctx->gemm_ws, 0, cb, ctx->stream));
    ctx->gemm_count_bytes = cb;
    ctx->gemm_part_bytes = pb;
  }
  *count = (int*)ctx->gemm_ws;
  *part = (float*)((char*)ctx->gemm_ws + ctx->gemm_count_bytes);
  return STRICTB200_OK;
}

template <int BT, int STAGES>
int launch(strictb200_ctx* ctx, const GemmArgs& g, TmemArgs ta) {
  constexpr int STAGE_BYTES = BN * BK + BT * BK;
  size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;  // + slack for the 1024-byte round-up
  static SbDeviceOnce once;  // one per instantiation
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(gemm_tmem_kernel<BT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  CUtensorMap mw, mx;
  SB_TRY(make_map(&mw, g.wq, g.N, g.K, g.ldw, BN));
  SB_TRY(make_map(&mx, g.xq, ta.Mq, g.K, g.ldx, BT));
  const int64_t tiles_n = (g.N + BN - 1) / BN, tiles_t = (ta.Mq + BT - 1) / BT, tiles = tiles_n * tiles_t;
  if (tiles > INT32_MAX / 2) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: too many output tiles");
  ta.tiles_n = (int)tiles_n;
  ta.total = tiles * (g.K / BK);
  ta.stream_k = tiles < ctx->sm_count;
  int64_t cap = ta.stream_k ? ta.total : tiles;
  int64_t grid = ctx->sm_count < cap ? ctx->sm_count : cap;  // one persistent block per SM
  SB_TRY(gemm_workspace(ctx, (size_t)tiles * sizeof(int), (size_t)2 * grid * (BT / 2) * BN * sizeof(float), &ta.ws_count, &ta.ws_part));
  SB_CUDA(sb_launch(ctx, gemm_tmem_kernel<BT, STAGES>, dim3((unsigned)grid), dim3(192), smem, mw, mx, ta));
  ctx->launches++;
  return STRICTB200_OK;
}

}  // namespace

int k_gemm_fp8_tmem_split(strictb200_ctx* ctx, const GemmArgs& g);  // gemm_tmem_split.cu
int k_gemm_fp8_tmem_pair(strictb200_ctx* ctx, const GemmArgs& g);   // gemm_tmem_pair.cu

int k_gemm_fp8_tmem(strictb200_ctx* ctx, const GemmArgs& g) {
  if (g.K % BK) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "tensor-memory GEMM needs K to be a multiple of 128");
  if (sb_qrows(g.M) <= 256) return k_gemm_fp8_tmem_split(ctx, g);  // one tile of tokens: one tile per block + K splits
  if (g.splits != 1 || g.raw) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "the persistent tensor-memory GEMM produces complete outputs");
  if (((uintptr_t)g.xq | (uintptr_t)g.wq | (uintptr_t)g.ldx | (uintptr_t)g.ldw) & 15)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: operands and row strides must be 16-byte aligned");
  // many tokens: two SMs per 256 x 256 tile (half the operand bytes per flop through each SM)
  if (ctx->opt.gemm_pair && g.N >= 256 && ctx->sm_count >= 2) return k_gemm_fp8_tmem_pair(ctx, g);
  SB_TRY(get_encode());
  const int prefetch = ctx->opt.prefetch;
  TmemArgs ta{};
  ta.M = (int)g.M; ta.Mq = (int)sb_qrows(g.M); ta.N = (int)g.N; ta.K = (int)g.K;
  ta.sx = g.sx; ta.sw = g.sw; ta.out = g.out; ta.out_f32 = g.out_f32; ta.status = ctx->d_status; ta.prefetch = prefetch;
  return launch<256, 4>(ctx, g, ta);  // 128 x 256 tiles, 4 stages x 48 KB, two 256-column accumulators
}
