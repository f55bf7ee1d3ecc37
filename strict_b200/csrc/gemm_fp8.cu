// bf16-activation x E4M3-weight GEMM on the FP8 tensor cores, Y[M,N] = ((X . Wq^T) * sx[M]) * sw[N],
// fp32 accumulation. The bf16 activations arrive as two E4M3 terms, X = sx*(hi + lo/16) with sx
// a power of two (norm.cu), laid out in groups of 8 hi rows + 8 lo rows: the MMA runs over
// 2M operand rows and the epilogue adds acc_hi + acc_lo/16, so every product is exact and no
// weight is ever dequantised in the kernel.
//
// Three kernels, chosen by shape:
//  * skinny (M <= 32, decode): an HBM stream over the weights. Each warp owns 16 output
//    channels and walks K with 128-bit loads straight from global memory into mma.sync
//    m16n8k32 A-fragments (weights are the A operand, tokens the B operand, so no row of
//    the 16x32 tile is padding); the token block is staged once per K-chunk in shared memory.
//    K can be split across blocks; raw fp32 partial accumulators are then reduced by the
//    row-wise consumer kernel (norm.cu / rope.cu) that also applies the scales.
//  * mma.sync tiles (any M): 128x128 block tiles through a cp.async pipeline; the portable
//    fallback and the cross-check for
//  * tcgen05/TMEM tiles (gemm_tmem.cu): TMA-fed UMMA with the accumulator in tensor memory.
//
// The k index inside a 64-byte unit is permuted identically for both operands (lane t of a
// quad holds bytes [16t,16t+16) of the unit and feeds them to two consecutive MMAs), which is
// legal because a dot product does not depend on the order of its terms.
#include <cstdlib>

#include "common.cuh"

int k_gemm_fp8_tmem(strictb200_ctx* ctx, const GemmArgs& a);  // gemm_tmem.cu

namespace {

__device__ __forceinline__ void mma_e4m3(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

struct GemmDev {
  int M, Mq, N, K;  // Mq = 16*ceil(M/8) rows of the split activation buffer
  const uint8_t* xq;
  int64_t ldx;
  const float* sx;
  const uint8_t* wq;
  int64_t ldw;
  const float* sw;
  void* out;
  int out_f32;
  float* part;
  int splits;
  int raw;
};

// ------------------------------------------------------------------ skinny stream kernel
constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = SK_WARPS * 16;  // output channels per block
constexpr int SK_PF = 8;                // 64-byte units of weights in flight per thread

template <int NT>  // NT tiles of 8 operand rows = NT*4 tokens (hi tile, lo tile alternating)
__global__ void __launch_bounds__(SK_WARPS * 32) gemm_skinny_kernel(GemmDev a, int kc_max) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int Ks = a.K / a.splits;
  const int k_begin = blockIdx.y * Ks;
  const int n0 = blockIdx.x * SK_ROWS + warp * 16;
  const bool rows_ok = n0 < a.N;  // N % 16 == 0: a warp's 16 rows are all valid or all outside
  const int stride = (kc_max % 128 == 0) ? kc_max + 64 : kc_max;  // == 64 mod 128: rows g, g+1 hit disjoint banks
  const int MP = NT * 8;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[j][i] = 0.f;

  const uint8_t* w_lo = a.wq + (int64_t)(rows_ok ? n0 + g : 0) * a.ldw + k_begin + 16 * tig;
  const uint8_t* w_hi = w_lo + (rows_ok ? 8 * a.ldw : 0);
  const int nunits = Ks / 64;
  uint4 wa[SK_PF][2];
#pragma unroll
  for (int i = 0; i < SK_PF; i++)
    if (rows_ok && i < nunits) { wa[i][0] = ldg_stream(w_lo + 64 * i); wa[i][1] = ldg_stream(w_hi + 64 * i); }

  int u_base = 0;  // first unit of the current activation chunk
  for (int kc0 = 0; kc0 < Ks; kc0 += kc_max) {
    const int kc_len = min(kc_max, Ks - kc0);
    __syncthreads();
    // stage tokens [MP][kc_len] (zero rows beyond M)
    const int chunks_per_row = kc_len / 16;
    for (int c = threadIdx.x; c < MP * chunks_per_row; c += blockDim.x) {
      int r = c / chunks_per_row, cc = c - r * chunks_per_row;
      bool valid = r < a.Mq;
      const uint8_t* src = a.xq + (int64_t)(valid ? r : 0) * a.ldx + k_begin + kc0 + 16 * cc;
      cp_async16(smem + r * stride + 16 * cc, src, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (rows_ok) {
      const int cu = kc_len / 64;
      for (int u0 = 0; u0 < cu; u0 += SK_PF) {
#pragma unroll
        for (int i = 0; i < SK_PF; i++) {
          int u = u0 + i;
          if (u < cu) {
            uint4 lo = wa[i][0], hi = wa[i][1];
            int nxt = u_base + u + SK_PF;
            if (nxt < nunits) { wa[i][0] = ldg_stream(w_lo + 64 * nxt); wa[i][1] = ldg_stream(w_hi + 64 * nxt); }
            const uint8_t* bs = smem + g * stride + 64 * u + 16 * tig;
#pragma unroll
            for (int j = 0; j < NT; j++) {
              uint4 b = *(const uint4*)(bs + j * 8 * stride);
              mma_e4m3(acc[j], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
              mma_e4m3(acc[j], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
            }
          }
        }
      }
    }
    u_base += kc_len / 64;
  }
  if (!rows_ok) return;
  // epilogue. Tile pair (2jp, 2jp+1) = hi and lo rows of tokens 8jp..8jp+7.
  // acc[.][0]: (channel n0+g, token 8jp+2tig) [1]: token+1  [2],[3]: channel n0+g+8
  const bool raw = a.raw || a.splits > 1;
#pragma unroll
  for (int jp = 0; jp < NT / 2; jp++) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int tok = 8 * jp + 2 * tig + (i & 1);
      int n = n0 + g + ((i >> 1) << 3);
      if (tok < a.M) {
        float v = __fadd_rn(acc[2 * jp][i], __fmul_rn(0.0625f, acc[2 * jp + 1][i]));
        if (raw) {
          a.part[((int64_t)blockIdx.y * a.M + tok) * a.N + n] = v;
        } else {
          float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), a.sw[n]);
          if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
          else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

// The prefetch ring above indexes units per activation chunk; it relies on kc_max being a
// multiple of 64*SK_PF so that ring slot i always holds unit (u_base + u) with u % SK_PF == i.

// ------------------------------------------------------------------ mma.sync tile kernel
constexpr int TL_BN = 128, TL_BM = 128, TL_STAGES = 4;

__global__ void __launch_bounds__(256) gemm_tiles_kernel(GemmDev a) {
  extern __shared__ __align__(128) uint8_t smem[];
  // stage layout: W tile [128 rows][64 B] then X tile [128 operand rows = 64 tokens][64 B]; consecutive rows are
  // 64 B apart, so the two rows a quarter-warp reads form one conflict-free 128-byte line.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int wn = warp & 3, wm = warp >> 2;  // 4 warps along N (32 channels each), 2 along M (64 tokens each)
  const int n0 = blockIdx.x * TL_BN, m0 = blockIdx.y * TL_BM;
  const int Ks = a.K / a.splits, k_begin = blockIdx.z * Ks;
  const int nunits = Ks / 64;

  float acc[2][8][4];
#pragma unroll
  for (int i = 0; i < 2; i++)
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int k = 0; k < 4; k++) acc[i][j][k] = 0.f;

  auto load_stage = [&](int stage, int u) {
    uint8_t* ws = smem + stage * (TL_BN + TL_BM) * 64;
    uint8_t* xs = ws + TL_BN * 64;
#pragma unroll
    for (int it = 0; it < 2; it++) {
      int c = threadIdx.x + it * 256;  // 512 chunks of 16 B per operand
      int r = c >> 2, cc = c & 3;
      bool vw = n0 + r < a.N;
      cp_async16(ws + r * 64 + cc * 16, a.wq + (int64_t)(vw ? n0 + r : 0) * a.ldw + k_begin + u * 64 + cc * 16, vw);
      bool vx = m0 + r < a.Mq;
      cp_async16(xs + r * 64 + cc * 16, a.xq + (int64_t)(vx ? m0 + r : 0) * a.ldx + k_begin + u * 64 + cc * 16, vx);
    }
  };
#pragma unroll
  for (int s = 0; s < TL_STAGES - 1; s++) {
    if (s < nunits) load_stage(s, s);
    cp_async_commit();
  }
  for (int u = 0; u < nunits; u++) {
    cp_async_wait<TL_STAGES - 2>();
    __syncthreads();
    int nu = u + TL_STAGES - 1;
    if (nu < nunits) load_stage(nu % TL_STAGES, nu);
    cp_async_commit();
    const uint8_t* ws = smem + (u % TL_STAGES) * (TL_BN + TL_BM) * 64;
    const uint8_t* xs = ws + TL_BN * 64;
    uint4 af[2][2];
#pragma unroll
    for (int mi = 0; mi < 2; mi++) {
      af[mi][0] = *(const uint4*)(ws + (wn * 32 + mi * 16 + g) * 64 + 16 * tig);
      af[mi][1] = *(const uint4*)(ws + (wn * 32 + mi * 16 + g + 8) * 64 + 16 * tig);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      uint4 b = *(const uint4*)(xs + (wm * 64 + j * 8 + g) * 64 + 16 * tig);
#pragma unroll
      for (int mi = 0; mi < 2; mi++) {
        mma_e4m3(acc[mi][j], af[mi][0].x, af[mi][1].x, af[mi][0].y, af[mi][1].y, b.x, b.y);
        mma_e4m3(acc[mi][j], af[mi][0].z, af[mi][1].z, af[mi][0].w, af[mi][1].w, b.z, b.w);
      }
    }
  }
  const bool raw = a.raw || a.splits > 1;
#pragma unroll
  for (int mi = 0; mi < 2; mi++)
#pragma unroll
    for (int jp = 0; jp < 4; jp++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int tok = ((m0 + wm * 64 + 16 * jp) >> 1) + 2 * tig + (i & 1);  // operand rows 16g.. hold tokens 8g..
        int n = n0 + wn * 32 + mi * 16 + g + ((i >> 1) << 3);
        if (tok < a.M && n < a.N) {
          float v = __fadd_rn(acc[mi][2 * jp][i], __fmul_rn(0.0625f, acc[mi][2 * jp + 1][i]));
          if (raw) {
            a.part[((int64_t)blockIdx.z * a.M + tok) * a.N + n] = v;
          } else {
            float y = __fmul_rn(__fmul_rn(v, a.sx[tok]), a.sw[n]);
            if (a.out_f32) ((float*)a.out)[(int64_t)tok * a.N + n] = y;
            else ((bf16*)a.out)[(int64_t)tok * a.N + n] = __float2bfloat16_rn(y);
          }
        }
      }
}

template <int NT>
int launch_skinny(strictb200_ctx* ctx, const GemmDev& d) {
  const int MP = NT * 8;
  int Ks = d.K / d.splits;
  // activation chunk: a multiple of 64*SK_PF bytes of K, at most ~96 KB of shared memory
  int kc_max = (96 * 1024 / MP - 64) / (64 * SK_PF) * (64 * SK_PF);
  if (kc_max > Ks) kc_max = (Ks + 64 * SK_PF - 1) / (64 * SK_PF) * (64 * SK_PF);
  int stride = (kc_max % 128 == 0) ? kc_max + 64 : kc_max;
  size_t smem = (size_t)MP * stride;
  static SbDeviceOnce once;  // one per instantiation
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(gemm_skinny_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); }));
  dim3 grid((d.N + SK_ROWS - 1) / SK_ROWS, d.splits);
  gemm_skinny_kernel<NT><<<grid, SK_WARPS * 32, smem, ctx->stream>>>(d, kc_max);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

}  // namespace

// Number of K splits for a skinny GEMM so that the grid covers the SMs about twice.
int sb_gemm_pick_splits(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K) {
  if (M > 128 || K % 128) return 1;
  const int64_t tiles = (N + SK_ROWS - 1) / SK_ROWS, nkb = K / 128;
  if (M > 32) {
    // 33..128 tokens: one block per SM fits (its ring fills the shared memory); split K until the grid covers the GPU
    int64_t s = ctx->sm_count / tiles;
    if (s > nkb / 2) s = nkb / 2;
    return (int)(s < 1 ? 1 : (s > 8 ? 8 : s));
  }
  // About 1.6 blocks per SM (two blocks of this kernel fit an SM, so all of them are resident
  // at once and share its bandwidth) measured best on the decode shapes; more than 8 partial
  // results are not taken by the kernels that sum them.
  const int target = ctx->opt.split_target;
  const int64_t want = target ? target : (int64_t)ctx->sm_count * 13 / 8;
  int64_t s = (want + tiles - 1) / tiles;
  while (s > 1 && tiles * s > 2 * (int64_t)ctx->sm_count) s--;
  if (s > nkb / 2) s = nkb / 2;  // at least two k-blocks per split
  return (int)(s < 1 ? 1 : (s > 8 ? 8 : s));
}

int k_gemm_fp8(strictb200_ctx* ctx, const GemmArgs& g) {
  if (g.K % 64 || g.N % 16) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: K must be a multiple of 64 and N of 16");
  if (g.splits < 1) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: splits must be positive");
  if ((g.splits > 1 || g.raw) && !g.part) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: split-K needs a partial buffer");
  if (((uintptr_t)g.xq | (uintptr_t)g.wq | (uintptr_t)g.ldx | (uintptr_t)g.ldw) & 15)
    return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: operands and row strides must be 16-byte aligned");
  if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: dimension too large");
  int kernel = g.kernel;
  if (kernel == 0) kernel = 3;
  if (kernel == 3) {
    int st = k_gemm_fp8_tmem(ctx, g);
    if (st != STRICTB200_ERR_UNSUPPORTED || g.kernel == 3) return st;
    kernel = g.M <= 32 ? 1 : 2;  // shapes the tensor-memory kernel does not cover (K % 128 != 0)
  }
  if (g.K % (g.splits * 64)) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: K/splits must be a multiple of 64 for this kernel");
  GemmDev d{(int)g.M, (int)sb_qrows(g.M), (int)g.N, (int)g.K, g.xq, g.ldx, g.sx, g.wq, g.ldw, g.sw, g.out, g.out_f32, g.part, g.splits, g.raw};
  if (kernel == 1) {
    if (g.M > 32) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: the skinny kernel takes at most 32 rows");
    if (g.M <= 8) return launch_skinny<2>(ctx, d);
    if (g.M <= 16) return launch_skinny<4>(ctx, d);
    return launch_skinny<8>(ctx, d);
  }
  static SbDeviceOnce once;
  size_t smem = (size_t)TL_STAGES * (TL_BN + TL_BM) * 64;
  SB_CUDA(once.run(ctx->device, [&] { return cudaFuncSetAttribute(gemm_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
  dim3 grid((unsigned)((g.N + TL_BN - 1) / TL_BN), (unsigned)((d.Mq + TL_BM - 1) / TL_BM), g.splits);
  if (grid.y > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_fp8: M too large for the tile kernel");
  gemm_tiles_kernel<<<grid, 256, smem, ctx->stream>>>(d);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
