// fp32 linear layer of the GPT-2 path: Y[M,N] = X[M,K] . W[N,K]^T + bias. Decode (M = 1) is
// a pure HBM stream over W; one warp (or 2-8 for a long row) per output channel, lanes split K with 128-bit loads,
// warp-shuffle reduction. Up to 8 token rows share one pass over a weight row. `accumulate`: 0
// stores the result, 1 adds it to Y (residual), 2 stores GELU(result) (the MLP's first layer).
#include "common.cuh"

namespace {
constexpr int F32_MT = 8;

constexpr int F32_PRE = 8;  // float4 of its weight row a lane fetches before the dependency wait (covers K <= 1024)

__global__ void __launch_bounds__(256) gemm_f32_kernel(int M, int N, int K, const float* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ bias, float* __restrict__ y, int accumulate, int ks) {
  // The block's 8 warps are 8/ks output channels x ks slices of K: a long row (K > 1024) is
  // walked by several warps at once so that every lane still has all its loads in flight in one
  // round trip; the slices' sums meet in shared memory and are added in slice order.
  __shared__ float part[8][F32_MT];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = 8 / ks, slice = warp % ks;
  const int n = blockIdx.x * rows + warp / ks;
  const int m0 = blockIdx.y * F32_MT;
  const bool live = n < N;
  const int nk4 = K / 4, per = (nk4 + ks - 1) / ks;
  const int k4_lo = slice * per, k4_hi = min(nk4, k4_lo + per);
  const float4* wr = (const float4*)(w + (int64_t)(live ? n : 0) * K);
  // the weights are constants: the head of the slice streams in while the previous kernel still runs
  // (streaming loads: a step reads its 0.5 GB of weights once each, and they should not push the
  // kernels' code and the activations out of L2)
  float4 wpre[F32_PRE];
#pragma unroll
  for (int i = 0; i < F32_PRE; i++)
    if (live && k4_lo + lane + 32 * i < k4_hi) wpre[i] = __ldcs(wr + k4_lo + lane + 32 * i);
  const float bn = bias && live ? bias[n] : 0.f;
  pdl_wait();
  float acc[F32_MT];
#pragma unroll
  for (int i = 0; i < F32_MT; i++) acc[i] = 0.f;
  const int mt = min(F32_MT, M - m0);
  auto fma_row = [&](int k4, const float4& wv) {
#pragma unroll
    for (int i = 0; i < F32_MT; i++) {
      if (i < mt) {
        float4 xv = *((const float4*)(x + (int64_t)(m0 + i) * K) + k4);
        acc[i] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
      }
    }
  };
  if (live) {
#pragma unroll
    for (int i = 0; i < F32_PRE; i++)
      if (k4_lo + lane + 32 * i < k4_hi) fma_row(k4_lo + lane + 32 * i, wpre[i]);
#pragma unroll 4
    for (int k4 = k4_lo + lane + 32 * F32_PRE; k4 < k4_hi; k4 += 32) fma_row(k4, __ldcs(wr + k4));
  }
#pragma unroll
  for (int i = 0; i < F32_MT; i++) {
    const float v = warp_sum(acc[i]);
    if (lane == 0) part[warp][i] = v;
  }
  __syncthreads();
  if (live && slice == 0 && lane < mt) {
    float v = 0.f;
    for (int s2 = 0; s2 < ks; s2++) v += part[warp + s2][lane];
    const int64_t o = (int64_t)(m0 + lane) * N + n;
    v += bn;
    y[o] = accumulate == 1 ? y[o] + v : accumulate == 2 ? sb_gelu_tanh(v) : v;
  }
}
}  // namespace

int k_gemm_f32(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const float* x, const float* w, const float* bias, float* y,
               int accumulate) {
  if (K % 4) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_f32: K must be a multiple of 4");
  int ks = 1;  // warps per output channel: slices of at most 1024 columns, as long as the grid stays small
  while (ks < 8 && K > 1024 * (int64_t)ks && (N * ks * 2 + 7) / 8 <= 8 * (int64_t)ctx->sm_count) ks *= 2;
  const int rows = 8 / ks;
  dim3 grid((unsigned)((N + rows - 1) / rows), (unsigned)((M + F32_MT - 1) / F32_MT));
  if (grid.y > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_f32: M too large");
  SB_CUDA(sb_launch(ctx, gemm_f32_kernel, grid, dim3(256), 0, (int)M, (int)N, (int)K, x, w, bias, y, accumulate, ks));
  ctx->launches++;
  return STRICTB200_OK;
}
