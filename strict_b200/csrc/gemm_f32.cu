// fp32 linear layer of the GPT-2 path: Y[M,N] = X[M,K] . W[N,K]^T + bias. Decode (M = 1) is
// a pure HBM stream over W; one warp per output channel, lanes split K with 128-bit loads,
// warp-shuffle reduction. Up to 8 token rows share one pass over a weight row.
#include "common.cuh"

namespace {
constexpr int F32_MT = 8;

__global__ void __launch_bounds__(256) gemm_f32_kernel(int M, int N, int K, const float* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ bias, float* __restrict__ y, int accumulate) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n = blockIdx.x * 8 + warp;
  int m0 = blockIdx.y * F32_MT;
  if (n >= N) return;
  float acc[F32_MT];
#pragma unroll
  for (int i = 0; i < F32_MT; i++) acc[i] = 0.f;
  const float4* wr = (const float4*)(w + (int64_t)n * K);
  int mt = min(F32_MT, M - m0);
  for (int k4 = lane; k4 < K / 4; k4 += 32) {
    float4 wv = __ldg(wr + k4);
#pragma unroll
    for (int i = 0; i < F32_MT; i++) {
      if (i < mt) {
        float4 xv = *((const float4*)(x + (int64_t)(m0 + i) * K) + k4);
        acc[i] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < F32_MT; i++) {
    float v = warp_sum(acc[i]);
    if (lane == 0 && i < mt) {
      int64_t o = (int64_t)(m0 + i) * N + n;
      v += bias ? bias[n] : 0.f;
      y[o] = accumulate ? y[o] + v : v;
    }
  }
}
}  // namespace

int k_gemm_f32(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const float* x, const float* w, const float* bias, float* y,
               int accumulate) {
  if (K % 4) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_f32: K must be a multiple of 4");
  dim3 grid((unsigned)((N + 7) / 8), (unsigned)((M + F32_MT - 1) / F32_MT));
  if (grid.y > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gemm_f32: M too large");
  gemm_f32_kernel<<<grid, 256, 0, ctx->stream>>>((int)M, (int)N, (int)K, x, w, bias, y, accumulate);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
