// bf16-activation x int8-weight linear layer on the integer tensor cores:
// Y[M,N] = ((X . Wq^T) * sx[M]) * sw[N] with Wq signed 8-bit integers, one fp32 scale per output
// channel (sw = absmax / 127), and the bf16 activations carried as two int8 terms per element,
// x ~ sx * (128 * hi + lo) with sx a power of two chosen per token so that |x| / sx <= 16256
// (hi in [-127, 127], lo in [-64, 63]: a 15-bit fixed-point value per element, exact wherever
// |x| / sx >= 128, which covers every element within a factor 63 of the row's largest). No weight is dequantised in the kernel: the
// MMA (tcgen05 kind::i8, gemm_tmem_split.cu) runs over the hi rows and the lo rows with exact
// 32-bit integer sums, and the epilogue forms 128 * sum_hi + sum_lo in 64-bit integers before the
// one conversion to fp32. Every intermediate is an exact integer, so the result is the same bit
// pattern for every K split and every summation order, and equals the CPU restatement exactly.
// The split-activation buffer has the layout of the FP8 path: tokens in groups of 8, 8 hi rows
// then 8 lo rows of width K.
#include "common.cuh"

int k_gemm_fp8_tmem_split(strictb200_ctx* ctx, const GemmArgs& g);  // gemm_tmem_split.cu

namespace {

constexpr int QT = 256;

__device__ __forceinline__ float block_absmax(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = 0.f;
  for (int i = 0; i < QT / 32; i++) m = fmaxf(m, red[i]);
  __syncthreads();
  return m;
}

// Smallest power of two s with absmax / s <= 16256 (= 127 * 128); 1 for a row of zeros.
__device__ __forceinline__ float int8_row_scale(float absmax) {
  if (!(absmax > 0.f)) return 1.f;
  int e;
  const float m = frexpf(absmax, &e);  // absmax = m * 2^e, m in [0.5, 1)
  return ldexpf(1.f, m <= 0.9921875f ? e - 14 : e - 13);
}

// One block per token row.
__global__ void __launch_bounds__(QT) quantize_rows_int8_kernel(const bf16* __restrict__ x, int64_t K, int8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float red[QT / 32];
  const int64_t row = blockIdx.x;
  const bf16* xr = x + row * K;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += QT) amax = fmaxf(amax, fabsf(__bfloat162float(xr[k])));
  amax = block_absmax(amax, red);
  const float s = int8_row_scale(amax), inv = 1.f / s;  // a power of two: the division and the product below are exact
  if (threadIdx.x == 0) scale[row] = s;
  int8_t* hi = q + ((row >> 3) * 16 + (row & 7)) * K;
  int8_t* lo = hi + 8 * K;
  for (int64_t k = threadIdx.x; k < K; k += QT) {
    const int v = __float2int_rn(__fmul_rn(__bfloat162float(xr[k]), inv));
    const int h = (v + 64) >> 7;
    hi[k] = (int8_t)h;
    lo[k] = (int8_t)(v - (h << 7));
  }
}
// Rows of the last group that hold no token are zeroed, so the MMA reads defined bytes.
__global__ void zero_pad_rows_kernel(int8_t* __restrict__ q, int64_t M, int64_t K) {
  const int64_t pad = (8 - (M & 7)) & 7, g = M >> 3;
  const int64_t total = pad * 2 * K, step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t r = i / K, k = i - r * K;  // r in [0, 2*pad): hi pads then lo pads
    const int64_t slot = (M & 7) + (r % pad) + (r / pad) * 8;
    q[(g * 16 + slot) * K + k] = 0;
  }
}

// One block per output channel: sw = absmax / 127 (1 for a row of zeros), q = round-to-nearest-even(w / sw) clamped to [-127, 127].
__global__ void __launch_bounds__(QT) quantize_weights_int8_kernel(const float* __restrict__ w, int64_t K, int8_t* __restrict__ q, float* __restrict__ sw) {
  __shared__ float red[QT / 32];
  const int64_t row = blockIdx.x;
  const float* wr = w + row * K;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += QT) amax = fmaxf(amax, fabsf(wr[k]));
  amax = block_absmax(amax, red);
  const float s = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
  if (threadIdx.x == 0) sw[row] = s;
  for (int64_t k = threadIdx.x; k < K; k += QT) {
    int v = __float2int_rn(__fdiv_rn(wr[k], s));
    v = v > 127 ? 127 : (v < -127 ? -127 : v);
    q[row * K + k] = (int8_t)v;
  }
}

// Sum of the K splits' integer partials, [split][hi, lo][M, N], joined and scaled.
__global__ void finish_int8_kernel(const int32_t* __restrict__ part, int splits, int64_t M, int64_t N, const float* __restrict__ sx,
                                   const float* __restrict__ sw, bf16* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  const int64_t total = M * N, step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    int64_t hi = 0, lo = 0;
    for (int s = 0; s < splits; s++) {
      hi += part[((int64_t)s * 2 + 0) * total + i];
      lo += part[((int64_t)s * 2 + 1) * total + i];
    }
    const int64_t m = i / N, n = i - m * N;
    y[i] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(__ll2float_rn(hi * 128 + lo), sx[m]), sw[n]));
  }
}

}  // namespace

int k_quantize_rows_int8(strictb200_ctx* ctx, const bf16* x, int64_t M, int64_t K, int8_t* q, float* scale) {
  quantize_rows_int8_kernel<<<(unsigned)M, QT, 0, ctx->stream>>>(x, K, q, scale);
  SB_LAUNCHED(ctx);
  if (M & 7) {
    zero_pad_rows_kernel<<<64, 256, 0, ctx->stream>>>(q, M, K);
    SB_LAUNCHED(ctx);
  }
  return STRICTB200_OK;
}

int k_gemm_int8w(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const int8_t* xq, const float* sx, const int8_t* wq, const float* sw, bf16* y,
                 int splits, int32_t* part) {
  GemmArgs g;
  g.M = M; g.N = N; g.K = K;
  g.xq = (const uint8_t*)xq; g.ldx = K; g.sx = sx;
  g.wq = (const uint8_t*)wq; g.ldw = K; g.sw = sw;
  g.out = y; g.out_f32 = 0; g.part = (float*)part; g.splits = splits; g.raw = 0; g.kernel = 3; g.i8 = 1;
  SB_TRY(k_gemm_fp8_tmem_split(ctx, g));
  if (splits > 1) {
    const int64_t total = M * N;
    int64_t blocks = (total + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    SB_CUDA(sb_launch(ctx, finish_int8_kernel, dim3((unsigned)(blocks > cap ? cap : blocks)), dim3(256), 0, (const int32_t*)part, splits, M, N, sx, sw, y));
    ctx->launches++;
  }
  return STRICTB200_OK;
}

extern "C" {

int strictb200_quantize_weights_int8(strictb200_ctx* ctx, const float* d_w, int64_t N, int64_t K, int8_t* d_wq, float* d_sw) {
  SB_ENTER(ctx);
  SB_REQUIRE(N >= 0 && K > 0 && N <= INT32_MAX, "bad shape");
  if (!N) return STRICTB200_OK;
  SB_REQUIRE(d_w && d_wq && d_sw, "null pointer");
  quantize_weights_int8_kernel<<<(unsigned)N, QT, 0, ctx->stream>>>(d_w, K, d_wq, d_sw);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

int strictb200_quantize_rows_int8(strictb200_ctx* ctx, const uint16_t* d_x_bf16, int64_t M, int64_t K, int8_t* d_split, float* d_scale) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && K > 0 && M <= INT32_MAX, "bad shape");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(d_x_bf16 && d_split && d_scale, "null pointer");
  return k_quantize_rows_int8(ctx, (const bf16*)d_x_bf16, M, K, d_split, d_scale);
}

int strictb200_gemm_int8(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const int8_t* d_split, const float* d_sx, const int8_t* d_wq,
                         const float* d_sw, uint16_t* d_y_bf16) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 128 == 0 && N % 16 == 0, "bad shape (K must be a multiple of 128, N of 16)");
  SB_REQUIRE(K <= 131072 && M <= INT32_MAX && N <= INT32_MAX, "K is limited to 131072 (exact 32-bit sums), M and N to 2^31 - 1");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(d_split && d_sx && d_wq && d_sw && d_y_bf16, "null pointer");
  SB_REQUIRE((((uintptr_t)d_wq | (uintptr_t)d_split) & 15) == 0, "the operands must be 16-byte aligned");
  const int splits = sb_gemm_pick_splits(ctx, M, N, K);
  void* ws = nullptr;
  if (splits > 1) SB_TRY(sb_ws(ctx, (size_t)splits * 2 * M * N * 4, &ws));
  return k_gemm_int8w(ctx, M, N, K, d_split, d_sx, d_wq, d_sw, (bf16*)d_y_bf16, splits, (int32_t*)ws);
}

int strictb200_gemm_int8w(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* d_x_bf16, const int8_t* d_wq, const float* d_sw,
                          uint16_t* d_y_bf16) {
  SB_ENTER(ctx);
  SB_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 128 == 0 && N % 16 == 0, "bad shape (K must be a multiple of 128, N of 16)");
  // 127 * 127 * K must stay below 2^31: the 32-bit accumulators hold the hi and the lo sums exactly
  SB_REQUIRE(K <= 131072 && M <= INT32_MAX && N <= INT32_MAX, "K is limited to 131072 (exact 32-bit sums), M and N to 2^31 - 1");
  if (!M) return STRICTB200_OK;
  SB_REQUIRE(d_x_bf16 && d_wq && d_sw && d_y_bf16, "null pointer");
  SB_REQUIRE(((uintptr_t)d_wq & 15) == 0, "the weights must be 16-byte aligned");
  const int splits = sb_gemm_pick_splits(ctx, M, N, K);
  const size_t qbytes = ((size_t)sb_qrows(M) * K + 255) & ~(size_t)255, sbytes = ((size_t)M * 4 + 255) & ~(size_t)255;
  const size_t pbytes = splits > 1 ? (size_t)splits * 2 * M * N * 4 : 0;
  void* ws;
  SB_TRY(sb_ws(ctx, qbytes + sbytes + pbytes, &ws));
  int8_t* xq = (int8_t*)ws;
  float* sx = (float*)((char*)ws + qbytes);
  int32_t* part = (int32_t*)((char*)ws + qbytes + sbytes);
  SB_TRY(k_quantize_rows_int8(ctx, (const bf16*)d_x_bf16, M, K, xq, sx));
  return k_gemm_int8w(ctx, M, N, K, xq, sx, d_wq, d_sw, (bf16*)d_y_bf16, splits, part);
}

}  // extern "C"
