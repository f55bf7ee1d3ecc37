// Seeded synthetic-tensor generator on the device.
//
// Specification (integer arithmetic is exact; every floating operation is a single IEEE-754
// binary32 round-to-nearest operation written with an explicit intrinsic so the compiler can
// neither contract nor reorder it — the same bits come out of any conforming implementation):
//   mix64(z)      z=(z^(z>>30))*0xBF58476D1CE4E5B9; z=(z^(z>>27))*0x94D049BB133111EB; z^(z>>31)
//   key(seed,t)   mix64(mix64(seed+GOLD) ^ (t*0xD6E8FEB86659FD93)), GOLD = 0x9E3779B97F4A7C15
//   rand64(key,c) mix64(key + (c+1)*GOLD)
//   normal pair j: r = rand64(key,j); k = (low32(r)>>8)+1; b = high32(r);
//                  radius = sqrt(-2*(ln k - 24 ln 2)), ln by an atanh series on the mantissa;
//                  angle = (b>>29) eighth-turns + ((b>>5)&0xFFFFFF)/2^24 of one, sin/cos by
//                  Taylor polynomials on [0, pi/4] and octant symmetry;
//                  element 2j = radius*cos, element 2j+1 = radius*sin.
//   uniform int   (high32(rand64(key,i)) * range) >> 32
#include "common.cuh"

#define GOLD 0x9E3779B97F4A7C15ull

__host__ __device__ static inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
uint64_t sb_stream_key(uint64_t seed, uint64_t tensor) { return mix64(mix64(seed + GOLD) ^ (tensor * 0xD6E8FEB86659FD93ull)); }

__device__ __forceinline__ uint64_t rand64(uint64_t key, uint64_t ctr) { return mix64(key + (ctr + 1) * GOLD); }

__device__ __forceinline__ float gen_log_u(uint32_t k) {
  float f = __uint2float_rn(k);
  uint32_t b = __float_as_uint(f);
  int e = (int)(b >> 23) - 127;
  float m = __uint_as_float((b & 0x7FFFFFu) | 0x3F800000u);
  if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
  float t = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
  float t2 = __fmul_rn(t, t);
  float p = __fmaf_rn(t2, 0.111111111f, 0.142857143f);
  p = __fmaf_rn(t2, p, 0.2f);
  p = __fmaf_rn(t2, p, 0.333333343f);
  p = __fmaf_rn(t2, p, 1.0f);
  float lnm = __fmul_rn(__fadd_rn(t, t), p);
  return __fmaf_rn(__int2float_rn(e - 24), 0.693147182f, lnm);
}

__device__ __forceinline__ void gen_sincos(uint32_t oct, uint32_t frac, float* c_out, float* s_out) {
  uint32_t fr = (oct & 1u) ? (16777216u - frac) : frac;
  float a = __fmul_rn(__fmul_rn(__uint2float_rn(fr), 5.9604644775390625e-08f), 0.785398185f);
  float z = __fmul_rn(a, a);
  float ps = __fmaf_rn(z, 2.75573188e-06f, -1.98412701e-04f);
  ps = __fmaf_rn(z, ps, 8.33333377e-03f);
  ps = __fmaf_rn(z, ps, -1.66666672e-01f);
  ps = __fmaf_rn(z, ps, 1.0f);
  float s = __fmul_rn(a, ps);
  float pc = __fmaf_rn(z, -2.75573188e-07f, 2.48015876e-05f);
  pc = __fmaf_rn(z, pc, -1.38888892e-03f);
  pc = __fmaf_rn(z, pc, 4.16666679e-02f);
  pc = __fmaf_rn(z, pc, -0.5f);
  float c = __fmaf_rn(z, pc, 1.0f);
  float cq = (oct & 1u) ? s : c, sq = (oct & 1u) ? c : s;
  switch (oct >> 1) {
    case 0: *c_out = cq; *s_out = sq; break;
    case 1: *c_out = -sq; *s_out = cq; break;
    case 2: *c_out = -cq; *s_out = -sq; break;
    default: *c_out = sq; *s_out = -cq; break;
  }
}

__device__ __forceinline__ void normal_pair(uint64_t key, uint64_t j, float* z0, float* z1) {
  uint64_t r = rand64(key, j);
  uint32_t k = ((uint32_t)r >> 8) + 1u;
  uint32_t b = (uint32_t)(r >> 32);
  float rad = __fsqrt_rn(__fmul_rn(-2.0f, gen_log_u(k)));
  float c, s;
  gen_sincos(b >> 29, (b >> 5) & 0xFFFFFFu, &c, &s);
  *z0 = __fmul_rn(rad, c);
  *z1 = __fmul_rn(rad, s);
}

// Elements [first, first+count) of the stream; one thread per normal pair.
template <typename T>
__global__ void gen_normal_kernel(uint64_t key, int64_t first, int64_t count, float std_, T* out) {
  int64_t p0 = first >> 1;
  int64_t npairs = ((first + count + 1) >> 1) - p0;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < npairs; p += (int64_t)gridDim.x * blockDim.x) {
    float z0, z1;
    normal_pair(key, (uint64_t)(p0 + p), &z0, &z1);
    int64_t i0 = 2 * (p0 + p) - first;
    float v0 = __fmul_rn(std_, z0), v1 = __fmul_rn(std_, z1);
    if (i0 >= 0 && i0 < count) out[i0] = (T)v0;
    if (i0 + 1 >= 0 && i0 + 1 < count) out[i0 + 1] = (T)v1;
  }
}

__global__ void gen_tokens_kernel(uint64_t key, int64_t count, uint32_t range, int32_t* out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = (int32_t)(((rand64(key, (uint64_t)i) >> 32) * (uint64_t)range) >> 32);
}

// One block per weight row: generate the whole row (row-major index r*K+k), reduce its
// absmax, quantise the requested column window. The row is regenerated in the second pass
// rather than staged, which keeps shared memory independent of K.
__global__ void gen_weight_e4m3_kernel(uint64_t key, int64_t row0, int64_t K, int64_t col0, int64_t cols, float std_, uint8_t* q,
                                       int64_t ldq, float* scale) {
  __shared__ float red[32];
  int64_t r = row0 + blockIdx.x;
  int64_t base = r * K;  // even or odd; pairs are aligned on even global indices
  float amax = 0.f;
  int64_t p_lo = base >> 1, p_hi = (base + K - 1) >> 1;
  for (int64_t p = p_lo + threadIdx.x; p <= p_hi; p += blockDim.x) {
    float z0, z1;
    normal_pair(key, (uint64_t)p, &z0, &z1);
    int64_t i0 = 2 * p;
    if (i0 >= base && i0 < base + K) amax = fmaxf(amax, fabsf(__fmul_rn(std_, z0)));
    if (i0 + 1 >= base && i0 + 1 < base + K) amax = fmaxf(amax, fabsf(__fmul_rn(std_, z1)));
  }
  amax = block_max(amax, red);
  float inv = 1.0f, sc = 1.0f;
  if (amax > 0.f) { inv = __fdiv_rn(448.0f, amax); sc = __fdiv_rn(amax, 448.0f); }
  if (threadIdx.x == 0) scale[blockIdx.x] = sc;
  int64_t w0 = base + col0, w1 = w0 + cols;
  uint8_t* qr = q + (int64_t)blockIdx.x * ldq;
  for (int64_t p = (w0 >> 1) + threadIdx.x; p <= ((w1 - 1) >> 1); p += blockDim.x) {
    float z0, z1;
    normal_pair(key, (uint64_t)p, &z0, &z1);
    uint32_t e = f32x2_to_e4m3x2(__fmul_rn(__fmul_rn(std_, z0), inv), __fmul_rn(__fmul_rn(std_, z1), inv));
    int64_t i0 = 2 * p;
    if (i0 >= w0 && i0 < w1) qr[i0 - w0] = (uint8_t)(e & 0xFF);
    if (i0 + 1 >= w0 && i0 + 1 < w1) qr[i0 + 1 - w0] = (uint8_t)(e >> 8);
  }
}

static int grid_for(strictb200_ctx* ctx, int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  int64_t cap = (int64_t)ctx->sm_count * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

int k_gen_normal_f32(strictb200_ctx* ctx, uint64_t key, int64_t first, int64_t count, float std_, float* out) {
  gen_normal_kernel<float><<<grid_for(ctx, count / 2 + 1, 256), 256, 0, ctx->stream>>>(key, first, count, std_, out);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_gen_normal_bf16(strictb200_ctx* ctx, uint64_t key, int64_t first, int64_t count, float std_, bf16* out) {
  gen_normal_kernel<bf16><<<grid_for(ctx, count / 2 + 1, 256), 256, 0, ctx->stream>>>(key, first, count, std_, out);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_gen_tokens(strictb200_ctx* ctx, uint64_t key, int64_t count, uint32_t range, int32_t* out) {
  gen_tokens_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>(key, count, range, out);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_gen_weight_e4m3(strictb200_ctx* ctx, uint64_t key, int64_t row0, int64_t rows, int64_t K, int64_t col0, int64_t cols, float std_,
                      uint8_t* q, int64_t ldq, float* scale) {
  const int64_t MAXG = 1 << 30;
  for (int64_t done = 0; done < rows; done += MAXG) {
    int64_t n = rows - done < MAXG ? rows - done : MAXG;
    gen_weight_e4m3_kernel<<<(unsigned)n, 256, 0, ctx->stream>>>(key, row0 + done, K, col0, cols, std_, q + done * ldq, ldq, scale + done);
    SB_LAUNCHED(ctx);
  }
  return STRICTB200_OK;
}
