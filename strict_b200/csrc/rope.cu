// Per-head RMS norm of q and k, rotary embedding, and append of k/v to the cache, fused with
// the dequantising reduction of the qkv GEMM's split-K partials. One warp per (token row, head): a lane owns 4 of the 128 dims, the rotary partner (i, i+64) lives in lane^16.
#include <cmath>
#include <vector>

#include "common.cuh"

namespace {

struct RopeDev {
  const bf16* qkv;
  const float* qkv_f32;
  const float* part;
  int splits;
  const float* sx;
  const float* sw;
  const int32_t* seq;
  const int32_t* pos;
  const int32_t* lens;
  const float* cos_t;
  const float* sin_t;
  const float* qgain;
  const float* kgain;
  float eps;
  int Hq, Hkv, maxlen, max_pos;
  bf16* q_out;
  bf16* kcache;
  bf16* vcache;
};

__global__ void __launch_bounds__(256) rope_kernel(RopeDev a, int64_t T) {
  constexpr int D = 128;
  pdl_trigger();
  pdl_wait();
  int64_t t = blockIdx.x;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int h_first = blockIdx.y * nwarps + warp, h_step = gridDim.y * nwarps;
  int b = a.seq ? a.seq[t] : (int)t;
  int p = a.pos ? a.pos[t] : a.lens[b];
  if (p < 0 || p >= a.maxlen || p >= a.max_pos) return;  // host validates; never index outside the cache
  int nheads = a.Hq + 2 * a.Hkv;
  int64_t nqkv = (int64_t)nheads * D;
  for (int h = h_first; h < nheads; h += h_step) {
    int64_t col = (int64_t)h * D + lane * 4;
    float x[4];
    if (a.part) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int s = 0; s < a.splits; s++) {
        float4 v = *(const float4*)(a.part + ((int64_t)s * T + t) * nqkv + col);
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      }
      float sxr = a.sx[t];
      float4 w = *(const float4*)(a.sw + col);
      x[0] = __fmul_rn(__fmul_rn(acc[0], sxr), w.x);
      x[1] = __fmul_rn(__fmul_rn(acc[1], sxr), w.y);
      x[2] = __fmul_rn(__fmul_rn(acc[2], sxr), w.z);
      x[3] = __fmul_rn(__fmul_rn(acc[3], sxr), w.w);
    } else if (a.qkv_f32) {
      float4 v = *(const float4*)(a.qkv_f32 + t * nqkv + col);
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
      uint2 u = *(const uint2*)(a.qkv + t * nqkv + col);
      x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xFFFF0000u);
      x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xFFFF0000u);
    }
    bool is_v = h >= a.Hq + a.Hkv;
    float o[4];
    if (!is_v) {
      const float* g = h < a.Hq ? a.qgain : a.kgain;
      float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
      float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)D), a.eps)));
      float4 gv = *(const float4*)(g + lane * 4);
      float n[4] = {__fmul_rn(__fmul_rn(x[0], r), gv.x), __fmul_rn(__fmul_rn(x[1], r), gv.y), __fmul_rn(__fmul_rn(x[2], r), gv.z),
                    __fmul_rn(__fmul_rn(x[3], r), gv.w)};
      int i0 = (lane & 15) * 4;
      float4 c = *(const float4*)(a.cos_t + (int64_t)p * (D / 2) + i0);
      float4 s = *(const float4*)(a.sin_t + (int64_t)p * (D / 2) + i0);
      float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float other = __shfl_xor_sync(0xffffffffu, n[j], 16);
        // first half: n_i*c - n_{i+64}*s ; second half: n_{i+64}*c + n_i*s
        o[j] = lane < 16 ? __fsub_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j]))
                         : __fadd_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) o[j] = x[j];
    }
    uint2 w;
    w.x = f32_to_bf16_bits(o[0]) | (f32_to_bf16_bits(o[1]) << 16);
    w.y = f32_to_bf16_bits(o[2]) | (f32_to_bf16_bits(o[3]) << 16);
    if (h < a.Hq) {
      *(uint2*)(a.q_out + (t * a.Hq + h) * D + lane * 4) = w;
    } else {
      int hk = is_v ? h - a.Hq - a.Hkv : h - a.Hq;
      bf16* cache = is_v ? a.vcache : a.kcache;
      *(uint2*)(cache + (((int64_t)b * a.Hkv + hk) * a.maxlen + p) * D + lane * 4) = w;
    }
  }
}

// The decode-step shape of the above: token t is sequence t at position lens[t], the input is
// at most 8 split-K partials or the finished fp32 projection, one head per warp. The constants (weight scales, gains) are
// fetched before the dependency wait and every load of the head is issued in one batch after
// it; the arithmetic is that of the kernel above, operation for operation.
__global__ void __launch_bounds__(256) rope_decode_kernel(RopeDev a, int64_t T) {
  constexpr int D = 128;
  SB_TRACE_BEGIN();
  pdl_trigger();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 8 + warp, nheads = a.Hq + 2 * a.Hkv;
  if (h >= nheads) return;
  const int64_t nqkv = (int64_t)nheads * D, col = (int64_t)h * D + lane * 4;
  const bool is_v = h >= a.Hq + a.Hkv;
  float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
  if (a.part) w = *(const float4*)(a.sw + col);
  float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!is_v) gv = *(const float4*)((h < a.Hq ? a.qgain : a.kgain) + lane * 4);
  pdl_wait();
  SB_TRACE_WAITED();
  const int p = a.lens[t];
  float4 v[8];
  float sxr = 1.f;
  if (a.part) {
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) v[s] = *(const float4*)(a.part + ((int64_t)s * T + t) * nqkv + col);
    sxr = a.sx[t];
  } else {
    v[0] = *(const float4*)(a.qkv_f32 + t * nqkv + col);
  }
  if (p < 0 || p >= a.maxlen || p >= a.max_pos) return;  // host validates; never index outside the cache
  float4 c = make_float4(0.f, 0.f, 0.f, 0.f), sn4 = c;
  if (!is_v) {
    const int i0 = (lane & 15) * 4;
    c = *(const float4*)(a.cos_t + (int64_t)p * (D / 2) + i0);
    sn4 = *(const float4*)(a.sin_t + (int64_t)p * (D / 2) + i0);
  }
  float x[4];
  if (a.part) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; s++)
      if (s < a.splits) { acc[0] += v[s].x; acc[1] += v[s].y; acc[2] += v[s].z; acc[3] += v[s].w; }
    x[0] = __fmul_rn(__fmul_rn(acc[0], sxr), w.x); x[1] = __fmul_rn(__fmul_rn(acc[1], sxr), w.y);
    x[2] = __fmul_rn(__fmul_rn(acc[2], sxr), w.z); x[3] = __fmul_rn(__fmul_rn(acc[3], sxr), w.w);
  } else {
    x[0] = v[0].x; x[1] = v[0].y; x[2] = v[0].z; x[3] = v[0].w;
  }
  float o[4];
  if (!is_v) {
    float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)D), a.eps)));
    float n[4] = {__fmul_rn(__fmul_rn(x[0], r), gv.x), __fmul_rn(__fmul_rn(x[1], r), gv.y), __fmul_rn(__fmul_rn(x[2], r), gv.z),
                  __fmul_rn(__fmul_rn(x[3], r), gv.w)};
    float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {sn4.x, sn4.y, sn4.z, sn4.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float other = __shfl_xor_sync(0xffffffffu, n[j], 16);
      o[j] = lane < 16 ? __fsub_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j]))
                       : __fadd_rn(__fmul_rn(n[j], cs[j]), __fmul_rn(other, sn[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) o[j] = x[j];
  }
  uint2 wv;
  wv.x = f32_to_bf16_bits(o[0]) | (f32_to_bf16_bits(o[1]) << 16);
  wv.y = f32_to_bf16_bits(o[2]) | (f32_to_bf16_bits(o[3]) << 16);
  if (h < a.Hq) {
    *(uint2*)(a.q_out + (t * a.Hq + h) * D + lane * 4) = wv;
  } else {
    const int hk = is_v ? h - a.Hq - a.Hkv : h - a.Hq;
    bf16* cache = is_v ? a.vcache : a.kcache;
    *(uint2*)(cache + ((t * a.Hkv + hk) * a.maxlen + p) * D + lane * 4) = wv;
  }
  SB_TRACE_END(SB_K_ROPE, 0);
}

}  // namespace

SB_TRACE_TU(rope)

int k_rope_qknorm_kvappend(strictb200_ctx* ctx, const RopeArgs& a, int64_t T) {
  if (a.D != 128) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "rope: head_dim must be 128");
  RopeDev v{a.qkv, a.qkv_f32, a.part, a.splits, a.sx, a.sw, a.seq, a.pos, a.lens, a.cos_t, a.sin_t, a.qgain, a.kgain,
            a.eps, a.Hq, a.Hkv, a.maxlen, a.max_pos, a.q_out, a.kcache, a.vcache};
  int nheads = a.Hq + 2 * a.Hkv;
  // few rows (decode): spread the heads of a row over several blocks, one head per warp
  dim3 grid((unsigned)T, T <= 256 ? (unsigned)((nheads + 7) / 8) : 1u);
  if (T <= 256 && ((a.part && a.splits <= 8) || (!a.part && a.qkv_f32)) && !a.seq && !a.pos) {
    SB_CUDA(sb_launch(ctx, rope_decode_kernel, grid, dim3(256), 0, v, T));
    ctx->launches++;
    return STRICTB200_OK;
  }
  SB_CUDA(sb_launch(ctx, rope_kernel, grid, dim3(256), 0, v, T));
  ctx->launches++;
  return STRICTB200_OK;
}

// cos/sin of pos * theta^(-2i/D), evaluated in double on the host and rounded to fp32: part of
// the model constants (like the weights), not of the per-token path.
int sb_rope_table(strictb200_ctx* ctx, int max_pos, int D, float theta, float** d_cos, float** d_sin) {
  int h = D / 2;
  std::vector<float> c((size_t)max_pos * h), s((size_t)max_pos * h);
  std::vector<double> inv(h);
  for (int i = 0; i < h; i++) inv[i] = std::pow((double)theta, -2.0 * (double)i / (double)D);
  for (int p = 0; p < max_pos; p++)
    for (int i = 0; i < h; i++) {
      double ang = (double)p * inv[i];
      c[(size_t)p * h + i] = (float)std::cos(ang);
      s[(size_t)p * h + i] = (float)std::sin(ang);
    }
  size_t bytes = c.size() * sizeof(float);
  SB_CUDA(cudaMalloc((void**)d_cos, bytes));
  SB_CUDA(cudaMalloc((void**)d_sin, bytes));
  SB_CUDA(cudaMemcpyAsync(*d_cos, c.data(), bytes, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaMemcpyAsync(*d_sin, s.data(), bytes, cudaMemcpyHostToDevice, ctx->stream));
  SB_CUDA(cudaStreamSynchronize(ctx->stream));
  return STRICTB200_OK;
}
