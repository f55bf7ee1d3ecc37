// Embedding gathers, greedy argmax and small index utilities.
#include "common.cuh"

namespace {

__global__ void embedding_bf16_kernel(const bf16* __restrict__ table, const int32_t* __restrict__ ids, int64_t d, int64_t vocab,
                                      bf16* __restrict__ out) {
  int64_t t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // host validates prompt ids; never index outside the table
  const uint4* src = (const uint4*)(table + id * d);
  uint4* dst = (uint4*)(out + t * d);
  for (int64_t i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void embedding_bf16_f32_kernel(const bf16* __restrict__ table, const int32_t* __restrict__ ids, int64_t d, int64_t vocab,
                                          float* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int64_t t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint2* src = (const uint2*)(table + id * d);
  float4* dst = (float4*)(out + t * d);
  for (int64_t i = threadIdx.x; i < d / 4; i += blockDim.x) {
    uint2 u = src[i];
    dst[i] = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                         __uint_as_float(u.y & 0xFFFF0000u));
  }
}

__global__ void embedding_f32_kernel(const float* __restrict__ wte, const float* __restrict__ wpe, const int32_t* __restrict__ ids,
                                     const int32_t* __restrict__ pos, const int32_t* __restrict__ lens, int64_t d, int64_t vocab, int max_pos,
                                     float* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int64_t t = blockIdx.x;
  int64_t id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  int p = pos ? pos[t] : lens[t];
  if (p < 0 || p >= max_pos) p = 0;
  for (int64_t i = threadIdx.x; i < d; i += blockDim.x) out[t * d + i] = __fadd_rn(wte[id * d + i], wpe[(int64_t)p * d + i]);
}

// One block per row; ties resolve to the lowest index (strict > while scanning upwards and
// an index comparison in the reductions).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ x, int64_t N, int64_t ldx, int32_t* __restrict__ out,
                                                      float* __restrict__ val_out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  int64_t row = blockIdx.x;
  const float* xr = x + row * ldx;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
    float v = xr[i];
    if (v > best || (v == best && (int)i < bi)) { best = v; bi = (int)i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -INFINITY;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (l == 0) {
      out[row] = bi == 0x7fffffff ? 0 : bi;
      if (val_out) val_out[row] = best;
    }
  }
}

__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ rows, int64_t row_vec, uint4* __restrict__ dst) {
  int64_t r = blockIdx.x;
  int64_t s = rows[r];
  for (int64_t i = threadIdx.x; i < row_vec; i += blockDim.x) dst[r * row_vec + i] = src[s * row_vec + i];
}
__global__ void add_i32_kernel(int32_t* x, const int32_t* inc, int32_t c, int64_t n) {
  pdl_trigger();
  pdl_wait();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += inc ? inc[i] : c;
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, int64_t n, bf16* __restrict__ y) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = __float2bfloat16_rn(x[i]);
}
__global__ void bf16_to_f32_kernel(const bf16* __restrict__ x, int64_t n, float* __restrict__ y) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = __bfloat162float(x[i]);
}
int sgrid(strictb200_ctx* ctx, int64_t n) {
  int64_t b = (n + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
}  // namespace

int k_embedding_bf16(strictb200_ctx* ctx, const bf16* table, const int32_t* ids, int64_t T, int64_t d, int64_t vocab, bf16* out) {
  if (d % 8) return sb_fail(STRICTB200_ERR_INVALID_ARG, "embedding: d must be a multiple of 8");
  embedding_bf16_kernel<<<(unsigned)T, 128, 0, ctx->stream>>>(table, ids, d, vocab, out);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_embedding_bf16_f32(strictb200_ctx* ctx, const bf16* table, const int32_t* ids, int64_t T, int64_t d, int64_t vocab, float* out) {
  if (d % 8) return sb_fail(STRICTB200_ERR_INVALID_ARG, "embedding: d must be a multiple of 8");
  SB_CUDA(sb_launch(ctx, embedding_bf16_f32_kernel, dim3((unsigned)T), dim3(128), 0, table, ids, d, vocab, out));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_embedding_f32(strictb200_ctx* ctx, const float* wte, const float* wpe, const int32_t* ids, const int32_t* pos, const int32_t* lens,
                    int64_t T, int64_t d, int64_t vocab, int max_pos, float* out) {
  SB_CUDA(sb_launch(ctx, embedding_f32_kernel, dim3((unsigned)T), dim3(256), 0, wte, wpe, ids, pos, lens, d, vocab, max_pos, out));
  ctx->launches++;
  return STRICTB200_OK;
}
// Two-stage pick for wide rows: blocks of 256 threads scan 4096-column chunks, then one block
// per row merges the chunk winners (chunks ascend, ties keep the lower index).
namespace {
constexpr int AM_CHUNK = 4096;
__global__ void __launch_bounds__(256) argmax_chunk_kernel(const float* __restrict__ x, int64_t N, int64_t ldx, float* __restrict__ cval,
                                                           int32_t* __restrict__ cidx, int nchunks) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_trigger();
  pdl_wait();
  int64_t row = blockIdx.y;
  int64_t c0 = (int64_t)blockIdx.x * AM_CHUNK, c1 = c0 + AM_CHUNK < N ? c0 + AM_CHUNK : N;
  const float* xr = x + row * ldx;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = c0 + threadIdx.x; i < c1; i += 256) {
    float v = xr[i];
    if (v > best) { best = v; bi = (int)i; }  // a thread's indices ascend: strict > keeps the lowest
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; k++)
      if (sv[k] > best || (sv[k] == best && si[k] < bi)) { best = sv[k]; bi = si[k]; }
    cval[row * nchunks + blockIdx.x] = best;
    cidx[row * nchunks + blockIdx.x] = bi;
  }
}
__global__ void argmax_merge_kernel(const float* __restrict__ cval, const int32_t* __restrict__ cidx, int nchunks, int32_t* __restrict__ out,
                                    float* __restrict__ val_out) {
  pdl_trigger();
  pdl_wait();
  int64_t row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int k = threadIdx.x; k < nchunks; k += 32) {
    float v = cval[row * nchunks + k];
    int i = cidx[row * nchunks + k];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (threadIdx.x == 0) {
    out[row] = bi == 0x7fffffff ? 0 : bi;
    if (val_out) val_out[row] = best;
  }
}
}  // namespace
size_t sb_argmax_scratch(int64_t M, int64_t N) { return (size_t)M * ((N + AM_CHUNK - 1) / AM_CHUNK) * 8; }
int k_argmax(strictb200_ctx* ctx, const float* x, int64_t M, int64_t N, int64_t ldx, int32_t* out, float* val_out, void* scratch) {
  if (!scratch || N <= 2 * AM_CHUNK) {
    argmax_kernel<<<(unsigned)M, 1024, 0, ctx->stream>>>(x, N, ldx, out, val_out);
    SB_LAUNCHED(ctx);
    return STRICTB200_OK;
  }
  int nchunks = (int)((N + AM_CHUNK - 1) / AM_CHUNK);
  float* cval = (float*)scratch;
  int32_t* cidx = (int32_t*)(cval + (size_t)M * nchunks);
  if (M > 65535) return sb_fail(STRICTB200_ERR_INVALID_ARG, "argmax: too many rows");
  SB_CUDA(sb_launch(ctx, argmax_chunk_kernel, dim3(nchunks, (unsigned)M), dim3(256), 0, x, N, ldx, cval, cidx, nchunks));
  ctx->launches++;
  SB_CUDA(sb_launch(ctx, argmax_merge_kernel, dim3((unsigned)M), dim3(32), 0, (const float*)cval, (const int32_t*)cidx, nchunks, out, val_out));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_gather_rows(strictb200_ctx* ctx, const void* src, const int32_t* rows, int64_t n_rows, int64_t row_bytes, void* dst) {
  if (row_bytes % 16) return sb_fail(STRICTB200_ERR_INVALID_ARG, "gather_rows: rows must be multiples of 16 bytes");
  gather_rows_kernel<<<(unsigned)n_rows, 128, 0, ctx->stream>>>((const uint4*)src, rows, row_bytes / 16, (uint4*)dst);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_add_i32(strictb200_ctx* ctx, int32_t* x, const int32_t* inc, int32_t c, int64_t n) {
  SB_CUDA(sb_launch(ctx, add_i32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, x, inc, c, n));
  ctx->launches++;
  return STRICTB200_OK;
}
int k_f32_to_bf16(strictb200_ctx* ctx, const float* x, int64_t n, bf16* y) {
  f32_to_bf16_kernel<<<sgrid(ctx, n), 256, 0, ctx->stream>>>(x, n, y);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
int k_bf16_to_f32(strictb200_ctx* ctx, const bf16* x, int64_t n, float* y) {
  bf16_to_f32_kernel<<<sgrid(ctx, n), 256, 0, ctx->stream>>>(x, n, y);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
