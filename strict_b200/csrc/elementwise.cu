// Element-wise fp32 kernels: what the CUDA C text emitted by the reference's
// InstructionsToCuda computes (Strict.Compiler.Cuda/InstructionsToCuda.cs:58-73), compiled
// ahead of time. Pure HBM streams: 128-bit loads/stores, grid sized from the SM count.
#include "common.cuh"

template <int OP>
__device__ __forceinline__ float apply(float a, float b) {
  if (OP == 0) return __fadd_rn(a, b);
  if (OP == 1) return __fsub_rn(a, b);
  if (OP == 2) return __fmul_rn(a, b);
  return __fdiv_rn(a, b);
}

template <int OP>
__global__ void ew_binary_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t n, int vec) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    int64_t n4 = n >> 2;
    const float4* a4 = (const float4*)a;
    const float4* b4 = (const float4*)b;
    float4* o4 = (float4*)out;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 x = __ldcs(a4 + i), y = __ldcs(b4 + i), r;
      r.x = apply<OP>(x.x, y.x); r.y = apply<OP>(x.y, y.y); r.z = apply<OP>(x.z, y.z); r.w = apply<OP>(x.w, y.w);
      __stcs(o4 + i, r);
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = apply<OP>(a[i], b[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = apply<OP>(a[i], b[i]);
  }
}

int k_ew_binary(strictb200_ctx* ctx, int op, const float* a, const float* b, float* out, int64_t n) {
  int vec = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
  int64_t work = vec ? (n + 3) / 4 : n;
  int64_t blocks = (work + 255) / 256;
  int64_t cap = (int64_t)ctx->sm_count * 8;
  int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  switch (op) {
    case 0: ew_binary_kernel<0><<<grid, 256, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case 1: ew_binary_kernel<1><<<grid, 256, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case 2: ew_binary_kernel<2><<<grid, 256, 0, ctx->stream>>>(a, b, out, n, vec); break;
    case 3: ew_binary_kernel<3><<<grid, 256, 0, ctx->stream>>>(a, b, out, n, vec); break;
    default: return sb_fail(STRICTB200_ERR_UNSUPPORTED, "unsupported instruction");
  }
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}

struct EwProgram {
  int32_t code[64 * 4];
  const float* arrays[8];
  float scalars[8];
  float consts[16];
  int n_instr;
};

__global__ void ew_program_kernel(const __grid_constant__ EwProgram p, float* __restrict__ out, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    float r[16];
#pragma unroll
    for (int i = 0; i < 16; i++) r[i] = 0.f;
    float res = 0.0f;
    for (int i = 0; i < p.n_instr; i++) {
      int op = p.code[4 * i], a = p.code[4 * i + 1], b = p.code[4 * i + 2], c = p.code[4 * i + 3];
      float v;
      switch (op) {
        case 0: v = p.arrays[a][idx]; break;
        case 1: v = p.scalars[a]; break;
        case 2: v = p.consts[a]; break;
        case 3: v = __fadd_rn(r[a], r[b]); break;
        case 4: v = __fsub_rn(r[a], r[b]); break;
        case 5: v = __fmul_rn(r[a], r[b]); break;
        case 6: v = __fdiv_rn(r[a], r[b]); break;
        default: v = r[a]; break;
      }
      if (op == 7) res = v; else r[c] = v;
    }
    out[idx] = res;
  }
}

int k_ew_program(strictb200_ctx* ctx, const int32_t* h_code, int n_instr, const float* const* h_arrays, int n_arrays,
                 const float* h_scalars, int n_scalars, const float* h_consts, int n_consts, float* out, int64_t n) {
  EwProgram p;
  memset(&p, 0, sizeof(p));
  p.n_instr = n_instr;
  for (int i = 0; i < n_instr; i++) {
    const int32_t* q = h_code + 4 * i;
    int op = q[0];
    if (op < 0 || op > 7) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "unsupported instruction " + std::to_string(op));
    bool ok = true;
    if (op == 0) ok = q[1] >= 0 && q[1] < n_arrays && h_arrays && h_arrays[q[1]];
    if (op == 1) ok = q[1] >= 0 && q[1] < n_scalars && h_scalars;
    if (op == 2) ok = q[1] >= 0 && q[1] < n_consts && h_consts;
    if (op >= 3 && op <= 6) ok = q[1] >= 0 && q[1] < 16 && q[2] >= 0 && q[2] < 16;
    if (op == 7) ok = q[1] >= 0 && q[1] < 16;
    if (op != 7) ok = ok && q[3] >= 0 && q[3] < 16;
    if (!ok) return sb_fail(STRICTB200_ERR_INVALID_ARG, "instruction " + std::to_string(i) + " has an operand out of range");
    for (int j = 0; j < 4; j++) p.code[4 * i + j] = q[j];
  }
  for (int i = 0; i < n_arrays; i++) p.arrays[i] = h_arrays[i];
  for (int i = 0; i < n_scalars; i++) p.scalars[i] = h_scalars[i];
  for (int i = 0; i < n_consts; i++) p.consts[i] = h_consts[i];
  int64_t blocks = (n + 255) / 256;
  int64_t cap = (int64_t)ctx->sm_count * 8;
  int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  ew_program_kernel<<<grid, 256, 0, ctx->stream>>>(p, out, n);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
