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

// ---------------------------------------------------------------- the larger instruction set
// Register programs with conditionals, loops, loads at computed indices and variables: what the
// reference's plan lists as missing from its emitter (Strict.Compiler.Assembly/GpuSupportPlan.md:
// 63-67). One thread interprets the program for its element. 32 slots (16 registers,
// Strict.Bytecode/Register.cs:8-26, and 16 variables), a condition flag as in the reference's VM,
// four nested loops. Every program ends: a thread executes at most EW2_MAX_STEPS instructions,
// then writes 0 and sets the context's error word.
namespace {
constexpr int EW2_MAX_INSTR = 256, EW2_SLOTS = 32, EW2_MAX_LOOPS = 4, EW2_MAX_STEPS = 1 << 16;
struct EwProgram2 {  // travels as the kernel's parameter block (4.4 KB; large parameter blocks need CUDA 12.1+)
  int4 code[EW2_MAX_INSTR];
  const float* arrays[8];
  float scalars[8];
  float consts[16];
  int n_instr;
  int* status;
};

__global__ void ew_program2_kernel(const __grid_constant__ EwProgram2 p, float* __restrict__ out, int64_t n) {
  __shared__ int4 code[EW2_MAX_INSTR];  // threads diverge in pc: shared memory serves that better than the constant bank
  for (int i = threadIdx.x; i < p.n_instr; i += blockDim.x) code[i] = p.code[i];
  __syncthreads();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    float r[EW2_SLOTS];
#pragma unroll
    for (int i = 0; i < EW2_SLOTS; i++) r[i] = 0.f;
    int loop_begin[EW2_MAX_LOOPS], loop_count[EW2_MAX_LOOPS], loop_i[EW2_MAX_LOOPS], depth = 0;
    bool flag = false;
    float res = 0.0f;
    int pc = 0, steps = 0;
    while (pc < p.n_instr) {
      if (++steps > EW2_MAX_STEPS) {
        *(volatile int*)p.status = 7;
        res = 0.0f;
        break;
      }
      const int4 q = code[pc];
      const int op = q.x, a = q.y, b = q.z, c = q.w;
      int next = pc + 1;
      switch (op) {
        case 0: r[c] = p.arrays[a][idx]; break;
        case 1: r[c] = p.scalars[a]; break;
        case 2: r[c] = p.consts[a]; break;
        case 3: r[c] = __fadd_rn(r[a], r[b]); break;
        case 4: r[c] = __fsub_rn(r[a], r[b]); break;
        case 5: r[c] = __fmul_rn(r[a], r[b]); break;
        case 6: r[c] = __fdiv_rn(r[a], r[b]); break;
        case 7: res = r[a]; next = p.n_instr; break;
        case 8: r[c] = fmodf(r[a], r[b]); break;
        case 9: flag = r[a] == r[b]; break;
        case 10: flag = r[a] != r[b]; break;
        case 11: flag = r[a] < r[b]; break;
        case 12: flag = r[a] > r[b]; break;
        case 13: next = a; break;
        case 14: if (flag) next = a; break;
        case 15: if (!flag) next = a; break;
        case 16: {  // LOOP_BEGIN: count in r[a], b = pc after the loop, c = slot of the index
          const float cf = r[a];
          const int count = cf >= 1.0f ? (cf < 1048576.0f ? (int)cf : 1048576) : 0;
          if (count <= 0 || depth >= EW2_MAX_LOOPS) { next = b; break; }
          loop_begin[depth] = pc; loop_count[depth] = count; loop_i[depth] = 0; depth++;
          r[c] = 0.0f;
          break;
        }
        case 17: {  // LOOP_END: a = pc of the matching LOOP_BEGIN
          if (depth > 0 && loop_begin[depth - 1] == a) {
            if (++loop_i[depth - 1] < loop_count[depth - 1]) {
              r[code[a].w] = (float)loop_i[depth - 1];
              next = a + 1;
            } else {
              depth--;
            }
          }
          break;
        }
        case 18: {  // LOAD_AT: arrays[a][(int)r[b]], 0 outside [0, n)
          const float f = r[b];
          r[c] = (f >= 0.0f && f < (float)n) ? p.arrays[a][(int64_t)f] : 0.0f;
          break;
        }
        case 19: r[c] = r[a]; break;
        case 20: r[c] = (float)idx; break;
        default: next = p.n_instr; break;
      }
      pc = next;
    }
    out[idx] = res;
  }
}
}  // namespace

int k_ew_program2(strictb200_ctx* ctx, const int32_t* h_code, int n_instr, const float* const* h_arrays, int n_arrays,
                  const float* h_scalars, int n_scalars, const float* h_consts, int n_consts, float* out, int64_t n) {
  if (n_instr > EW2_MAX_INSTR) return sb_fail(STRICTB200_ERR_INVALID_ARG, "program longer than 256 instructions");
  EwProgram2 p;
  memset(&p, 0, sizeof(p));
  p.n_instr = n_instr;
  p.status = ctx->d_status;
  int depth = 0;
  for (int i = 0; i < n_instr; i++) {
    const int32_t* q = h_code + 4 * i;
    const int op = q[0], a = q[1], b = q[2], c = q[3];
    if (op < 0 || op > 20) return sb_fail(STRICTB200_ERR_UNSUPPORTED, "unsupported instruction " + std::to_string(op));
    auto slot = [](int s) { return s >= 0 && s < EW2_SLOTS; };
    auto target = [&](int t) { return t >= 0 && t <= n_instr; };
    bool ok = true;
    switch (op) {
      case 0: ok = a >= 0 && a < n_arrays && h_arrays && h_arrays[a] && slot(c); break;
      case 1: ok = a >= 0 && a < n_scalars && h_scalars && slot(c); break;
      case 2: ok = a >= 0 && a < n_consts && h_consts && slot(c); break;
      case 3: case 4: case 5: case 6: case 8: ok = slot(a) && slot(b) && slot(c); break;
      case 7: ok = slot(a); break;
      case 9: case 10: case 11: case 12: ok = slot(a) && slot(b); break;
      case 13: case 14: case 15: ok = target(a); break;
      case 16: ok = slot(a) && slot(c) && target(b) && b > i && ++depth <= EW2_MAX_LOOPS; break;
      case 17: ok = a >= 0 && a < i && h_code[4 * a] == 16 && h_code[4 * a + 2] == i + 1 && depth-- > 0; break;
      case 18: ok = a >= 0 && a < n_arrays && h_arrays && h_arrays[a] && slot(b) && slot(c); break;
      case 19: ok = slot(a) && slot(c); break;
      case 20: ok = slot(c); break;
    }
    if (!ok) return sb_fail(STRICTB200_ERR_INVALID_ARG, "instruction " + std::to_string(i) + " has an operand out of range or unbalanced loops");
  }
  if (depth != 0) return sb_fail(STRICTB200_ERR_INVALID_ARG, "a loop is not closed");
  for (int i = 0; i < n_arrays; i++) p.arrays[i] = h_arrays[i];
  for (int i = 0; i < n_scalars; i++) p.scalars[i] = h_scalars[i];
  for (int i = 0; i < n_consts; i++) p.consts[i] = h_consts[i];
  for (int i = 0; i < n_instr; i++) p.code[i] = make_int4(h_code[4 * i], h_code[4 * i + 1], h_code[4 * i + 2], h_code[4 * i + 3]);
  int64_t blocks = (n + 255) / 256;
  int64_t cap = (int64_t)ctx->sm_count * 8;
  int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  ew_program2_kernel<<<grid, 256, 0, ctx->stream>>>(p, out, n);
  SB_LAUNCHED(ctx);
  return STRICTB200_OK;
}
