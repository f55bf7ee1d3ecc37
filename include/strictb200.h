/* strictb200 — C ABI of the B200 (sm_100a) LLM forward path behind the Strict CUDA surface.
 *
 * One shared library, `libstrictb200.so`, plain C linkage, plain pointers and sizes. It is
 * what a `[DllImport("strictb200")]` class inside Strict.Compiler.Cuda binds instead of the
 * ManagedCuda + NVRTC objects the reference uses. Every function returns a status code
 * (0 = ok); no exception crosses the boundary; `strictb200_last_error()` gives the text of
 * the calling thread's last failure. All kernels are compiled ahead of time for sm_100a;
 * there is no CPU fallback: without a B200-class device `strictb200_create` fails.
 *
 * Threading: a context is bound to one device and one stream; calls on one context must be
 * serialised by the caller; different contexts may be driven from different threads.
 * Pointers named d_* are device pointers of that context's device, h_* are host pointers.
 */
#ifndef STRICTB200_H
#define STRICTB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STRICTB200_VERSION 100

enum strictb200_status {
  STRICTB200_OK = 0,
  STRICTB200_ERR_INVALID_ARG = 1, /* null handle, bad size/alignment, unknown name */
  STRICTB200_ERR_UNSUPPORTED = 2, /* maps to NotSupportedException (InstructionsToCuda.cs:108) */
  STRICTB200_ERR_CUDA = 3,
  STRICTB200_ERR_NCCL = 4,
  STRICTB200_ERR_OOM = 5,
  STRICTB200_ERR_TIMEOUT = 6 /* a bounded device-side wait gave up */
};

typedef struct strictb200_ctx strictb200_ctx;
typedef struct strictb200_model strictb200_model;
typedef struct strictb200_kv strictb200_kv;

/* ---- library ---- */
int strictb200_version(void);
const char* strictb200_last_error(void);
/* "<16 hex digits> <date> <time>": a hash of the sources this binary was built from (every file
 * under csrc/ and this header; python -m strict_b200.build computes and stamps it) and when it was
 * compiled. bench.py prints it beside the hash of the sources it finds next to the library. */
const char* strictb200_build_id(void);

/* Compiles CUDA C text to PTX with NVRTC, as the reference does through ManagedCuda's
 * CudaRuntimeCompiler(code, name).Compile(options) / GetPTXAsString / GetLogAsString
 * (Strict.Compiler.Cuda/Kernel.cs:29-33,43,57). Needs no GPU and no context. `options` are NVRTC
 * options such as "--gpu-architecture=compute_100a". With d_ptx_out NULL only *ptx_size (bytes
 * including the final NUL) is returned. A compile error returns ERR_INVALID_ARG with the
 * compiler's log as last_error; a machine without libnvrtc returns ERR_UNSUPPORTED. The kernels
 * this library runs are compiled ahead of time and do not go through this call. */
int strictb200_compile_to_ptx(const char* cuda_c, const char* name, const char* const* options, int n_options, char* ptx_out,
                              size_t ptx_capacity, size_t* ptx_size);

/* ---- context: replaces `new CudaContext(0)` (Strict.Compiler.Cuda/Kernel.cs:9) and
 * Kernel.Dispose (Kernel.cs:13-17). destroy(NULL) is a no-op. */
int strictb200_create(int device, strictb200_ctx** out);
int strictb200_destroy(strictb200_ctx* ctx);
int strictb200_synchronize(strictb200_ctx* ctx);
/* Device memory: replaces CudaDeviceVariable<T> ctor / implicit host<->device conversions
 * (Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:64,75-76,56). Copies are
 * synchronous with respect to the host. */
int strictb200_malloc(strictb200_ctx* ctx, size_t bytes, void** d_out);
int strictb200_free(strictb200_ctx* ctx, void* d_ptr);
int strictb200_memset(strictb200_ctx* ctx, void* d_ptr, int byte, size_t bytes);
int strictb200_upload(strictb200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes);
int strictb200_download(strictb200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes);
/* Asynchronous copies on the context's stream (pinned host memory recommended). */
int strictb200_upload_async(strictb200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes);
int strictb200_download_async(strictb200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes);
int strictb200_host_alloc(strictb200_ctx* ctx, size_t bytes, void** h_out); /* pinned */
int strictb200_host_free(strictb200_ctx* ctx, void* h_ptr);
/* Device timing on the context's stream: begin records an event, end records a second one,
 * waits for it and returns the milliseconds in between. */
int strictb200_timer_begin(strictb200_ctx* ctx);
int strictb200_timer_end(strictb200_ctx* ctx, float* ms_out);
/* Number of kernels this context launched since creation (library kernels only). */
int strictb200_launch_count(strictb200_ctx* ctx, uint64_t* out);
/* Waits for the stream, then returns (and clears) the error word kernels set when one of their
 * bounded waits expired: 0 = none; non-zero also returns ERR_TIMEOUT. strictb200_prefill,
 * _decode_step and _generate make the same check themselves after their own synchronise, so a
 * rank that never arrived shows as ERR_TIMEOUT from the call, not as silently wrong tokens. */
int strictb200_device_status(strictb200_ctx* ctx, int* out);
/* Writes `bytes` to a private buffer (> L2) so the next kernel starts with a cold L2. */
int strictb200_flush_l2(strictb200_ctx* ctx);
/* Diagnostics: time stamps of the decode step's kernels, per block. Between _trace_begin and
 * _trace_end thread 0 of every block of the instrumented kernels (decode GEMM, row kernels, RoPE,
 * decode attention and its merge, SwiGLU) stores eight 64-bit words: the global timer in ns at block
 * start, after the block's dependency wait, at block end, (kernel id | tag << 8 | SM << 48), up to
 * three optional marks inside the kernel (0 when unused) and a zero,
 * with ids 1 GEMM, 2 row kernel, 3 RoPE, 4 attention, 5 merge, 6 SwiGLU, 7 row kernel with the
 * fused all-reduce; the tag tells launches of one kernel apart (GEMM: N ^ K << 12). A recorded
 * graph can be replayed under a trace as it is. _trace_end copies at most max_records records
 * (8 words each) and returns in *out_count how many blocks reported. One trace per process at a
 * time (the switch is a device variable). The reference has no counterpart. */
int strictb200_trace_begin(strictb200_ctx* ctx, int capacity);
int strictb200_trace_end(strictb200_ctx* ctx, uint64_t* out_records, int max_records, int* out_count);
/* Switches of a context. Each is read ONCE from the environment variable STRICTB200_<NAME IN
 * CAPITALS> when the context is created; no launch path reads the environment. -1 = the
 * library's own choice. Names: "pdl" (programmatic dependent launch, 1), "attn_tc" (prefill
 * attention kernel: 0 mma.sync, 1 tcgen05 one query tile per block, 2 two tiles per block, -1),
 * "gemm_pair" (many-token GEMM on SM pairs, 1), "prefetch" (1), "deep_ring" (1),
 * "attn_blocks_per_sm" (0), "split_target" (0), "tp_two_shot" (fused all-reduce in two shots,
 * -1: with more than four ranks), "wait_limit" (polls of a cross-rank wait before it gives up,
 * 4194304), "prefill_chunk" (token rows per prefill chunk, 16384), "fuse_rope" (decode attention applies
 * QK-norm and RoPE and appends to the cache itself, 0), "row_cluster" (blocks of one cluster that share a row in the decode row
 * kernels, 4), "attn_prefetch" (decode attention loads its first key/value
 * tiles before the dependency wait, 1), "blur_rows" (image rows per block of the
 * blur kernel, 0 = 8), "host_timeout_ms" (under tensor
 * parallelism: a synchronising call polls the stream and NCCL's asynchronous error state and, after
 * this many milliseconds, aborts the communicator and returns ERR_TIMEOUT instead of waiting for
 * ever; 0 = wait without limit). Unknown name -> ERR_INVALID_ARG.
 * The reference has no counterpart (its one switch is a compile flag, Kernel.cs:43). */
int strictb200_set_option(strictb200_ctx* ctx, const char* name, int value);
int strictb200_get_option(strictb200_ctx* ctx, const char* name, int* out);

/* ---- recorded call sequences. The reference launches one kernel per `kernel.Run` call
 * (Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:77,86) and has no counterpart of
 * this: the calls made on the context between begin and end are recorded into a CUDA graph
 * instead of being run, and graph_launch replays them `times` times on the context's stream
 * with one submission each. While recording, make no call that synchronises, copies to or from
 * host memory, or grows a scratch buffer: run the sequence once before recording it. */
typedef struct strictb200_graph strictb200_graph;
int strictb200_graph_begin(strictb200_ctx* ctx);
int strictb200_graph_end(strictb200_ctx* ctx, strictb200_graph** out);
int strictb200_graph_launch(strictb200_ctx* ctx, strictb200_graph* g, int times);
int strictb200_graph_destroy(strictb200_graph* g);

/* ---- element-wise surface: what the kernels emitted by InstructionsToCuda compute
 * (Strict.Compiler.Cuda/InstructionsToCuda.cs:58-73,101-109), compiled ahead of time. */
enum strictb200_ew_op { STRICTB200_ADD = 0, STRICTB200_SUBTRACT = 1, STRICTB200_MULTIPLY = 2, STRICTB200_DIVIDE = 3 };
/* out[i] = a[i] op b[i], fp32, i < count. Unknown op -> ERR_UNSUPPORTED. */
int strictb200_ew_binary(strictb200_ctx* ctx, int op, const float* d_a, const float* d_b, float* d_out, int64_t count);
/* Register program over the instruction subset the emitter handles (InstructionsToCuda.cs:31-53).
 * code = n_instr quadruples (opcode, a, b, c):
 *   0 LOAD_ARRAY  r[c] = arrays[a][idx]      (LoadVariableToRegister of an array parameter)
 *   1 LOAD_SCALAR r[c] = scalars[a]          (width / height / initialDepth, cs:97-98)
 *   2 LOAD_CONST  r[c] = consts[a]           (LoadConstantInstruction)
 *   3 ADD 4 SUBTRACT 5 MULTIPLY 6 DIVIDE     r[c] = r[a] op r[b]
 *   7 RETURN      output[idx] = r[a]         (without one the output is 0.0f, cs:30)
 * 16 registers (Strict.Bytecode/Register.cs:8-26), at most 64 instructions, 8 arrays,
 * 8 scalars, 16 constants. h_arrays is a host array of device pointers. */
int strictb200_ew_program(strictb200_ctx* ctx, const int32_t* h_code, int n_instr, const float* const* h_arrays,
                          int n_arrays, const float* h_scalars, int n_scalars, const float* h_consts, int n_consts,
                          float* d_out, int64_t count);

/* The larger instruction set: what the reference's plan lists as missing from its emitter for real
 * data-parallel kernels (Strict.Compiler.Assembly/GpuSupportPlan.md:63-67) — conditionals, loops,
 * variables, loads at computed indices (calls are placed inline by the host). Same quadruples and
 * the opcodes 0..7 of strictb200_ew_program, over 32 slots (16 registers + 16 variables), plus
 *   8 MODULO r[c] = fmodf(r[a], r[b])        9 EQUAL 10 NOT_EQUAL 11 LESS 12 GREATER   flag = r[a] op r[b]
 *   13 JUMP pc = a     14 JUMP_IF_TRUE     15 JUMP_IF_FALSE      (absolute targets, 0..n_instr)
 *   16 LOOP_BEGIN  r[a] iterations (at most 2^20), b = pc after the loop, r[c] = the index, from 0
 *   17 LOOP_END    a = pc of its LOOP_BEGIN (at most 4 nested)
 *   18 LOAD_AT     r[c] = arrays[a][(int)r[b]], 0.0f where that index is outside [0, count)
 *   19 MOVE        r[c] = r[a]                20 LOAD_INDEX  r[c] = (float)idx
 * RETURN ends the program for the element. At most 256 instructions. A thread that executes more
 * than 65536 instructions for one element writes 0 and sets the context's error word
 * (strictb200_device_status then returns ERR_TIMEOUT): no program can hang the GPU. */
int strictb200_ew_program2(strictb200_ctx* ctx, const int32_t* h_code, int n_instr, const float* const* h_arrays, int n_arrays,
                           const float* h_scalars, int n_scalars, const float* h_consts, int n_consts, float* d_out, int64_t count);

/* ---- image workloads of the reference's samples ---- */
/* 5x5 box blur over interleaved RGB bytes, d_src -> d_dst (two different buffers of
 * width*height*3 bytes): what the reference's CPU harness computes
 * (Strict.Compiler.Assembly.Tests/BlurPerformanceTests.cs:52-141 — sum/25 where all 25
 * neighbours exist, sum/count of the neighbours inside the image at the edges, integer division
 * per channel) and what its CUDA harness was meant to (its kernel is a byte copy,
 * Strict.Compiler.Cuda.Tests/BlurPerformanceTests.cs:111-117). Bit-exact with the CPU form.
 * Rows whose byte length is a multiple of 16 (width % 16 == 0) with 16-byte aligned buffers
 * take the packed strip kernel; other images take the generic per-byte kernel. */
int strictb200_blur5x5_rgb8(strictb200_ctx* ctx, const uint8_t* d_src, uint8_t* d_dst, int width, int height);
/* AdjustBrightness (ImageProcessing/AdjustBrightness.strict:10,16) over the flat number layout of
 * Strict.Expressions/ValueArrayInstance.cs:9-16,128,339: fp32 array of structs, element i member
 * m at d_flat[offset + i*flat_width + m]; the first `channels` members of `count` elements get
 * `brightness` added in place (Color: flat_width 4 = Red, Green, Blue, Alpha; channels 3). The
 * sum is taken in double and stored as float, as the reference's VM does. clamp01 != 0 keeps
 * results inside [0,1] (the range Color.strict allows; the .strict code does not clamp). */
int strictb200_adjust_brightness(strictb200_ctx* ctx, float* d_flat, int64_t offset, int64_t count, int flat_width, int channels,
                                 double brightness, int clamp01);

/* ---- seeded generator (device side of the synthetic-tensor specification) ---- */
int strictb200_gen_normal_f32(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t first, int64_t count, float std, float* d_out);
int strictb200_gen_normal_bf16(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t first, int64_t count, float std, uint16_t* d_out);
int strictb200_gen_tokens(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t count, uint32_t range, int32_t* d_out);
/* rows [row0,row0+rows) x columns [col0,col0+cols) of an E4M3 weight [*,K] whose source is
 * std*N(0,1); d_scale[r] = absmax(full row)/448 for the generated rows. */
int strictb200_gen_weight_e4m3(strictb200_ctx* ctx, uint64_t seed, uint64_t tensor, int64_t row0, int64_t rows, int64_t K,
                               int64_t col0, int64_t cols, float std, uint8_t* d_q, float* d_scale);

/* ---- activation split and GEMM (no reference counterpart; new surface) ----
 * A linear layer is y = (x . W^T) * sw with bf16 x, E4M3 W and one fp32 scale per output
 * channel. To feed the FP8 tensor cores without dequantising weights in the kernel, a bf16 row
 * is carried as two E4M3 terms with a power-of-two scale, x = s*(hi + lo/16), which is exact
 * for every element at or above absmax/14336. The split buffer holds tokens in groups of 8:
 * group g occupies rows [16g,16g+16) of width K, 8 hi rows then 8 lo rows, so it has
 * 16*ceil(M/8) rows in total. */
int strictb200_quantize_rows(strictb200_ctx* ctx, const uint16_t* d_x_bf16, int64_t M, int64_t K, uint8_t* d_split, float* d_scale);
/* Y[M,N] = ((X . Wq[N,K]^T) * sx[M]) * sw[N] with X given as the split of M rows (above);
 * fp32 accumulation. out_dtype: 0 bf16, 1 fp32. K % 64 == 0 (K % 128 == 0 for the
 * tensor-memory kernel), N % 16 == 0.
 * kernel: 0 auto, 1 skinny stream (M <= 32), 2 mma.sync tiles, 3 tcgen05/TMEM tiles. */
int strictb200_gemm_fp8(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint8_t* d_split, const float* d_sx,
                        const uint8_t* d_wq, const float* d_sw, void* d_out, int out_dtype, int kernel);
/* bf16 activations in (split inside, using context scratch); bf16 out. */
int strictb200_gemm_fp8w(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                         const float* d_sw, uint16_t* d_y_bf16, int kernel);
/* ---- int8-weight linear layer (no reference counterpart; new surface) ----
 * y = (x . Wq^T) * sw with bf16 x, signed 8-bit Wq and one fp32 scale per output channel
 * (absmax / 127). The integer tensor cores take the activations as two int8 terms per element,
 * x ~ s * (128 * hi + lo) with s a power of two per token (|x| / s <= 16256, hi in [-127, 127],
 * lo in [-64, 63]; exact for every element within a factor 63 of the row's largest); the sums are exact 32-bit integers joined in 64 bits, so the result does
 * not depend on how K is split and equals the CPU restatement bit for bit. The split buffer has
 * the layout of strictb200_quantize_rows (groups of 8 tokens: 8 hi rows, 8 lo rows).
 * K % 128 == 0, K <= 131072, N % 16 == 0. */
int strictb200_quantize_weights_int8(strictb200_ctx* ctx, const float* d_w, int64_t N, int64_t K, int8_t* d_wq, float* d_sw);
int strictb200_quantize_rows_int8(strictb200_ctx* ctx, const uint16_t* d_x_bf16, int64_t M, int64_t K, int8_t* d_split, float* d_scale);
/* Y[M,N] bf16 from the split of M rows (above). */
int strictb200_gemm_int8(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const int8_t* d_split, const float* d_sx, const int8_t* d_wq,
                         const float* d_sw, uint16_t* d_y_bf16);
/* bf16 activations in (split inside, using context scratch); bf16 out. */
int strictb200_gemm_int8w(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* d_x_bf16, const int8_t* d_wq, const float* d_sw,
                          uint16_t* d_y_bf16);
/* fp32 Y[M,N] = X[M,K] . W[N,K]^T + bias[N] (bias may be NULL). */
int strictb200_gemm_f32(strictb200_ctx* ctx, int64_t M, int64_t N, int64_t K, const float* d_x, const float* d_w,
                        const float* d_bias, float* d_y);

/* ---- norms / activations ---- */
/* y = (x * rsqrt(mean(x^2)+eps)) * gain, bf16 in/out, fp32 statistics. If d_residual is not
 * NULL it is first updated in place: residual = bf16(residual + x), and the norm is taken
 * of the updated residual. This is the stand-alone operator with a bf16 residual; the model's
 * own path keeps its residual stream in fp32 and fuses the split-K sum, the residual update, the
 * norm and the activation split in one row kernel (the fp32-residual form of the same kernel is
 * reachable through strictb200_tp_allreduce_rownorm under tensor parallelism). */
int strictb200_rmsnorm(strictb200_ctx* ctx, const uint16_t* d_x, uint16_t* d_residual, const float* d_gain, float eps, int64_t M,
                       int64_t d, uint16_t* d_y);
int strictb200_layernorm(strictb200_ctx* ctx, const float* d_x, const float* d_gain, const float* d_bias, float eps, int64_t M,
                         int64_t d, float* d_y);
/* y = bf16(silu(gate) * up); gate_up is [M, 2*I] with gate in columns [0,I). */
int strictb200_swiglu(strictb200_ctx* ctx, const uint16_t* d_gate_up, int64_t M, int64_t I, uint16_t* d_y);
int strictb200_gelu_tanh(strictb200_ctx* ctx, const float* d_x, int64_t count, float* d_y);
/* Per-head RMS norm, rotary embedding (pairs (i, i+D/2), angle pos*theta^(-2i/D)) and cache
 * append. qkv is bf16 [T, (Hq+2Hkv)*D]; token t belongs to sequence seq[t] at position pos[t];
 * q_out is bf16 [T,Hq,D]; caches are bf16 [B,Hkv,maxlen,D]. */
int strictb200_rope_qknorm_kvappend(strictb200_ctx* ctx, const uint16_t* d_qkv, const int32_t* d_seq, const int32_t* d_pos, int64_t T,
                                    int Hq, int Hkv, int D, const float* d_qgain, const float* d_kgain, float eps, float theta,
                                    int max_pos, uint16_t* d_q_out, uint16_t* d_kcache, uint16_t* d_vcache, int maxlen);

/* ---- attention (bf16, GQA, D = 128) ---- */
/* Causal prefill: q [B,S,Hq,D]; caches [B,Hkv,maxlen,D] already hold positions [0,lens[b]);
 * the query at row i of sequence b has position past[b]+i (past may be NULL = 0) and the
 * rows i < lens[b]-past[b] are computed. out [B,S,Hq,D]. */
int strictb200_attn_prefill(strictb200_ctx* ctx, const uint16_t* d_q, const uint16_t* d_kcache, const uint16_t* d_vcache,
                            const int32_t* d_lens, const int32_t* d_past, int B, int S, int Hq, int Hkv, int D, int maxlen,
                            float scale, uint16_t* d_out);
/* Split-KV decode: one query per sequence, q [B,Hq,D], keys [0,lens[b]). out [B,Hq,D].
 * Uses context scratch for the per-split partial results. */
int strictb200_attn_decode(strictb200_ctx* ctx, const uint16_t* d_q, const uint16_t* d_kcache, const uint16_t* d_vcache,
                           const int32_t* d_lens, int B, int Hq, int Hkv, int D, int maxlen, float scale, uint16_t* d_out);

/* Same computation as strictb200_attn_decode for hosts that must not allocate while serving:
 * a decode loop that cannot absorb the device-wide stall cudaMalloc/cudaFree cause, or a host
 * that gave all device memory to its own pool at start-up. This entry point has no counterpart
 * in the reference. It calls no allocator of any kind: the split-KV partial results go to a
 * 4 MiB array built into the library image (every GPU that loads the library holds it until
 * exit). A call whose B * Hq * key-chunks * 130 floats exceed 4 MiB is rejected with
 * ERR_INVALID_ARG. The first call on a device looks up the array's device address; make that
 * first call before starting any stream capture. All calls on a device share the array and
 * its previous contents (none of it needs clearing), so two calls whose kernels overlap on
 * the GPU — different contexts or streams on one device — race; serialise them. */
int strictb200_attn_decode_noalloc(strictb200_ctx* ctx, const uint16_t* d_q, const uint16_t* d_kcache, const uint16_t* d_vcache,
                                   const int32_t* d_lens, int B, int Hq, int Hkv, int D, int maxlen, float scale, uint16_t* d_out);

/* ---- embedding / sampling ---- */
int strictb200_embedding_bf16(strictb200_ctx* ctx, const uint16_t* d_table, const int32_t* d_ids, int64_t T, int64_t d, int64_t vocab,
                              uint16_t* d_out);
/* argmax over the last dimension of fp32 [M,N]; ties go to the lowest index. */
int strictb200_argmax(strictb200_ctx* ctx, const float* d_x, int64_t M, int64_t N, int32_t* d_out);

/* ---- model / KV-cache objects (new API in the style of the existing surface) ---- */
enum strictb200_arch { STRICTB200_GPT2 = 0, STRICTB200_QWEN3 = 1 };
typedef struct strictb200_model_config {
  int32_t arch;       /* strictb200_arch */
  int32_t n_layers, d_model, n_q_heads, n_kv_heads, head_dim, d_ff, vocab;
  int32_t max_pos;    /* positions the model can address (learned table / RoPE table) */
  int32_t tied;       /* LM head shares the embedding matrix */
  float eps;          /* norm epsilon */
  float rope_theta;
} strictb200_model_config;

int strictb200_model_create(strictb200_ctx* ctx, const strictb200_model_config* cfg, strictb200_model** out);
int strictb200_model_destroy(strictb200_model* m);
/* Fill every tensor from the seeded generator (std 0.02, norm gains 1, biases 0). Under
 * tensor parallelism each rank generates only its own shard. */
int strictb200_model_init_random(strictb200_model* m, uint64_t seed);
/* Set / read one full (unsharded) tensor by name from / to host memory; the library slices
 * it for this rank. Names: "embed", "wpe", "normf.g", "normf.b", "head.q", "head.s",
 * "layers.<i>.{norm1.g,norm1.b,norm2.g,norm2.b,qnorm.g,knorm.g}", Qwen3:
 * "layers.<i>.{wqkv,wo,wgu,wdown}.{q,s}", GPT-2: "layers.<i>.{wqkv,wo,wfc,wproj}.{w,b}".
 * fp32 host data except ".q" (E4M3 bytes); "embed" of a Qwen3 model is given as fp32 and
 * rounded to bf16. */
int strictb200_model_set_tensor(strictb200_model* m, const char* name, const void* h_data, size_t bytes);
int strictb200_model_get_tensor(strictb200_model* m, const char* name, void* h_data, size_t bytes);
int strictb200_model_weight_bytes(strictb200_model* m, uint64_t* out);

int strictb200_kv_create(strictb200_model* m, int batch, int maxlen, strictb200_kv** out);
int strictb200_kv_destroy(strictb200_kv* kv);
int strictb200_kv_reset(strictb200_kv* kv);
int strictb200_kv_lens(strictb200_kv* kv, int32_t* h_lens);
/* Fill positions [0,len) of every sequence with seeded N(0,1) keys/values and set the
 * lengths to len (benchmark set-up of a long context without running the prefill). */
int strictb200_kv_fill_synthetic(strictb200_kv* kv, uint64_t seed, int len);

/* Prefill: h_tokens [B,S] row-major, the first h_lens[b] of each row are real. Appends to the
 * cache, writes the greedy next token of every sequence to h_next[B] and, if not NULL, the
 * fp32 logits [B,vocab] to h_logits. */
int strictb200_prefill(strictb200_model* m, strictb200_kv* kv, const int32_t* h_tokens, const int32_t* h_lens, int B, int S,
                       int32_t* h_next, float* h_logits);
/* One decode step for every sequence of the cache: h_ids[B] in, greedy next ids out. */
int strictb200_decode_step(strictb200_model* m, strictb200_kv* kv, const int32_t* h_ids, int32_t* h_next, float* h_logits);
/* n_steps greedy steps entirely on the device starting from h_ids; h_out [n_steps,B]. */
int strictb200_generate(strictb200_model* m, strictb200_kv* kv, const int32_t* h_ids, int n_steps, int32_t* h_out);
/* Same, with ids already on the device and no host copy: d_ids[B] is read and overwritten
 * each step (benchmark `value` leg). */
int strictb200_decode_steps_device(strictb200_model* m, strictb200_kv* kv, int32_t* d_ids, int n_steps);
int strictb200_kv_device_ids(strictb200_kv* kv, int32_t** d_ids_out);
/* 1 = capture the decode step in a CUDA graph and replay it (default), 0 = plain launches. */
int strictb200_model_set_graph(strictb200_model* m, int enabled);
/* Kernel classes of the Qwen3 decode step, for strictb200_profile_decode. */
enum strictb200_kernel_class {
  STRICTB200_K_EMBED = 0,     /* embedding gather, length update */
  STRICTB200_K_GEMM_QKV = 1,
  STRICTB200_K_ROPE = 2,      /* split-K reduce + QK-norm + RoPE + cache append */
  STRICTB200_K_ATTN = 3,      /* split-KV attention (the kernel that streams the cache) */
  STRICTB200_K_GEMM_O = 4,
  STRICTB200_K_ROWNORM = 5,   /* split-K reduce + residual + RMSNorm + quantise */
  STRICTB200_K_GEMM_GU = 6,
  STRICTB200_K_SWIGLU = 7,
  STRICTB200_K_GEMM_DOWN = 8,
  STRICTB200_K_HEAD = 9,      /* LM head GEMM + argmax */
  STRICTB200_K_ALLREDUCE = 10,
  STRICTB200_K_ATTN_MERGE = 11, /* merge of the key chunks + quantise */
  STRICTB200_K_COUNT = 12
};
/* Runs n_steps greedy decode steps as plain launches with a pair of CUDA events around every
 * call, and returns the summed device milliseconds and the number of calls per kernel class
 * (arrays of at least STRICTB200_K_COUNT entries). Advances the cache like decode does. */
int strictb200_profile_decode(strictb200_model* m, strictb200_kv* kv, int n_steps, float* h_ms, uint64_t* h_calls, int n_classes);
/* Algorithmic bytes one decode step reads at the cache's current lengths (weights + KV). */
int strictb200_decode_bytes(strictb200_model* m, strictb200_kv* kv, uint64_t* out);

/* ---- tensor parallelism: one context per GPU/rank, NCCL over NVLink ---- */
/* 128-byte NCCL unique id, created on rank 0 and handed to every rank by the host. */
int strictb200_tp_unique_id(void* h_id128);
/* Must be called before model_create on that context. world in {1,2,4,8}. */
int strictb200_tp_init(strictb200_ctx* ctx, int world, int rank, const void* h_id128);
int strictb200_tp_info(strictb200_ctx* ctx, int* world, int* rank);
/* Optional all-reduce over peer memory for the decode step (messages of a few hundred KB, where
 * NCCL's launch latency dominates): after tp_init every rank asks for the 64-byte CUDA IPC handle
 * of its exchange buffer, the host gathers the handles of all ranks (rank order, world x 64 bytes)
 * and hands them to every rank. From then on the all-reduce after o_proj and down_proj happens
 * inside the residual/RMSNorm kernel that consumes the sum: the block of a token row adds the
 * rank's own split-K partials, pushes every value into the peers' buffers over NVLink as one
 * 32-bit word whose two lowest mantissa bits carry the row's call count modulo 4 (plain stores;
 * no multicast), polls its own buffer until the same row's words of every peer carry the
 * current tag, and adds the ranks' values, those two bits cleared in every one of them, in rank
 * order, so every rank computes bit-identical sums (a partial sum loses at most 3 units of its
 * last place, 3.6e-7 relative; the NCCL path adds the unmodified values). With more than four ranks the exchange takes two
 * shots: each column slice goes to the rank that owns it, which returns the finished sums.
 * Every poll is bounded ("wait_limit"); if a rank never shows up the kernel sets the error word
 * and the call that synchronises next returns ERR_TIMEOUT. All ranks must be processes on one
 * NVLink-connected box. Batches that do not fit the buffers (more than 1M values per result)
 * and contexts without these two calls use NCCL. */
int strictb200_tp_comm_handle(strictb200_ctx* ctx, void* h_handle64);
int strictb200_tp_comm_open(strictb200_ctx* ctx, const void* h_handles);
/* The fused op by itself: out = RMSNorm(residual + sum over ranks of ((sum of this rank's
 * `splits` partials [splits][M,d]) * sx[M] * sw[d])) * gain. d_residual_f32 (may be NULL) is
 * updated in place; the normalised row is written as bf16 (d_y, may be NULL) and/or as the
 * two-term E4M3 split with its scales (d_split + d_split_scale, may both be NULL). Every rank
 * calls it with the same shapes, in the same order. Needs open peer buffers. */
int strictb200_tp_allreduce_rownorm(strictb200_ctx* ctx, const float* d_part, int splits, const float* d_sx, const float* d_sw,
                                    float* d_residual_f32, const float* d_gain, float eps, int64_t M, int64_t d, uint16_t* d_y,
                                    uint8_t* d_split, float* d_split_scale);
/* Failure injection on the host side, for tests of the bounded waits: sets the context up as
 * rank 0 of `world` ranks whose peers are local buffers that nothing ever writes, i.e. ranks
 * that never show up. No NCCL, no other process; only strictb200_tp_allreduce_rownorm may be
 * used on such a context, and with a small "wait_limit" it returns its (meaningless) result
 * quickly while strictb200_device_status reports ERR_TIMEOUT. Nothing faults or hangs. */
int strictb200_tp_comm_open_absent_peers(strictb200_ctx* ctx, int world);
/* fp32 sum all-reduce in place on the context's stream (the collective the model uses). */
int strictb200_tp_allreduce_f32(strictb200_ctx* ctx, float* d_buf, int64_t count);

#ifdef __cplusplus
}
#endif
#endif /* STRICTB200_H */
