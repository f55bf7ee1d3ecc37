// Run-time compilation of emitted CUDA C text to PTX, the step the reference performs through
// ManagedCuda's CudaRuntimeCompiler (Strict.Compiler.Cuda/Kernel.cs:29-33,43,57;
// Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:89-98): NVRTC is bound with dlopen,
// so the library loads on machines without it and the entry point then reports ERR_UNSUPPORTED
// (the reference's ToolNotFoundException case). Compiling needs no GPU. The kernels this
// library runs are compiled ahead of time; this entry exists so that the text InstructionsToCuda
// emits can be checked to be valid CUDA C for sm_100a, and for Kernel.CompileKernelAndSaveAsPtxFile.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace {
typedef struct _nvrtcProgram* nvrtc_program;
struct Nvrtc {
  void* lib = nullptr;
  int (*CreateProgram)(nvrtc_program*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*DestroyProgram)(nvrtc_program*) = nullptr;
  int (*CompileProgram)(nvrtc_program, int, const char* const*) = nullptr;
  int (*GetPTXSize)(nvrtc_program, size_t*) = nullptr;
  int (*GetPTX)(nvrtc_program, char*) = nullptr;
  int (*GetProgramLogSize)(nvrtc_program, size_t*) = nullptr;
  int (*GetProgramLog)(nvrtc_program, char*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
Nvrtc g_rtc;
std::mutex g_rtc_mutex;

int load_nvrtc() {
  std::lock_guard<std::mutex> lock(g_rtc_mutex);
  if (g_rtc.lib) return STRICTB200_OK;
  void* h = nullptr;
  for (const char* name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"}) {
    h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (h) break;
  }
  if (!h) return sb_fail(STRICTB200_ERR_UNSUPPORTED, std::string("NVRTC is not installed (") + dlerror() + ")");
#define SYM(field, name)                                                                          \
  *(void**)(&g_rtc.field) = dlsym(h, name);                                                       \
  if (!g_rtc.field) return sb_fail(STRICTB200_ERR_UNSUPPORTED, std::string("libnvrtc lacks ") + name);
  SYM(CreateProgram, "nvrtcCreateProgram")
  SYM(DestroyProgram, "nvrtcDestroyProgram")
  SYM(CompileProgram, "nvrtcCompileProgram")
  SYM(GetPTXSize, "nvrtcGetPTXSize")
  SYM(GetPTX, "nvrtcGetPTX")
  SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
  SYM(GetProgramLog, "nvrtcGetProgramLog")
  SYM(GetErrorString, "nvrtcGetErrorString")
#undef SYM
  g_rtc.lib = h;
  return STRICTB200_OK;
}
}  // namespace

extern "C" int strictb200_compile_to_ptx(const char* cuda_c, const char* name, const char* const* options, int n_options, char* ptx_out,
                                         size_t ptx_capacity, size_t* ptx_size) {
  if (!cuda_c || !name || n_options < 0 || (n_options && !options)) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null argument");
  SB_TRY(load_nvrtc());
  nvrtc_program prog = nullptr;
  int rc = g_rtc.CreateProgram(&prog, cuda_c, name, 0, nullptr, nullptr);
  if (rc) return sb_fail(STRICTB200_ERR_CUDA, std::string("nvrtcCreateProgram: ") + g_rtc.GetErrorString(rc));
  rc = g_rtc.CompileProgram(prog, n_options, options);
  if (rc) {
    // the compiler's log is the error text, as the reference prints GetLogAsString
    size_t n = 0;
    std::string log;
    if (!g_rtc.GetProgramLogSize(prog, &n) && n > 1) {
      std::vector<char> buf(n);
      if (!g_rtc.GetProgramLog(prog, buf.data())) log.assign(buf.data());
    }
    std::string msg = std::string("NVRTC: ") + g_rtc.GetErrorString(rc) + (log.empty() ? "" : ": " + log);
    g_rtc.DestroyProgram(&prog);
    return sb_fail(STRICTB200_ERR_INVALID_ARG, msg);
  }
  size_t n = 0;
  rc = g_rtc.GetPTXSize(prog, &n);
  if (!rc && ptx_size) *ptx_size = n;
  if (!rc && ptx_out) {
    if (n > ptx_capacity) {
      g_rtc.DestroyProgram(&prog);
      return sb_fail(STRICTB200_ERR_INVALID_ARG, "PTX needs " + std::to_string(n) + " bytes; the buffer holds " + std::to_string(ptx_capacity));
    }
    rc = g_rtc.GetPTX(prog, ptx_out);
  }
  g_rtc.DestroyProgram(&prog);
  if (rc) return sb_fail(STRICTB200_ERR_CUDA, std::string("nvrtcGetPTX: ") + g_rtc.GetErrorString(rc));
  return STRICTB200_OK;
}
