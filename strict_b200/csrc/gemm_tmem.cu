// Placeholder translation unit: the tcgen05/TMEM GEMM lands here.
#include "common.cuh"
int k_gemm_fp8_tmem(strictb200_ctx*, const GemmArgs&) { return sb_fail(STRICTB200_ERR_UNSUPPORTED, "tensor-memory GEMM not built"); }
