"""ctypes binding of libstrictb200.so — the same entry points a C# [DllImport] class binds.

The library is the only compute path: if it is missing or no B200 is present, loading or
`Context()` raises; nothing here falls back to the CPU.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libstrictb200.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_NCCL, ERR_OOM, ERR_TIMEOUT = range(7)


class KernelException(RuntimeError):
    """Non-zero status from the native library (carries strictb200_last_error)."""

    def __init__(self, status, message):
        super().__init__(f"strictb200 status {status}: {message}")
        self.status = status


class ModelConfig(C.Structure):
    _fields_ = [("arch", C.c_int32), ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_q_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("vocab", C.c_int32),
                ("max_pos", C.c_int32), ("tied", C.c_int32), ("eps", C.c_float), ("rope_theta", C.c_float)]


_lib = None

vp, i32, i64, u64, f32, u32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float, C.c_uint32, C.c_size_t

# name -> argtypes; every function returns int except where noted
SIGNATURES = {
    "strictb200_compile_to_ptx": [C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p), i32, vp, sz, C.POINTER(sz)],
    "strictb200_create": [i32, C.POINTER(vp)],
    "strictb200_destroy": [vp],
    "strictb200_synchronize": [vp],
    "strictb200_malloc": [vp, sz, C.POINTER(vp)],
    "strictb200_free": [vp, vp],
    "strictb200_memset": [vp, vp, i32, sz],
    "strictb200_upload": [vp, vp, vp, sz],
    "strictb200_download": [vp, vp, vp, sz],
    "strictb200_upload_async": [vp, vp, vp, sz],
    "strictb200_download_async": [vp, vp, vp, sz],
    "strictb200_host_alloc": [vp, sz, C.POINTER(vp)],
    "strictb200_host_free": [vp, vp],
    "strictb200_timer_begin": [vp],
    "strictb200_timer_end": [vp, C.POINTER(f32)],
    "strictb200_launch_count": [vp, C.POINTER(u64)],
    "strictb200_flush_l2": [vp],
    "strictb200_device_status": [vp, C.POINTER(i32)],
    "strictb200_set_option": [vp, C.c_char_p, i32],
    "strictb200_get_option": [vp, C.c_char_p, C.POINTER(i32)],
    "strictb200_graph_begin": [vp],
    "strictb200_graph_end": [vp, C.POINTER(vp)],
    "strictb200_graph_launch": [vp, vp, i32],
    "strictb200_graph_destroy": [vp],
    "strictb200_ew_binary": [vp, i32, vp, vp, vp, i64],
    "strictb200_ew_program": [vp, vp, i32, vp, i32, vp, i32, vp, i32, vp, i64],
    "strictb200_ew_program2": [vp, vp, i32, vp, i32, vp, i32, vp, i32, vp, i64],
    "strictb200_blur5x5_rgb8": [vp, vp, vp, i32, i32],
    "strictb200_adjust_brightness": [vp, vp, i64, i64, i32, i32, C.c_double, i32],
    "strictb200_gen_normal_f32": [vp, u64, u64, i64, i64, f32, vp],
    "strictb200_gen_normal_bf16": [vp, u64, u64, i64, i64, f32, vp],
    "strictb200_gen_tokens": [vp, u64, u64, i64, u32, vp],
    "strictb200_gen_weight_e4m3": [vp, u64, u64, i64, i64, i64, i64, i64, f32, vp, vp],
    "strictb200_quantize_rows": [vp, vp, i64, i64, vp, vp],
    "strictb200_gemm_fp8": [vp, i64, i64, i64, vp, vp, vp, vp, vp, i32, i32],
    "strictb200_gemm_fp8w": [vp, i64, i64, i64, vp, vp, vp, vp, i32],
    "strictb200_trace_begin": [vp, i32],
    "strictb200_trace_end": [vp, vp, i32, vp],
    "strictb200_quantize_weights_int8": [vp, vp, i64, i64, vp, vp],
    "strictb200_quantize_rows_int8": [vp, vp, i64, i64, vp, vp],
    "strictb200_gemm_int8": [vp, i64, i64, i64, vp, vp, vp, vp, vp],
    "strictb200_gemm_int8w": [vp, i64, i64, i64, vp, vp, vp, vp],
    "strictb200_gemm_f32": [vp, i64, i64, i64, vp, vp, vp, vp],
    "strictb200_rmsnorm": [vp, vp, vp, vp, f32, i64, i64, vp],
    "strictb200_layernorm": [vp, vp, vp, vp, f32, i64, i64, vp],
    "strictb200_swiglu": [vp, vp, i64, i64, vp],
    "strictb200_gelu_tanh": [vp, vp, i64, vp],
    "strictb200_rope_qknorm_kvappend": [vp, vp, vp, vp, i64, i32, i32, i32, vp, vp, f32, f32, i32, vp, vp, vp, i32],
    "strictb200_attn_prefill": [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp],
    "strictb200_attn_decode": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp],
    "strictb200_attn_decode_noalloc": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp],
    "strictb200_embedding_bf16": [vp, vp, vp, i64, i64, i64, vp],
    "strictb200_argmax": [vp, vp, i64, i64, vp],
    "strictb200_model_create": [vp, C.POINTER(ModelConfig), C.POINTER(vp)],
    "strictb200_model_destroy": [vp],
    "strictb200_model_init_random": [vp, u64],
    "strictb200_model_set_tensor": [vp, C.c_char_p, vp, sz],
    "strictb200_model_get_tensor": [vp, C.c_char_p, vp, sz],
    "strictb200_model_weight_bytes": [vp, C.POINTER(u64)],
    "strictb200_model_set_graph": [vp, i32],
    "strictb200_kv_create": [vp, i32, i32, C.POINTER(vp)],
    "strictb200_kv_destroy": [vp],
    "strictb200_kv_reset": [vp],
    "strictb200_kv_lens": [vp, vp],
    "strictb200_kv_fill_synthetic": [vp, u64, i32],
    "strictb200_prefill": [vp, vp, vp, vp, i32, i32, vp, vp],
    "strictb200_decode_step": [vp, vp, vp, vp, vp],
    "strictb200_generate": [vp, vp, vp, i32, vp],
    "strictb200_decode_steps_device": [vp, vp, vp, i32],
    "strictb200_kv_device_ids": [vp, C.POINTER(vp)],
    "strictb200_decode_bytes": [vp, vp, C.POINTER(u64)],
    "strictb200_profile_decode": [vp, vp, i32, vp, vp, i32],
    "strictb200_tp_unique_id": [vp],
    "strictb200_tp_init": [vp, i32, i32, vp],
    "strictb200_tp_info": [vp, C.POINTER(i32), C.POINTER(i32)],
    "strictb200_tp_comm_handle": [vp, vp],
    "strictb200_tp_comm_open": [vp, vp],
    "strictb200_tp_allreduce_f32": [vp, vp, i64],
    "strictb200_tp_allreduce_rownorm": [vp, vp, i32, vp, vp, vp, vp, f32, i64, i64, vp, vp, vp],
    "strictb200_tp_comm_open_absent_peers": [vp, i32],
}


def lib():
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m strict_b200.build` (there is no CPU path)")
        L = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        L.strictb200_version.restype = C.c_int
        L.strictb200_version.argtypes = []
        L.strictb200_last_error.restype = C.c_char_p
        L.strictb200_last_error.argtypes = []
        L.strictb200_build_id.restype = C.c_char_p
        L.strictb200_build_id.argtypes = []
        _lib = L
    return _lib


def check(status):
    if status == OK:
        return
    msg = lib().strictb200_last_error().decode(errors="replace")
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)  # the reference throws NotSupportedException here
    if status == ERR_INVALID_ARG:
        raise ValueError(msg)
    if status == ERR_OOM:
        raise MemoryError(msg)
    raise KernelException(status, msg)


def compile_to_ptx(cuda_c, name, options=("--gpu-architecture=compute_100a",)):
    """CUDA C text -> PTX text through NVRTC (no GPU needed). Raises ValueError with the compiler's
    log on a compile error, NotImplementedError where NVRTC is not installed."""
    opts = (C.c_char_p * max(1, len(options)))(*[o.encode() for o in options])
    size = sz()
    check(lib().strictb200_compile_to_ptx(cuda_c.encode(), name.encode(), opts, len(options), None, 0, C.byref(size)))
    buf = C.create_string_buffer(size.value)
    check(lib().strictb200_compile_to_ptx(cuda_c.encode(), name.encode(), opts, len(options), buf, size.value, C.byref(size)))
    return buf.value.decode()


def ptr(a):
    """Host pointer of a C-contiguous numpy array (or None)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)
