"""ctypes view of the CPU oracle (oracle/oracle.cpp).

TEST INFRASTRUCTURE: imported only by tests, the smoke check and the benchmark's
cpu_baseline / reference arm. The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ARCH_GPT2, ARCH_QWEN3 = 0, 1


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("oracle.cpp", "oracle_num.h")]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        _LIB = C.CDLL(so)
        L = _LIB
        L.or_stream_key.restype = C.c_uint64
        L.or_stream_key.argtypes = [C.c_uint64, C.c_uint64]
        L.or_model_create.restype = C.c_void_p
        L.or_model_create.argtypes = [C.c_void_p, C.c_float, C.c_float, C.c_uint64]
        L.or_model_free.argtypes = [C.c_void_p]
        L.or_model_tensor.restype = C.c_int64
        L.or_model_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
        L.or_model_retie.argtypes = [C.c_void_p]
        L.or_state_create.restype = C.c_void_p
        L.or_state_create.argtypes = [C.c_void_p, C.c_int, C.c_int]
        for f in (L.or_state_free, L.or_state_reset):
            f.argtypes = [C.c_void_p]
        L.or_state_lens.argtypes = [C.c_void_p, C.c_void_p]
        L.or_state_fill_synthetic.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int]
        L.or_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.or_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ------------------------------------------------------------------ generator / formats
def gen_normal(seed, tensor, count, std=1.0, first=0):
    out = np.empty(count, np.float32)
    lib().or_gen_normal(C.c_uint64(seed), C.c_uint64(tensor), C.c_int64(first), C.c_int64(count), C.c_float(std), _p(out))
    return out


def gen_tokens(seed, tensor, count, vocab):
    out = np.empty(count, np.int32)
    lib().or_gen_tokens(C.c_uint64(seed), C.c_uint64(tensor), C.c_int64(count), C.c_uint32(vocab), _p(out))
    return out


def gen_qlinear(seed, tensor, rows, K, std=0.02):
    q = np.empty((rows, K), np.uint8)
    s = np.empty(rows, np.float32)
    lib().or_gen_qlinear(C.c_uint64(seed), C.c_uint64(tensor), C.c_int64(rows), C.c_int64(K), C.c_float(std), _p(q), _p(s))
    return q, s


def f32_to_bf16(x):
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().or_f32_to_bf16(_p(x), C.c_int64(x.size), _p(out))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().or_bf16_to_f32(_p(x), C.c_int64(x.size), _p(out))
    return out


def round_bf16(x):
    return bf16_to_f32(f32_to_bf16(x))


def f32_to_e4m3(x):
    x = _f32(x)
    out = np.empty(x.shape, np.uint8)
    lib().or_f32_to_e4m3(_p(x), C.c_int64(x.size), _p(out))
    return out


def e4m3_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint8)
    out = np.empty(x.shape, np.float32)
    lib().or_e4m3_to_f32(_p(x), C.c_int64(x.size), _p(out))
    return out


# ------------------------------------------------------------------ element-wise surface
def ew_binary(op, a, b):
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    if lib().or_ew_binary(C.c_int(op), _p(a), _p(b), _p(out), C.c_int64(a.size)):
        raise NotImplementedError(op)
    return out


def ew_program(code, arrays, scalars, consts, n):
    code = np.ascontiguousarray(code, dtype=np.int32).reshape(-1, 4)
    arrs = [_f32(a) for a in arrays]
    ptrs = (C.c_void_p * max(1, len(arrs)))(*[a.ctypes.data for a in arrs])
    sc = _f32(scalars if len(scalars) else [0])
    co = _f32(consts if len(consts) else [0])
    out = np.empty(n, np.float32)
    if lib().or_ew_program(_p(code), C.c_int(len(code)), ptrs, _p(sc), _p(co), _p(out), C.c_int64(n)):
        raise NotImplementedError("opcode")
    return out


def ew_program2(code, arrays, scalars, consts, n):
    """The larger instruction set (conditionals, loops, indexed loads); raises RuntimeError if an
    element ran past the step budget."""
    code = np.ascontiguousarray(code, dtype=np.int32).reshape(-1, 4)
    arrs = [_f32(a) for a in arrays]
    ptrs = (C.c_void_p * max(1, len(arrs)))(*[a.ctypes.data for a in arrs])
    sc = _f32(scalars if len(scalars) else [0])
    co = _f32(consts if len(consts) else [0])
    out = np.empty(n, np.float32)
    rc = lib().or_ew_program2(_p(code), C.c_int(len(code)), ptrs, _p(sc), _p(co), _p(out), C.c_int64(n))
    if rc == 1:
        raise NotImplementedError("opcode")
    if rc == 2:
        raise RuntimeError("step budget exceeded")
    return out


# ------------------------------------------------------------------ image workloads
def blur5x5_rgb8(pixels, width, height, iterations=1):
    """pixels uint8 [height*width*3]; returns the image after `iterations` in-place blur passes."""
    px = np.array(pixels, dtype=np.uint8).reshape(-1).copy()
    assert px.size == width * height * 3
    lib().or_blur5x5_rgb8_inplace(_p(px), C.c_int(width), C.c_int(height), C.c_int(iterations))
    return px


def adjust_brightness(flat, offset, count, flat_width, channels, brightness, clamp01=False):
    out = _f32(flat).reshape(-1).copy()
    lib().or_adjust_brightness(_p(out), C.c_int64(offset), C.c_int64(count), C.c_int(flat_width), C.c_int(channels),
                               C.c_double(brightness), C.c_int(1 if clamp01 else 0))
    return out


# ------------------------------------------------------------------ primitives
def split_rows(x):
    """Two-term E4M3 split of bf16-valued rows: returns (hi codes, lo codes, hi+lo/16 as fp32, scale)."""
    x = _f32(x)
    M, K = x.shape
    hi = np.empty((M, K), np.uint8)
    lo = np.empty((M, K), np.uint8)
    eff = np.empty((M, K), np.float32)
    s = np.empty(M, np.float32)
    lib().or_split_rows(_p(x), C.c_int64(M), C.c_int64(K), _p(hi), _p(lo), _p(eff), _p(s))
    return hi, lo, eff, s


def split_rows_device_layout(x):
    """The split in the row order the device kernels use: tokens in groups of 8, each group as
    8 hi rows followed by 8 lo rows; rows of padding tokens are zero."""
    hi, lo, _, s = split_rows(x)
    M, K = hi.shape
    G = (M + 7) // 8
    out = np.zeros((G * 16, K), np.uint8)
    for m in range(M):
        out[16 * (m // 8) + m % 8] = hi[m]
        out[16 * (m // 8) + 8 + m % 8] = lo[m]
    return out, s


def quant_weight_rows(x):
    x = _f32(x)
    M, K = x.shape
    q = np.empty((M, K), np.uint8)
    s = np.empty(M, np.float32)
    lib().or_quant_weight_rows(_p(x), C.c_int64(M), C.c_int64(K), _p(q), _p(s))
    return q, s


def linear_fp8w(x, wq, sw):
    """(x . W^T) * sw with bf16-valued x and E4M3 weights; fp32, unrounded."""
    x = _f32(x)
    M, K = x.shape
    N = wq.shape[0]
    out = np.empty((M, N), np.float32)
    lib().or_linear_fp8w(_p(x), _p(np.ascontiguousarray(wq)), _p(_f32(sw)), C.c_int64(M), C.c_int64(N), C.c_int64(K), _p(out))
    return out


def quantize_weights_int8(w):
    """int8 weights with one fp32 scale per output channel (absmax / 127)."""
    w = _f32(w)
    N, K = w.shape
    q = np.empty((N, K), np.int8)
    s = np.empty(N, np.float32)
    lib().or_quantize_weights_int8(_p(w), C.c_int64(N), C.c_int64(K), _p(q), _p(s))
    return q, s


def quantize_rows_int8(x):
    """Two int8 terms per element of bf16-valued rows, x ~ s * (128 * hi + lo): (hi, lo, s)."""
    x = _f32(x)
    M, K = x.shape
    hi = np.empty((M, K), np.int8)
    lo = np.empty((M, K), np.int8)
    s = np.empty(M, np.float32)
    lib().or_quantize_rows_int8(_p(x), C.c_int64(M), C.c_int64(K), _p(hi), _p(lo), _p(s))
    return hi, lo, s


def gemm_int8w(x, wq, sw):
    """bf16 bit patterns of ((x . Wq^T) * sx) * sw with bf16-valued x and int8 weights."""
    x = _f32(x)
    M, K = x.shape
    wq = np.ascontiguousarray(wq, dtype=np.int8)
    N = wq.shape[0]
    out = np.empty((M, N), np.uint16)
    lib().or_gemm_int8w(_p(x), _p(wq), _p(_f32(sw)), C.c_int64(M), C.c_int64(N), C.c_int64(K), _p(out))
    return out


def gemm_f32(x, w, b=None):
    x, w = _f32(x), _f32(w)
    M, K = x.shape
    N = w.shape[0]
    out = np.empty((M, N), np.float32)
    bb = _f32(b) if b is not None else None
    lib().or_gemm_f32(_p(x), _p(w), _p(bb) if bb is not None else None, C.c_int64(M), C.c_int64(N), C.c_int64(K), _p(out))
    return out


def rmsnorm(x, g, eps):
    x, g = _f32(x), _f32(g)
    y = np.empty_like(x)
    lib().or_rmsnorm(_p(x), _p(g), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_float(eps), _p(y))
    return y


def layernorm(x, g, b, eps):
    x, g, b = _f32(x), _f32(g), _f32(b)
    y = np.empty_like(x)
    lib().or_layernorm(_p(x), _p(g), _p(b), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_float(eps), _p(y))
    return y


def gelu_tanh(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().or_gelu_tanh(_p(x), C.c_int64(x.size), _p(y))
    return y


def swiglu(gate, up):
    gate, up = _f32(gate), _f32(up)
    y = np.empty_like(gate)
    lib().or_swiglu(_p(gate), _p(up), C.c_int64(gate.size), _p(y))
    return y


def rope_table(n_pos, D, theta):
    c = np.empty((n_pos, D // 2), np.float32)
    s = np.empty((n_pos, D // 2), np.float32)
    lib().or_rope_table(C.c_int(n_pos), C.c_int(D), C.c_float(theta), _p(c), _p(s))
    return c, s


def qknorm_rope(x, g, pos, eps, theta):
    x, g = _f32(x), _f32(g)
    T, H, D = x.shape
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    out = np.empty_like(x)
    lib().or_qknorm_rope(_p(x), _p(g), _p(pos), C.c_int64(T), C.c_int(H), C.c_int(D), C.c_float(eps), C.c_float(theta), _p(out))
    return out


def attn_prefill(q, k, v, lens, scale):
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    out = np.zeros_like(q)
    lib().or_attn_prefill(_p(q), _p(k), _p(v), _p(lens), C.c_int(B), C.c_int(S), C.c_int(Hq), C.c_int(Hkv), C.c_int(D), C.c_float(scale), _p(out))
    return out


def attn_decode(q, kc, vc, lens, scale):
    q, kc, vc = _f32(q), _f32(kc), _f32(vc)
    B, Hq, D = q.shape
    _, Hkv, maxlen, _ = kc.shape
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    out = np.empty_like(q)
    lib().or_attn_decode(_p(q), _p(kc), _p(vc), _p(lens), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(maxlen), C.c_int(D), C.c_float(scale), _p(out))
    return out


def argmax(x):
    x = _f32(x)
    out = np.empty(x.shape[0], np.int32)
    lib().or_argmax(_p(x), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), _p(out))
    return out


def num_threads():
    return lib().or_num_threads()


# ------------------------------------------------------------------ model
class Model:
    """CPU restatement of a GPT-2 / Qwen3 stack. cfg keys: arch, n_layers, d_model, n_q_heads,
    n_kv_heads, head_dim, d_ff, vocab, max_pos, tied, eps, rope_theta."""

    def __init__(self, cfg, seed):
        self.cfg = dict(cfg)
        icfg = np.array([cfg["arch"], cfg["n_layers"], cfg["d_model"], cfg["n_q_heads"], cfg["n_kv_heads"],
                         cfg["head_dim"], cfg["d_ff"], cfg["vocab"], cfg["max_pos"], cfg["tied"]], np.int32)
        self.h = lib().or_model_create(_p(icfg), C.c_float(cfg["eps"]), C.c_float(cfg["rope_theta"]), C.c_uint64(seed))
        self.states = []

    def tensor(self, name, dtype):
        ptr = C.c_void_p()
        n = lib().or_model_tensor(self.h, name.encode(), C.byref(ptr))
        if not ptr.value:
            raise KeyError(name)
        buf = (C.c_uint8 * n).from_address(ptr.value)
        return np.frombuffer(buf, dtype=dtype)

    def retie(self):
        lib().or_model_retie(self.h)

    def new_state(self, B, maxlen):
        return State(self, B, maxlen)

    def close(self):
        if self.h:
            lib().or_model_free(self.h)
            self.h = None


class State:
    def __init__(self, model, B, maxlen):
        self.model, self.B = model, B
        self.h = lib().or_state_create(model.h, C.c_int(B), C.c_int(maxlen))

    def prefill(self, tokens, lens):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        B, S = tokens.shape
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        logits = np.empty((B, self.model.cfg["vocab"]), np.float32)
        if lib().or_prefill(self.model.h, self.h, _p(tokens), _p(lens), C.c_int(B), C.c_int(S), _p(logits)):
            raise ValueError("prefill does not fit the cache")
        return logits

    def decode(self, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        logits = np.empty((self.B, self.model.cfg["vocab"]), np.float32)
        if lib().or_decode(self.model.h, self.h, _p(ids), C.c_int(self.B), _p(logits)):
            raise ValueError("cache full")
        return logits

    def fill_synthetic(self, seed, length):
        """Benchmark set-up: cheap pseudo-random keys/values at positions [0,length)."""
        if lib().or_state_fill_synthetic(self.model.h, self.h, C.c_uint64(seed), C.c_int(length)):
            raise ValueError("length outside the cache")

    def lens(self):
        out = np.empty(self.B, np.int32)
        lib().or_state_lens(self.h, _p(out))
        return out

    def reset(self):
        lib().or_state_reset(self.h)

    def close(self):
        if self.h:
            lib().or_state_free(self.h)
            self.h = None
