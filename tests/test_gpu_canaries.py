"""Guard words around outputs: kernels write inside their output buffers only. Every output is
carved out of a larger poisoned allocation; after the call the bytes in front of and behind it
must still hold the poison (the memory-checker tools are not available on the GPU pool, so
out-of-bounds writes are looked for this way, on shapes that do not fill the kernels' tiles)."""
import ctypes as C

import numpy as np
import pytest

from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV

pytestmark = pytest.mark.gpu
L = N.lib
GUARD = 4096  # bytes on each side
POISON = 0xA5


class Guarded:
    """A device buffer of `nbytes` with GUARD poisoned bytes on both sides."""

    def __init__(self, ctx, nbytes):
        self.ctx, self.nbytes = ctx, nbytes
        self.whole = DV(ctx, nbytes + 2 * GUARD, np.uint8)
        N.check(L().strictb200_memset(ctx.h, self.whole.p, POISON, nbytes + 2 * GUARD))
        self.p = C.c_void_p(self.whole.p.value + GUARD)

    def check(self):
        host = self.whole.to_host()
        assert (host[:GUARD] == POISON).all(), "write in front of the buffer"
        assert (host[GUARD + self.nbytes:] == POISON).all(), "write behind the buffer"
        return host[GUARD:GUARD + self.nbytes]

    def free(self):
        self.whole.free()


def test_outputs_stay_inside_their_buffers(ctx, oracle, rng):
    # GEMM, tokens and channels that do not fill a tile, fp32 and bf16 outputs, all kernels
    M, N_, K = 37, 1008, 1536
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xq, sx = oracle.split_rows_device_layout(x)
    wq, sw = oracle.gen_qlinear(2, 5, N_, K)
    dxq, dsx, dwq, dsw = DV.of(ctx, xq), DV.of(ctx, sx), DV.of(ctx, wq), DV.of(ctx, sw)
    for kernel in (0, 2, 3):
        for out_dtype, esz in ((0, 2), (1, 4)):
            g = Guarded(ctx, M * N_ * esz)
            N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, dxq.p, dsx.p, dwq.p, dsw.p, g.p, out_dtype, kernel))
            g.check()
            g.free()
    # skinny kernel
    g = Guarded(ctx, 7 * N_ * 4)
    N.check(L().strictb200_gemm_fp8(ctx.h, 7, N_, K, dxq.p, dsx.p, dwq.p, dsw.p, g.p, 1, 1))
    g.check(), g.free()
    # the split of odd row counts: 16*ceil(M/8) rows are the buffer
    for m in (1, 9, 37):
        xb = DV.of(ctx, oracle.f32_to_bf16(x[:m]))
        q, s = Guarded(ctx, 16 * ((m + 7) // 8) * K), Guarded(ctx, m * 4)
        N.check(L().strictb200_quantize_rows(ctx.h, xb.p, m, K, q.p, s.p))
        q.check(), s.check(), q.free(), s.free(), xb.free()
    # row kernels
    d = 1024
    xb, gain = DV.of(ctx, oracle.f32_to_bf16(rng.standard_normal((5, d)).astype(np.float32))), DV.of(ctx, np.ones(d, np.float32))
    y = Guarded(ctx, 5 * d * 2)
    N.check(L().strictb200_rmsnorm(ctx.h, xb.p, None, gain.p, 1e-6, 5, d, y.p))
    y.check(), y.free()
    gu = DV.of(ctx, oracle.f32_to_bf16(rng.standard_normal((3, 2 * 3072)).astype(np.float32)))
    y = Guarded(ctx, 3 * 3072 * 2)
    N.check(L().strictb200_swiglu(ctx.h, gu.p, 3, 3072, y.p))
    y.check(), y.free()
    # attention: ragged lengths, outputs of both phases
    B, S, Hq, Hkv, D, maxlen = 2, 200, 8, 2, 128, 256
    q = DV.of(ctx, oracle.f32_to_bf16(rng.standard_normal((B, S, Hq, D)).astype(np.float32)))
    kc = DV.of(ctx, oracle.f32_to_bf16(rng.standard_normal((B, Hkv, maxlen, D)).astype(np.float32)))
    lens = DV.of(ctx, np.array([200, 129], np.int32))
    for mode in (0, 1, 2):
        with ctx.option("attn_tc", mode):
            o = Guarded(ctx, B * S * Hq * D * 2)
            N.check(L().strictb200_attn_prefill(ctx.h, q.p, kc.p, kc.p, lens.p, None, B, S, Hq, Hkv, D, maxlen, 0.088, o.p))
            o.check(), o.free()
    o = Guarded(ctx, B * Hq * D * 2)
    N.check(L().strictb200_attn_decode(ctx.h, q.p, kc.p, kc.p, lens.p, B, Hq, Hkv, D, maxlen, 0.088, o.p))
    o.check(), o.free()
    # element-wise and image kernels on sizes that do not fill a vector or a strip
    a = DV.of(ctx, rng.standard_normal(1003).astype(np.float32))
    o = Guarded(ctx, 1003 * 4)
    N.check(L().strictb200_ew_binary(ctx.h, 0, a.p, a.p, o.p, 1003))
    o.check(), o.free()
    for w, h in ((48, 37), (1000, 33), (16, 5)):
        px = DV.of(ctx, rng.integers(0, 256, w * h * 3, dtype=np.uint8))
        o = Guarded(ctx, w * h * 3)
        N.check(L().strictb200_blur5x5_rgb8(ctx.h, px.p, o.p, w, h))
        assert np.array_equal(o.check(), oracle.blur5x5_rgb8(px.to_host(), w, h))
        o.free(), px.free()
    argm = Guarded(ctx, 9 * 4)
    logits = DV.of(ctx, rng.standard_normal((9, 50257)).astype(np.float32))
    N.check(L().strictb200_argmax(ctx.h, logits.p, 9, 50257, argm.p))
    argm.check(), argm.free()
    assert ctx.device_status() == 0
