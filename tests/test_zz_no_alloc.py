"""strictb200_attn_decode_noalloc — decode attention for hosts that cannot allocate.

Some users of the library run it from a serving loop that must never hit cudaMalloc/cudaFree
(both stall every stream of the process while they run), or from a host that reserved all GPU
memory for its own pool before the library was loaded, so the driver has nothing left to hand out.
The entry point keeps its split-KV partial results in a 4 MiB array compiled into the library
instead. Its output must be the same as strictb200_attn_decode's, call after call, even though
the array keeps whatever the previous call left in it, and within the attention tests' bars of
the CPU oracle.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest

from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV

pytestmark = pytest.mark.gpu
L = N.lib


def _case(ctx, oracle, seed, B, Hq, Hkv, maxlen, lens):
    D = 128
    rng = np.random.default_rng(seed)
    q = oracle.f32_to_bf16(rng.standard_normal((B, Hq, D)).astype(np.float32))
    kc = oracle.f32_to_bf16(rng.standard_normal((B, Hkv, maxlen, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((B, Hkv, maxlen, D)).astype(np.float32))
    dq, dk, dv, dl = DV.of(ctx, q), DV.of(ctx, kc), DV.of(ctx, vc), DV.of(ctx, np.array(lens, np.int32))
    want, got = DV(ctx, B * Hq * D, np.uint16), DV(ctx, B * Hq * D, np.uint16)
    scale = float(1.0 / np.sqrt(D))
    N.check(L().strictb200_attn_decode(ctx.h, dq.p, dk.p, dv.p, dl.p, B, Hq, Hkv, D, maxlen, scale, want.p))
    N.check(L().strictb200_attn_decode_noalloc(ctx.h, dq.p, dk.p, dv.p, dl.p, B, Hq, Hkv, D, maxlen, scale, got.p))
    a, b = oracle.bf16_to_f32(want.to_host()), oracle.bf16_to_f32(got.to_host())
    for v in (dq, dk, dv, dl, want, got):
        v.free()
    # the entry against the CPU oracle as well (not only against the allocating entry): the bars of the attention tests
    ref = oracle.round_bf16(oracle.attn_decode(oracle.bf16_to_f32(q), oracle.bf16_to_f32(kc), oracle.bf16_to_f32(vc), np.array(lens, np.int32), scale))
    err = np.abs(b.reshape(ref.shape) - ref)
    assert err.max() <= 2e-2 and err.mean() / np.abs(ref).mean() <= 5e-3, (err.max(), err.mean())
    return a, b


def test_noalloc_matches_allocating_entry_twice_in_a_row(ctx, oracle):
    # first call: long ragged contexts, several key chunks per sequence fill the built-in scratch
    a, b = _case(ctx, oracle, 1, 4, 32, 8, 4096, [4096, 1, 2049, 777])
    assert np.isfinite(b).all()
    assert np.abs(a - b).max() <= 2e-2 and np.abs(a - b).mean() / np.abs(a).mean() <= 5e-3  # the attention tests' tolerance
    assert np.array_equal(a, b)  # same kernels, same order of operations
    # second call right after it: other shapes and lengths read the scratch the first call left behind
    a, b = _case(ctx, oracle, 2, 3, 8, 2, 1024, [100, 1024, 65])
    assert np.abs(a - b).max() <= 2e-2 and np.abs(a - b).mean() / np.abs(a).mean() <= 5e-3
    assert np.array_equal(a, b)


def test_noalloc_rejects_what_does_not_fit(ctx):
    # 4096 sequences x 32 heads x 130 floats of partial results per key chunk is far beyond 4 MiB;
    # the size check comes before any pointer is touched
    dummy = DV(ctx, 16, np.uint16)
    with pytest.raises(ValueError, match="built-in scratch"):
        N.check(L().strictb200_attn_decode_noalloc(ctx.h, dummy.p, dummy.p, dummy.p, dummy.p, 4096, 32, 8, 128, 4096, 0.1, dummy.p))
    dummy.free()
