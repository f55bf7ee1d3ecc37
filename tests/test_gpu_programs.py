"""GPU parity of the larger element-wise instruction set (conditionals, loops, calls placed
inline, loads at computed indices) through the C ABI against the oracle's interpreter, bit for
bit; the step budget that keeps any program from hanging the GPU; routing by the reference's
complexity rule; a model loaded from tensors packaged beside the bytecode."""
import ctypes as C
import zipfile

import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import native as N, packaging
from strict_b200.kernel import DeviceVariable as DV
from test_host_mirror import FILTERS

pytestmark = pytest.mark.gpu
L = N.lib


@pytest.mark.parametrize("name,n_arrays,scalars", [("Clamp", 1, []), ("Brighten", 1, [0.3]), ("Blur5", 1, []), ("Checker", 2, []), ("Triangle", 1, []),
                                                   ("Twice", 1, [])])
@pytest.mark.parametrize("n", [1, 1000, (1 << 20) + 3])
def test_program_matches_oracle(ctx, oracle, rng, name, n_arrays, scalars, n):
    compiled = sb.InstructionsToCuda().compile(FILTERS.by_name[name], FILTERS)
    arrays = [rng.standard_normal(n).astype(np.float32) for _ in range(n_arrays)]
    want = oracle.ew_program2(np.array(compiled.code, np.int32), arrays, scalars, compiled.consts, n)
    dv = [DV.of(ctx, a) for a in arrays]
    out = DV(ctx, n)
    compiled.launch(ctx, *dv, *scalars, out, n)
    assert np.array_equal(out.to_host(), want)
    assert ctx.device_status() == 0
    for v in dv + [out]:
        v.free()


def test_step_budget_ends_a_runaway_program(ctx, oracle):
    """A loop of a million iterations per element runs past the 65536-instruction budget: the
    element gets 0, the error word is set, nothing hangs, and the context keeps working."""
    m = sb.InstructionsToCuda().compile(sb.Method("Spin(a Number) Number", ["\tmutable t = 0", "\tfor 1000000", "\t\tt = t + a", "\tt"]))
    a, out = DV.of(ctx, np.ones(64, np.float32)), DV(ctx, 64)
    m.launch(ctx, a, out, 64)
    with pytest.raises(N.KernelException) as e:
        ctx.device_status()
    assert e.value.status == N.ERR_TIMEOUT
    assert (out.to_host() == 0).all()
    with pytest.raises(RuntimeError):
        oracle.ew_program2(np.array(m.code, np.int32), [np.ones(4, np.float32)], [], m.consts, 4)
    ok = sb.InstructionsToCuda().compile(sb.Method("Sum(a Number) Number", ["\tmutable t = 0", "\tfor 1000", "\t\tt = t + a", "\tt"]))
    ok.launch(ctx, a, out, 64)
    assert ctx.device_status() == 0 and (out.to_host() == 1000).all()


def test_malformed_programs_are_rejected(ctx):
    out = DV(ctx, 4)
    ptrs = (C.c_void_p * 1)(out.p.value)

    def run(code):
        code = np.array(code, np.int32)
        N.check(L().strictb200_ew_program2(ctx.h, N.ptr(code), len(code), ptrs, 1, None, 0, None, 0, out.p, 4))
    with pytest.raises(ValueError):
        run([[13, 9, 0, 0]])                       # jump beyond the program
    with pytest.raises(ValueError):
        run([[16, 0, 2, 16], [7, 0, 0, 0]])        # loop without its end
    with pytest.raises(ValueError):
        run([[19, 0, 0, 32]])                      # slot out of range
    with pytest.raises(ValueError):
        run([[18, 3, 0, 0]])                       # array out of range
    with pytest.raises(NotImplementedError):
        run([[21, 0, 0, 0]])
    run([[20, 0, 0, 0], [7, 0, 0, 0]])             # LOAD_INDEX; RETURN
    assert out.to_host().tolist() == [0.0, 1.0, 2.0, 3.0]


def test_runner_routes_by_complexity(ctx, oracle, rng, tmp_path):
    r = sb.Runner(str(tmp_path / "Filters.strict"), FILTERS)
    small = DV.of(ctx, rng.standard_normal(1000).astype(np.float32))
    out = DV(ctx, 1000)
    assert r.TryRunOnGpu(ctx, "Blur5", small, out, 1000) is None  # below the threshold: stays with the host's VM
    n = 1 << 20
    x = rng.standard_normal(n).astype(np.float32)
    big, out = DV.of(ctx, x), DV(ctx, n)
    plan, compiled = r.Plan("Blur5", n)
    assert plan == "gpu.launch"
    assert r.TryRunOnGpu(ctx, "Blur5", big, out, n) is out
    assert np.array_equal(out.to_host(), oracle.ew_program2(np.array(compiled.code, np.int32), [x], [], compiled.consts, n))


def test_model_from_tensors_beside_the_bytecode(ctx, oracle, tmp_path):
    cfg = dict(arch=1, n_layers=2, d_model=256, n_q_heads=4, n_kv_heads=2, head_dim=128, d_ff=512, vocab=1024, max_pos=128, tied=0, eps=1e-6,
               rope_theta=1e6)
    source = sb.Model(ctx, cfg).init_random(4)
    names = {"embed": (np.float32, 1024 * 256), "normf.g": (np.float32, 256), "head.q": (np.uint8, 1024 * 256), "head.s": (np.float32, 1024)}
    for l in range(2):
        for n_, (rows, cols) in {"wqkv": (1024, 256), "wo": (256, 512), "wgu": (1024, 256), "wdown": (256, 512)}.items():
            names[f"layers.{l}.{n_}.q"] = (np.uint8, rows * cols)
            names[f"layers.{l}.{n_}.s"] = (np.float32, rows)
        for g, k in (("norm1.g", 256), ("norm2.g", 256), ("qnorm.g", 128), ("knorm.g", 128)):
            names[f"layers.{l}.{g}"] = (np.float32, k)
    path = str(tmp_path / "Chat.strictbinary")
    with zipfile.ZipFile(path, "w") as z:
        z.writestr("Chat.bytecode", b"\x00\x01")
    packaging.save_model(path, source, names)
    assert packaging.bytecode_entries(path) == ["Chat"]
    loaded = packaging.load_model(ctx, path)
    toks = oracle.gen_tokens(5, 1, 2 * 8, cfg["vocab"]).reshape(2, 8)
    a, b = source.new_cache(2, 32), loaded.new_cache(2, 32)
    na, la = a.prefill(toks, want_logits=True)
    nb, lb = b.prefill(toks, want_logits=True)
    assert np.array_equal(la, lb) and np.array_equal(na, nb)
    assert np.array_equal(a.generate(na, 6), b.generate(nb, 6))
    for o in (a, b, source, loaded):
        o.dispose()
