"""GPU parity tests of the individual kernels, called through the C ABI, against the CPU oracle
on the same seeded inputs. Integer/byte results must be bit-exact; floating point uses the
tolerance written next to each check."""
import json
import os

import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "reference_known_answers.json")))
L = N.lib


def bf16_dev(ctx, O, x):
    return DV.of(ctx, O.f32_to_bf16(x))


def bf16_host(O, dv, shape):
    return O.bf16_to_f32(dv.to_host()).reshape(shape)


# ------------------------------------------------------------------ reference known answers
@pytest.mark.parametrize("case", GOLD["execute"], ids=lambda c: c["case"])
def test_reference_known_answers(ctx, case):
    """ParseGenerateCudaAndExecute (Strict.Compiler.Cuda.Tests/CSharpToCudaTranspilerTests.cs:46-57)."""
    method = sb.InstructionsToCuda().compile(sb.Method(case["signature"], ["\t" + case["body"]]))
    kernel = sb.Kernel.__new__(sb.Kernel)
    kernel.Context = ctx
    output = DV(ctx, 1)
    if "first" in case:
        first, second = DV.of(ctx, np.array([case["first"]], np.float32)), DV.of(ctx, np.array([case["second"]], np.float32))
        kernel.Run(method, first, second, output, case["count"])
    else:
        inp = DV.of(ctx, np.array([case["input"]], np.float32))
        kernel.Run(method, inp, case["width"], case["height"], case["initialDepth"], output)
    assert output[0] == case["expected"]


def test_stale_fixture_ten_elements(ctx):
    n = GOLD["stale_fixture_n"]
    a, b, out = DV.of(ctx, np.full(n, 1.0, np.float32)), DV.of(ctx, np.full(n, 2.0, np.float32)), DV(ctx, n)
    for op, want in ((0, 3.0), (1, -1.0), (2, 2.0)):
        N.check(L().strictb200_ew_binary(ctx.h, op, a.p, b.p, out.p, n))
        assert np.all(np.abs(out.to_host() - want) < 1e-6)


@pytest.mark.parametrize("n", [0, 1, 3, 1000, 1 << 20, (1 << 22) + 5])
def test_ew_binary_bit_exact(ctx, oracle, rng, n):
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    da, db, do = DV.of(ctx, a), DV.of(ctx, b), DV(ctx, max(n, 1))
    for op in range(4):
        N.check(L().strictb200_ew_binary(ctx.h, op, da.p, db.p, do.p, n))
        if n:
            assert np.array_equal(do.to_host()[:n], oracle.ew_binary(op, a, b))
    with pytest.raises(NotImplementedError):
        N.check(L().strictb200_ew_binary(ctx.h, 7, da.p, db.p, do.p, n))
    for v in (da, db, do):
        v.free()


def test_ew_binary_unaligned_views(ctx, oracle, rng):
    a = rng.standard_normal(1001).astype(np.float32)
    da, do = DV.of(ctx, a), DV(ctx, 1001)
    import ctypes as C
    pa = C.c_void_p(da.p.value + 4)
    N.check(L().strictb200_ew_binary(ctx.h, 2, pa, pa, do.p, 1000))
    assert np.array_equal(do.to_host()[:1000], a[1:] * a[1:])


def test_ew_program_matches_oracle(ctx, oracle, rng):
    m = sb.InstructionsToCuda().compile(sb.Method("F(a Number, b Number, c Number, width Number) Number", ["\t(a + b) * c / width - 1.5"]))
    n = 5000
    arrs = [rng.standard_normal(n).astype(np.float32) for _ in range(3)]
    dv = [DV.of(ctx, x) for x in arrs]
    out = DV(ctx, n)
    m.launch(ctx, dv[0], dv[1], dv[2], 3, out, n)
    want = oracle.ew_program(np.array(m.code, np.int32), arrs, [3.0], m.consts, n)
    assert np.array_equal(out.to_host(), want)


def test_invalid_arguments(ctx):
    with pytest.raises(ValueError):
        N.check(L().strictb200_ew_binary(ctx.h, 0, None, None, None, 4))
    with pytest.raises(ValueError):
        N.check(L().strictb200_gemm_fp8(ctx.h, 4, 100, 64, None, None, None, None, None, 0, 0))
    out = DV(ctx, 4)
    code = np.array([[0, 3, 0, 0], [7, 0, 0, 0]], np.int32)  # array index out of range
    import ctypes as C
    with pytest.raises(ValueError):
        N.check(L().strictb200_ew_program(ctx.h, N.ptr(code), 2, (C.c_void_p * 1)(out.p.value), 1, None, 0, None, 0, out.p, 4))


# ------------------------------------------------------------------ generator: bit-exact with the oracle
def test_generator_bit_exact(ctx, oracle):
    for seed, tensor, first, count in ((0, 1, 0, 100001), (5, 40, 12345, 4096), (2, 17, 1, 7)):
        out = DV(ctx, count)
        N.check(L().strictb200_gen_normal_f32(ctx.h, seed, tensor, first, count, 0.02, out.p))
        assert np.array_equal(out.to_host(), oracle.gen_normal(seed, tensor, count, std=0.02, first=first))
        ob = DV(ctx, count, np.uint16)
        N.check(L().strictb200_gen_normal_bf16(ctx.h, seed, tensor, first, count, 0.02, ob.p))
        assert np.array_equal(ob.to_host(), oracle.f32_to_bf16(oracle.gen_normal(seed, tensor, count, std=0.02, first=first)))
    t = DV(ctx, 5000, np.int32)
    N.check(L().strictb200_gen_tokens(ctx.h, 1, 1, 5000, 50257, t.p))
    assert np.array_equal(t.to_host(), oracle.gen_tokens(1, 1, 5000, 50257))


@pytest.mark.parametrize("K", [256, 1023, 4096])
def test_weight_generator_bit_exact(ctx, oracle, K):
    rows = 37
    q, s = DV(ctx, rows * K, np.uint8), DV(ctx, rows)
    N.check(L().strictb200_gen_weight_e4m3(ctx.h, 2, 17, 0, rows, K, 0, K, 0.02, q.p, s.p))
    wq, ws = oracle.gen_qlinear(2, 17, rows, K)
    assert np.array_equal(q.to_host().reshape(rows, K), wq) and np.array_equal(s.to_host(), ws)
    # a window of rows and columns (a tensor-parallel shard) equals the slice of the whole
    r0, nr, c0, nc = 5, 9, K // 4, K // 2
    q2, s2 = DV(ctx, nr * nc, np.uint8), DV(ctx, nr)
    N.check(L().strictb200_gen_weight_e4m3(ctx.h, 2, 17, r0, nr, K, c0, nc, 0.02, q2.p, s2.p))
    assert np.array_equal(q2.to_host().reshape(nr, nc), wq[r0:r0 + nr, c0:c0 + nc])
    assert np.array_equal(s2.to_host(), ws[r0:r0 + nr])


# ------------------------------------------------------------------ quantisation and GEMM
@pytest.mark.parametrize("M,K", [(1, 64), (5, 4096), (33, 12288), (8, 256)])
def test_quantize_rows_bit_exact(ctx, oracle, rng, M, K):
    x = oracle.round_bf16((rng.standard_normal((M, K)) * rng.uniform(0.01, 30, (M, 1))).astype(np.float32))
    if M > 1:
        x[0, :] = 0
    rows = 16 * ((M + 7) // 8)
    dx, dq, ds = bf16_dev(ctx, oracle, x), DV(ctx, rows * K, np.uint8), DV(ctx, M)
    dq.zero()
    N.check(L().strictb200_quantize_rows(ctx.h, dx.p, M, K, dq.p, ds.p))
    q, s = oracle.split_rows_device_layout(x)
    assert np.array_equal(ds.to_host(), s)
    assert np.array_equal(dq.to_host().reshape(rows, K), q)


def _gemm_case(ctx, oracle, rng, M, N_, K, kernel, out_dtype=0, seed=2):
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xq, sx = oracle.split_rows_device_layout(x)
    wq, sw = oracle.gen_qlinear(seed, 100 + N_ % 97, N_, K)
    want = oracle.linear_fp8w(x, wq, sw)
    dxq, dsx, dwq, dsw = DV.of(ctx, xq), DV.of(ctx, sx), DV.of(ctx, wq), DV.of(ctx, sw)
    out = DV(ctx, M * N_, np.float32 if out_dtype else np.uint16)
    N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, dxq.p, dsx.p, dwq.p, dsw.p, out.p, out_dtype, kernel))
    got = out.to_host().reshape(M, N_) if out_dtype else oracle.bf16_to_f32(out.to_host()).reshape(M, N_)
    for v in (dxq, dsx, dwq, dsw, out):
        v.free()
    return got, want


@pytest.mark.parametrize("M", [1, 7, 8, 9, 16, 25, 32])
@pytest.mark.parametrize("N_,K", [(128, 256), (4096, 4096), (1008, 1536), (144, 12288)])
def test_gemm_skinny_vs_oracle(ctx, oracle, rng, M, N_, K):
    got, want = _gemm_case(ctx, oracle, rng, M, N_, K, kernel=1, out_dtype=1)
    # exact bf16 x E4M3 products, fp32 accumulation: only the summation order differs
    assert np.allclose(got, want, rtol=2e-5, atol=1e-5 * np.abs(want).max())
    got, want = _gemm_case(ctx, oracle, rng, M, N_, K, kernel=1, out_dtype=0)
    ref = oracle.round_bf16(want)
    # bf16 output: equal except where the fp32 value sits on a rounding boundary (then 1 ulp)
    assert np.abs(got - ref).max() <= np.abs(ref).max() * 2 ** -7
    assert (got != ref).mean() < 1e-3


@pytest.mark.parametrize("M,N_,K", [(33, 128, 128), (64, 256, 512), (200, 1008, 1536), (2048, 4096, 4096), (300, 144, 12288), (5, 4096, 4096)])
@pytest.mark.parametrize("kernel", [2, 3])
def test_gemm_tiles_vs_oracle(ctx, oracle, rng, M, N_, K, kernel):
    got, want = _gemm_case(ctx, oracle, rng, M, N_, K, kernel=kernel, out_dtype=1)
    assert np.allclose(got, want, rtol=2e-5, atol=1e-5 * np.abs(want).max())


@pytest.mark.parametrize("M,N_,K", [(300, 1008, 1536), (2048, 4096, 4096)])
def test_gemm_one_sm_persistent_kernel_vs_oracle(ctx, oracle, rng, M, N_, K):
    """The one-SM persistent tcgen05 kernel (the fallback of the paired kernel) stays correct."""
    with ctx.option("gemm_pair", 0):
        got, want = _gemm_case(ctx, oracle, rng, M, N_, K, kernel=3, out_dtype=1)
    assert np.allclose(got, want, rtol=2e-5, atol=1e-5 * np.abs(want).max())


@pytest.mark.parametrize("pair", [1, 0], ids=["sm-pairs", "one-sm"])
def test_gemm_prefill_benchmark_shape_vs_oracle(ctx, oracle, rng, pair):
    """The many-token tcgen05 kernels at the benchmark's second shape (M=2048, N=14336, K=4096,
    device-generated weights from seed 2): 256 random output channels against the oracle, and
    every channel against the few-token kernel path run on a slice of the rows."""
    M, N_, K = 2048, 14336, 4096
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xq, sx = oracle.split_rows_device_layout(x)
    dwq, dsw = DV(ctx, N_ * K, np.uint8), DV(ctx, N_)
    N.check(L().strictb200_gen_weight_e4m3(ctx.h, 2, 7, 0, N_, K, 0, K, 0.02, dwq.p, dsw.p))
    dxq, dsx, out = DV.of(ctx, xq), DV.of(ctx, sx), DV(ctx, M * N_)
    with ctx.option("gemm_pair", pair):
        N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, dxq.p, dsx.p, dwq.p, dsw.p, out.p, 1, 3))
    got = out.to_host().reshape(M, N_)
    cols = np.sort(rng.choice(N_, 256, replace=False))
    cols[:4] = [0, 127, 128, N_ - 1]  # tile edges
    wq = dwq.to_host().reshape(N_, K)[cols]
    want = oracle.linear_fp8w(x, wq, dsw.to_host()[cols])
    assert np.allclose(got[:, cols], want, rtol=2e-5, atol=1e-5 * np.abs(want).max())
    # all 14336 channels of 32 rows spread over the token tiles, against the few-token kernel
    rows = np.sort(rng.choice(M, 32, replace=False))
    xq2, sx2 = oracle.split_rows_device_layout(x[rows])
    d2, s2, o2 = DV.of(ctx, xq2), DV.of(ctx, sx2), DV(ctx, 32 * N_)
    N.check(L().strictb200_gemm_fp8(ctx.h, 32, N_, K, d2.p, s2.p, dwq.p, dsw.p, o2.p, 1, 1))
    small = o2.to_host().reshape(32, N_)
    assert np.allclose(got[rows], small, rtol=2e-5, atol=1e-5 * np.abs(small).max())
    for v in (dwq, dsw, dxq, dsx, out, d2, s2, o2):
        v.free()


def test_gemm_kernels_agree_and_linearity(ctx, oracle, rng):
    """Size-independent properties at a benchmark shape: the three kernels agree, and the GEMM
    is linear in the activation scale."""
    M, N_, K = 32, 14336, 4096
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    xq, sx = oracle.split_rows_device_layout(x)
    dwq, dsw = DV(ctx, N_ * K, np.uint8), DV(ctx, N_)
    N.check(L().strictb200_gen_weight_e4m3(ctx.h, 2, 7, 0, N_, K, 0, K, 0.02, dwq.p, dsw.p))
    dxq, dsx, dsx2 = DV.of(ctx, xq), DV.of(ctx, sx), DV.of(ctx, sx * 2)
    outs = []
    for kernel in (1, 2, 3):
        o = DV(ctx, M * N_)
        N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, dxq.p, dsx.p, dwq.p, dsw.p, o.p, 1, kernel))
        outs.append(o.to_host())
    scale = np.abs(outs[0]).max()
    assert np.allclose(outs[0], outs[1], rtol=2e-5, atol=1e-5 * scale) and np.allclose(outs[0], outs[2], rtol=2e-5, atol=1e-5 * scale)
    o2 = DV(ctx, M * N_)
    N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, dxq.p, dsx2.p, dwq.p, dsw.p, o2.p, 1, 1))
    assert np.array_equal(o2.to_host(), outs[0] * 2)
    # spot-check 64 output channels against the oracle
    rows = rng.choice(N_, 64, replace=False)
    wq = dwq.to_host().reshape(N_, K)[rows]
    want = oracle.linear_fp8w(x, wq, dsw.to_host()[rows])
    assert np.allclose(outs[0].reshape(M, N_)[:, rows], want, rtol=2e-5, atol=1e-5 * scale)


@pytest.mark.parametrize("M,N_,K", [(1, 4096, 4096), (8, 1024, 3072), (32, 4096, 4096), (32, 1008, 1536), (17, 6144, 4096), (100, 4096, 4096), (128, 1008, 1536)])
@pytest.mark.parametrize("out_dtype", [0, 1])
def test_gemm_auto_split_k_vs_oracle(ctx, oracle, rng, M, N_, K, out_dtype):
    """kernel 0 with few tokens: K splits (uneven where K/128 does not divide) and a summing kernel."""
    got, want = _gemm_case(ctx, oracle, rng, M, N_, K, kernel=0, out_dtype=out_dtype)
    if out_dtype:
        assert np.allclose(got, want, rtol=2e-5, atol=1e-5 * np.abs(want).max())
    else:
        ref = oracle.round_bf16(want)
        assert np.abs(got - ref).max() <= np.abs(ref).max() * 2 ** -7 and (got != ref).mean() < 1e-3


def test_recorded_sequence_replays(ctx, oracle, rng):
    """Calls made while recording do not run; a replay runs them, `times` times, and counts its launches."""
    n = 1 << 12
    a = rng.standard_normal(n).astype(np.float32)
    da, dout = DV.of(ctx, a), DV(ctx, n)
    N.check(L().strictb200_ew_binary(ctx.h, 0, da.p, da.p, dout.p, n))  # out = 2a
    ctx.synchronize()
    launches0 = ctx.launch_count()
    with ctx.record():
        N.check(L().strictb200_ew_binary(ctx.h, 0, dout.p, da.p, dout.p, n))  # out += a
        N.check(L().strictb200_ew_binary(ctx.h, 0, dout.p, da.p, dout.p, n))
    graph = ctx.last_graph
    assert ctx.launch_count() == launches0
    assert np.array_equal(dout.to_host(), a + a)  # nothing ran yet
    ctx.replay(graph, 3)
    want = a + a
    for _ in range(6):
        want = want + a
    assert np.array_equal(dout.to_host(), want)
    assert ctx.launch_count() == launches0 + 6
    ctx.free_graph(graph)
    for v in (da, dout):
        v.free()


def test_gemm_fp8w_entry(ctx, oracle, rng):
    M, N_, K = 8, 512, 1024
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    wq, sw = oracle.gen_qlinear(2, 3, N_, K)
    want = oracle.round_bf16(oracle.linear_fp8w(x, wq, sw))
    dx, dwq, dsw, dy = bf16_dev(ctx, oracle, x), DV.of(ctx, wq), DV.of(ctx, sw), DV(ctx, M * N_, np.uint16)
    N.check(L().strictb200_gemm_fp8w(ctx.h, M, N_, K, dx.p, dwq.p, dsw.p, dy.p, 0))
    got = bf16_host(oracle, dy, (M, N_))
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -7 and (got != want).mean() < 1e-3


@pytest.mark.parametrize("M,N_,K", [(1, 512, 1024), (8, 4096, 4096), (32, 1536, 4096), (33, 144, 256), (128, 4096, 12288), (200, 1024, 1024),
                                    (300, 256, 128), (2048, 512, 512)])
def test_gemm_int8w_bit_exact(ctx, oracle, rng, M, N_, K):
    """int8 weights on the integer tensor cores (tcgen05 kind::i8): quantisers and linear layer
    equal the CPU restatement bit for bit, for one and several K splits, one and several token
    tiles, token counts that are not multiples of 8 and channel counts that are not multiples of
    the 128-channel tile."""
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32) * rng.choice([1e-2, 1.0, 50.0], (M, 1)).astype(np.float32))
    if M > 2:
        x[2] = 0.0
    w = (rng.standard_normal((N_, K)) * 0.02).astype(np.float32)
    w[min(5, N_ - 1)] = 0.0
    wq, sw = oracle.quantize_weights_int8(w)
    dw, dwq, dsw = DV.of(ctx, w), DV(ctx, N_ * K, np.int8), DV(ctx, N_)
    N.check(L().strictb200_quantize_weights_int8(ctx.h, dw.p, N_, K, dwq.p, dsw.p))
    assert np.array_equal(dwq.to_host().reshape(N_, K), wq) and np.array_equal(dsw.to_host(), sw)
    hi, lo, s = oracle.quantize_rows_int8(x)
    rows = 16 * ((M + 7) // 8)
    dx, dsplit, dsx = bf16_dev(ctx, oracle, x), DV(ctx, rows * K, np.int8), DV(ctx, M)
    N.check(L().strictb200_memset(ctx.h, dsplit.p, 0x55, rows * K))  # the padding rows must be written too
    N.check(L().strictb200_quantize_rows_int8(ctx.h, dx.p, M, K, dsplit.p, dsx.p))
    split = dsplit.to_host().reshape(rows // 16, 2, 8, K)
    want_split = np.zeros((rows // 16 * 8, 2, K), np.int8)
    want_split[:M, 0], want_split[:M, 1] = hi, lo
    assert np.array_equal(split, want_split.reshape(rows // 16, 8, 2, K).transpose(0, 2, 1, 3)) and np.array_equal(dsx.to_host(), s)
    want = oracle.gemm_int8w(x, wq, sw)
    dy = DV(ctx, M * N_, np.uint16)
    N.check(L().strictb200_gemm_int8w(ctx.h, M, N_, K, dx.p, dwq.p, dsw.p, dy.p))
    got = dy.to_host().reshape(M, N_)
    assert np.array_equal(got, want), (np.argwhere(got != want)[:5], (got != want).sum())
    N.check(L().strictb200_memset(ctx.h, dy.p, 0, M * N_ * 2))
    N.check(L().strictb200_gemm_int8(ctx.h, M, N_, K, dsplit.p, dsx.p, dwq.p, dsw.p, dy.p))
    assert np.array_equal(dy.to_host().reshape(M, N_), want)
    for v in (dw, dwq, dsw, dx, dsplit, dsx, dy):
        v.free()


def test_gemm_int8w_extreme_sums(ctx, oracle):
    """Every product at its largest magnitude over the longest K of the configurations: the hi and
    lo sums stay inside 32 bits and the joined 64-bit value is converted once."""
    M, N_, K = 8, 256, 12288
    x = np.full((M, K), 16256.0, np.float32)
    x[1] = -x[1]
    x[2, ::2] = 63.0 * 2.0 ** -7 * 128  # lo at its largest with hi zero
    w = np.ones((N_, K), np.float32)
    w[1::2] = -1.0
    wq, sw = oracle.quantize_weights_int8(w)
    assert np.abs(wq).min() == 127
    want = oracle.gemm_int8w(x, wq, sw)
    dx, dwq, dsw, dy = bf16_dev(ctx, oracle, x), DV.of(ctx, wq), DV.of(ctx, sw), DV(ctx, M * N_, np.uint16)
    N.check(L().strictb200_gemm_int8w(ctx.h, M, N_, K, dx.p, dwq.p, dsw.p, dy.p))
    got = dy.to_host().reshape(M, N_)
    assert np.array_equal(got, want)
    assert oracle.bf16_to_f32(got)[0, 0] == oracle.round_bf16(np.float32(16256.0 * K))
    for v in (dx, dwq, dsw, dy):
        v.free()


@pytest.mark.parametrize("M,N_,K", [(1, 2304, 768), (3, 50257, 768), (128, 768, 3072), (9, 10, 4), (5, 7, 1500), (2, 13, 8200)])
def test_gemm_f32_vs_oracle(ctx, oracle, rng, M, N_, K):
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N_, K)) * 0.02).astype(np.float32)
    b = rng.standard_normal(N_).astype(np.float32)
    dx, dw, db, dy = DV.of(ctx, x), DV.of(ctx, w), DV.of(ctx, b), DV(ctx, M * N_)
    N.check(L().strictb200_gemm_f32(ctx.h, M, N_, K, dx.p, dw.p, db.p, dy.p))
    assert np.allclose(dy.to_host().reshape(M, N_), oracle.gemm_f32(x, w, b), rtol=1e-5, atol=1e-5)
    N.check(L().strictb200_gemm_f32(ctx.h, M, N_, K, dx.p, dw.p, None, dy.p))
    assert np.allclose(dy.to_host().reshape(M, N_), oracle.gemm_f32(x, w), rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------ norms / activations
@pytest.mark.parametrize("M,d", [(1, 128), (5, 1024), (33, 4096), (2, 16384)])
def test_rmsnorm_vs_oracle(ctx, oracle, rng, M, d):
    x = oracle.round_bf16(rng.standard_normal((M, d)).astype(np.float32) * 3)
    res = oracle.round_bf16(rng.standard_normal((M, d)).astype(np.float32))
    g = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    dx, dg, dy = bf16_dev(ctx, oracle, x), DV.of(ctx, g), DV(ctx, M * d, np.uint16)
    N.check(L().strictb200_rmsnorm(ctx.h, dx.p, None, dg.p, 1e-6, M, d, dy.p))
    want = oracle.round_bf16(oracle.rmsnorm(x, g, 1e-6))
    got = bf16_host(oracle, dy, (M, d))
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -7 and (got != want).mean() < 2e-3
    # fused residual: residual <- bf16(residual + x); y = norm(residual)
    dr = bf16_dev(ctx, oracle, res)
    N.check(L().strictb200_rmsnorm(ctx.h, dx.p, dr.p, dg.p, 1e-6, M, d, dy.p))
    h = oracle.round_bf16(res + x)
    assert np.array_equal(bf16_host(oracle, dr, (M, d)), h)
    want = oracle.round_bf16(oracle.rmsnorm(h, g, 1e-6))
    got = bf16_host(oracle, dy, (M, d))
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -7 and (got != want).mean() < 2e-3


@pytest.mark.parametrize("M,d", [(1, 768), (7, 100), (128, 768)])
def test_layernorm_vs_oracle(ctx, oracle, rng, M, d):
    x = rng.standard_normal((M, d)).astype(np.float32) * 2 + 0.5
    g, b = rng.standard_normal(d).astype(np.float32), rng.standard_normal(d).astype(np.float32)
    dx, dg, db, dy = DV.of(ctx, x), DV.of(ctx, g), DV.of(ctx, b), DV(ctx, M * d)
    N.check(L().strictb200_layernorm(ctx.h, dx.p, dg.p, db.p, 1e-5, M, d, dy.p))
    assert np.allclose(dy.to_host().reshape(M, d), oracle.layernorm(x, g, b, 1e-5), rtol=1e-5, atol=1e-5)


def test_swiglu_gelu_vs_oracle(ctx, oracle, rng):
    M, I = 5, 3072
    gu = oracle.round_bf16(rng.standard_normal((M, 2 * I)).astype(np.float32) * 2)
    dgu, dy = bf16_dev(ctx, oracle, gu), DV(ctx, M * I, np.uint16)
    N.check(L().strictb200_swiglu(ctx.h, dgu.p, M, I, dy.p))
    want = oracle.round_bf16(oracle.swiglu(gu[:, :I], gu[:, I:]))
    got = bf16_host(oracle, dy, (M, I))
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -7 and (got != want).mean() < 2e-3
    x = rng.standard_normal(10007).astype(np.float32) * 3
    dx, dg = DV.of(ctx, x), DV(ctx, x.size)
    N.check(L().strictb200_gelu_tanh(ctx.h, dx.p, x.size, dg.p))
    assert np.allclose(dg.to_host(), oracle.gelu_tanh(x), rtol=1e-5, atol=1e-6)


def test_rope_qknorm_kvappend_vs_oracle(ctx, oracle, rng):
    T, Hq, Hkv, D, B, maxlen = 6, 4, 2, 128, 3, 64
    nqkv = (Hq + 2 * Hkv) * D
    qkv = oracle.round_bf16(rng.standard_normal((T, nqkv)).astype(np.float32))
    seq = np.array([0, 0, 1, 2, 2, 2], np.int32)
    pos = np.array([0, 1, 5, 61, 62, 63], np.int32)
    qg = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kg = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    dqkv, dseq, dpos, dqg, dkg = bf16_dev(ctx, oracle, qkv), DV.of(ctx, seq), DV.of(ctx, pos), DV.of(ctx, qg), DV.of(ctx, kg)
    dq = DV(ctx, T * Hq * D, np.uint16)
    dk, dv = DV(ctx, B * Hkv * maxlen * D, np.uint16), DV(ctx, B * Hkv * maxlen * D, np.uint16)
    dk.zero(), dv.zero()
    N.check(L().strictb200_rope_qknorm_kvappend(ctx.h, dqkv.p, dseq.p, dpos.p, T, Hq, Hkv, D, dqg.p, dkg.p, 1e-6, 1e6, 4096, dq.p, dk.p,
                                                dv.p, maxlen))
    q_want = oracle.qknorm_rope(qkv[:, :Hq * D].reshape(T, Hq, D), qg, pos, 1e-6, 1e6)
    k_want = oracle.qknorm_rope(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D), kg, pos, 1e-6, 1e6)
    v_want = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    q_got = bf16_host(oracle, dq, (T, Hq, D))
    kc, vc = bf16_host(oracle, dk, (B, Hkv, maxlen, D)), bf16_host(oracle, dv, (B, Hkv, maxlen, D))
    k_got = np.stack([kc[seq[t], :, pos[t]] for t in range(T)])
    v_got = np.stack([vc[seq[t], :, pos[t]] for t in range(T)])
    assert np.array_equal(v_got, v_want)
    for got, want in ((q_got, q_want), (k_got, k_want)):
        assert np.abs(got - want).max() <= 2 ** -6 and (got != want).mean() < 5e-3
    # nothing else in the cache was touched
    mask = np.ones((B, maxlen), bool)
    mask[seq, pos] = False
    assert not kc.transpose(0, 2, 1, 3)[mask].any() and not vc.transpose(0, 2, 1, 3)[mask].any()


# ------------------------------------------------------------------ attention
def _attn_tol(got, want):
    # P is rounded to bf16 before the PV product on the tensor cores, outputs to bf16
    err = np.abs(got - want)
    return err.max() <= 2e-2 and err.mean() / np.abs(want).mean() <= 5e-3


@pytest.mark.parametrize("B,S,Hq,Hkv,lens", [(1, 1, 4, 2, [1]), (2, 65, 4, 1, [65, 3]), (2, 200, 8, 2, [200, 129]), (1, 64, 2, 2, [64]),
                                             (2, 256, 4, 2, [256, 130]), (1, 250, 8, 8, [250])])
@pytest.mark.parametrize("tensor_memory_kernel", [1, 0, 2])
def test_attn_prefill_vs_oracle(ctx, oracle, rng, B, S, Hq, Hkv, lens, tensor_memory_kernel):
    # tcgen05 one tile per block / mma.sync / tcgen05 two tiles per block
    with ctx.option("attn_tc", tensor_memory_kernel):
        _attn_prefill_case(ctx, oracle, rng, B, S, Hq, Hkv, lens)


def _attn_prefill_case(ctx, oracle, rng, B, S, Hq, Hkv, lens):
    D, maxlen = 128, 256
    q = oracle.round_bf16(rng.standard_normal((B, S, Hq, D)).astype(np.float32))
    k = oracle.round_bf16(rng.standard_normal((B, S, Hkv, D)).astype(np.float32))
    v = oracle.round_bf16(rng.standard_normal((B, S, Hkv, D)).astype(np.float32))
    lens = np.array(lens, np.int32)
    scale = 1.0 / np.sqrt(D)
    want = oracle.round_bf16(oracle.attn_prefill(q, k, v, lens, scale))
    kc = np.zeros((B, Hkv, maxlen, D), np.float32)
    vc = np.zeros((B, Hkv, maxlen, D), np.float32)
    kc[:, :, :S], vc[:, :, :S] = k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3)
    dq, dk, dv, dl = bf16_dev(ctx, oracle, q), bf16_dev(ctx, oracle, kc), bf16_dev(ctx, oracle, vc), DV.of(ctx, lens)
    do = DV(ctx, B * S * Hq * D, np.uint16)
    do.zero()
    N.check(L().strictb200_attn_prefill(ctx.h, dq.p, dk.p, dv.p, dl.p, None, B, S, Hq, Hkv, D, maxlen, scale, do.p))
    got = bf16_host(oracle, do, (B, S, Hq, D))
    for b in range(B):
        assert _attn_tol(got[b, :lens[b]], want[b, :lens[b]])
        assert not got[b, lens[b]:].any()  # rows beyond the sequence are not written
    # chunked continuation: the last 5 queries with past = len-5 reproduce the same rows
    if lens.min() > 5:
        past = (lens - 5).astype(np.int32)
        q2 = np.zeros((B, 5, Hq, D), np.float32)
        for b in range(B):
            q2[b] = q[b, past[b]:lens[b]]
        dq2, dp, do2 = bf16_dev(ctx, oracle, q2), DV.of(ctx, past), DV(ctx, B * 5 * Hq * D, np.uint16)
        N.check(L().strictb200_attn_prefill(ctx.h, dq2.p, dk.p, dv.p, dl.p, dp.p, B, 5, Hq, Hkv, D, maxlen, scale, do2.p))
        got2 = bf16_host(oracle, do2, (B, 5, Hq, D))
        for b in range(B):
            assert _attn_tol(got2[b], want[b, past[b]:lens[b]])


def _spiked_qkv(oracle, rng, B, S, Hq, Hkv, lens, spikes):
    """bf16-valued N(0,1) q, k, v [B,S,H,128]. `spikes` = (sequence, query row, key index < row):
    that key is set to 2.5 x the query of head 0 of every KV group, so the row's running maximum
    jumps by ~28 (40 in the exp2 domain) when the key's tile comes up, late in the row's pass."""
    D = 128
    q = oracle.round_bf16(rng.standard_normal((B, S, Hq, D)).astype(np.float32))
    k = oracle.round_bf16(rng.standard_normal((B, S, Hkv, D)).astype(np.float32))
    v = oracle.round_bf16(rng.standard_normal((B, S, Hkv, D)).astype(np.float32))
    G = Hq // Hkv
    for b, row, key in spikes:
        assert key <= row < lens[b]
        for hk in range(Hkv):
            k[b, key, hk] = oracle.round_bf16(2.5 * q[b, row, hk * G])
    return q, k, v


@pytest.mark.parametrize("B,S,Hq,Hkv,lens", [(2, 1024, 8, 2, [1024, 700]), (2, 2048, 8, 2, [2048, 1337]), (1, 8192, 4, 1, [8192])],
                         ids=["s1024", "s2048", "s8192"])
def test_attn_prefill_long_vs_oracle(ctx, oracle, rng, B, S, Hq, Hkv, lens):
    """Prefill attention at the prompt lengths of the benchmark (8 to 64 key tiles per query
    tile), four query heads per KV head, ragged lengths, for both tcgen05 kernels; rows whose
    maximum grows by far more than 2^8 late in the sequence exercise the lazy rescaling of the
    running output; a continuation with past > 0 of 300 new tokens reproduces the same rows."""
    D, maxlen = 128, S
    lens = np.array(lens, np.int32)
    spikes = []
    for b in range(B):
        n = int(lens[b])
        spikes += [(b, n - 1, n - 7), (b, n - 130, n - 135), (b, n // 2 + 3, n // 2 - 40), (b, n - 50, 5), (b, 200, 199)]
    q, k, v = _spiked_qkv(oracle, rng, B, S, Hq, Hkv, lens, spikes)
    scale = 1.0 / np.sqrt(D)
    want = oracle.round_bf16(oracle.attn_prefill(q, k, v, lens, scale))
    kc = np.ascontiguousarray(k.transpose(0, 2, 1, 3))
    vc = np.ascontiguousarray(v.transpose(0, 2, 1, 3))
    dq, dk, dv, dl = bf16_dev(ctx, oracle, q), bf16_dev(ctx, oracle, kc), bf16_dev(ctx, oracle, vc), DV.of(ctx, lens)
    do = DV(ctx, B * S * Hq * D, np.uint16)
    new = 300
    past = (lens - new).astype(np.int32)
    q2 = np.stack([q[b, past[b]:lens[b]] for b in range(B)])
    dq2, dp, do2 = bf16_dev(ctx, oracle, q2), DV.of(ctx, past), DV(ctx, B * new * Hq * D, np.uint16)
    for mode in (1, 2, -1):
        with ctx.option("attn_tc", mode):
            do.zero()
            N.check(L().strictb200_attn_prefill(ctx.h, dq.p, dk.p, dv.p, dl.p, None, B, S, Hq, Hkv, D, maxlen, scale, do.p))
            got = bf16_host(oracle, do, (B, S, Hq, D))
            N.check(L().strictb200_attn_prefill(ctx.h, dq2.p, dk.p, dv.p, dl.p, dp.p, B, new, Hq, Hkv, D, maxlen, scale, do2.p))
            got2 = bf16_host(oracle, do2, (B, new, Hq, D))
        for b in range(B):
            assert _attn_tol(got[b, :lens[b]], want[b, :lens[b]]), (mode, b)
            assert not got[b, lens[b]:].any()
            assert _attn_tol(got2[b], want[b, past[b]:lens[b]]), (mode, b, "continuation")
            for _, row, _ in [s for s in spikes if s[0] == b]:  # the spiked rows one by one
                assert np.abs(got[b, row] - want[b, row]).max() <= 2e-2, (mode, b, row)
    assert ctx.device_status() == 0
    for x in (dq, dk, dv, dl, do, dq2, dp, do2):
        x.free()


@pytest.mark.parametrize("B,Hq,Hkv,maxlen,lens", [(1, 4, 2, 64, [1]), (3, 8, 2, 1024, [1, 64, 1000]), (2, 32, 8, 4096, [4096, 2049]),
                                                  (2, 16, 1, 512, [511, 65])])
def test_attn_decode_vs_oracle(ctx, oracle, rng, B, Hq, Hkv, maxlen, lens):
    D = 128
    lens = np.array(lens, np.int32)
    q = oracle.round_bf16(rng.standard_normal((B, Hq, D)).astype(np.float32))
    kc = oracle.round_bf16(rng.standard_normal((B, Hkv, maxlen, D)).astype(np.float32))
    vc = oracle.round_bf16(rng.standard_normal((B, Hkv, maxlen, D)).astype(np.float32))
    scale = 1.0 / np.sqrt(D)
    want = oracle.round_bf16(oracle.attn_decode(q, kc, vc, lens, scale))
    dq, dk, dv, dl = bf16_dev(ctx, oracle, q), bf16_dev(ctx, oracle, kc), bf16_dev(ctx, oracle, vc), DV.of(ctx, lens)
    do = DV(ctx, B * Hq * D, np.uint16)
    N.check(L().strictb200_attn_decode(ctx.h, dq.p, dk.p, dv.p, dl.p, B, Hq, Hkv, D, maxlen, scale, do.p))
    assert _attn_tol(bf16_host(oracle, do, (B, Hq, D)), want)


def test_attn_decode_microbench_shape_properties(ctx, oracle, rng):
    """Benchmark shape (32 query / 8 KV heads, ragged long contexts): a one-hot V column makes
    every output equal to the softmax mass on that key set — independent of the size."""
    B, Hq, Hkv, D, maxlen = 4, 32, 8, 128, 32768
    lens = np.array([1024, 32768, 20001, 7777], np.int32)
    dq = DV(ctx, B * Hq * D, np.uint16)
    dk, dv = DV(ctx, B * Hkv * maxlen * D, np.uint16), DV(ctx, B * Hkv * maxlen * D, np.uint16)
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 1, 0, B * Hq * D, 1.0, dq.p))
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 2, 0, B * Hkv * maxlen * D, 1.0, dk.p))
    ones = np.full(B * Hkv * maxlen * D, 0x3F80, np.uint16)  # V = 1 everywhere -> output must be exactly 1
    dv.upload(ones)
    dl, do = DV.of(ctx, lens), DV(ctx, B * Hq * D, np.uint16)
    N.check(L().strictb200_attn_decode(ctx.h, dq.p, dk.p, dv.p, dl.p, B, Hq, Hkv, D, maxlen, 1.0 / np.sqrt(D), do.p))
    got = bf16_host(oracle, do, (B, Hq, D))
    assert np.abs(got - 1.0).max() <= 2 ** -7
    # and a spot check of two (sequence, head) pairs against the oracle with random V
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 3, 0, B * Hkv * maxlen * D, 1.0, dv.p))
    N.check(L().strictb200_attn_decode(ctx.h, dq.p, dk.p, dv.p, dl.p, B, Hq, Hkv, D, maxlen, 1.0 / np.sqrt(D), do.p))
    got = bf16_host(oracle, do, (B, Hq, D))
    q = bf16_host(oracle, dq, (B, Hq, D))
    kc, vc = bf16_host(oracle, dk, (B, Hkv, maxlen, D)), bf16_host(oracle, dv, (B, Hkv, maxlen, D))
    for b, hk in ((1, 3), (2, 7)):
        want = oracle.attn_decode(q[b:b + 1, hk * 4:hk * 4 + 4], kc[b:b + 1, hk:hk + 1], vc[b:b + 1, hk:hk + 1], lens[b:b + 1], 1.0 / np.sqrt(D))
        assert np.abs(got[b, hk * 4:hk * 4 + 4] - want[0]).max() < 5e-3


# ------------------------------------------------------------------ embedding / argmax
def test_embedding_and_argmax(ctx, oracle, rng):
    V, d, T = 1000, 256, 17
    table = oracle.f32_to_bf16(rng.standard_normal((V, d)).astype(np.float32))
    ids = rng.integers(0, V, T).astype(np.int32)
    dt, di, do = DV.of(ctx, table), DV.of(ctx, ids), DV(ctx, T * d, np.uint16)
    N.check(L().strictb200_embedding_bf16(ctx.h, dt.p, di.p, T, d, V, do.p))
    assert np.array_equal(do.to_host().reshape(T, d), table[ids])
    x = rng.standard_normal((9, 151936)).astype(np.float32)
    x[0, 5] = x[0, 77] = 100.0  # tie -> lowest index
    x[1, :] = -3.0              # all equal -> 0
    x[2, 151935] = 50.0
    dx, da = DV.of(ctx, x), DV(ctx, 9, np.int32)
    N.check(L().strictb200_argmax(ctx.h, dx.p, 9, 151936, da.p))
    assert np.array_equal(da.to_host(), oracle.argmax(x))
    assert da.to_host()[:3].tolist() == [5, 0, 151935]
