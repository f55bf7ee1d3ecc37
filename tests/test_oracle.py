"""CPU tests of the oracle: pinned to the reference's known answers where the reference has
any (the element-wise surface), cross-checked against torch used as a calculator everywhere
else (the LLM path is unpinned by the reference), and frozen by tests/golden/oracle_vectors.npz."""
import json
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "reference_known_answers.json")))

TINY_QWEN = dict(arch=1, n_layers=2, d_model=256, n_q_heads=4, n_kv_heads=2, head_dim=128, d_ff=512, vocab=1024,
                 max_pos=128, tied=0, eps=1e-6, rope_theta=1e6)
TINY_GPT2 = dict(arch=0, n_layers=2, d_model=128, n_q_heads=2, n_kv_heads=2, head_dim=64, d_ff=512, vocab=512,
                 max_pos=64, tied=1, eps=1e-5, rope_theta=0.0)


# ------------------------------------------------------------------ reference-pinned surface
@pytest.mark.parametrize("case", [c for c in GOLD["execute"] if "first" in c], ids=lambda c: c["case"])
def test_known_answers_binary(oracle, case):
    op = {"+": 0, "-": 1, "*": 2, "/": 3}[case["body"].split()[1]]
    n = GOLD["stale_fixture_n"]
    out = oracle.ew_binary(op, np.full(n, case["first"], np.float32), np.full(n, case["second"], np.float32))
    assert np.all(out == np.float32(case["expected"]))


def test_known_answer_initialize_depths(oracle):
    case = [c for c in GOLD["execute"] if c["case"] == "InitializeDepths"][0]
    # LOAD_SCALAR initialDepth -> r0 ; RETURN r0
    out = oracle.ew_program([[1, 2, 0, 0], [7, 0, 0, 0]], [np.full(1, case["input"], np.float32)],
                            [case["width"], case["height"], case["initialDepth"]], [], 1)
    assert out[0] == np.float32(case["expected"])


def test_program_without_return_is_zero(oracle):
    out = oracle.ew_program([[2, 0, 0, 0]], [], [], [3.0], 4)
    assert np.all(out == 0.0)


def test_ew_unknown_op(oracle):
    with pytest.raises(NotImplementedError):
        oracle.ew_binary(9, np.zeros(1, np.float32), np.zeros(1, np.float32))


def test_ew_float_semantics(oracle, rng):
    a = rng.standard_normal(1000).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    for op, f in enumerate([np.add, np.subtract, np.multiply, np.divide]):
        assert np.array_equal(oracle.ew_binary(op, a, b), f(a, b).astype(np.float32))


# ------------------------------------------------------------------ formats and generator
def test_e4m3_codec_matches_torch(oracle, rng):
    allb = np.arange(256, dtype=np.uint8)
    want = torch.tensor(allb).view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_to_f32(allb)
    assert np.array_equal(np.isnan(want), np.isnan(got))
    assert np.array_equal(want[~np.isnan(want)], got[~np.isnan(got)])
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 1e-2, 0.1, 1, 10, 100)])
    x = x[np.abs(x) <= 448]
    assert np.array_equal(oracle.f32_to_e4m3(x), torch.tensor(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    # saturation instead of NaN beyond the largest finite value
    assert oracle.f32_to_e4m3(np.array([1e6, -1e6, 449.0], np.float32)).tolist() == [0x7E, 0xFE, 0x7E]
    # every code point round-trips
    finite = ~np.isnan(got)
    assert np.array_equal(oracle.f32_to_e4m3(got[finite]) & 0x7F, allb[finite] & 0x7F)


def test_bf16_codec_matches_torch(oracle, rng):
    x = (rng.standard_normal(100000) * 10.0 ** rng.integers(-20, 20, 100000)).astype(np.float32)
    want = torch.tensor(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(x), want)


def test_generator_statistics(oracle):
    z = oracle.gen_normal(0, 1, 1_000_000)
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1) < 5e-3
    assert abs((z ** 3).mean()) < 2e-2 and abs((z ** 4).mean() - 3) < 5e-2
    assert np.abs(z).max() < 6.0
    # streams differ by seed and by tensor; a window of a stream equals the same slice of the whole
    assert not np.array_equal(oracle.gen_normal(1, 1, 64), z[:64])
    assert not np.array_equal(oracle.gen_normal(0, 2, 64), z[:64])
    assert np.array_equal(oracle.gen_normal(0, 1, 100, first=12345), z[12345:12445])
    t = oracle.gen_tokens(1, 1, 100000, 50257)
    assert t.min() >= 0 and t.max() < 50257 and abs(t.mean() / 50257 - 0.5) < 0.01


def test_weight_quantiser(oracle):
    q, s = oracle.gen_qlinear(2, 17, 8, 256, std=0.02)
    w = oracle.gen_normal(2, 17, 8 * 256, std=0.02).reshape(8, 256)
    assert np.allclose(s, np.abs(w).max(1) / 448, rtol=1e-6)
    dq = oracle.e4m3_to_f32(q) * s[:, None]
    assert np.abs(dq - w).max() <= np.abs(w).max() * 0.0625 + 1e-9  # half an E4M3 ulp at the top binade
    assert (np.abs(oracle.e4m3_to_f32(q)).max(1) == 448).all()


def test_golden_vectors(oracle):
    g = np.load(os.path.join(HERE, "golden", "oracle_vectors.npz"))
    assert np.array_equal(oracle.gen_normal(7, 3, 64), g["normal_seed7_t3"])
    assert np.array_equal(oracle.gen_tokens(1, 1, 32, 50257), g["tokens_seed1_t1"])
    q, s = oracle.gen_qlinear(2, 17, 4, 128)
    assert np.array_equal(q, g["qlinear_q"]) and np.array_equal(s, g["qlinear_s"])
    for name, cfg, seed, B in (("qwen", TINY_QWEN, 4, 2), ("gpt2", TINY_GPT2, 0, 1)):
        m = oracle.Model(cfg, seed)
        toks = g[name + "_tokens"]
        st = m.new_state(B, toks.shape[1] + 4)
        logits = st.prefill(toks, np.full(B, toks.shape[1], np.int32))
        ids = [oracle.argmax(logits)]
        for _ in range(4):
            logits = st.decode(ids[-1])
            ids.append(oracle.argmax(logits))
        assert np.array_equal(np.stack(ids), g[name + "_ids"])
        assert np.array_equal(logits, g[name + "_last_logits"])
        st.close()
        m.close()


# ------------------------------------------------------------------ primitives vs torch (calculator)
def test_split_rows_and_linear(oracle, rng):
    """The two-term E4M3 split reproduces bf16 rows exactly (above absmax/14336), its scale is
    the smallest power of two that fits 448, and the linear layer equals the float64 product of
    the bf16 activations with the dequantised weights."""
    x = oracle.round_bf16((rng.standard_normal((6, 512)) * rng.uniform(0.01, 30, (6, 1))).astype(np.float32))
    x[5] = 0
    hi, lo, eff, s = oracle.split_rows(x)
    amax = np.abs(x).max(1)
    assert s[5] == 1.0 and not hi[5].any() and not lo[5].any()
    assert np.all(np.log2(s) == np.round(np.log2(s)))
    assert np.all(amax[:5] / s[:5] <= 448) and np.all(amax[:5] / s[:5] > 224)
    assert np.array_equal(eff, oracle.e4m3_to_f32(hi) + oracle.e4m3_to_f32(lo) / 16)
    big = np.abs(x) >= (amax / 14336)[:, None]
    assert np.array_equal((eff * s[:, None])[big], x[big])
    assert np.abs(eff * s[:, None] - x).max() <= amax.max() * 2.0 ** -22
    # hi is the nearest E4M3 value of x/s
    assert np.array_equal(hi, torch.tensor(x / s[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    wq, sw = oracle.gen_qlinear(2, 1, 48, 512)
    y = oracle.linear_fp8w(x, wq, sw)
    want = (x.astype(np.float64) @ oracle.e4m3_to_f32(wq).astype(np.float64).T) * sw[None, :]
    assert np.allclose(y, want, rtol=2e-6, atol=1e-6 * np.abs(want).max())
    packed, s2 = oracle.split_rows_device_layout(x)
    assert packed.shape == (16, 512) and np.array_equal(s2, s)
    assert np.array_equal(packed[:6], hi) and np.array_equal(packed[8:14], lo) and not packed[6:8].any()


def test_norms_and_activations(oracle, rng):
    x = rng.standard_normal((7, 96)).astype(np.float32)
    g = rng.standard_normal(96).astype(np.float32)
    b = rng.standard_normal(96).astype(np.float32)
    tx = torch.tensor(x, dtype=torch.float64)
    want = tx * torch.rsqrt((tx * tx).mean(-1, keepdim=True) + 1e-6) * torch.tensor(g, dtype=torch.float64)
    assert np.allclose(oracle.rmsnorm(x, g, 1e-6), want.numpy(), rtol=2e-6, atol=1e-6)
    want = torch.nn.functional.layer_norm(tx, (96,), torch.tensor(g, dtype=torch.float64), torch.tensor(b, dtype=torch.float64), 1e-5)
    assert np.allclose(oracle.layernorm(x, g, b, 1e-5), want.numpy(), rtol=2e-6, atol=2e-6)
    assert np.allclose(oracle.gelu_tanh(x), torch.nn.functional.gelu(tx, approximate="tanh").numpy(), rtol=2e-6, atol=1e-6)
    u = rng.standard_normal((7, 96)).astype(np.float32)
    assert np.allclose(oracle.swiglu(x, u), (torch.nn.functional.silu(tx) * torch.tensor(u, dtype=torch.float64)).numpy(), rtol=2e-6, atol=1e-6)
    # RMSNorm output has RMS |gain| when the gain is constant
    y = oracle.rmsnorm(x, np.full(96, 3.0, np.float32), 0.0)
    assert np.allclose(np.sqrt((y ** 2).mean(1)), 3.0, rtol=1e-5)


def test_rope(oracle, rng):
    D = 128
    x = oracle.round_bf16(rng.standard_normal((6, 3, D)).astype(np.float32))
    pos = np.array([0, 1, 5, 100, 1000, 4095], np.int32)
    g = np.ones(D, np.float32)
    y = oracle.qknorm_rope(x, g, pos, 1e-6, 1e6)
    # independent: normalise, then rotate pairs (i, i+64) as complex numbers
    xn = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)
    inv = 1e6 ** (-2.0 * np.arange(D // 2) / D)
    ang = pos[:, None, None] * inv[None, None, :]
    z = (xn[..., :64] + 1j * xn[..., 64:]) * np.exp(1j * ang)
    want = np.concatenate([z.real, z.imag], -1)
    assert np.abs(y - want).max() < 0.02  # bf16 output rounding (|y| < 4)
    # position 0 is the identity rotation; rotation keeps the norm of every pair
    assert np.allclose(y[0], oracle.round_bf16(xn[0].astype(np.float32)), atol=1e-6)
    n_in = xn[..., :64] ** 2 + xn[..., 64:] ** 2
    n_out = y[..., :64].astype(np.float64) ** 2 + y[..., 64:].astype(np.float64) ** 2
    assert np.allclose(n_in, n_out, rtol=0.02, atol=0.02)
    c, s = oracle.rope_table(16, D, 1e6)
    assert np.allclose(c ** 2 + s ** 2, 1.0, atol=1e-6) and c[0].min() == 1.0


def test_attention_matches_torch(oracle, rng):
    B, S, Hq, Hkv, D = 2, 9, 4, 2, 128
    q = rng.standard_normal((B, S, Hq, D)).astype(np.float32)
    k = rng.standard_normal((B, S, Hkv, D)).astype(np.float32)
    v = rng.standard_normal((B, S, Hkv, D)).astype(np.float32)
    lens = np.array([9, 4], np.int32)
    scale = 1.0 / np.sqrt(D)
    out = oracle.attn_prefill(q, k, v, lens, scale)
    tq = torch.tensor(q, dtype=torch.float64).permute(0, 2, 1, 3)
    tk = torch.tensor(k, dtype=torch.float64).permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    tv = torch.tensor(v, dtype=torch.float64).permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    want = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv, is_causal=True, scale=scale).permute(0, 2, 1, 3).numpy()
    for b in range(B):
        assert np.allclose(out[b, :lens[b]], want[b, :lens[b]], rtol=1e-5, atol=1e-6)
    # decode = last row of the prefill
    kc = np.zeros((B, Hkv, 16, D), np.float32)
    vc = np.zeros((B, Hkv, 16, D), np.float32)
    kc[:, :, :S] = k.transpose(0, 2, 1, 3)
    vc[:, :, :S] = v.transpose(0, 2, 1, 3)
    qd = np.stack([q[b, lens[b] - 1] for b in range(B)])
    od = oracle.attn_decode(qd, kc, vc, lens, scale)
    for b in range(B):
        assert np.allclose(od[b], out[b, lens[b] - 1], rtol=1e-6, atol=1e-7)


def test_argmax_ties_lowest(oracle):
    x = np.array([[1, 5, 5, 2], [7, 7, 7, 7], [0, -1, 3, 3]], np.float32)
    assert oracle.argmax(x).tolist() == [1, 0, 2]


# ------------------------------------------------------------------ whole models vs an independent torch forward
def _torch_qwen_forward(oracle, m, cfg, tokens):
    """Full-sequence forward of one sequence in float64 torch with the oracle's weights and the
    same quantisation points; returns logits at the last position."""
    T = len(tokens)
    d, D, Hq, Hkv, I = cfg["d_model"], cfg["head_dim"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["d_ff"]
    f64 = torch.float64

    def t(name, dt=np.float32):
        return torch.tensor(np.array(m.tensor(name, dt)))

    def rb(x):  # round to bf16
        return x.to(torch.float32).to(torch.bfloat16).to(f64)

    def qlin(x, name, N, K):  # exact bf16 x E4M3 products, per-channel scale
        w = t(name + ".q", np.uint8).view(torch.float8_e4m3fn).to(f64).reshape(N, K)
        return (x @ w.T) * t(name + ".s").reshape(1, N).to(f64)

    def rms(x, g):
        x32 = x.to(torch.float32)
        r = 1.0 / torch.sqrt((x.to(f64) ** 2).mean(-1, keepdim=True).to(torch.float32) + cfg["eps"])
        return rb(((x32 * r) * g).to(f64))

    x = t("embed").reshape(cfg["vocab"], d)[torch.tensor(tokens, dtype=torch.long)].to(f64)
    pos = torch.arange(T, dtype=f64)
    inv = torch.tensor(1e6, dtype=f64) ** (-2.0 * torch.arange(D // 2, dtype=f64) / D)
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(torch.float32).to(f64), torch.sin(ang).to(torch.float32).to(f64)

    def rope(h, g):  # h [T,H,D]
        n = rms(h, g)
        a, b = n[..., : D // 2], n[..., D // 2:]
        return rb(torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None]], -1))

    nq, nkv = Hq * D, Hkv * D
    for l in range(cfg["n_layers"]):
        p = f"layers.{l}."
        a = rms(x, t(p + "norm1.g"))
        qkv = qlin(a, p + "wqkv", nq + 2 * nkv, d).to(torch.float32).to(f64)
        q = rope(qkv[:, :nq].reshape(T, Hq, D), t(p + "qnorm.g"))
        k = rope(qkv[:, nq:nq + nkv].reshape(T, Hkv, D), t(p + "knorm.g"))
        v = rb(qkv[:, nq + nkv:]).reshape(T, Hkv, D)
        kk = k.repeat_interleave(Hq // Hkv, 1).permute(1, 0, 2)
        vv = v.repeat_interleave(Hq // Hkv, 1).permute(1, 0, 2)
        s = ((q.permute(1, 0, 2) @ kk.transpose(1, 2)).to(torch.float32) * np.float32(1.0 / np.sqrt(D))).to(f64)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        att = rb((torch.softmax(s, -1) @ vv).permute(1, 0, 2).reshape(T, nq))
        x = x + qlin(att, p + "wo", d, nq).to(torch.float32).to(f64)
        a = rms(x, t(p + "norm2.g"))
        gu = qlin(a, p + "wgu", 2 * I, d)
        g32, u32 = gu[:, :I].to(torch.float32), gu[:, I:].to(torch.float32)
        h = rb(((g32 / (1.0 + torch.exp(-g32))) * u32).to(f64))
        x = x + qlin(h, p + "wdown", d, I).to(torch.float32).to(f64)
    a = rms(x[-1:], t("normf.g"))
    return qlin(a, "head", cfg["vocab"], d)[0].numpy()


def test_qwen_forward_matches_independent_torch(oracle, rng):
    cfg = TINY_QWEN
    m = oracle.Model(cfg, 11)
    # non-trivial gains
    for l in range(cfg["n_layers"]):
        for n in ("norm1.g", "norm2.g", "qnorm.g", "knorm.g"):
            t = m.tensor(f"layers.{l}.{n}", np.float32)
            t[:] = 1.0 + 0.1 * rng.standard_normal(t.size).astype(np.float32)
    toks = oracle.gen_tokens(3, 1, 12, cfg["vocab"])
    st = m.new_state(1, 16)
    logits = st.prefill(toks[None, :], np.array([12], np.int32))[0]
    want = _torch_qwen_forward(oracle, m, cfg, toks.tolist())
    # identical up to occasional 1-ulp bf16 rounding flips from the different summation order
    assert np.abs(logits - want).max() < 2e-2
    assert np.abs(logits - want).mean() / np.abs(want).mean() < 5e-3
    st.close()
    m.close()


def test_gpt2_forward_matches_independent_torch(oracle):
    cfg = TINY_GPT2
    m = oracle.Model(cfg, 5)
    d, H, Dh, T = cfg["d_model"], cfg["n_q_heads"], cfg["head_dim"], 10
    toks = oracle.gen_tokens(9, 1, T, cfg["vocab"])
    st = m.new_state(1, 16)
    logits = st.prefill(toks[None, :], np.array([T], np.int32))[0]
    f64 = torch.float64
    t = lambda n: torch.tensor(np.array(m.tensor(n, np.float32)), dtype=f64)  # noqa: E731
    wte, wpe = t("embed").reshape(-1, d), t("wpe").reshape(-1, d)
    x = wte[torch.tensor(toks.astype(np.int64))] + wpe[:T]
    for l in range(cfg["n_layers"]):
        p = f"layers.{l}."
        a = torch.nn.functional.layer_norm(x, (d,), t(p + "norm1.g"), t(p + "norm1.b"), cfg["eps"])
        qkv = a @ t(p + "wqkv.w").reshape(3 * d, d).T + t(p + "wqkv.b")
        q, k, v = [z.reshape(T, H, Dh).permute(1, 0, 2) for z in qkv.split(d, -1)]
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).permute(1, 0, 2).reshape(T, d)
        x = x + o @ t(p + "wo.w").reshape(d, d).T + t(p + "wo.b")
        a = torch.nn.functional.layer_norm(x, (d,), t(p + "norm2.g"), t(p + "norm2.b"), cfg["eps"])
        h = torch.nn.functional.gelu(a @ t(p + "wfc.w").reshape(-1, d).T + t(p + "wfc.b"), approximate="tanh")
        x = x + h @ t(p + "wproj.w").reshape(d, -1).T + t(p + "wproj.b")
    a = torch.nn.functional.layer_norm(x[-1:], (d,), t("normf.g"), t("normf.b"), cfg["eps"])
    want = (a @ wte.T)[0].numpy()
    assert np.allclose(logits, want, rtol=1e-4, atol=2e-5)
    st.close()
    m.close()


@pytest.mark.parametrize("cfg,seed", [(TINY_QWEN, 4), (TINY_GPT2, 0)], ids=["qwen", "gpt2"])
def test_decode_continues_prefill(oracle, cfg, seed):
    """Incremental decoding and ragged prompts give the logits of a single long prefill."""
    m = oracle.Model(cfg, seed)
    toks = oracle.gen_tokens(seed + 1, 1, 2 * 10, cfg["vocab"]).reshape(2, 10)
    full = m.new_state(2, 16)
    want = full.prefill(toks, np.array([10, 7], np.int32))
    inc = m.new_state(2, 16)
    inc.prefill(toks[:, :6], np.array([6, 6], np.int32))
    step = inc.decode(toks[:, 6])
    assert inc.lens().tolist() == [7, 7]
    tol = dict(atol=2e-2) if cfg["arch"] == 1 else dict(rtol=1e-4, atol=1e-5)
    assert np.allclose(step[1], want[1], **tol)  # sequence 1 has 7 tokens
    for i in range(7, 10):
        step = inc.decode(toks[:, i])
    assert np.allclose(step[0], want[0], **tol)
    for s in (full, inc):
        s.close()
    m.close()


# ------------------------------------------------------------------ image workloads (reference-pinned)
def test_adjust_brightness_known_answers(oracle):
    """ImageProcessing/AdjustBrightness.strict:6-7,12-14,23 and Strict.Tests/RunnerTests.cs:270-289."""
    g = GOLD["adjust_brightness"]
    for case in g["cases"]:
        out = oracle.adjust_brightness(np.array(g["test_color"], np.float32), 0, 1, 4, 3, case["brightness"])
        assert out.tolist() == case["expected"]
    run = g["run"]
    n = run["width"] * run["height"]
    image = np.tile(np.array(run["default_color"], np.float32), n)
    out = oracle.adjust_brightness(image, 0, n, 4, 3, run["brightness"]).reshape(run["height"], run["width"], 4)
    assert out[run["height"] // 2, run["width"] // 2, :3].tolist() == run["expected_centre"]
    assert (out[..., 3] == 1.0).all()  # Alpha is not touched
    # a view that starts inside the backing array (offset) and a struct of another width
    flat = np.arange(20, dtype=np.float32)
    out = oracle.adjust_brightness(flat, 2, 3, 5, 2, 0.5)
    want = flat.copy()
    for i in range(3):
        want[2 + 5 * i:2 + 5 * i + 2] += 0.5
    assert np.array_equal(out, want)
    # double sum, one rounding: 0.1 is not a float, so float(x) + float(0.1) would differ
    x = np.array([1.0000001, 0, 0, 1], np.float32)
    assert oracle.adjust_brightness(x, 0, 1, 4, 3, 0.1)[0] == np.float32(np.float64(x[0]) + 0.1)
    assert oracle.adjust_brightness(np.array([0.9, 0.5, 0.1, 1], np.float32), 0, 1, 4, 3, 0.25, clamp01=True).tolist()[:3] == [1.0, 0.75, np.float32(np.float64(np.float32(0.1)) + 0.25)]


def _blur_python(px, w, h):
    """Pixel-by-pixel restatement in Python of BlurInteriorPixel / BlurEdgePixel for small images."""
    src = px.reshape(h, w, 3).astype(np.int64)
    out = np.zeros_like(src)
    for r in range(h):
        for c in range(w):
            r0, r1, c0, c1 = max(r - 2, 0), min(r + 3, h), max(c - 2, 0), min(c + 3, w)
            win = src[r0:r1, c0:c1]
            out[r, c] = win.sum(axis=(0, 1)) // ((r1 - r0) * (c1 - c0))
    return out.astype(np.uint8).reshape(-1)


@pytest.mark.parametrize("w,h", [tuple(s) for s in GOLD["blur"]["sizes"][:3]] + [(1, 1), (3, 7), (5, 5), (6, 4)])
def test_blur_restatement_matches_python_and_is_thread_independent(oracle, w, h):
    """The reference's own check (BlurProducesCorrectResults, :193-206) is that the single-thread
    and the row-parallel blur agree byte for byte; here the C restatement on all threads, on one
    thread, and a Python restatement of the two pixel functions agree on seeded bytes."""
    px = (oracle.gen_tokens(42, 9, w * h * 3, 256)).astype(np.uint8)
    many = oracle.blur5x5_rgb8(px, w, h)
    oracle.lib().or_set_threads(1)
    one = oracle.blur5x5_rgb8(px, w, h)
    oracle.lib().or_set_threads(oracle.num_threads() if oracle.num_threads() > 1 else os.cpu_count() or 1)
    assert np.array_equal(many, one)
    assert np.array_equal(many, _blur_python(px, w, h))
    twice = oracle.blur5x5_rgb8(px, w, h, iterations=2)
    assert np.array_equal(twice, _blur_python(_blur_python(px, w, h), w, h))


def test_noise_floor_of_the_numerics_contract_at_qwen3_8b_width(oracle):
    """The contract rounds activations to bf16 between operators. At Qwen3-8B's width, four layers
    deep, an oracle whose RMSNorm gains are 1 + 1e-6 (eight fp32 ulps) instead of 1 ends up with
    logits that differ from the unperturbed oracle's by about 7e-3 mean-rel: a difference far
    below a bf16 ulp flips some roundings, every flip is a whole bf16 ulp, the next operator
    spreads it. Two faithful implementations with different fp32 summation orders are therefore
    this far apart, which is above the 5e-3 mean-rel bar of the FP8 path; the GPU parity tests
    take 1.5 x this measured floor as their bar where it exceeds 5e-3. (Vocabulary cut to 32768
    rows so that the test runs in seconds; the logits' statistics do not depend on it.)"""
    cfg = dict(arch=1, n_layers=4, d_model=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, d_ff=12288, vocab=32768, max_pos=128, tied=0,
               eps=1e-6, rope_theta=1e6)
    toks = oracle.gen_tokens(105, 1, 32, cfg["vocab"]).reshape(1, 32)
    lens = np.array([32], np.int32)
    logits = []
    for gain in (1.0, 1.0 + 1e-6):
        om = oracle.Model(cfg, 5)
        for l in range(cfg["n_layers"]):
            for name in ("norm1.g", "norm2.g"):
                om.tensor(f"layers.{l}.{name}", np.float32)[:] = np.float32(gain)
        st = om.new_state(1, 40)
        logits.append(st.prefill(toks, lens).copy())
        st.close(), om.close()
    err = np.abs(logits[0] - logits[1])
    mean_rel = err.mean() / np.abs(logits[0]).mean()
    assert 3e-3 < mean_rel < 2e-2, mean_rel   # at or above the 5e-3 bar's order of magnitude, far above fp32 noise (1e-6)
    assert err.max() < 5e-2                    # the max-abs bar of the FP8 path still holds


def test_int8_weight_linear_contract(oracle, rng):
    """The integer path's restatement against plain numpy integer arithmetic: ranges of the two
    activation terms, exactness of the split for elements within a factor 63 of the row's largest, the
    weight quantiser, and the linear layer as exact integer sums (float64 holds them exactly)."""
    M, N, K = 5, 48, 256
    x = oracle.round_bf16(rng.standard_normal((M, K)).astype(np.float32) * np.array([[1e-3], [1.0], [300.0], [0.0], [7.0]], np.float32))
    x[4, 3] = 16256.0 * 2.0 ** -6  # a row maximum whose mantissa is the largest that keeps the smaller scale
    hi, lo, s = oracle.quantize_rows_int8(x)
    assert hi.min() >= -127 and hi.max() <= 127 and lo.min() >= -64 and lo.max() <= 63
    assert s[3] == 1.0 and not hi[3].any() and not lo[3].any()
    v = 128 * hi.astype(np.int64) + lo
    assert np.abs(v).max() <= 16256 and (np.log2(s) % 1 == 0).all()
    amax = np.abs(x).max(axis=1, keepdims=True)
    assert (np.abs(v).max(axis=1)[[0, 1, 2, 4]] > 8128).all()  # the smallest power of two that fits
    rec = v * s[:, None].astype(np.float64)
    big = np.abs(x) >= amax / 63  # |x| / s >= 128: the eight significant bits of a bf16 value are all kept
    assert np.array_equal(rec[big], x.astype(np.float64)[big])
    assert (np.abs(rec - x) <= s[:, None] / 2).all()
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    w[7] = 0.0
    wq, sw = oracle.quantize_weights_int8(w)
    assert np.array_equal(sw, np.where(np.abs(w).max(axis=1) > 0, np.abs(w).max(axis=1) / np.float32(127), np.float32(1)).astype(np.float32))
    assert np.array_equal(wq, np.clip(np.rint(w / sw[:, None]), -127, 127).astype(np.int8)) and np.abs(wq).max() == 127 and not wq[7].any()
    got = oracle.gemm_int8w(x, wq, sw)
    t = (v @ wq.astype(np.int64).T).astype(np.float32)  # exact integers, one rounding to fp32
    want = oracle.f32_to_bf16((t * s[:, None]) * sw[None, :])
    assert np.array_equal(got, want)
    # and the quantised layer stays close to the unquantised one
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(oracle.bf16_to_f32(got) - ref).max() <= 0.02 * np.abs(ref).max()
