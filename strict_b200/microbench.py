"""Kernel microbenchmarks at the shapes of BASELINE.json configs[1] (GEMM/GEMV) and configs[2]
(GQA attention), through the C ABI, timed with CUDA events on the library's stream.

    python -m strict_b200.microbench [gemm] [attn] [--iters N] [--shape M,N,K]

Every timed call reads buffers that were not touched by the previous call (weights rotate
through enough distinct copies to exceed the 126 MB L2; the attention caches are GBs), so the
HBM figures are not L2 figures. The GEMM calls are recorded once (one call per weight copy)
and replayed, so the figure is device time, not the host's submission rate. One JSON line
per case.
"""
import argparse
import json
import os
import sys

import numpy as np

from . import native as N
from .kernel import Context, DeviceVariable as DV

L = N.lib


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def gemm_cases(ctx, iters, shape=None):
    hbm, bf16_tf, kind = _peaks()
    for N_, K in ((4096, 4096), (14336, 4096)) if shape is None else ((shape[1], shape[2]),):
        copies = max(2, int(np.ceil(300e6 / (N_ * K))))  # > 2x L2 of distinct weights
        wq = [DV(ctx, N_ * K, np.uint8) for _ in range(copies)]
        sw = DV(ctx, N_)
        for i, w in enumerate(wq):
            N.check(L().strictb200_gen_weight_e4m3(ctx.h, 2, 10 + i, 0, N_, K, 0, K, 0.02, w.p, sw.p))
        for M in (1, 8, 32, 128, 2048) if shape is None else (shape[0],):
            x = DV(ctx, M * K, np.uint16)
            N.check(L().strictb200_gen_normal_bf16(ctx.h, 2, 99, 0, M * K, 1.0, x.p))
            y = DV(ctx, M * N_, np.uint16)
            rows = 16 * ((M + 7) // 8)
            xq, sx = DV(ctx, rows * K, np.uint8), DV(ctx, M)
            N.check(L().strictb200_quantize_rows(ctx.h, x.p, M, K, xq.p, sx.p))
            for it in range(copies):  # also sizes every scratch buffer before the recording
                N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, xq.p, sx.p, wq[it].p, sw.p, y.p, 0, 0))
            ctx.synchronize()
            with ctx.record():
                for it in range(copies):
                    N.check(L().strictb200_gemm_fp8(ctx.h, M, N_, K, xq.p, sx.p, wq[it].p, sw.p, y.p, 0, 0))
            graph = ctx.last_graph
            reps = max(1, iters // copies)
            ctx.replay(graph, 2)
            ctx.synchronize()
            ctx.timer_begin()
            ctx.replay(graph, reps)
            ms = ctx.timer_end() / (reps * copies)
            ctx.free_graph(graph)
            byts = N_ * K + 4 * N_ + 2 * M * K + 2 * M * N_
            flops = 2.0 * M * N_ * K
            print(json.dumps({"case": "gemm_fp8w", "M": M, "N": N_, "K": K, "us": ms * 1e3, "GBps": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm,
                              "useful_TFLOPs": flops / ms / 1e9, "executed_fp8_TFLOPs": 2 * flops / ms / 1e9,
                              "frac_of_bf16_peak": flops / ms / 1e9 / bf16_tf, "peaks": kind,
                              "note": "split of the activations not included; weights rotate over %d copies" % copies}), flush=True)
            for v in (x, y, xq, sx):
                v.free()
        for w in wq:
            w.free()
        sw.free()


def attn_cases(ctx, iters):
    hbm, bf16_tf, kind = _peaks()
    Hq, Hkv, D = 32, 8, 128
    scale = float(1.0 / np.sqrt(D))
    # decode: batch 64, lengths uniform in [1024, 32768] from the seeded generator (seed 3)
    B, maxlen = 64, 32768
    tok = DV(ctx, B, np.int32)
    N.check(L().strictb200_gen_tokens(ctx.h, 3, 7, B, 32768 - 1024 + 1, tok.p))
    lens = (tok.to_host() + 1024).astype(np.int32)
    q = DV(ctx, B * Hq * D, np.uint16)
    kc, vc = DV(ctx, B * Hkv * maxlen * D, np.uint16), DV(ctx, B * Hkv * maxlen * D, np.uint16)
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 1, 0, B * Hq * D, 1.0, q.p))
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 2, 0, B * Hkv * maxlen * D, 1.0, kc.p))
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 3, 0, B * Hkv * maxlen * D, 1.0, vc.p))
    dl, out = DV.of(ctx, lens), DV(ctx, B * Hq * D, np.uint16)
    for _ in range(3):
        N.check(L().strictb200_attn_decode(ctx.h, q.p, kc.p, vc.p, dl.p, B, Hq, Hkv, D, maxlen, scale, out.p))
    ctx.synchronize()
    ctx.timer_begin()
    for _ in range(iters):
        N.check(L().strictb200_attn_decode(ctx.h, q.p, kc.p, vc.p, dl.p, B, Hq, Hkv, D, maxlen, scale, out.p))
    ms = ctx.timer_end() / iters
    byts = int(lens.sum()) * Hkv * D * 2 * 2
    print(json.dumps({"case": "attn_decode", "B": B, "sum_len": int(lens.sum()), "us": ms * 1e3, "GBps": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm,
                      "peaks": kind, "note": "4.4 GB of K/V per call, far beyond L2"}), flush=True)
    for v in (q, kc, vc, dl, out, tok):
        v.free()
    # prefill: batch 4 x 8192, causal
    B, S = 4, 8192
    q = DV(ctx, B * S * Hq * D, np.uint16)
    kc, vc = DV(ctx, B * Hkv * S * D, np.uint16), DV(ctx, B * Hkv * S * D, np.uint16)
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 4, 0, B * S * Hq * D, 1.0, q.p))
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 5, 0, B * Hkv * S * D, 1.0, kc.p))
    N.check(L().strictb200_gen_normal_bf16(ctx.h, 3, 6, 0, B * Hkv * S * D, 1.0, vc.p))
    dl, out = DV.of(ctx, np.full(B, S, np.int32)), DV(ctx, B * S * Hq * D, np.uint16)
    n = max(2, iters // 5)
    N.check(L().strictb200_attn_prefill(ctx.h, q.p, kc.p, vc.p, dl.p, None, B, S, Hq, Hkv, D, S, scale, out.p))
    ctx.synchronize()
    ctx.timer_begin()
    for _ in range(n):
        N.check(L().strictb200_attn_prefill(ctx.h, q.p, kc.p, vc.p, dl.p, None, B, S, Hq, Hkv, D, S, scale, out.p))
    ms = ctx.timer_end() / n
    flops = 4.0 * B * Hq * D * S * S / 2
    print(json.dumps({"case": "attn_prefill", "B": B, "S": S, "ms": ms, "useful_TFLOPs": flops / ms / 1e9, "frac_of_bf16_peak": flops / ms / 1e9 / bf16_tf,
                      "peaks": kind}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="*", default=["gemm", "attn"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--shape", default=None, help="M,N,K: run the GEMM case for this one shape only")
    args = ap.parse_args()
    ctx = Context(0)
    if "gemm" in args.what:
        gemm_cases(ctx, args.iters, tuple(int(v) for v in args.shape.split(",")) if args.shape else None)
    if "attn" in args.what:
        attn_cases(ctx, args.iters)
    ctx.dispose()


if __name__ == "__main__":
    main()
