"""Kernel microbenchmarks at the shapes of BASELINE.json configs[1] (GEMM/GEMV) and configs[2]
(GQA attention), through the C ABI, timed with CUDA events on the library's stream.

    python -m strict_b200.microbench [gemm] [attn] [ew] [image] [--iters N] [--shape M,N,K]

Every timed call reads buffers that were not touched by the previous call (weights rotate
through enough distinct copies to exceed the 126 MB L2; the attention caches are GBs), so the
HBM figures are not L2 figures. The GEMM calls are recorded once (one call per weight copy)
and replayed, so the figure is device time, not the host's submission rate. One JSON line
per case. `ew` times the element-wise surface in the six ways of the reference's own
performance harness (Strict.Compiler.Cuda.Tests/TestPerformance.cs:13-61): one element at a
time and in chunks, on one host thread and on all of them, on the GPU, and GPU + host together.
"""
import argparse
import json
import os
import sys

import numpy as np

from . import native as N
from .clocks import ClockSampler
from .kernel import Context, DeviceVariable as DV

L = N.lib
MIN_TIMED_S = 0.6  # every timed region lasts at least this long, so that the 200 ms clock samples fall inside it


def timed(ctx, run, first_reps):
    """run(reps) enqueues the work; returns (ms per rep-unit of the long run, clock record)."""
    run(max(1, first_reps // 4))  # warm-up
    ctx.synchronize()
    ctx.timer_begin()
    run(first_reps)
    ms = ctx.timer_end()
    reps = max(first_reps, int(first_reps * MIN_TIMED_S * 1e3 / max(ms, 1e-3)) + 1)
    sampler = ClockSampler(ctx.device)
    sampler.start()
    ctx.synchronize()
    ctx.timer_begin()
    run(reps)
    ms = ctx.timer_end()
    return ms / reps, sampler.stop()


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
            ms, clocks = timed(ctx, lambda reps: ctx.replay(graph, reps), max(1, iters // copies))
            ms /= copies
            ctx.free_graph(graph)
            byts = N_ * K + 4 * N_ + 2 * M * K + 2 * M * N_
            flops = 2.0 * M * N_ * K
            print(json.dumps({"case": "gemm_fp8w", "M": M, "N": N_, "K": K, "us": ms * 1e3, "GBps": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm,
                              "useful_TFLOPs": flops / ms / 1e9, "executed_fp8_TFLOPs": 2 * flops / ms / 1e9,
                              "frac_of_bf16_peak": flops / ms / 1e9 / bf16_tf, "peaks": kind, "clocks": clocks,
                              "note": "split of the activations not included; weights rotate over %d copies" % copies}), flush=True)
            for v in (x, y, xq, sx):
                v.free()
        for w in wq:
            w.free()
        sw.free()


def gemm_int8_cases(ctx, iters):
    """The int8-weight linear layer (tcgen05 kind::i8) on the two microbenchmark shapes; weights
    N(0, 0.02) from the seeded generator quantised on the device, activations split beforehand."""
    hbm, bf16_tf, kind = _peaks()
    for N_, K in ((4096, 4096), (14336, 4096)):
        copies = max(2, int(np.ceil(300e6 / (N_ * K))))
        wf = DV(ctx, N_ * K)
        wq = [DV(ctx, N_ * K, np.int8) for _ in range(copies)]
        sw = DV(ctx, N_)
        for i, w in enumerate(wq):
            N.check(L().strictb200_gen_normal_f32(ctx.h, 2, 10 + i, 0, N_ * K, 0.02, wf.p))
            N.check(L().strictb200_quantize_weights_int8(ctx.h, wf.p, N_, K, w.p, sw.p))
        wf.free()
        for M in (1, 8, 32, 128, 2048):
            x = DV(ctx, M * K, np.uint16)
            N.check(L().strictb200_gen_normal_bf16(ctx.h, 2, 99, 0, M * K, 1.0, x.p))
            y = DV(ctx, M * N_, np.uint16)
            rows = 16 * ((M + 7) // 8)
            xq, sx = DV(ctx, rows * K, np.int8), DV(ctx, M)
            N.check(L().strictb200_quantize_rows_int8(ctx.h, x.p, M, K, xq.p, sx.p))
            for it in range(copies):
                N.check(L().strictb200_gemm_int8(ctx.h, M, N_, K, xq.p, sx.p, wq[it].p, sw.p, y.p))
            ctx.synchronize()
            with ctx.record():
                for it in range(copies):
                    N.check(L().strictb200_gemm_int8(ctx.h, M, N_, K, xq.p, sx.p, wq[it].p, sw.p, y.p))
            graph = ctx.last_graph
            ms, clocks = timed(ctx, lambda reps: ctx.replay(graph, reps), max(1, iters // copies))
            ms /= copies
            ctx.free_graph(graph)
            byts = N_ * K + 4 * N_ + 2 * M * K + 2 * M * N_
            flops = 2.0 * M * N_ * K
            print(json.dumps({"case": "gemm_int8w", "M": M, "N": N_, "K": K, "us": ms * 1e3, "GBps": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm,
                              "useful_TOPs": flops / ms / 1e9, "executed_int8_TOPs": 2 * flops / ms / 1e9, "peaks": kind, "clocks": clocks,
                              "note": "split of the activations not included; weights rotate over %d copies; the K-split sum is a second kernel" % copies}),
                  flush=True)
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
    def run_decode(reps):
        for _ in range(reps):
            N.check(L().strictb200_attn_decode(ctx.h, q.p, kc.p, vc.p, dl.p, B, Hq, Hkv, D, maxlen, scale, out.p))
    ms, clocks = timed(ctx, run_decode, iters)
    byts = int(lens.sum()) * Hkv * D * 2 * 2
    print(json.dumps({"case": "attn_decode", "B": B, "sum_len": int(lens.sum()), "us": ms * 1e3, "GBps": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm,
                      "peaks": kind, "clocks": clocks, "note": "4.4 GB of K/V per call, far beyond L2"}), flush=True)
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
    def run_prefill(reps):
        for _ in range(reps):
            N.check(L().strictb200_attn_prefill(ctx.h, q.p, kc.p, vc.p, dl.p, None, B, S, Hq, Hkv, D, S, scale, out.p))
    ms, clocks = timed(ctx, run_prefill, max(2, iters // 5))
    flops = 4.0 * B * Hq * D * S * S / 2
    print(json.dumps({"case": "attn_prefill", "B": B, "S": S, "ms": ms, "useful_TFLOPs": flops / ms / 1e9, "frac_of_bf16_peak": flops / ms / 1e9 / bf16_tf,
                      "peaks": kind, "clocks": clocks}), flush=True)


def ew_cases(ctx, count=1 << 24, chunk=100):
    """The reference's six timings (TestPerformance.cs:16-21: SingleThread, SingleThreadChunks,
    ParallelCpu, ParallelCpuChunks, CudaGpu, CudaGpuAndCpu) for out = a + b over `count` floats.
    The host legs are numpy on slices (one element per call for the unchunked ones, on a bounded
    prefix whose size is reported); the GPU legs include the copies in both directions, as the
    reference's RunGpu does through CudaDeviceVariable (CSharpToCudaTranspilerTests.cs:64-77)."""
    import time
    from concurrent.futures import ThreadPoolExecutor
    hbm, _, kind = _peaks()
    rng = np.random.default_rng(6)
    a, b = rng.standard_normal(count, np.float32), rng.standard_normal(count, np.float32)
    out = np.empty_like(a)
    threads = os.cpu_count() or 1
    pool = ThreadPoolExecutor(threads)

    def run_chunk(start, n):
        np.add(a[start:start + n], b[start:start + n], out=out[start:start + n])

    def spread(lo, hi, step):  # Parallel.For over [lo, hi) in steps of `step`, one span per thread
        idx = list(range(lo, hi, step))
        per = (len(idx) + threads - 1) // threads
        list(pool.map(lambda part: [run_chunk(i, step) for i in part], [idx[t * per:(t + 1) * per] for t in range(threads)]))

    da, db, do = DV(ctx, count), DV(ctx, count), DV(ctx, count)

    def run_gpu(n):
        if n <= 0:
            return
        N.check(L().strictb200_upload(ctx.h, da.p, N.ptr(a), 4 * n))
        N.check(L().strictb200_upload(ctx.h, db.p, N.ptr(b), 4 * n))
        N.check(L().strictb200_ew_binary(ctx.h, 0, da.p, db.p, do.p, n))
        N.check(L().strictb200_download(ctx.h, N.ptr(out), do.p, 4 * n))

    small = min(count, 1 << 18)  # one numpy call per element is ~1 us: bound the unchunked legs
    legs = [
        ("SingleThread", small, lambda: [run_chunk(i, 1) for i in range(small)]),
        ("SingleThreadChunks", count, lambda: [run_chunk(i, chunk) for i in range(0, count - chunk + 1, chunk)]),
        ("ParallelCpu", small, lambda: spread(0, small, 1)),
        ("ParallelCpuChunks", count, lambda: spread(0, count - chunk + 1, chunk)),
        ("CudaGpu", count, lambda: run_gpu(count)),
    ]
    gpu_n = int(count * 0.97) // chunk * chunk  # the reference's GpuFactor (TestPerformance.cs:56)

    def both():
        f = pool.submit(run_gpu, gpu_n)
        for i in range(gpu_n, count - chunk + 1, chunk):
            run_chunk(i, chunk)
        f.result()
    legs.append(("CudaGpuAndCpu", count, both))
    run_gpu(count)  # warm the context and page the host arrays in
    for name, n, fn in legs:
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        print(json.dumps({"case": "ew_add", "variant": name, "elements": n, "chunk": chunk, "host_threads": threads,
                          "ms": dt * 1e3, "Melem_per_s": n / dt / 1e6}), flush=True)
    assert np.array_equal(out[:count // chunk * chunk], (a + b)[:count // chunk * chunk])
    # the kernel alone, device-resident (3 x 4 bytes per element), larger than L2
    ctx.synchronize()
    reps = 20
    N.check(L().strictb200_ew_binary(ctx.h, 0, da.p, db.p, do.p, count))
    ctx.timer_begin()
    for _ in range(reps):
        N.check(L().strictb200_ew_binary(ctx.h, 0, da.p, db.p, do.p, count))
    ms = ctx.timer_end() / reps
    print(json.dumps({"case": "ew_add", "variant": "kernel_only_device_resident", "elements": count, "us": ms * 1e3,
                      "GBps": 12.0 * count / ms / 1e6, "hbm_frac": 12.0 * count / ms / 1e6 / hbm, "peaks": kind}), flush=True)
    for v in (da, db, do):
        v.free()
    pool.shutdown()


def image_cases(ctx, iters):
    """The image workloads: the 5x5 box blur over RGB bytes on an image larger than L2 (one byte
    read and one written per byte of image) and at the reference harness's size and iteration
    count (2048x1024, 200 passes, Strict.Compiler.Cuda.Tests/BlurPerformanceTests.cs:20-26, with
    the copies to and from the device, as its RunGpu has); AdjustBrightness over 2^26 colours."""
    import time
    hbm, _, kind = _peaks()
    w, h = 8192, 8192
    n = w * h * 3
    a, b = DV(ctx, n, np.uint8), DV(ctx, n, np.uint8)
    N.check(L().strictb200_gen_tokens(ctx.h, 42, 11, n // 4, 1 << 31, a.p))

    def run_blur(reps):
        for _ in range(reps):
            N.check(L().strictb200_blur5x5_rgb8(ctx.h, a.p, b.p, w, h))
    ms, clocks = timed(ctx, run_blur, max(4, iters // 4))
    print(json.dumps({"case": "blur5x5_rgb8", "width": w, "height": h, "us": ms * 1e3, "GBps": 2.0 * n / ms / 1e6, "hbm_frac": 2.0 * n / ms / 1e6 / hbm,
                      "bytes_per_pixel_byte": 2, "peaks": kind, "clocks": clocks, "note": "201 MB read + 201 MB written per pass, larger than L2"}), flush=True)
    for v in (a, b):
        v.free()
    w, h, passes = 2048, 1024, 200
    n = w * h * 3
    host = np.random.default_rng(42).integers(0, 256, n, dtype=np.uint8)
    a, b = DV(ctx, n, np.uint8), DV(ctx, n, np.uint8)
    out = np.empty(n, np.uint8)

    def harness():
        N.check(L().strictb200_upload(ctx.h, a.p, N.ptr(host), n))
        x, y = a, b
        for _ in range(passes):
            N.check(L().strictb200_blur5x5_rgb8(ctx.h, x.p, y.p, w, h))
            x, y = y, x
        N.check(L().strictb200_download(ctx.h, N.ptr(out), x.p, n))
    harness()
    t0 = time.perf_counter()
    harness()
    dt = time.perf_counter() - t0
    print(json.dumps({"case": "blur5x5_rgb8", "variant": "CudaGpu (reference harness: 2048x1024, 200 passes, copies included)", "ms": dt * 1e3,
                      "pixel_passes_per_s": w * h * passes / dt, "note": "6.3 MB image: resident in L2 between passes"}), flush=True)
    for v in (a, b):
        v.free()
    count = 1 << 26
    flat = DV(ctx, count * 4)
    N.check(L().strictb200_gen_normal_f32(ctx.h, 6, 1, 0, count * 4, 0.1, flat.p))

    def run_brightness(reps):
        for _ in range(reps):
            N.check(L().strictb200_adjust_brightness(ctx.h, flat.p, 0, count, 4, 3, 1e-6, 0))
    ms, clocks = timed(ctx, run_brightness, max(4, iters // 4))
    print(json.dumps({"case": "adjust_brightness", "colors": count, "flat_width": 4, "us": ms * 1e3, "GBps": 32.0 * count / ms / 1e6,
                      "hbm_frac": 32.0 * count / ms / 1e6 / hbm, "peaks": kind, "clocks": clocks,
                      "note": "16 bytes read and written per colour (the 128-bit access also carries Alpha)"}), flush=True)
    flat.free()


def model_cases(ctx):
    """Decode throughput of the two single-GPU model configurations as they are specified: GPT-2
    small (fp32, batch 1, prompt 128, 128 decoded tokens) and Qwen3-0.6B (FP8 weights, batch 8,
    prompts of 512, 256 decoded tokens); seeded weights and prompts, greedy steps with the ids
    resident on the device (graph replay), CUDA events around the whole decode loop."""
    from .model import CONFIGS, Model
    hbm, _, kind = _peaks()
    for name, B, prompt, new, seed in (("gpt2-small", 1, 128, 128, 0), ("qwen3-0.6b", 8, 512, 256, 4)):
        cfg = CONFIGS[name]
        m = Model(ctx, cfg).init_random(seed)
        kv = m.new_cache(B, prompt + new + 8)
        tok = DV(ctx, B * prompt, np.int32)
        N.check(L().strictb200_gen_tokens(ctx.h, seed + 1, 1, B * prompt, cfg["vocab"], tok.p))
        first, _ = kv.prefill(tok.to_host().reshape(B, prompt))
        kv.decode_step(first)            # plain launches once (set-up)
        kv.decode_steps_device(3)        # includes the graph capture
        ctx.synchronize()
        bytes_step = kv.decode_bytes()
        sampler = ClockSampler(ctx.device)
        sampler.start()
        ctx.synchronize()
        ctx.timer_begin()
        kv.decode_steps_device(new - 4)
        ms = ctx.timer_end()
        clocks = sampler.stop()
        steps = new - 4
        print(json.dumps({"case": "model_decode", "model": name, "batch": B, "prompt": prompt, "steps": steps, "ms_per_step": ms / steps,
                          "tokens_per_s": B * steps / (ms / 1e3), "bytes_per_step": bytes_step, "GBps": bytes_step / (ms / steps) / 1e6,
                          "hbm_frac": bytes_step / (ms / steps) / 1e6 / hbm, "peaks": kind, "clocks": clocks,
                          "note": "a step streams %.2f GB (weights + cache); below ~1 GB a step is a chain of launch-bound kernels" % (bytes_step / 1e9)}),
              flush=True)
        tok.free()
        kv.dispose()
        m.dispose()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="*", default=["gemm", "attn"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--shape", default=None, help="M,N,K: run the GEMM case for this one shape only")
    args = ap.parse_args()
    ctx = Context(0)
    if "gemm" in args.what:
        gemm_cases(ctx, args.iters, tuple(int(v) for v in args.shape.split(",")) if args.shape else None)
    if "int8" in args.what:
        gemm_int8_cases(ctx, args.iters)
    if "attn" in args.what:
        attn_cases(ctx, args.iters)
    if "ew" in args.what:
        ew_cases(ctx)
    if "image" in args.what:
        image_cases(ctx, args.iters)
    if "models" in args.what:
        model_cases(ctx)
    ctx.dispose()


if __name__ == "__main__":
    main()
