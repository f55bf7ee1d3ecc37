"""Headline benchmark: Qwen3-8B-architecture FP8 greedy decode, batch 32, context 2048, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (torchrun for N > 1, tensor-parallel over NCCL). A step is one decode step
of all 32 sequences. `value` is timed on the device with the token ids resident in HBM
(CUDA-graph replay of the step); `e2e` goes through the public decode_step call with host ids
in and host ids out every step. The workload streams ~17.8 GB per step, far beyond the 126 MB
L2, so no flush is needed between steps. Weights, prompts and the reference arm's tensors are
synthetic (seeded generator), random-initialised, of the architecture's exact shapes.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, PROMPT, NEW_TOKENS = 32, 2048, 256
SEED = 5
METRIC = "qwen3_8b_fp8_decode_tokens_per_s"
WORKLOAD = "qwen3-8b fp8 greedy decode, batch 32, prompt 2048 (BASELINE.json configs[4])"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


from strict_b200.clocks import ClockSampler  # noqa: E402


# ---------------------------------------------------------------------------------- CPU arm
CPU_TIME_BUDGET_S = 150.0  # wall time the timed steps of the CPU arm may take; fewer steps are run (and reported) beyond it


def workload_config(n_gpus):
    """The keys that name the workload; identical in both arms."""
    return {"workload": WORKLOAD, "batch": BATCH, "prompt": PROMPT, "layers": 36, "parallelism": f"tp{n_gpus}",
            "l2": "inputs larger than L2 (17.8 GB streamed per step)"}


def mem_available_gb():
    try:
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable:"):
                return int(ln.split()[1]) / 1e6
    except OSError:
        pass
    return None


def cpu_reference(steps, warmup):
    """The reference has no implementation of this path; its stand-in is this repository's CPU
    oracle (kind "port"). What is timed is the oracle's own decode step of the whole model — all
    36 layers with their norms, RoPE, SwiGLU and attention, the LM head and the greedy pick — at
    batch 32 and context 2048 on all host threads, step after step, each step feeding the next.
    Set-up (untimed): the seeded weights of the full architecture; the cache is filled with
    pseudo-random keys and values instead of a CPU prefill of 65,536 tokens, which would take
    hours. Every reported step was executed; nothing is multiplied. If the requested steps would
    take longer than CPU_TIME_BUDGET_S, fewer are run and the line says how many."""
    from oracle import oracle as O
    import strict_b200 as sb
    O.build()
    cfg = dict(sb.CONFIGS["qwen3-8b"])
    ctx_len = PROMPT
    n_max = warmup + steps + 1
    kv_gb = 2 * cfg["n_layers"] * BATCH * cfg["n_kv_heads"] * (ctx_len + n_max) * cfg["head_dim"] * 4 / 1e9
    need_gb = kv_gb + 7.6 + 2.5 + 4.0
    avail = mem_available_gb()
    note = ""
    if avail is not None and avail < need_gb:
        # keep the host alive: shorten the context to what fits and say so
        per_pos_gb = 2 * cfg["n_layers"] * BATCH * cfg["n_kv_heads"] * cfg["head_dim"] * 4 / 1e9
        ctx_len = max(64, int((avail - 16.0) / per_pos_gb) - n_max)
        note = f"; host has {avail:.0f} GB free, context cut to {ctx_len}"
    t0 = time.perf_counter()
    om = O.Model(cfg, SEED)
    st = om.new_state(BATCH, ctx_len + n_max)
    st.fill_synthetic(SEED + 2, ctx_len)
    setup_s = time.perf_counter() - t0
    ids = O.gen_tokens(SEED + 1, 2, BATCH, cfg["vocab"])
    times = []
    t_begin = None
    for it in range(warmup + steps):
        if it == warmup:
            t_begin = time.perf_counter()
        if it > warmup and time.perf_counter() - t_begin > CPU_TIME_BUDGET_S:
            break
        t1 = time.perf_counter()
        ids = O.argmax(st.decode(ids))
        if it >= warmup:
            times.append(time.perf_counter() - t1)
    st.close(), om.close()
    step_s = float(np.mean(times))
    return {"value": BATCH / step_s, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{len(times)} whole decode steps (36 layers + LM head + greedy pick, batch {BATCH}, context {ctx_len}+) of the CPU oracle on "
                      f"{O.num_threads()} threads after {warmup} warm-up steps; every step executed, wall clock; set-up {setup_s:.0f} s untimed "
                      f"(seeded weights, pseudo-random cache){note}",
            "steps_run": len(times), "timed_s": float(np.sum(times))}, step_s


def run_reference(args, rank):
    if rank != 0:
        return
    base, step_s = cpu_reference(max(1, args.steps), max(0, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": base["steps_run"],
            "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 x fp8_e4m3 -> f32", "data": "synthetic", "config": workload_config(args.gpus),
            "timing": "host wall clock around every step", "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------- GPU arm
# DRAM traffic per launch over algorithmic bytes, from the ncu captures summarised in profiles/
# (attn_decode_kernel: 269.5 MB read + 4.5 MB written for 270.5 MB of keys and values; the decode
# GEMMs: 101.05 + 4.06 MB for 100.66 MB of weights).
TRAFFIC_RATIO = {"attn_decode": 1.013, "gemm_gate_up": 1.044}


def run_ours(args, rank, world, local_rank):
    import strict_b200 as sb
    from strict_b200 import native as N, tp
    # Libraries (NCCL prints its version banner) write to file descriptor 1 while the job runs:
    # send that to stderr and give stdout back just before the one JSON line.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist:
            dist.barrier()

    def max_over_ranks(x):
        return tp.max_over_ranks(dist, x, "cuda") if dist else x

    ctx = sb.Context(local_rank)
    if world > 1:
        def make_id():
            h = np.zeros(128, np.uint8)
            N.check(N.lib().strictb200_tp_unique_id(N.ptr(h)))
            return h
        ctx.tp_init(world, rank, N.ptr(tp.share_unique_id(dist, rank, make_id, "cuda")))
        if not args.nccl_allreduce:
            # decode all-reduces: one-shot over peer memory, fused into the consuming row kernel
            ctx.tp_open_peer_buffers(lambda mine: tp.all_gather_bytes(dist, mine, "cuda"))
    if args.two_shot >= 0:
        ctx.set_option("tp_two_shot", args.two_shot)
    cfg = dict(sb.CONFIGS["qwen3-8b"])
    if args.layers:
        cfg["n_layers"] = args.layers  # profiling aid: same kernels and shapes, fewer layers resident
    model = sb.Model(ctx, cfg).init_random(SEED)
    if args.no_graph:
        model.set_graph(False)
    total_steps = 2 * (max(args.warmup, 3) + args.steps) + 16 + (NEW_TOKENS if not args.no_sustained else 0)
    kv = model.new_cache(BATCH, PROMPT + total_steps + 8)
    # prompts: 32 x 2048 uniform ids from the seeded generator; real prefill fills the cache
    toks = np.empty((BATCH, PROMPT), np.int32)
    d_tok = sb.DeviceVariable(ctx, BATCH * PROMPT, np.int32)
    N.check(N.lib().strictb200_gen_tokens(ctx.h, SEED + 1, 1, BATCH * PROMPT, cfg["vocab"], d_tok.p))
    toks[:] = d_tok.to_host().reshape(BATCH, PROMPT)
    d_tok.free()
    t0 = time.perf_counter()
    prefill_dev_s, prefill_clocks = None, None
    if args.synthetic_kv:
        kv.fill_synthetic(SEED + 2, PROMPT)  # profiling aid: seeded N(0,1) keys/values instead of the prefill
        first = toks[:, -1].copy()
    else:
        pf_sampler = ClockSampler(local_rank)
        if rank == 0:
            pf_sampler.start()
        ctx.timer_begin()
        first, _ = kv.prefill(toks)
        prefill_dev_s = ctx.timer_end() / 1e3
        if rank == 0:
            prefill_clocks = pf_sampler.stop()  # the prefill is tensor-bound: its time follows the SM clock under the power cap
            if prefill_clocks.get("sm_mhz"):
                prefill_clocks["device_s_x_sm_mhz"] = prefill_dev_s * prefill_clocks["sm_mhz"]
    ctx.synchronize()
    prefill_s = time.perf_counter() - t0
    barrier()  # the ranks leave the set-up together: a rank's first decode step waits for its peers inside a kernel, with a bounded wait

    # ---- value: device-resident ids, graph replay
    ids_dev = first.copy()
    kv.decode_step(ids_dev)  # plain-launch step (one-time set-up), leaves next ids on the device
    kv.decode_steps_device(max(args.warmup, 3))  # includes the graph capture
    ctx.synchronize()
    bytes_step = kv.decode_bytes()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count()
    ctx.synchronize()
    barrier()
    ctx.timer_begin()
    kv.decode_steps_device(args.steps)
    ms = ctx.timer_end()
    barrier()
    launches = ctx.launch_count() - launches0
    ms = max_over_ranks(ms)
    clocks = sampler.stop() if rank == 0 else None
    value = BATCH * args.steps / (ms / 1e3)

    # ---- sustained: the specification's 256 decoded tokens in one timed region (same method, graph replay)
    sustained = None
    if not args.no_sustained:
        barrier()
        s_sampler = ClockSampler(local_rank)
        if rank == 0:
            s_sampler.start()
        ctx.synchronize()
        barrier()
        ctx.timer_begin()
        kv.decode_steps_device(NEW_TOKENS)
        s_ms = max_over_ranks(ctx.timer_end())
        barrier()
        sustained = {"value": BATCH * NEW_TOKENS / (s_ms / 1e3), "unit": "tokens/s", "steps": NEW_TOKENS, "ms_per_step": s_ms / NEW_TOKENS,
                     "clocks": s_sampler.stop() if rank == 0 else None}

    # ---- e2e: host ids in, host ids out, every step, through the public decode_step call
    h_in = np.zeros(BATCH, np.int32)
    h_out = np.zeros(BATCH, np.int32)
    nxt, _ = kv.decode_step(first)
    for _ in range(max(args.warmup, 3)):
        nxt, _ = kv.decode_step(nxt)
    ctx.synchronize()
    barrier()
    t0 = time.perf_counter()
    h_in[:] = nxt
    for _ in range(args.steps):
        kv.decode_step(h_in, out=h_out)
        h_in[:] = h_out
    ctx.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    e2e = {"value": BATCH * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4,
           "ms_per_step": e2e_s / args.steps * 1e3}

    # ---- optional: where one graph-replayed step's time goes, from per-block time stamps (outside every timed region)
    timeline = None
    if not args.no_timeline:
        from strict_b200 import timeline as TL
        with ctx.trace(1 << 18) as tr:
            kv.decode_steps_device(1)
        Hkv_t, D_t = cfg["n_kv_heads"] // world, cfg["head_dim"]
        d_t, I_t, nq_t = cfg["d_model"], cfg["d_ff"] // world, cfg["n_q_heads"] // world * D_t
        names = {(nq_t + 2 * Hkv_t * D_t, d_t): "gemm_qkv", (d_t, nq_t): "gemm_o", (2 * I_t, d_t): "gemm_gate_up", (d_t, I_t): "gemm_down",
                 (cfg["vocab"] // world, d_t): "head"}
        ll = TL.launches(tr.records, names)
        timeline = {"blocks_reported": tr.reported, "launches": len(ll), "span_us": (ll[-1]["end"] / 1e3) if ll else 0.0,
                    "exposed_us": {k: [v[0] / 1e3, v[1]] for k, v in TL.per_kernel(ll).items()}}
        if args.timeline:
            with open(args.timeline + f".rank{rank}" if world > 1 else args.timeline, "w") as f:
                json.dump({"summary": timeline, "launches": ll}, f)

    # ---- per-kernel-class device times of the same step (plain launches, CUDA events on the launch stream)
    prof = kv.profile_decode(4)
    lens_now = kv.lens()
    Hkv_l, D, Ln = cfg["n_kv_heads"] // world, cfg["head_dim"], cfg["n_layers"]
    d, I_l, nq_l = cfg["d_model"], cfg["d_ff"] // world, cfg["n_q_heads"] // world * D
    alg = {  # algorithmic bytes per call of each class (weights or KV streamed once)
        "gemm_qkv": (nq_l + 2 * Hkv_l * D) * d, "gemm_o": d * nq_l, "gemm_gate_up": 2 * I_l * d, "gemm_down": d * I_l,
        "head": cfg["vocab"] // world * d, "attn_decode": int(lens_now.sum()) * Hkv_l * D * 2 * 2,
    }
    hbm, peak_kind = peaks()
    kernels = {}
    for k, (tot, calls) in prof.items():
        if calls:
            e = {"ms_per_call": tot / calls, "calls_per_step": calls / 4, "share": None}
            if k in alg:
                e["gbs"] = alg[k] / (tot / calls * 1e-3) / 1e9
                e["frac"] = e["gbs"] / hbm
            kernels[k] = e
    tot_ms = sum(v[0] for v in prof.values())
    for k in kernels:
        kernels[k]["share"] = prof[k][0] / tot_ms
    if timeline:
        # the same classes inside the graph-replayed step, from the kernels' own time stamps: how far each launch moved the
        # end of the chain (the traced replay is about 6 % slower than an untraced one, so these fractions are on the low side)
        total_us = {}
        for k, (us, n) in timeline["exposed_us"].items():
            k = {"rope": "rope_kvappend", "rownorm_allreduce": "rownorm", "attn_combine": "attn_merge"}.get(k, k)
            total_us[k] = total_us.get(k, 0.0) + us
        for k, us in total_us.items():
            if k in kernels and kernels[k]["calls_per_step"]:
                us = us / kernels[k]["calls_per_step"]  # per call of the class, as ms_per_call is
                kernels[k]["exposed_us_in_step"] = us
                if k in alg:
                    kernels[k]["frac_in_step"] = alg[k] / (us * 1e-6) / 1e9 / hbm
    dom = max((k for k in kernels if k in alg), key=lambda k: prof[k][0])
    roofline = {"bound": "hbm", "kernel": dom, "achieved": kernels[dom]["gbs"], "peak": hbm, "unit": "GB/s", "frac": kernels[dom]["frac"],
                "traffic": TRAFFIC_RATIO[dom] * alg[dom] if dom in TRAFFIC_RATIO else None,
                "traffic_note": "ncu dram__bytes_read+write per launch / algorithmic bytes of the same launch (profiles/), times this launch's algorithmic bytes",
                "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": alg[dom],
                "step": {"algorithmic_bytes": bytes_step, "achieved": bytes_step / (ms / args.steps * 1e-3) / 1e9,
                         "frac": bytes_step / (ms / args.steps * 1e-3) / 1e9 / hbm}}
    if rank != 0:
        barrier()
        kv.dispose(), model.dispose(), ctx.dispose()
        dist.destroy_process_group()
        return
    if dist:
        barrier()
    status = ctx.device_status()  # raises if a bounded device-side wait expired anywhere in the run
    base, _ = cpu_reference(2, 1) if world == 1 and not args.no_cpu else (None, None)
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 x fp8_e4m3 -> f32 (activations as two E4M3 terms on the FP8 tensor cores; bf16 KV)", "data": "synthetic",
            "config": dict(workload_config(world), layers=cfg["n_layers"]),
            "setup": {"context": int(lens_now.mean()), "prefill_s": prefill_s, "prefill_device_s": prefill_dev_s, "prefill_clocks": prefill_clocks,
                      "cuda_graph": not args.no_graph, "kv": "synthetic" if args.synthetic_kv else "prefill of the seeded prompts"},
            "roofline": roofline, "kernels": kernels, "e2e": e2e, "sustained": sustained, "gpu_launches": int(launches), "clocks": clocks,
            "device_status": status}
    if timeline:
        line["timeline"] = timeline
    from strict_b200 import build as _build
    stamp = N.lib().strictb200_build_id().decode()
    line["build"] = {"library": stamp, "sources_beside_it": _build.source_id(), "match": stamp.split()[0] == _build.source_id()}
    if base:
        line["cpu_baseline"] = base
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    os.close(saved_stdout)
    print(json.dumps(line), flush=True)
    kv.dispose()
    model.dispose()
    ctx.dispose()
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: run only this many of the 36 layers")
    ap.add_argument("--synthetic-kv", action="store_true", help="profiling aid: fill the cache with seeded values instead of the prefill")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 256-step sustained leg")
    ap.add_argument("--nccl-allreduce", action="store_true", help="decode all-reduces through NCCL instead of the fused peer-memory exchange")
    ap.add_argument("--two-shot", type=int, default=-1, help="fused all-reduce: 0 one shot, 1 two shots (default: two with more than four ranks)")
    ap.add_argument("--timeline", default=None, help="also write the per-launch timeline of one graph-replayed decode step (per-block time stamps) to this file")
    ap.add_argument("--no-timeline", action="store_true", help="skip the traced replay (outside every timed region) that gives the per-kernel exposed times")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of CUDA-graph replay of the decode step")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            # convenience: relaunch under torchrun when started as plain python with --gpus N
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
                   "--master-port", os.environ.get("MASTER_PORT", "29517"), os.path.abspath(__file__)] + sys.argv[1:]
            sys.exit(subprocess.call(cmd))
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
