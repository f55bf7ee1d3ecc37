"""Tensor-parallel parity on two GPUs (skipped on a one-GPU box): two processes, one context per
GPU, NCCL over NVLink; prefill logits and greedy tokens of a small Qwen3-shaped model against the
same CPU oracle as TP=1 (TP only changes the order of fp32 sums)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(arch=1, n_layers=3, d_model=512, n_q_heads=8, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=2048, max_pos=128, tied=0,
           eps=1e-6, rope_theta=1e6)


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, port, path, out, fused):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if fused:
        os.environ["STRICTB200_TP_TWO_SHOT"] = "1" if fused == 2 else "0"  # the two exchange patterns of the fused all-reduce
    import torch.distributed as dist
    import strict_b200 as sb
    from strict_b200 import native as N, tp
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ctx = sb.Context(rank)

        def make_id():
            h = np.zeros(128, np.uint8)
            N.check(N.lib().strictb200_tp_unique_id(N.ptr(h)))
            return h
        ctx.tp_init(world, rank, N.ptr(tp.share_unique_id(dist, rank, make_id)))
        if fused:
            ctx.tp_open_peer_buffers(lambda mine: tp.all_gather_bytes(dist, mine))
        m = sb.Model(ctx, CFG).init_random(11)
        from oracle import oracle as O
        toks = O.gen_tokens(12, 1, 3 * 20, CFG["vocab"]).reshape(3, 20)
        lens = np.array([20, 9, 14], np.int32)
        kv = m.new_cache(3, 64)
        nxt, logits = kv.prefill(toks, lens, want_logits=True)
        ids = kv.generate(nxt, 16)
        assert ctx.device_status() == 0
        if rank == 0:
            np.savez(path, nxt=nxt, logits=logits, ids=ids, toks=toks, lens=lens)
        dist.barrier()
        kv.dispose(), m.dispose(), ctx.dispose()
        out[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fused", [0, 1, 2], ids=["nccl", "peer-memory-one-shot", "peer-memory-two-shot"])
def test_tp2_matches_oracle(oracle, tmp_path, fused):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    path = str(tmp_path / "tp2.npz")
    mp.spawn(_worker, args=(2, port, path, out, fused), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}
    r = np.load(path)
    om = oracle.Model(CFG, 11)
    st = om.new_state(3, 64)
    want = st.prefill(r["toks"], r["lens"])
    err = np.abs(r["logits"] - want)
    assert err.max() <= 5e-2 and err.mean() / np.abs(want).mean() <= 5e-3, (err.max(), err.mean())
    pick = oracle.argmax(want)
    alive = np.ones(3, bool)
    seq = np.vstack([r["nxt"][None], r["ids"]])
    for s_ in range(17):
        for b in range(3):
            if alive[b] and pick[b] != seq[s_, b]:
                alive[b] = False  # compared against the oracle's margin below
                assert logits_margin(st_logits, b, pick[b], seq[s_, b]) <= 5e-2
        if s_ < 16:
            st_logits = st.decode(pick)
            pick = oracle.argmax(st_logits)
    st.close(), om.close()


def logits_margin(logits, b, a, c):
    return float(logits[b, a] - logits[b, c])
