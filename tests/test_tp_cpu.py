"""World-size-2 tests on CPU ranks (gloo): the sharding arithmetic of the tensor-parallel layer
and the launcher's small collectives, with no GPU involved. Each rank takes its slice of the
oracle's weights, computes its partial projection, the partials are summed with an all-reduce —
the result must equal the unsharded oracle (fp32 sums in a different order only)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from strict_b200 import tp

CFG = dict(arch=1, n_layers=1, d_model=256, n_q_heads=4, n_kv_heads=2, head_dim=128, d_ff=512, vocab=1024, max_pos=64, tied=0,
           eps=1e-6, rope_theta=1e6)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        m = O.Model(CFG, 7)
        d, D, I = CFG["d_model"], CFG["head_dim"], CFG["d_ff"]
        nq = CFG["n_q_heads"] * D
        spec = tp.shard_ranges(CFG, world, rank)
        rng = np.random.default_rng(0)  # same activations on every rank
        att = O.round_bf16(rng.standard_normal((5, nq)).astype(np.float32))
        h = O.round_bf16(rng.standard_normal((5, I)).astype(np.float32))
        a = O.round_bf16(rng.standard_normal((5, d)).astype(np.float32))
        res = {}
        # row-parallel projections: slice of the input columns, partial sums all-reduced
        for name, x in (("wo", att), ("wdown", h)):
            wq = np.array(m.tensor(f"layers.0.{name}.q", np.uint8)).reshape(d, -1)
            sw = np.array(m.tensor(f"layers.0.{name}.s", np.float32))
            c0, nc = spec[name][1]
            part = torch.from_numpy(O.linear_fp8w(x[:, c0:c0 + nc], tp.take_shard(wq, spec[name]), sw))
            dist.all_reduce(part)
            res[name] = (part.numpy(), O.linear_fp8w(x, wq, sw))
        # column-parallel projections: each rank owns output channels; gathered they equal the whole
        for name in ("wqkv", "wgu", "head"):
            key = "head" if name == "head" else f"layers.0.{name}"
            wq = np.array(m.tensor(key + ".q", np.uint8)).reshape(-1, d)
            sw = np.array(m.tensor(key + ".s", np.float32))
            rows = spec[name][0]
            mine = O.linear_fp8w(a, tp.take_shard(wq, spec[name]), np.concatenate([sw[r0:r0 + n] for r0, n in rows]))
            full = O.linear_fp8w(a, wq, sw)
            want = np.concatenate([full[:, r0:r0 + n] for r0, n in rows], 1)
            res[name] = (mine, want)
        uid = tp.share_unique_id(dist, rank, lambda: np.arange(128, dtype=np.uint8) ^ 0x5A)
        mx = tp.max_over_ranks(dist, 1.5 + rank)
        gathered = tp.all_gather_bytes(dist, np.full(64, rank, np.uint8))
        ok = all(np.allclose(g, w, rtol=1e-5, atol=1e-6 * np.abs(w).max()) for g, w in res.values())
        ok = ok and np.array_equal(res["wqkv"][0], res["wqkv"][1])  # column shards are exact
        ok = ok and np.array_equal(uid, np.arange(128, dtype=np.uint8) ^ 0x5A) and mx == 1.5 + world - 1
        ok = ok and gathered.shape == (world, 64) and all((gathered[r] == r).all() for r in range(world))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_projections_equal_unsharded_on_two_cpu_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_shard_ranges_cover_every_tensor_once():
    cfg = dict(CFG, n_q_heads=32, n_kv_heads=8, d_model=4096, d_ff=12288, vocab=151936)
    D = cfg["head_dim"]
    for world in (1, 2, 4, 8):
        seen = {k: [] for k in ("wqkv", "wo", "wgu", "wdown", "head")}
        for r in range(world):
            for k, (rows, cols) in tp.shard_ranges(cfg, world, r).items():
                seen[k].append((rows, cols))
        qkv_rows = sorted(x for rows, _ in seen["wqkv"] for x in rows)
        assert sum(n for _, n in qkv_rows) == (32 + 16) * D and all(a + n == b for (a, n), (b, _) in zip(qkv_rows, qkv_rows[1:]))
        assert sorted(c for _, c in seen["wo"]) == [(r * 4096 // world, 4096 // world) for r in range(world)]
        assert sorted(c for _, c in seen["wdown"]) == [(r * 12288 // world, 12288 // world) for r in range(world)]
        assert sum(n for rows, _ in seen["head"] for _, n in rows) == 151936
    with pytest.raises(ValueError):
        tp.shard_ranges(dict(cfg, n_kv_heads=2), 4, 0)
