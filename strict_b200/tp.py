"""Host-side helpers for tensor parallelism: which slice of every tensor a rank owns (the same
arithmetic the library applies in strictb200_model_set_tensor / _init_random), and the small
collectives the launcher needs (hand-out of the NCCL id, max of a timing over ranks). The
collectives take any torch.distributed backend, so the logic is testable with gloo on CPUs."""
import numpy as np


def shard_ranges(cfg, world, rank):
    """Row/column windows of the full tensors held by `rank`:
    name -> (list of (src_row, n_rows), (col0, n_cols)). Qwen3 layout only."""
    D, d, I = cfg["head_dim"], cfg["d_model"], cfg["d_ff"]
    Hq, Hkv, V = cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab"]
    if Hkv % world or I % (world * 64) or V % (world * 16):
        raise ValueError("heads, d_ff/64 and vocab/16 must divide by the world size")
    nq, nkv = Hq * D, Hkv * D
    nq_l, nkv_l, I_l, V_l = nq // world, nkv // world, I // world, V // world
    r = rank
    return {
        "wqkv": ([(r * nq_l, nq_l), (nq + r * nkv_l, nkv_l), (nq + nkv + r * nkv_l, nkv_l)], (0, d)),
        "wo": ([(0, d)], (r * nq_l, nq_l)),
        "wgu": ([(r * I_l, I_l), (I + r * I_l, I_l)], (0, d)),
        "wdown": ([(0, d)], (r * I_l, I_l)),
        "head": ([(r * V_l, V_l)], (0, d)),
    }


def take_shard(full, spec):
    rows, (c0, nc) = spec
    return np.concatenate([full[r0:r0 + n, c0:c0 + nc] for r0, n in rows], 0)


def share_unique_id(dist, rank, make_id, device="cpu"):
    """Rank 0 creates the 128-byte NCCL id (make_id() -> uint8[128]); every rank returns it."""
    import torch
    t = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        t.copy_(torch.from_numpy(np.ascontiguousarray(make_id(), dtype=np.uint8)))
    dist.broadcast(t, 0)
    return np.ascontiguousarray(t.cpu().numpy())


def max_over_ranks(dist, value, device="cpu"):
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_gather_bytes(dist, mine, device="cpu"):
    """Gather a small uint8 array from every rank, rank order -> uint8[world, len]."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(mine, dtype=np.uint8)).to(device)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return np.stack([o.cpu().numpy() for o in out])
