"""Reads a trace of per-block time stamps (Context.trace) as a timeline of kernel launches.

A launch is a run of blocks of one (kernel id, tag) whose start times follow each other without a
gap longer than the blocks before them ran; launches are ordered by the end of their last block,
and each one's "exposed" time is how far it moved the end of the chain: end(launch) - end(previous
launch). The exposed times add up to the step, so they say where the step's time goes when
dependent launches overlap (programmatic dependent launch, loads issued before the dependency
wait), which per-kernel timings of separate launches cannot."""
import numpy as np

KERNELS = {1: "gemm", 2: "rownorm", 3: "rope", 4: "attn_decode", 5: "attn_combine", 6: "swiglu", 7: "rownorm_allreduce"}


def launches(records, gemm_names=None):
    """records: (n, 8) uint64. gemm_names: {(N, K): name} to label the GEMM launches.
    Returns a list of dicts ordered by end time; times are ns from the first block's start."""
    if len(records) == 0:
        return []
    rec = np.asarray(records, dtype=np.uint64)
    word = rec[:, 3]
    kid = (word & np.uint64(0xFF)).astype(np.int64)
    tag = ((word >> np.uint64(8)) & np.uint64(0xFFFFFFFFFF)).astype(np.int64)
    t0 = rec[:, 0].astype(np.int64)
    tw = rec[:, 1].astype(np.int64)
    t2 = rec[:, 2].astype(np.int64)
    origin = t0.min()
    tags = {}
    for (n, k), name in (gemm_names or {}).items():
        tags[(n ^ (k << 12)) & 0xFFFFFFFF] = name
    out = []
    for key in sorted(set(zip(kid.tolist(), tag.tolist()))):
        sel = np.flatnonzero((kid == key[0]) & (tag == key[1]))
        sel = sel[np.argsort(t0[sel], kind="stable")]
        groups, cur, cur_end = [], [sel[0]], t2[sel[0]]
        for i in sel[1:]:
            if t0[i] > cur_end:  # every block of the previous launch had ended: a new launch
                groups.append(cur)
                cur, cur_end = [i], t2[i]
            else:
                cur.append(i)
                cur_end = max(cur_end, t2[i])
        groups.append(cur)
        name = KERNELS.get(key[0], "kernel%d" % key[0])
        if key[0] == 1:
            name = tags.get(key[1] & 0xFFFFFFFF, "gemm_%x" % key[1])
        for g in groups:
            g = np.array(g)
            waited = tw[g][tw[g] > 0]
            marks = [int(np.median(rec[g, 4 + j].astype(np.int64)[rec[g, 4 + j] > 0]) - origin) if (rec[g, 4 + j] > 0).any() else None for j in range(3)]
            out.append({"kernel": name, "blocks": int(len(g)), "marks": marks, "first_start": int(t0[g].min() - origin), "last_start": int(t0[g].max() - origin),
                        "waited": int(np.median(waited) - origin) if len(waited) else None, "first_end": int(t2[g].min() - origin),
                        "end": int(t2[g].max() - origin)})
    out.sort(key=lambda d: d["end"])
    prev = 0
    for d in out:
        d["exposed"] = d["end"] - prev
        prev = d["end"]
    return out


def per_kernel(launch_list):
    """Sum of the exposed time and launch count per kernel name, largest first: {name: (ns, launches)}."""
    acc = {}
    for d in launch_list:
        a = acc.setdefault(d["kernel"], [0, 0])
        a[0] += d["exposed"]
        a[1] += 1
    return dict(sorted(((k, (v[0], v[1])) for k, v in acc.items()), key=lambda kv: -kv[1][0]))
