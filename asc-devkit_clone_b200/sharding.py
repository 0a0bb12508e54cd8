"""Host-side planner for running the hot path on several GPUs of one box without communication.

Large GEMMs shard by N-slab (rank r owns the B rows / per-channel parameters / C columns
[r*N/g, (r+1)*N/g); A and the per-token scales are replicated), the grouped matmul by expert group.
In the reference the corresponding split is the multi-core block split of the tiling
(examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul/matmul.asc:114-141) and the round-robin
of group blocks over cores (quant_group_matmul_custom.asc:254-286).
"""
import numpy as np


def n_slab(n, rank, world, align=16):
    """Column range [lo, hi) of `rank`; slabs are equal when world divides n/align, else the last ranks get less."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world")
    per = -(-n // world)
    per = -(-per // align) * align
    lo = min(n, rank * per)
    return lo, min(n, lo + per)


def dirichlet_counts(groups, total, seed):
    """Deterministic Dirichlet(1) split of `total` rows over `groups`: normalised Exp(1) draws, floored, the
    remainder handed out by largest fraction.  Groups may be empty."""
    e = np.random.default_rng(seed).exponential(1.0, groups)
    w = e / e.sum() * total
    c = np.floor(w).astype(np.int64)
    rem = total - int(c.sum())
    c[np.argsort(-(w - c), kind="stable")[:rem]] += 1
    return c


def lpt_partition(counts, parts):
    """Greedy longest-processing-time assignment of groups to ranks by row count; returns sorted group ids per rank."""
    counts = np.asarray(counts)
    load = [0] * parts
    owner = [[] for _ in range(parts)]
    for g in np.argsort(-counts, kind="stable"):
        r = int(np.argmin(load))
        owner[r].append(int(g))
        load[r] += int(counts[g])
    return [sorted(o) for o in owner]


def group_rows(counts):
    """Start row of every group in the packed activation matrix."""
    counts = np.maximum(np.asarray(counts, np.int64), 0)
    return np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int64)
