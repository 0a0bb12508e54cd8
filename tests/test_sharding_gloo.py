"""Multi-rank host logic on CPU: two gloo ranks each take their shard from the C ABI's planners (ascb200_shard_nslab,
ascb200_shard_groups_lpt: host functions, no device) and compute it with the CPU oracle standing in for the GPU kernel; the
union must equal the unsharded result, and the timing reduction is a max over ranks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    for p in (os.path.join(ROOT, "asc-devkit_clone_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    import ascb200 as ab
    import oracle as orc
    import sharding
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # --- N-slab sharded A8W8 GEMM ---
        M, K, N = 48, 64, 160
        rng = np.random.default_rng(1)
        a = rng.integers(-127, 128, (M, K)).astype(np.int8)
        b = rng.integers(-127, 128, (N, K)).astype(np.int8)
        tok = rng.uniform(1e-3, 1e-2, M).astype(np.float32)
        ch = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
        lo, hi = ab.shard_nslab(N, rank, world, 16)
        slab = orc.dequant_tok_ch(orc.gemm_i8(a, b[lo:hi], trans_b=True), tok, ch[lo:hi], orc.BF16)
        parts = [torch.zeros((M, hi - lo), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(slab.astype(np.int32)))   # the optional gather of output slabs
        full = torch.cat(parts, dim=1).numpy().astype(np.uint16)
        ref = orc.dequant_tok_ch(orc.gemm_i8(a, b, trans_b=True), tok, ch, orc.BF16)
        ok_gemm = bool((full == ref).all())
        # --- grouped matmul sharded by group ---
        G, Kg, Ng = 8, 32, 48
        counts = sharding.dirichlet_counts(G, 200, 5)
        mine = np.flatnonzero(ab.shard_groups_lpt(counts, world) == rank).tolist()
        starts = sharding.group_rows(counts)
        x = rng.integers(-127, 128, (200, Kg)).astype(np.int8)
        w = rng.integers(-127, 128, (G, Ng, Kg)).astype(np.int8)
        tk = rng.uniform(1e-3, 1e-2, 200).astype(np.float32)
        cs = rng.uniform(1e-3, 1e-2, (G, Ng)).astype(np.float32)
        rows = np.concatenate([np.arange(starts[g], starts[g] + counts[g]) for g in mine]) if mine else np.zeros(0, np.int64)
        local = orc.grouped_i8(np.ascontiguousarray(x[rows]), np.ascontiguousarray(w[mine]), counts[mine], tk[rows], cs[mine], orc.BF16)
        ref_g = orc.grouped_i8(x, w, counts, tk, cs, orc.BF16)
        ok_group = bool((local == ref_g[rows]).all())
        covered = torch.zeros(200, dtype=torch.int32)
        covered[torch.from_numpy(rows)] = 1
        dist.all_reduce(covered)                      # every row owned exactly once across ranks
        ok_cover = bool((covered == 1).all())
        # --- timing reduction: max over ranks ---
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ret[rank] = (ok_gemm, ok_group, ok_cover, float(t.item()))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, 29541 + os.getpid() % 500, ret), nprocs=world, join=True)
    for rank in range(world):
        ok_gemm, ok_group, ok_cover, tmax = ret[rank]
        assert ok_gemm and ok_group and ok_cover
        assert tmax == float(world)


def test_planner_properties():
    sys.path.insert(0, os.path.join(ROOT, "asc-devkit_clone_b200"))
    import sharding
    for n, world in ((11008, 1), (11008, 2), (11008, 4), (11008, 8), (8192, 8), (100, 3)):
        edges = [sharding.n_slab(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
    assert sharding.n_slab(11008, 3, 8) == (4128, 5504)   # 1376 columns per rank
    counts = sharding.dirichlet_counts(64, 32768, 0xA5C00003)
    assert counts.sum() == 32768 and (counts >= 0).all() and len(counts) == 64
    for parts in (1, 2, 4, 8):
        owner = sharding.lpt_partition(counts, parts)
        assert sorted(g for o in owner for g in o) == list(range(64))
        loads = [int(counts[o].sum()) for o in owner]
        assert max(loads) - min(loads) <= counts.max()
    with pytest.raises(ValueError):
        sharding.n_slab(10, 2, 2)
