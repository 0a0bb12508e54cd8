"""Benchmark of the ascb200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload a8w8|grouped|mxfp4|softmax_quant|fp16] [--impl reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the A8W8 dense GEMM of the baseline (A[4096,4096] int8, B[11008,4096] int8 K-major,
int32 accumulation, fused bf16(acc * ch_scale[n] * tok_scale[m]) epilogue), sharded by N-slab
across ranks with no communication; `value` is the whole-job rate (all ranks' operations divided
by the slowest rank's device time, CUDA events on the launching stream).

Rank 0 prints ONE JSON line.  Under "others" it carries the same measurement for the other baseline
configurations: at N=1 grouped A8W8, MXFP4, SoftMax+AscendQuant (and its 64 x rows companion), the fp16
Matmul and the reference's published fp16 8192^3 shape; at N>1 the other two sharded configurations
(grouped A8W8 by expert group, MXFP4 by N-slab).  `--all` adds the kernels that lie outside the baseline
configurations.  The last key, "summary", repeats workload / value / fraction of every configuration in
a few characters each.

Timing: the K steps are captured into one CUDA graph; the graph is replayed R >= 10 times (about 0.4 s
in total), every replay bracketed by a barrier and a synchronisation on both sides and timed with CUDA
events on the launching stream, maximum over ranks.  `ms_per_step` and `value` come from the median
replay, `ms_per_step_range` gives the fastest and slowest one.  SM clocks are sampled only while these
replays run.  Every rank rotates through enough buffer sets that their total size is at least twice the
L2 capacity, so no step finds its operands in cache.  Because the timed region is a long back-to-back
sequence under the board's power cap, `roofline.peak` of the tensor-bound kernels is the SUSTAINED
measured cuBLAS figure (scaled by the hardware's rate ratio for int8 / fp4); `roofline.frac_of_burst_peak`
gives the same rate against the burst figure, and `roofline.best_replay` the fastest replay (normally the
first one, before the cap pulls the clock down) against the burst figure, which is itself a best-of-ten.

`--impl reference` times the CPU restatement of the reference arithmetic (oracle/, OpenMP, all host
threads) on a bounded row sample of the same workload; the reference's own CPU-debug executable
needs the closed CANN CPU twin and cannot be built.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "asc-devkit_clone_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

L2_BYTES = 126 * 1024 * 1024


def cold_sets(bytes_per_set):
    """Number of rotating buffer sets whose total size is at least twice the L2 capacity (at least two)."""
    return max(2, -(-2 * L2_BYTES // max(int(bytes_per_set), 1)))


def plan_nslab(n, rank, world):
    """Column range of this rank's N-slab from the C ABI's planner (a host function: the CPU arm calls it too)."""
    import ascb200
    lo, hi = ascb200.shard_nslab(n, rank, world, 16)
    assert (hi - lo) * world == n, "the baseline shapes split into equal slabs"
    return lo, hi


def cache_label(sets, bytes_per_set):
    total = sets * bytes_per_set
    rel = ">= 2 x L2" if total >= 2 * L2_BYTES else ("> L2" if total > L2_BYTES else "fits L2: warm")
    return f"{sets} rotating buffer sets ({total // 2**20} MiB {rel} of {L2_BYTES // 2**20} MiB)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks: NVML samples taken by a thread while the timed region runs
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.002)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
from sharding import dirichlet_counts  # noqa: E402  (the seeded group sizes of the baseline; the shard plans come from the C ABI)


class Workload:
    """Holds device buffers for `sets` rotating input/output sets and launches one step."""
    name = metric = unit = dtype = ""
    unit_scale = 1e12            # value = units / seconds / unit_scale (1e12: TOPS / TFLOPS, 1e9: GB/s)
    bound = "tensor"
    scaling = "strong"
    kernels_per_step = 1
    published = None  # (value, note) of a like-for-like number the reference publishes (other hardware)
    # dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, per launch, from one ncu capture of the whole
    # configuration on 1 GPU; None where no capture exists
    traffic_1gpu = None

    def units_total(self):       # algorithmic operations (or bytes) of the whole job per step
        raise NotImplementedError

    def units_rank(self):        # of this rank per step (roofline of the dominant kernel)
        raise NotImplementedError

    def step(self, i):
        raise NotImplementedError

    def e2e_step(self, i):
        raise NotImplementedError

    def peak(self, peaks):
        raise NotImplementedError


class A8W8(Workload):
    name = "a8w8_gemm_4096x4096x11008_dequant_bf16"
    metric, unit, dtype = "quant-GEMM throughput (int8, fused per-token x per-channel dequant)", "TOPS", "s8"
    M, K, N = 4096, 4096, 11008
    traffic_1gpu = 62.05e6 + 49.67e6   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of gemm_tc_pair_kernel<int8>

    def __init__(self, ab, rank, world, sets):
        self.ab, self.rank, self.world = ab, rank, world
        self.n_lo, n_hi = plan_nslab(self.N, rank, world)
        self.n_loc = n_hi - self.n_lo
        rng = np.random.default_rng(0xA5C00002)
        self.a_h = rng.integers(-127, 128, (self.M, self.K)).astype(np.int8)
        self.tok_h = rng.uniform(1e-3, 1e-2, self.M).astype(np.float32)
        ch = rng.uniform(1e-3, 1e-2, self.N).astype(np.float32)
        rng_b = np.random.default_rng(0xA5C00002 + 1000 + rank)   # each rank draws its own B slab
        self.b_h = rng_b.integers(-127, 128, (self.n_loc, self.K)).astype(np.int8)
        self.ch_h = ch[self.n_lo:self.n_lo + self.n_loc].copy()
        self.sets = sets = cold_sets(self.bytes_rank())
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.tok, self.ch = ab.to_dev(self.tok_h), ab.to_dev(self.ch_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}",
                       "cache": cache_label(sets, self.bytes_rank())}
        self.pin = None

    def units_total(self):
        return 2.0 * self.M * self.K * self.N

    def units_rank(self):
        return 2.0 * self.M * self.K * self.n_loc

    def bytes_rank(self):
        return self.M * self.K + self.n_loc * self.K + 2 * self.M * self.n_loc + 4 * (self.M + self.n_loc)

    def peak(self, peaks):
        return 2.0 * peaks["bf16_tflops"], "TOPS", "2 x measured bf16 cuBLAS burst (int8 runs at twice the bf16 rate)"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_S8, self.M, self.n_loc, self.K, self.a[s], self.b[s], self.c[s], ab.BF16,
                         epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, tok=self.tok, ch=self.ch, stream=stream))

    def e2e_bytes(self):
        return self.a_h.nbytes + self.b_h.nbytes + self.tok_h.nbytes + self.ch_h.nbytes, self.M * self.n_loc * 2

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.a_h, self.b_h, self.tok_h, self.ch_h], self.M * self.n_loc * 2)

    def e2e_step(self, i, stream):
        ab, s = self.ab, i % self.sets
        self.pin.h2d([self.a[s], self.b[s], self.tok, self.ch], stream)
        self.step(i, stream)
        self.pin.d2h(self.c[s], stream)

    def cpu_sample(self, orc, rows):
        t0 = time.perf_counter()
        acc = orc.gemm_i8(self.a_h[:rows], self.b_h, trans_b=True)
        orc.dequant_tok_ch(acc, self.tok_h[:rows], self.ch_h, orc.BF16)
        return time.perf_counter() - t0, 2.0 * rows * self.K * self.n_loc, f"{rows} of {self.M} rows of A x all {self.n_loc} columns"

    def verify(self, orc):
        """Spot check of set 0 against the oracle: first 32 rows."""
        got = self.c[0].download()[:32]
        ref = orc.dequant_tok_ch(orc.gemm_i8(self.a_h[:32], self.b_h, trans_b=True), self.tok_h[:32], self.ch_h, orc.BF16)
        return bool((got == ref).all())


class Grouped(Workload):
    name = "grouped_a8w8_64groups_M32768_K7168_N2048"
    metric, unit, dtype = "grouped quant-GEMM throughput (int8, fused dequant)", "TOPS", "s8"
    G, MTOT, K, N = 64, 32768, 7168, 2048
    OUT, ACT = "BF16", 0
    traffic_1gpu = 1.2680e9 + 0.1266e9   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of gemm_tc_pair_kernel<int8>, grouped

    def counts(self):
        return dirichlet_counts(self.G, self.MTOT, 0xA5C00003)

    @staticmethod
    def plan_owner(counts, world):
        import ascb200
        return ascb200.shard_groups_lpt(counts, world)   # ascb200_shard_groups_lpt: a host function, also used by the CPU arm

    def __init__(self, ab, rank, world, sets):
        self.ab, self.rank, self.world = ab, rank, world
        counts = self.counts()
        mine = np.flatnonzero(self.plan_owner(counts, world) == rank)
        self.counts_h = counts[mine].astype(np.int64)
        self.m_loc = int(self.counts_h.sum())
        self.g_loc = len(mine)
        rng = np.random.default_rng(0xA5C00003 + 1000 + rank)
        self.x_h = rng.integers(-127, 128, (max(self.m_loc, 1), self.K)).astype(np.int8)
        self.w_h = rng.integers(-127, 128, (self.g_loc, self.N, self.K), dtype=np.int8)
        self.tok_h = rng.uniform(1e-3, 1e-2, max(self.m_loc, 1)).astype(np.float32)
        self.ch_h = rng.uniform(1e-3, 1e-2, (self.g_loc, self.N)).astype(np.float32)
        # every pass streams this rank's weights, rows and outputs once: all of them rotate
        per_set = self.x_h.nbytes + self.w_h.nbytes + 2 * max(self.m_loc, 1) * self.N
        self.sets = sets = cold_sets(per_set)
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.w = [ab.to_dev(self.w_h) for _ in range(sets)]
        self.c = [ab.empty((max(self.m_loc, 1), self.N), np.uint16) for _ in range(sets)]
        self.tok, self.ch, self.counts_d = ab.to_dev(self.tok_h), ab.to_dev(self.ch_h), ab.to_dev(self.counts_h)
        self.config = {"workload": self.name, "groups": self.G, "rows": self.MTOT, "K": self.K, "N": self.N,
                       "shard": f"groups x{world} (greedy by rows)", "rows_this_rank": self.m_loc, "cache": cache_label(sets, per_set)}

    def units_total(self):
        return 2.0 * self.MTOT * self.K * self.N

    def units_rank(self):
        return 2.0 * self.m_loc * self.K * self.N

    def peak(self, peaks):
        return 2.0 * peaks["bf16_tflops"], "TOPS", "2 x measured bf16 cuBLAS burst"

    def extra_roofline(self, ms_per_step, peaks):
        """The configuration's own bound: every group reads its K x N weights from HBM once whatever its row count, so a group
        of fewer than about 210 rows (2 x rows op/B below the ridge) is bound by that read, the others by the tensor
        cores: sum over this rank's groups of max(compute time at the sustained int8 rate, bytes / measured copy bandwidth)."""
        c = self.counts_h.astype(np.float64)
        tensor = 2.0 * (peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]) * 1e12
        comp = 2.0 * c * self.K * self.N / tensor
        mem = ((c > 0) * float(self.K * self.N) + c * (self.K + 2 * self.N)) / (peaks["hbm_gbs"] * 1e9)
        bound_ms = float(np.maximum(comp, mem).sum() * 1e3)
        return {"per_group_bound_ms": round(bound_ms, 4), "frac_of_per_group_bound": round(bound_ms / ms_per_step, 4),
                "groups_bound_by_weight_read": int((mem > comp).sum())}

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_S8, self.m_loc, self.N, self.K, self.x[s], self.w[s], self.c[s], getattr(ab, self.OUT),
                         epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, tok=self.tok, ch=self.ch, group_counts=self.counts_d,
                         groups=self.g_loc, act=self.ACT, stream=stream))

    def e2e_bytes(self):
        return self.x_h.nbytes + self.w_h.nbytes + self.tok_h.nbytes + self.ch_h.nbytes + self.counts_h.nbytes, self.m_loc * self.N * 2

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.x_h, self.w_h, self.tok_h, self.ch_h, self.counts_h], self.m_loc * self.N * 2)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.x[s], self.w[s], self.tok, self.ch, self.counts_d], stream)
        self.step(i, stream)
        self.pin.d2h(self.c[s], stream)

    def cpu_sample(self, orc, rows):
        # the first `rows` rows of every non-empty group
        take = np.minimum(self.counts_h, rows)
        starts = np.concatenate([[0], np.cumsum(self.counts_h)[:-1]])
        idx = np.concatenate([np.arange(s, s + t) for s, t in zip(starts, take)])
        x, tok = np.ascontiguousarray(self.x_h[idx]), self.tok_h[idx]
        t0 = time.perf_counter()
        orc.grouped_i8(x, self.w_h, take, tok, self.ch_h, getattr(orc, self.OUT), trans_b=True, act=self.ACT)
        return time.perf_counter() - t0, 2.0 * int(take.sum()) * self.K * self.N, f"first {rows} rows of each of {self.g_loc} groups"

    def verify(self, orc):
        got = self.c[0].download()
        take = np.minimum(self.counts_h, 2)
        starts = np.concatenate([[0], np.cumsum(self.counts_h)[:-1]])
        idx = np.concatenate([np.arange(s, s + t) for s, t in zip(starts, take)])
        ref = orc.grouped_i8(np.ascontiguousarray(self.x_h[idx]), self.w_h, take, self.tok_h[idx], self.ch_h, getattr(orc, self.OUT), trans_b=True,
                             act=self.ACT)
        if self.ACT:  # the activation uses fast exponentials: the example's own acceptance rule (rtol = atol = 1e-3)
            return bool(np.isclose(orc.f16_bits_to_f32(got[idx]), orc.f16_bits_to_f32(ref), rtol=1e-3, atol=1e-3).mean() > 0.9999)
        return bool((got[idx] == ref).all())


class MXFP4(Workload):
    name = "mxfp4_gemm_8192x8192x8192_requant_int8_bf16"
    metric, unit, dtype = "quant-GEMM throughput (MXFP4 e2m1 x ue8m0, int8 requant + bf16 out)", "TFLOPS", "fp4_e2m1"
    M = K = N = 8192
    kernels_per_step = 2  # re-tiling of A's scales + the GEMM (the weights' scales are prepacked once, outside the timed region)
    traffic_1gpu = 87.1e6 + 167.9e6    # ncu: dram__bytes_read.sum + dram__bytes_write.sum of gemm_tc_pair_kernel<mxf4>
    published = (1614.0, "Ascend 950PR basic-API MXFP4 8192^3, bf16 out; the reference's published figure")

    def __init__(self, ab, rank, world, sets):
        from gpu_util import mx_quantize, quant_params
        self.ab, self.rank, self.world = ab, rank, world
        self.n_lo, n_hi = plan_nslab(self.N, rank, world)
        self.n_loc = n_hi - self.n_lo
        rng = np.random.default_rng(0xA5C00004)
        self.a_h, self.sa_h = mx_quantize(rng.standard_normal((self.M, self.K), dtype=np.float32))
        rng_b = np.random.default_rng(0xA5C00004 + 1000 + rank)
        self.b_h, self.sb_h = mx_quantize(rng_b.standard_normal((self.n_loc, self.K), dtype=np.float32))
        # accumulators ~ N(0, K * E[a^2] E[b^2]); quantised unit normals keep E[x^2] ~ 1 -> sigma ~ sqrt(K)
        scales = (rng.uniform(0.5, 2.0, self.N) * 40.0 / np.sqrt(self.K)).astype(np.float32)
        self.q_h = quant_params(scales[self.n_lo:self.n_lo + self.n_loc])
        per_set = self.a_h.nbytes + self.b_h.nbytes + 3 * self.M * self.n_loc
        self.sets = sets = cold_sets(per_set)
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.sa, self.sb, self.q = ab.to_dev(self.sa_h), ab.to_dev(self.sb_h), ab.to_dev(self.q_h)
        # the weights' scale factors are static: re-tiled once here; a step re-tiles only A's
        self.sb_packed = ab.mx_scale_prepack(self.sb, self.n_loc, self.K) if self.sb is not None else None
        self.c = [ab.empty((self.M, self.n_loc), np.int8) for _ in range(sets)]
        self.c2 = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}",
                       "cache": cache_label(sets, per_set), "scales": "B prepacked once (static weights), A re-tiled every step"}

    def units_total(self):
        return 2.0 * self.M * self.K * self.N

    def units_rank(self):
        return 2.0 * self.M * self.K * self.n_loc

    def peak(self, peaks):
        return 4.0 * peaks["bf16_tflops"], "TFLOPS", "4 x measured bf16 cuBLAS burst (fp4 runs at four times the bf16 rate)"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_MXFP4, self.M, self.n_loc, self.K, self.a[s], self.b[s], self.c[s], ab.S8,
                         epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, scale_a=self.sa, scale_b=self.sb_packed, quant=self.q,
                         c2=self.c2[s], c2_dtype=ab.BF16, scale_flags=ab.SCALE_B_PREPACKED, stream=stream))

    def e2e_bytes(self):
        return (self.a_h.nbytes + self.b_h.nbytes + self.sa_h.nbytes + self.sb_h.nbytes + self.q_h.nbytes,
                self.M * self.n_loc * 3)

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.a_h, self.b_h, self.sa_h, self.sb_h, self.q_h], self.M * self.n_loc * 3)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.a[s], self.b[s], self.sa, self.sb, self.q], stream)
        self.step(i, stream)
        self.pin.d2h(self.c[s], stream, 0)
        self.pin.d2h(self.c2[s], stream, self.M * self.n_loc)

    def cpu_sample(self, orc, rows):
        t0 = time.perf_counter()
        acc = orc.gemm_mxf4(self.a_h[:rows], self.sa_h[:rows], self.b_h, self.sb_h, base_k=256)
        orc.fixpipe_qf322b8(acc, self.q_h)
        orc.cast_f32(acc, orc.BF16)
        return time.perf_counter() - t0, 2.0 * rows * self.K * self.n_loc, f"{rows} of {self.M} rows of A x all {self.n_loc} columns"

    def verify(self, orc):
        """Stage-wise and bit exact: the fp32 accumulators of the same GEMM (same tiles, fp32 output) agree with the oracle within
        the GEMM tolerance, and both timed outputs equal the oracle's output stage applied to those accumulators."""
        ab = self.ab
        d_acc = ab.empty((self.M, self.n_loc), np.float32)
        ab.check(ab.gemm(ab.KIND_MXFP4, self.M, self.n_loc, self.K, self.a[0], self.b[0], d_acc, ab.F32, trans_b=True, scale_a=self.sa,
                         scale_b=self.sb_packed, scale_flags=ab.SCALE_B_PREPACKED))
        ab.sync()
        acc_gpu = d_acc.download()[:16]
        d_acc.free()
        acc = orc.gemm_mxf4(self.a_h[:16], self.sa_h[:16], self.b_h, self.sb_h, base_k=256)
        ok_acc = np.allclose(acc_gpu, acc, rtol=1e-2, atol=1e-3)
        ok_q = (self.c[0].download()[:16] == orc.fixpipe_qf322b8(acc_gpu, self.q_h)).all()
        ok_bf = (self.c2[0].download()[:16] == orc.cast_f32(acc_gpu, orc.BF16)).all()
        return bool(ok_acc and ok_q and ok_bf)


class SoftmaxQuant(Workload):
    name = "softmax_ascendquant_4096x2048_fp16_int8"
    metric, unit, dtype = "SoftMax + AscendQuant row-op bandwidth (fused single pass)", "GB/s", "f16"
    bound = "hbm"
    unit_scale = 1e9
    scaling = "weak"  # rows are independent; every rank runs its own replica of the configuration
    M, K = 4096, 2048
    ROW_FACTOR = 1
    traffic_1gpu = 16.8e6               # ncu: dram bytes of softmax_rows_kernel (the outputs are still in L2 when the kernel ends)

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.M = self.M * self.ROW_FACTOR
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00001 + rank)
        self.x_h = np.tile(f16_bits(rng.standard_normal((4096, self.K), dtype=np.float32) * 3.0), (self.ROW_FACTOR, 1))
        self.sc_h = f16_bits((127.0 / rng.uniform(0.5, 2.0, self.K)).astype(np.float32))
        self.sets = sets = cold_sets(self.per_step_bytes())   # 42 MB per set at the baseline shape: 7 sets
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.y = [ab.empty((self.M, self.K), np.uint16) for _ in range(sets)]
        self.q = [ab.empty((self.M, self.K), np.int8) for _ in range(sets)]
        self.sm, self.mx = ab.empty((self.M,), np.float32), ab.empty((self.M,), np.float32)
        self.sc = ab.to_dev(self.sc_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "shard": f"replica per rank x{world}",
                       "cache": cache_label(sets, self.per_step_bytes())}

    def per_step_bytes(self):
        return self.M * self.K * (2 + 2 + 1) + 8 * self.M + 2 * self.K  # X in, Y + Q + sum + max out, scale in

    def units_total(self):
        return float(self.per_step_bytes()) * self.world

    def units_rank(self):
        return float(self.per_step_bytes())

    def peak(self, peaks):
        return peaks["hbm_gbs"], "GB/s", "measured STREAM-style copy"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.softmax_quant(self.x[s], self.y[s], self.sm, self.mx, self.q[s], self.sc, None, 0.0, self.M, self.K, stream=stream))

    def e2e_bytes(self):
        return self.x_h.nbytes + self.sc_h.nbytes, self.M * self.K * 3 + 8 * self.M

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.x_h, self.sc_h], self.M * self.K * 3 + 8 * self.M)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.x[s], self.sc], stream)
        self.step(i, stream)
        self.pin.d2h(self.y[s], stream, 0)
        self.pin.d2h(self.q[s], stream, self.M * self.K * 2)
        self.pin.d2h(self.sm, stream, self.M * self.K * 3)
        self.pin.d2h(self.mx, stream, self.M * self.K * 3 + 4 * self.M)

    def cpu_sample(self, orc, rows):
        rows = min(rows * 16, self.M)
        t0 = time.perf_counter()
        y, _, _ = orc.softmax(self.x_h[:rows], orc.F16)
        orc.quant_per_channel(y, orc.F16, self.sc_h, 0.0)
        # the CPU path is the unfused pair, counted with the same algorithmic bytes as the fused kernel
        return time.perf_counter() - t0, rows * self.K * 5.0, f"{rows} of {self.M} rows"

    def verify(self, orc):
        y, q = self.y[0].download()[:64], self.q[0].download()[:64]
        ry, _, _ = orc.softmax(self.x_h[:64], orc.F16)
        yf, rf = orc.f16_bits_to_f32(y), orc.f16_bits_to_f32(ry)
        return bool((np.abs(yf - rf) <= 1e-3 * np.abs(rf) + 2.0 ** -24).all() and (q == orc.quant_per_channel(y, orc.F16, self.sc_h, 0.0)).all())


class SoftmaxQuantLarge(SoftmaxQuant):
    """Companion of the baseline row-op configuration with 64 x the rows (2.7 GB per pass): the 42 MB
    baseline shape lasts only a few microseconds, so launch ramp-up and tail dominate its bandwidth figure."""
    name = "softmax_ascendquant_262144x2048_fp16_int8"
    ROW_FACTOR = 64
    traffic_1gpu = 1.0738e9 + 1.5580e9  # ncu: dram__bytes_read.sum + dram__bytes_write.sum of softmax_rows_kernel


class FP16(Workload):
    name = "matmul_fp16_512x512x1024_bias_fp32"
    metric, unit, dtype = "adv_api Matmul fp16 -> fp32 with bias", "TFLOPS", "f16"
    scaling = "weak"  # too small to shard: replicas only
    M, K, N = 512, 512, 1024

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00000)
        self.a_h = f16_bits(rng.uniform(-1, 1, (self.M, self.K)).astype(np.float32))
        self.b_h = f16_bits(rng.uniform(-1, 1, (self.K, self.N)).astype(np.float32))
        self.bias_h = rng.uniform(-1, 1, self.N).astype(np.float32)
        self.sets = sets = cold_sets(self.a_h.nbytes + self.b_h.nbytes + 4 * self.M * self.N)  # 3.5 MiB per set: 72 sets
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.N), np.float32) for _ in range(sets)]
        self.bias = ab.to_dev(self.bias_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"replica per rank x{world}",
                       "cache": cache_label(sets, self.a_h.nbytes + self.b_h.nbytes + 4 * self.M * self.N),
                       "note": "0.54 GFLOP: launch-latency bound"}

    def units_total(self):
        return 2.0 * self.M * self.K * self.N * self.world

    def units_rank(self):
        return 2.0 * self.M * self.K * self.N

    def peak(self, peaks):
        return peaks["bf16_tflops"], "TFLOPS", "measured bf16 cuBLAS burst"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_F16, self.M, self.N, self.K, self.a[s], self.b[s], self.c[s], ab.F32, bias=self.bias, stream=stream))

    def e2e_bytes(self):
        return self.a_h.nbytes + self.b_h.nbytes + self.bias_h.nbytes, self.M * self.N * 4

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.a_h, self.b_h, self.bias_h], self.M * self.N * 4)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.a[s], self.b[s], self.bias], stream)
        self.step(i, stream)
        self.pin.d2h(self.c[s], stream)

    def cpu_sample(self, orc, rows):
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 2.0:
            orc.gemm_f16(self.a_h, self.b_h, self.bias_h, base_k=64)
            reps += 1
        return time.perf_counter() - t0, reps * 2.0 * self.M * self.K * self.N, f"whole problem x{reps}"

    def verify(self, orc):
        ref = orc.gemm_f16(self.a_h, self.b_h, self.bias_h, base_k=64)
        return bool(np.allclose(self.c[0].download(), ref, rtol=1e-2, atol=1e-3))


class FP16Large(Workload):
    """The reference's own published Matmul shape (fp16 8192^3, B stored transposed, fp16 out):
    examples/01_simd_cpp_api/05_best_practices/01_matrix_compute/matmul_high_performance (scripts/gen_data.py:20-28)."""
    name = "matmul_fp16_8192x8192x8192_fp16_out"
    metric, unit, dtype = "adv_api Matmul fp16 -> fp16, 8192^3 (the reference's published shape)", "TFLOPS", "f16"
    M = K = N = 8192
    published = (427.0, "Ascend 950PR basic-API fp16 8192^3, 2572 us (the reference's published figure); Atlas A2 adv_api: 269")
    traffic_1gpu = 1.0571e9 + 0.1269e9   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of gemm_tc_pair_kernel<f16>, banded tile order

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        self.n_lo, n_hi = plan_nslab(self.N, rank, world)
        self.n_loc = n_hi - self.n_lo
        rng = np.random.default_rng(0xA5C00005)
        self.a_h = f16_bits(rng.uniform(1, 10, (self.M, self.K)).astype(np.float32))      # the example draws U[1,10)
        self.b_h = f16_bits(np.random.default_rng(0xA5C00005 + 1000 + rank).uniform(1, 10, (self.n_loc, self.K)).astype(np.float32))
        per_set = self.a_h.nbytes + self.b_h.nbytes + 2 * self.M * self.n_loc
        self.sets = sets = cold_sets(per_set)
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}", "cache": cache_label(sets, per_set)}

    def units_total(self):
        return 2.0 * self.M * self.K * self.N

    def units_rank(self):
        return 2.0 * self.M * self.K * self.n_loc

    def peak(self, peaks):
        return peaks["bf16_tflops"], "TFLOPS", "measured bf16 cuBLAS burst"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_F16, self.M, self.n_loc, self.K, self.a[s], self.b[s], self.c[s], ab.F16, trans_b=True, stream=stream))

    def e2e_bytes(self):
        return self.a_h.nbytes + self.b_h.nbytes, self.M * self.n_loc * 2

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.a_h, self.b_h], self.M * self.n_loc * 2)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.a[s], self.b[s]], stream)
        self.step(i, stream)
        self.pin.d2h(self.c[s], stream)

    def cpu_sample(self, orc, rows):
        t0 = time.perf_counter()
        acc = orc.gemm_f16(self.a_h[:rows], self.b_h, trans_b=True, base_k=64)
        orc.cast_f32(acc, orc.F16)
        return time.perf_counter() - t0, 2.0 * rows * self.K * self.n_loc, f"{rows} of {self.M} rows of A x all {self.n_loc} columns"

    def verify(self, orc):
        ref = orc.f16_bits_to_f32(orc.cast_f32(orc.gemm_f16(self.a_h[:8], self.b_h, trans_b=True, base_k=64), orc.F16))
        return bool(np.allclose(orc.f16_bits_to_f32(self.c[0].download()[:8]), ref, rtol=1e-2, atol=1e-3))


class GroupedRefShape(Grouped):
    """The grouped example's own shape and epilogue: 8 groups x 1024 rows, K=1024, N=8192, FasterGelu, fp16 out
    (quant_group_matmul_high_performance/scripts/gen_data.py:21-25); published 204.1 us on Ascend 950PR, 299.3 us on Atlas A2."""
    name = "grouped_a8w8_8groups_M8192_K1024_N8192_gelu_fp16"
    metric = "grouped quant-GEMM throughput (the reference example's shape, FasterGelu, fp16 out)"
    G, MTOT, K, N = 8, 8192, 1024, 8192
    traffic_1gpu = None
    published = (2.0 * 8192 * 1024 * 8192 / 204.129e-6 / 1e12, "Ascend 950PR, 204.129 us (the reference's published figure)")
    OUT, ACT = "F16", 1

    def counts(self):
        return np.full(self.G, self.MTOT // self.G, np.int64)


class RowOp(Workload):
    """Common part of the HBM-bound layout / quantisation kernels of the widened path: replicas per rank, bytes per second."""
    unit, bound, unit_scale, scaling = "GB/s", "hbm", 1e9, "weak"

    def units_total(self):
        return float(self.per_step_bytes()) * self.world

    def units_rank(self):
        return float(self.per_step_bytes())

    def peak(self, peaks):
        return peaks["hbm_gbs"], "GB/s", "measured STREAM-style copy"

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, self.h2d_arrays(), sum(n for _, n in self.d2h_buffers(0)))

    def e2e_bytes(self):
        return sum(a.nbytes for a in self.h2d_arrays()), sum(n for _, n in self.d2h_buffers(0))

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d(self.h2d_targets(s), stream)
        self.step(i, stream)
        off = 0
        for buf, n in self.d2h_buffers(s):
            self.pin.d2h(buf, stream, off)
            off += n


class QuantPerGroupFp4(RowOp):
    name = "ascendquant_per_group32_fp16_to_fp4_32768x8192"
    metric, dtype = "AscendQuant PER_GROUP (fp16 -> packed fp4 e2m1, fp32 scale per 32 columns) bandwidth", "f16"
    M, N, G = 32768, 8192, 32
    traffic_1gpu = 570.5e6 + 120.6e6   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of the kernel

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00010 + rank)
        self.x_h = np.tile(f16_bits(rng.standard_normal((4096, self.N), dtype=np.float32)), (self.M // 4096, 1))
        self.s_h = np.tile(rng.uniform(0.75, 1.5, (4096, self.N // self.G)).astype(np.float32), (self.M // 4096, 1))
        self.sets = sets = 2   # 704 MB per set
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.sc = [ab.to_dev(self.s_h) for _ in range(sets)]
        self.q = [ab.empty((self.M, self.N // 2), np.uint8) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "N": self.N, "group": self.G, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

    def per_step_bytes(self):
        return self.M * self.N * 2 + self.M * self.N // 2 + self.M * (self.N // self.G) * 4

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.quant_policy(self.x[s], self.q[s], self.M, self.N, ab.F16, ab.F32, ab.FP4, ab.QUANT_PER_GROUP, self.sc[s], k_dim=1,
                                 group_size=self.G, stream=stream))

    def h2d_arrays(self):
        return [self.x_h, self.s_h]

    def h2d_targets(self, s):
        return [self.x[s], self.sc[s]]

    def d2h_buffers(self, s):
        return [(self.q[s], self.M * self.N // 2)]

    def cpu_sample(self, orc, rows):
        rows = min(rows * 8, self.M)
        t0 = time.perf_counter()
        orc.quant_policy(self.x_h[:rows], self.s_h[:rows], orc.F16, orc.F32, orc.FP4_E2M1, 3, k_dim=1, group_size=self.G)
        return time.perf_counter() - t0, rows * (self.per_step_bytes() / self.M), f"{rows} of {self.M} rows"

    def verify(self, orc):
        ref = orc.quant_policy(self.x_h[:64], self.s_h[:64], orc.F16, orc.F32, orc.FP4_E2M1, 3, k_dim=1, group_size=self.G)
        return bool((self.q[0].download().reshape(self.M, self.N // 2)[:64] == ref).all())


class SoftmaxFlashStep(RowOp):
    name = "softmaxflashv2_update_262144x2048_fp16"
    metric, dtype = "SoftmaxFlashV2 update step (fp16 data, fp32 statistics) bandwidth", "f16"
    M, K = 262144, 2048
    traffic_1gpu = 1.0906e9 + 1.0412e9   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of the kernel

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00011 + rank)
        self.x_h = np.tile(f16_bits(rng.standard_normal((4096, self.K), dtype=np.float32) * 3.0), (self.M // 4096, 1))
        self.in_max_h = np.repeat(rng.uniform(2, 8, (self.M, 1)).astype(np.float32), 8, axis=1)
        self.in_sum_h = np.repeat(rng.uniform(100, 200, (self.M, 1)).astype(np.float32), 8, axis=1)
        self.sets = sets = 2   # 2.2 GB per set
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.y = [ab.empty((self.M, self.K), np.uint16) for _ in range(sets)]
        self.in_max, self.in_sum = ab.to_dev(self.in_max_h), ab.to_dev(self.in_sum_h)
        self.mx, self.sm = ab.empty((self.M, 8), np.float32), ab.empty((self.M, 8), np.float32)
        self.em = ab.empty((self.M, 16), np.uint16)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

    def per_step_bytes(self):
        return self.M * self.K * 4 + self.M * (4 * 32 + 32)  # x in, y out; four statistics blocks of 32 bytes and expMax per row

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.softmax_flash_v2(self.x[s], self.y[s], self.sm, self.mx, self.em, self.in_sum, self.in_max, self.M, self.K, ab.F16, ab.F32,
                                     True, True, stream=stream))

    def h2d_arrays(self):
        return [self.x_h, self.in_max_h, self.in_sum_h]

    def h2d_targets(self, s):
        return [self.x[s], self.in_max, self.in_sum]

    def d2h_buffers(self, s):
        return [(self.y[s], self.M * self.K * 2), (self.sm, self.M * 32), (self.mx, self.M * 32), (self.em, self.M * 32)]

    def cpu_sample(self, orc, rows):
        rows = min(rows * 16, self.M)
        t0 = time.perf_counter()
        orc.softmax_flash_v2(self.x_h[:rows], orc.F16, orc.F32, in_sum=self.in_sum_h[:rows], in_max=self.in_max_h[:rows])
        return time.perf_counter() - t0, rows * (self.per_step_bytes() / self.M), f"{rows} of {self.M} rows"

    def verify(self, orc):
        y, s, mx, em = orc.softmax_flash_v2(self.x_h[:64], orc.F16, orc.F32, in_sum=self.in_sum_h[:64], in_max=self.in_max_h[:64])
        got_y = orc.f16_bits_to_f32(self.y[0].download().reshape(self.M, self.K)[:64])
        got_s = self.sm.download().reshape(self.M, 8)[:64]
        return bool(np.allclose(got_y, orc.f16_bits_to_f32(y), rtol=1e-3, atol=1e-6) and np.allclose(got_s, s, rtol=2e-3) and
                    (self.mx.download().reshape(self.M, 8)[:64] == mx).all())


class SoftmaxGradStep(RowOp):
    name = "softmaxgrad_131072x2048_fp16"
    metric, dtype = "SoftmaxGrad (fp16 grad and softmax output in, fp16 out) bandwidth", "f16"
    M, K = 131072, 2048
    traffic_1gpu = 1.0738e9 + 0.4822e9   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of the kernel

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00013 + rank)
        x = rng.standard_normal((4096, self.K), dtype=np.float32) * 2.0
        e = np.exp(x - x.max(axis=1, keepdims=True))
        self.y_h = np.tile(f16_bits(e / e.sum(axis=1, keepdims=True)), (self.M // 4096, 1))
        self.g_h = np.tile(f16_bits(rng.uniform(-1, 1, (4096, self.K)).astype(np.float32)), (self.M // 4096, 1))
        self.sets = sets = 2   # 1.6 GB per set
        self.g = [ab.to_dev(self.g_h) for _ in range(sets)]
        self.y = [ab.to_dev(self.y_h) for _ in range(sets)]
        self.o = [ab.empty((self.M, self.K), np.uint16) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

    def per_step_bytes(self):
        return self.M * self.K * 6   # grad and y in, dst out

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.softmax_grad(self.g[s], self.y[s], self.o[s], self.M, self.K, ab.F16, False, stream=stream))

    def h2d_arrays(self):
        return [self.g_h, self.y_h]

    def h2d_targets(self, s):
        return [self.g[s], self.y[s]]

    def d2h_buffers(self, s):
        return [(self.o[s], self.M * self.K * 2)]

    def cpu_sample(self, orc, rows):
        rows = min(rows * 16, self.M)
        t0 = time.perf_counter()
        orc.softmax_grad(self.g_h[:rows], self.y_h[:rows], orc.F16)
        return time.perf_counter() - t0, rows * (self.per_step_bytes() / self.M), f"{rows} of {self.M} rows"

    def verify(self, orc):
        ref = orc.f16_bits_to_f32(orc.softmax_grad(self.g_h[:64], self.y_h[:64], orc.F16))
        got = orc.f16_bits_to_f32(self.o[0].download().reshape(self.M, self.K)[:64])
        return bool((np.abs(got - ref) <= 1e-3 * np.abs(ref) + 1e-5).all())


class AntiQuantPerChannel(RowOp):
    name = "ascendantiquant_per_channel_int8_to_fp16_131072x2048"
    metric, dtype = "AscendAntiQuant per channel (int8 -> fp16, fp16 scale and offset per column) bandwidth", "f16"
    M, N = 131072, 2048
    traffic_1gpu = 268.9e6 + 477.8e6   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of the kernel

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00014 + rank)
        self.x_h = np.tile(rng.integers(-128, 128, (4096, self.N), dtype=np.int8), (self.M // 4096, 1))
        self.sc_h = f16_bits(rng.uniform(-2, 2, self.N).astype(np.float32))
        self.of_h = f16_bits(rng.uniform(-8, 8, self.N).astype(np.float32))
        self.sets = sets = 2   # 805 MB per set
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.o = [ab.empty((self.M, self.N), np.uint16) for _ in range(sets)]
        self.sc, self.of = ab.to_dev(self.sc_h), ab.to_dev(self.of_h)
        self.config = {"workload": self.name, "M": self.M, "N": self.N, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

    def per_step_bytes(self):
        return self.M * self.N * 3 + self.N * 4

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.antiquant(self.x[s], self.o[s], self.M, self.N, ab.F16, 1, self.sc, self.of, stream=stream))

    def h2d_arrays(self):
        return [self.x_h, self.sc_h, self.of_h]

    def h2d_targets(self, s):
        return [self.x[s], self.sc, self.of]

    def d2h_buffers(self, s):
        return [(self.o[s], self.M * self.N * 2)]

    def cpu_sample(self, orc, rows):
        rows = min(rows * 16, self.M)
        t0 = time.perf_counter()
        orc.antiquant(self.x_h[:rows], orc.F16, 1, scale=self.sc_h, offset=self.of_h)
        return time.perf_counter() - t0, rows * (self.per_step_bytes() / self.M), f"{rows} of {self.M} rows"

    def verify(self, orc):
        ref = orc.antiquant(self.x_h[:64], orc.F16, 1, scale=self.sc_h, offset=self.of_h)
        return bool((self.o[0].download().reshape(self.M, self.N)[:64] == ref).all())


class NzUnpack(RowOp):
    name = "nz_weight_unpack_int8_16x7168x2048"
    metric, dtype = "fractal NZ -> K-major weight unpack bandwidth", "u8"
    G, K, N = 16, 7168, 2048
    traffic_1gpu = 234.9e6 + 181.7e6   # ncu: dram__bytes_read.sum + dram__bytes_write.sum of the kernel

    def __init__(self, ab, rank, world, sets):
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00012 + rank)
        self.w_h = rng.integers(-128, 128, (self.G, self.N // 32, self.K // 16, 16, 32), dtype=np.int8)  # already in NZ order
        self.sets = sets = 2   # 470 MB per set
        self.w = [ab.to_dev(self.w_h) for _ in range(sets)]
        self.o = [ab.empty((self.G, self.N, self.K), np.int8) for _ in range(sets)]
        self.config = {"workload": self.name, "groups": self.G, "K": self.K, "N": self.N, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

    def per_step_bytes(self):
        return 2 * self.G * self.K * self.N

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.nz_unpack(self.w[s], self.o[s], self.G, self.K, self.N, 1, True, stream=stream))

    def h2d_arrays(self):
        return [self.w_h]

    def h2d_targets(self, s):
        return [self.w[s]]

    def d2h_buffers(self, s):
        return [(self.o[s], self.G * self.K * self.N)]

    def cpu_sample(self, orc, rows):
        t0 = time.perf_counter()
        np.ascontiguousarray(self.w_h[:2].transpose(0, 1, 4, 2, 3))  # [g, n/32, 32, k/16, 16] = [g, n, k]
        return time.perf_counter() - t0, 2.0 * 2 * self.K * self.N, "2 of 16 groups (numpy transpose, one thread)"

    def verify(self, orc):
        ref = self.w_h[:1].transpose(0, 1, 4, 2, 3).reshape(1, self.N, self.K)
        return bool((self.o[0].download().reshape(self.G, self.N, self.K)[:1] == ref).all())


WORKLOADS = {"a8w8": A8W8, "grouped": Grouped, "mxfp4": MXFP4, "softmax_quant": SoftmaxQuant, "softmax_quant_x64": SoftmaxQuantLarge,
             "fp16": FP16, "fp16_8192": FP16Large, "grouped_ref_shape": GroupedRefShape, "quant_per_group_fp4": QuantPerGroupFp4,
             "softmax_flash_v2": SoftmaxFlashStep, "softmax_grad": SoftmaxGradStep, "antiquant": AntiQuantPerChannel, "nz_unpack": NzUnpack}


class PinnedSet:
    """Pinned host copies of one step's inputs and a pinned landing buffer for its outputs."""

    def __init__(self, ab, arrays, out_bytes):
        import ctypes as C
        self.ab, self.C = ab, C
        self.src = []
        for a in arrays:
            p = C.c_void_p()
            ab.check(ab.lib().ascb200_malloc_host(C.byref(p), max(a.nbytes, 1)))
            C.memmove(p.value, a.ctypes.data, a.nbytes)
            self.src.append((p.value, a.nbytes))
        self.outs = []
        for _ in range(2):   # one landing buffer per in-flight step (two streams alternate)
            p = C.c_void_p()
            ab.check(ab.lib().ascb200_malloc_host(C.byref(p), max(out_bytes, 1)))
            self.outs.append(p.value)
        self.out, self.out_bytes, self.slot = self.outs[0], out_bytes, 0

    def h2d(self, dev_bufs, stream):
        for (p, n), d in zip(self.src, dev_bufs):
            self.ab.check(self.ab.lib().ascb200_memcpy_h2d(d.ptr, p, n, stream))

    def d2h(self, dev_buf, stream, offset=0):
        n = min(dev_buf.nbytes, self.out_bytes - offset)
        self.ab.check(self.ab.lib().ascb200_memcpy_d2h(self.outs[self.slot] + offset, dev_buf.ptr, n, stream))


# ------------------------------------------------------------------------------------------------
# measurement
# ------------------------------------------------------------------------------------------------
def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class Comm:
    """torch.distributed (NCCL) used only for the barrier and the max over ranks of the measured time."""

    def __init__(self, world, local_rank):
        self.world = world
        self.torch = None
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            self.torch, self.dist = torch, dist

    def barrier(self):
        if self.torch:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max(self, v):
        if not self.torch:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def slab_comm(self, ab):
        """An NCCL communicator made through the C ABI (ascb200_comm_init); the 128-byte id travels over the rendezvous group."""
        import ctypes as C
        if getattr(self, "_slab_comm", None) is None:
            torch, dist = self.torch, self.dist
            ident = (C.c_uint8 * 128)()
            if dist.get_rank() == 0:
                ab.check(ab.lib().ascb200_comm_unique_id(ident), "comm_unique_id")
            t = torch.tensor(list(ident), dtype=torch.uint8, device="cuda")
            dist.broadcast(t, 0)
            ident = (C.c_uint8 * 128)(*t.cpu().tolist())
            comm = C.c_void_p()
            ab.check(ab.lib().ascb200_comm_init(C.byref(comm), self.world, dist.get_rank(), ident), "comm_init")
            self._slab_comm = comm
        return self._slab_comm

    def allgather_ms(self, ab, slab, m, n_loc, elem_bytes, stream, reps=5):
        """Times ascb200_allgather_slabs (NCCL all-gather + local re-layout into row-major [m][ranks * n_loc]) of one rank's output
        slab and checks the result: every rank's columns of the gathered C carry that rank's checksum."""
        torch, dist = self.torch, self.dist
        comm = self.slab_comm(ab)
        gathered = ab.empty((self.world, m, n_loc * elem_bytes), np.uint8)
        full = ab.empty((m, self.world * n_loc * elem_bytes), np.uint8)
        call = lambda: ab.check(ab.lib().ascb200_allgather_slabs(comm, self.world, slab.ptr, m, n_loc, elem_bytes, gathered.ptr, full.ptr, 0, stream),
                                "allgather_slabs")
        for _ in range(2):
            call()
        ab.sync(stream)
        self.barrier()
        timer = ab.Timer(stream)
        timer.start()
        for _ in range(reps):
            call()
        ms = self.max(timer.stop_ms() / reps)
        ab.sync(stream)
        mine = slab.download(shape=(m, n_loc * elem_bytes), dtype=np.uint8)
        sums = torch.zeros(self.world, dtype=torch.int64, device="cuda")
        sums[dist.get_rank()] = int(mine.astype(np.int64).sum())
        dist.all_reduce(sums)
        got = full.download().reshape(m, self.world, n_loc * elem_bytes)
        ok = bool((got[:, dist.get_rank()] == mine).all() and (got.astype(np.int64).sum(axis=(0, 2)) == sums.cpu().numpy()).all())
        gathered.free()
        full.free()
        return ms, ok

    def close(self):
        if getattr(self, "_slab_comm", None) is not None:
            import ascb200 as ab
            ab.lib().ascb200_comm_destroy(self._slab_comm)
        if self.torch:
            self.dist.destroy_process_group()


def time_e2e(ab, wl, comm, steps, warmup, stream, stream2):
    """End to end: every step copies its inputs from pinned host memory, runs the call and copies the outputs back.  Two
    streams (and two pinned landing buffers) alternate, so that the copy-out of one step overlaps the copy-in of the next on
    the full-duplex host link; timed on the first stream, which waits for the second before the closing event.  Returns the
    maximum over ranks (ms) for exactly `steps` steps."""
    import ctypes as C
    streams = [stream, stream2]

    def fn(i):
        wl.pin.slot = i % 2
        wl.e2e_step(i, streams[i % 2])

    for i in range(warmup):
        fn(i)
    ab.sync(stream)
    ab.sync(stream2)
    comm.barrier()
    timer = ab.Timer(stream)
    timer.start()
    ab.check(ab.lib().ascb200_stream_wait_event(stream2, timer.e0))   # the second stream starts after the opening event
    for i in range(steps):
        fn(warmup + i)
    ev = C.c_void_p()
    ab.check(ab.lib().ascb200_event_create(C.byref(ev)))
    ab.check(ab.lib().ascb200_event_record(ev, stream2))
    ab.check(ab.lib().ascb200_stream_wait_event(stream, ev))
    ms = timer.stop_ms()
    ab.sync(stream)
    ab.sync(stream2)
    comm.barrier()
    return comm.max(ms)


def time_resident(ab, wl, comm, steps, warmup, stream, clock_index, budget_s=0.4):
    """Device-resident timing.  The `steps` steps are captured into one CUDA graph (so that the host's per-call cost does not
    sit between kernels that last microseconds); after the warm-up steps and one untimed replay the graph is replayed R >= 10
    times (R chosen so that the replays last about `budget_s` in total), each replay bracketed by barrier + synchronise and
    timed with CUDA events on the launching stream, maximum over ranks.  Clocks are sampled only while the replays run.
    Returns (per-replay times in ms, clock summary)."""
    for i in range(warmup):
        wl.step(i, stream)
    ab.sync(stream)
    graph = ab.Graph(stream, lambda: [wl.step(warmup + i, stream) for i in range(steps)])
    timer = ab.Timer(stream)
    timer.start()
    graph.launch()                       # untimed: graph upload, and an estimate of one replay
    est_ms = max(timer.stop_ms(), 1e-3)
    ab.sync(stream)
    local_r = int(min(200, max(10, -(-budget_s * 1e3 // est_ms))))
    repeats = int(comm.max(float(local_r)))   # the same count on every rank
    sampler = ClockSampler(clock_index)
    sampler.start()
    times = []
    for _ in range(repeats):
        comm.barrier()
        timer.start()
        graph.launch()
        ms = timer.stop_ms()             # synchronises on the closing event
        ab.sync(stream)
        times.append(comm.max(ms))
    clocks = sampler.stop()
    comm.barrier()
    graph.destroy()
    return times, clocks


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(wl, target_s):
    import oracle as orc
    orc.set_num_threads(host_threads())   # a launcher may have exported OMP_NUM_THREADS=1
    rows = 2
    t, units, what = wl.cpu_sample(orc, rows)
    # grow the sample until it takes target_s (bounded), keeping the last measurement
    while t < target_s / 3 and rows < 4096:
        rows = min(4096, max(rows * 2, int(rows * target_s / max(t, 1e-3) * 0.7)))
        t, units, what = wl.cpu_sample(orc, rows)
        if "whole problem" in what:
            break
    return {"value": units / t / wl.unit_scale, "unit": wl.unit, "cores": orc.num_threads(), "kind": "port", "sample": what,
            "seconds": round(t, 3)}


def measure(ab, cls, comm, rank, world, args, peaks, with_cpu, clock_index):
    import ctypes as C
    stream_p = C.c_void_p()
    ab.check(ab.lib().ascb200_stream_create(C.byref(stream_p)))
    stream = stream_p.value
    wl = cls(ab, rank, world, sets=2)
    # untimed check that the configuration computes the right thing
    wl.step(0, stream)
    ab.sync(stream)
    import oracle as orc
    verified = wl.verify(orc)

    warmup = max(args.warmup, 3)
    times, clocks = time_resident(ab, wl, comm, args.steps, warmup, stream, clock_index)
    ms = float(np.median(times))

    e2e_steps = max(3, min(args.steps, 20))
    bi, bo = wl.e2e_bytes()
    if args.kernel_only:
        ms_e2e, with_cpu = float("nan"), False
    else:
        wl.e2e_setup()
        stream2_p = C.c_void_p()
        ab.check(ab.lib().ascb200_stream_create(C.byref(stream2_p)))
        ms_e2e = time_e2e(ab, wl, comm, e2e_steps, 4, stream, stream2_p.value)
        ab.lib().ascb200_stream_destroy(stream2_p.value)

    per_step_s = ms / 1e3 / args.steps
    value = wl.units_total() / per_step_s / wl.unit_scale
    achieved = wl.units_rank() / per_step_s / wl.unit_scale
    peak, punit, pnote = wl.peak(peaks)              # the burst figure
    roof = {"bound": wl.bound, "achieved": round(achieved, 3), "unit": punit, "traffic": (wl.traffic_1gpu if world == 1 else None),
            "algorithmic": wl.units_rank() if wl.bound == "hbm" else getattr(wl, "algorithmic_bytes", None)}
    sustained = peaks.get("bf16_tflops_sustained")
    if wl.bound == "tensor" and sustained:
        # the replays are a long back-to-back sequence under the power cap: the sustained cuBLAS figure is the denominator
        peak_s = peak * sustained / peaks["bf16_tflops"]
        roof.update(peak=round(peak_s, 1), frac=round(achieved / peak_s, 4), frac_of_burst_peak=round(achieved / peak, 4),
                    peak_source=f"{peaks['source']}, sustained: {pnote.replace('burst', 'sustained loop')}")
    else:
        roof.update(peak=round(peak, 1), frac=round(achieved / peak, 4), peak_source=f"{peaks['source']}: {pnote}")
    # the fastest replay (normally the first, before the power cap pulls the clock down) against the burst figure, which is
    # itself a best-of-ten
    best_rate = wl.units_rank() / (min(times) / 1e3 / args.steps) / wl.unit_scale
    roof["best_replay"] = {"ms_per_step": round(min(times) / args.steps, 6), "achieved": round(best_rate, 3), "frac_of_burst_peak": round(best_rate / peak, 4)}
    extra = wl.extra_roofline(ms / args.steps, peaks) if hasattr(wl, "extra_roofline") else None
    if extra:
        roof.update(extra)
    med_mhz = clocks.get("sm_mhz")
    line = {
        "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms / args.steps, 6), "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
        "repeats": len(times), "ms_per_step_range": [round(min(times) / args.steps, 6), round(max(times) / args.steps, 6)],
        "ms_x_sm_mhz": round(ms / args.steps * med_mhz, 3) if med_mhz else None,
        "roofline": roof,
        "e2e": {"value": round(wl.units_total() / (ms_e2e / 1e3 / e2e_steps) / wl.unit_scale, 4), "unit": wl.unit, "h2d_bytes_per_step": int(bi),
                "d2h_bytes_per_step": int(bo), "steps": e2e_steps},
        "gpu_launches": args.steps * wl.kernels_per_step, "clocks": clocks, "parity_spot_check": verified,
    }
    if world > 1 and hasattr(wl, "n_loc") and not args.no_allgather:
        # outside the timed region: the optional collective that gives every rank the whole row-major C
        esz = wl.c[0].nbytes // (wl.M * wl.n_loc)
        ms_ag, ok_ag = comm.allgather_ms(ab, wl.c[0], wl.M, wl.n_loc, esz, stream)
        slab_bytes = wl.c[0].nbytes
        line["allgather"] = {"ms": round(ms_ag, 4), "bytes_per_rank": slab_bytes, "layout": "row-major [M][N] on every rank", "ok": ok_ag,
                             "what": "ascb200_allgather_slabs: NCCL all-gather + local re-layout kernel",
                             "busbw_gbs": round(slab_bytes * (world - 1) / (ms_ag / 1e3) / 1e9, 1)}
    if wl.published:
        line["vs_published_other_hw"] = {"ratio": round(value / wl.published[0], 3), "what": wl.published[1]}
    if with_cpu:
        line["cpu_baseline"] = cpu_baseline(wl, 10.0)
    ab.lib().ascb200_stream_destroy(stream)
    return line


def run_reference_arm(args, rank, world, out):
    """CPU restatement of the reference arithmetic, all host threads, bounded sample per step.  Rank 0 alone runs it; the
    workload object is built for rank 0 of `world` ranks, so its configuration labels equal the ones of the GPU arm."""
    if rank != 0:
        return
    import oracle as orc
    orc.set_num_threads(host_threads())   # torchrun exports OMP_NUM_THREADS=1

    class HostOnly:
        """Stands in for the device binding: the reference arm allocates nothing on a GPU."""
        SCALE_B_PREPACKED = 2

        @staticmethod
        def to_dev(a):
            return None

        @staticmethod
        def empty(shape, dtype):
            return None

        @staticmethod
        def mx_scale_prepack(*a, **k):
            return None

    wl = WORKLOADS[args.workload](HostOnly, 0, world, sets=1)
    rows = 2
    t, units, what = wl.cpu_sample(orc, rows)
    while t < 0.7 and rows < 4096 and "whole problem" not in what:   # ~2 s per step
        rows = min(4096, max(rows * 2, int(rows * 2.0 / max(t, 1e-3) * 0.7)))
        t, units, what = wl.cpu_sample(orc, rows)
    for _ in range(min(args.warmup, 1)):
        wl.cpu_sample(orc, rows)
    tot_t = tot_u = 0.0
    for _ in range(args.steps):
        t, units, what = wl.cpu_sample(orc, rows)
        tot_t += t
        tot_u += units
    value = tot_u / tot_t / wl.unit_scale
    line = {
        "impl": "reference", "metric": wl.metric, "value": round(value, 6), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(tot_t / args.steps * 1e3, 3), "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
        "cpu_baseline": {"value": round(value, 6), "unit": wl.unit, "cores": orc.num_threads(), "kind": "port", "sample": what + " per step"},
        "e2e": {"value": round(value, 6), "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference arithmetic (oracle/asc_oracle.c, OpenMP); the reference's CPU-debug build needs the closed CANN CPU twin",
    }
    out.emit(json.dumps(line))


class OneLineStdout:
    """Everything that libraries print to stdout (NCCL's version banner, for one) is sent to stderr; the
    JSON line is written to the real stdout at the end, so that stdout carries exactly one line."""

    def __init__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)

    def emit(self, text):
        sys.stdout.flush()
        os.write(self.real, (text + "\n").encode())


BASELINE_OTHERS_1GPU = ["grouped", "mxfp4", "softmax_quant", "softmax_quant_x64", "fp16", "fp16_8192", "grouped_ref_shape"]
SHARDED = ["a8w8", "grouped", "mxfp4"]


def summary_entry(o):
    return {"workload": o["config"]["workload"], "value": o["value"], "unit": o["unit"], "ms_per_step": o["ms_per_step"],
            "frac": o["roofline"]["frac"], "best_replay_frac_of_burst": o["roofline"]["best_replay"]["frac_of_burst_peak"], "e2e": o["e2e"]["value"],
            "parity": o["parity_spot_check"]}


def main():
    out = OneLineStdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="a8w8", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ascb200", choices=["ascb200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the other baseline configurations")
    ap.add_argument("--all", action="store_true", help="N=1: also measure the kernels outside the baseline configurations")
    ap.add_argument("--no-allgather", action="store_true",
                    help="N>1, N-slab workloads: skip the (untimed-region) measurement of the all-gather that gives every rank the whole C")
    ap.add_argument("--kernel-only", action="store_true", help="time the device-resident step only (no e2e, no CPU baseline): profiling runs")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference_arm(args, rank, world, out)
        return

    import ascb200 as ab
    comm = Comm(world, local_rank)
    ab.init(local_rank)
    peaks = measured_peaks()
    line = measure(ab, WORKLOADS[args.workload], comm, rank, world, args, peaks, with_cpu=(world == 1 and rank == 0),
                   clock_index=local_rank)
    if not args.no_others and not args.kernel_only:
        if world == 1:
            names = list(WORKLOADS) if args.all else BASELINE_OTHERS_1GPU
        else:
            names = SHARDED   # the sharded configurations: the scaling record then carries all three at every N
        others = []
        for name in names:
            if name == args.workload:
                continue
            sub = argparse.Namespace(**vars(args))
            sub.steps = min(args.steps, 50)
            o = measure(ab, WORKLOADS[name], comm, rank, world, sub, peaks, with_cpu=(world == 1), clock_index=local_rank)
            others.append({k: o[k] for k in ("metric", "value", "unit", "n_gpus", "ms_per_step", "ms_per_step_range", "repeats", "ms_x_sm_mhz", "steps",
                                             "config", "roofline", "e2e", "cpu_baseline", "clocks", "parity_spot_check", "gpu_launches",
                                             "vs_published_other_hw", "allgather") if k in o})
        line["others"] = others
        # the same figures beside the headline kernel's roofline: a reader that keeps only the contract's keys still sees every configuration
        line["roofline"]["other_configs"] = {o["config"]["workload"]: {"achieved": o["value"], "unit": o["unit"], "ms_per_step": o["ms_per_step"],
                                                                       "peak": o["roofline"]["peak"], "frac": o["roofline"]["frac"],
                                                                       "bound": o["roofline"]["bound"]} for o in others}
        line["summary"] = [summary_entry(line)] + [summary_entry(o) for o in others]
    comm.close()
    if rank == 0:
        out.emit(json.dumps(line))


if __name__ == "__main__":
    main()
