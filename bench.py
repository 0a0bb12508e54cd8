"""Benchmark of the ascb200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload a8w8|grouped|mxfp4|softmax_quant|fp16] [--impl reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the A8W8 dense GEMM of the baseline (A[4096,4096] int8, B[11008,4096] int8 K-major,
int32 accumulation, fused bf16(acc * ch_scale[n] * tok_scale[m]) epilogue), sharded by N-slab
across ranks with no communication; `value` is the whole-job rate (all ranks' operations divided
by the slowest rank's device time, CUDA events on the launching stream).

Rank 0 prints ONE JSON line.  At N=1 it also carries, under "others", the same measurement for
the other baseline configurations (grouped A8W8, MXFP4, SoftMax+AscendQuant, fp16 Matmul).

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
from sharding import dirichlet_counts, lpt_partition  # noqa: E402


class Workload:
    """Holds device buffers for `sets` rotating input/output sets and launches one step."""
    name = metric = unit = dtype = ""
    unit_scale = 1e12            # value = units / seconds / unit_scale (1e12: TOPS / TFLOPS, 1e9: GB/s)
    bound = "tensor"
    scaling = "strong"
    kernels_per_step = 1
    published = None  # (value, note) of a like-for-like number the reference publishes (other hardware)
    # dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, per launch, from the ncu capture summarised in
    # profiles/ (1 GPU, whole configuration); None where no capture exists
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
    traffic_1gpu = 62.05e6 + 48.92e6   # profiles/gemm_tc_pair_kernel_int8_a8w8_4096x4096x11008.md

    def __init__(self, ab, rank, world, sets):
        self.ab, self.rank, self.world = ab, rank, world
        assert self.N % world == 0
        self.n_loc = self.N // world
        rng = np.random.default_rng(0xA5C00002)
        self.a_h = rng.integers(-127, 128, (self.M, self.K)).astype(np.int8)
        self.tok_h = rng.uniform(1e-3, 1e-2, self.M).astype(np.float32)
        ch = rng.uniform(1e-3, 1e-2, self.N).astype(np.float32)
        rng_b = np.random.default_rng(0xA5C00002 + 1000 + rank)   # each rank draws its own B slab
        self.b_h = rng_b.integers(-127, 128, (self.n_loc, self.K)).astype(np.int8)
        self.ch_h = ch[rank * self.n_loc:(rank + 1) * self.n_loc].copy()
        self.sets = sets
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.tok, self.ch = ab.to_dev(self.tok_h), ab.to_dev(self.ch_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.bytes_rank() // 2**20} MiB > L2)"}
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
    traffic_1gpu = 1.2107e9 + 0.1229e9   # profiles/gemm_tc_kernel_int8_grouped_64groups_M32768_K7168_N2048.md

    def counts(self):
        return dirichlet_counts(self.G, self.MTOT, 0xA5C00003)

    def __init__(self, ab, rank, world, sets):
        self.ab, self.rank, self.world = ab, rank, world
        counts = self.counts()
        mine = lpt_partition(counts, world)[rank]
        self.counts_h = counts[mine].astype(np.int64)
        self.m_loc = int(self.counts_h.sum())
        self.g_loc = len(mine)
        rng = np.random.default_rng(0xA5C00003 + 1000 + rank)
        self.x_h = rng.integers(-127, 128, (max(self.m_loc, 1), self.K)).astype(np.int8)
        self.w_h = rng.integers(-127, 128, (self.g_loc, self.N, self.K), dtype=np.int8)
        self.tok_h = rng.uniform(1e-3, 1e-2, max(self.m_loc, 1)).astype(np.float32)
        self.ch_h = rng.uniform(1e-3, 1e-2, (self.g_loc, self.N)).astype(np.float32)
        self.sets = sets
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.w = [ab.to_dev(self.w_h) for _ in range(1)]           # 0.94 GB of weights already exceed L2
        self.c = [ab.empty((max(self.m_loc, 1), self.N), np.uint16) for _ in range(sets)]
        self.tok, self.ch, self.counts_d = ab.to_dev(self.tok_h), ab.to_dev(self.ch_h), ab.to_dev(self.counts_h)
        self.config = {"workload": self.name, "groups": self.G, "rows": self.MTOT, "K": self.K, "N": self.N,
                       "shard": f"groups x{world} (greedy by rows)", "rows_this_rank": self.m_loc,
                       "cache": f"weights of one pass ({self.w_h.nbytes // 2**20} MiB on this rank)" + ("" if self.w_h.nbytes > L2_BYTES else ", may stay in L2")}

    def units_total(self):
        return 2.0 * self.MTOT * self.K * self.N

    def units_rank(self):
        return 2.0 * self.m_loc * self.K * self.N

    def peak(self, peaks):
        return 2.0 * peaks["bf16_tflops"], "TOPS", "2 x measured bf16 cuBLAS burst"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_S8, self.m_loc, self.N, self.K, self.x[s], self.w[0], self.c[s], getattr(ab, self.OUT),
                         epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, tok=self.tok, ch=self.ch, group_counts=self.counts_d,
                         groups=self.g_loc, act=self.ACT, stream=stream))

    def e2e_bytes(self):
        return self.x_h.nbytes + self.w_h.nbytes + self.tok_h.nbytes + self.ch_h.nbytes + self.counts_h.nbytes, self.m_loc * self.N * 2

    def e2e_setup(self):
        self.pin = PinnedSet(self.ab, [self.x_h, self.w_h, self.tok_h, self.ch_h, self.counts_h], self.m_loc * self.N * 2)

    def e2e_step(self, i, stream):
        s = i % self.sets
        self.pin.h2d([self.x[s], self.w[0], self.tok, self.ch, self.counts_d], stream)
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
    kernels_per_step = 3  # two scale re-tiling launches + the GEMM
    traffic_1gpu = 95.2e6 + 168.0e6    # profiles/gemm_tc_pair_kernel_mxfp4_8192x8192x8192.md
    published = (1614.0, "Ascend 950PR basic-API MXFP4 8192^3, bf16 out; the reference's published figure")

    def __init__(self, ab, rank, world, sets):
        from gpu_util import mx_quantize, quant_params
        self.ab, self.rank, self.world = ab, rank, world
        self.n_loc = self.N // world
        rng = np.random.default_rng(0xA5C00004)
        self.a_h, self.sa_h = mx_quantize(rng.standard_normal((self.M, self.K), dtype=np.float32))
        rng_b = np.random.default_rng(0xA5C00004 + 1000 + rank)
        self.b_h, self.sb_h = mx_quantize(rng_b.standard_normal((self.n_loc, self.K), dtype=np.float32))
        # accumulators ~ N(0, K * E[a^2] E[b^2]); quantised unit normals keep E[x^2] ~ 1 -> sigma ~ sqrt(K)
        scales = (rng.uniform(0.5, 2.0, self.N) * 40.0 / np.sqrt(self.K)).astype(np.float32)
        self.q_h = quant_params(scales[rank * self.n_loc:(rank + 1) * self.n_loc])
        self.sets = sets
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.sa, self.sb, self.q = ab.to_dev(self.sa_h), ab.to_dev(self.sb_h), ab.to_dev(self.q_h)
        self.c = [ab.empty((self.M, self.n_loc), np.int8) for _ in range(sets)]
        self.c2 = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}",
                       "cache": f"{sets} rotating buffer sets"}

    def units_total(self):
        return 2.0 * self.M * self.K * self.N

    def units_rank(self):
        return 2.0 * self.M * self.K * self.n_loc

    def peak(self, peaks):
        return 4.0 * peaks["bf16_tflops"], "TFLOPS", "4 x measured bf16 cuBLAS burst (fp4 runs at four times the bf16 rate)"

    def step(self, i, stream=None):
        ab, s = self.ab, i % self.sets
        ab.check(ab.gemm(ab.KIND_MXFP4, self.M, self.n_loc, self.K, self.a[s], self.b[s], self.c[s], ab.S8,
                         epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, scale_a=self.sa, scale_b=self.sb, quant=self.q,
                         c2=self.c2[s], c2_dtype=ab.BF16, stream=stream))

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
        acc = orc.gemm_mxf4(self.a_h[:16], self.sa_h[:16], self.b_h, self.sb_h, base_k=256)
        q = self.c[0].download()[:16]
        bf = self.c2[0].download()[:16]
        ref_q = orc.fixpipe_qf322b8(acc, self.q_h)
        d = np.abs(q.astype(np.int32) - ref_q.astype(np.int32))
        ok_bf = np.allclose(orc.bf16_bits_to_f32(bf), acc, rtol=1e-2, atol=1e-3)
        return bool(d.max() <= 1 and (d != 0).mean() < 1e-3 and ok_bf)


class SoftmaxQuant(Workload):
    name = "softmax_ascendquant_4096x2048_fp16_int8"
    metric, unit, dtype = "SoftMax + AscendQuant row-op bandwidth (fused single pass)", "GB/s", "f16"
    bound = "hbm"
    unit_scale = 1e9
    scaling = "weak"  # rows are independent; every rank runs its own replica of the configuration
    M, K = 4096, 2048
    ROW_FACTOR = 1
    traffic_1gpu = 16.8e6               # profiles/softmax_rows_kernel_fused_quant_4096x2048.md (outputs still in L2 at kernel end)

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.M = self.M * self.ROW_FACTOR
        self.ab, self.rank, self.world = ab, rank, world
        rng = np.random.default_rng(0xA5C00001 + rank)
        self.x_h = np.tile(f16_bits(rng.standard_normal((4096, self.K), dtype=np.float32) * 3.0), (self.ROW_FACTOR, 1))
        self.sc_h = f16_bits((127.0 / rng.uniform(0.5, 2.0, self.K)).astype(np.float32))
        self.sets = sets = max(sets, 8) if self.ROW_FACTOR == 1 else 2  # 42 MB per set: rotate 8 sets so no step finds its input in L2
        self.x = [ab.to_dev(self.x_h) for _ in range(sets)]
        self.y = [ab.empty((self.M, self.K), np.uint16) for _ in range(sets)]
        self.q = [ab.empty((self.M, self.K), np.int8) for _ in range(sets)]
        self.sm, self.mx = ab.empty((self.M,), np.float32), ab.empty((self.M,), np.float32)
        self.sc = ab.to_dev(self.sc_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets ({sets * self.per_step_bytes() // 2**20} MiB > L2)"}

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
    traffic_1gpu = 1.0738e9 + 1.5580e9  # profiles/softmax_rows_kernel_fused_quant_262144x2048.md


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
        self.sets = sets = 48  # 3.7 MB per set: 48 sets = 176 MB > L2
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.N), np.float32) for _ in range(sets)]
        self.bias = ab.to_dev(self.bias_h)
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"replica per rank x{world}",
                       "cache": f"{sets} rotating buffer sets (176 MiB > L2)", "note": "0.54 GFLOP: launch-latency bound"}

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

    def __init__(self, ab, rank, world, sets):
        from gpu_util import f16_bits
        self.ab, self.rank, self.world = ab, rank, world
        self.n_loc = self.N // world
        rng = np.random.default_rng(0xA5C00005)
        self.a_h = f16_bits(rng.uniform(1, 10, (self.M, self.K)).astype(np.float32))      # the example draws U[1,10)
        self.b_h = f16_bits(np.random.default_rng(0xA5C00005 + 1000 + rank).uniform(1, 10, (self.n_loc, self.K)).astype(np.float32))
        self.sets = sets
        self.a = [ab.to_dev(self.a_h) for _ in range(sets)]
        self.b = [ab.to_dev(self.b_h) for _ in range(sets)]
        self.c = [ab.empty((self.M, self.n_loc), np.uint16) for _ in range(sets)]
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shard": f"N-slab x{world}", "cache": f"{sets} rotating buffer sets"}

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
    traffic_1gpu = 570.5e6 + 120.6e6   # profiles/quant_policy_vec_kernel_per_group32_fp16_fp4_32768x8192.md

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
    traffic_1gpu = 1.0906e9 + 1.0412e9   # profiles/softmax_flash_rows_kernel_update_262144x2048_fp16.md

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
    traffic_1gpu = 1.0738e9 + 0.4822e9   # profiles/softmax_grad_rows_kernel_131072x2048_fp16.md

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
    traffic_1gpu = 268.9e6 + 477.8e6   # profiles/antiquant_i8_columns_kernel_int8_fp16_131072x2048.md

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
    traffic_1gpu = 234.9e6 + 181.7e6   # profiles/nz_unpack_kernel_int8_16x7168x2048.md

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

    def allgather_ms(self, ab, dev_buf, nbytes, reps=5):
        """Times all_gather_into_tensor of one rank's output slab (copied into a torch buffer once, outside the timing)."""
        torch, dist = self.torch, self.dist
        send = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        recv = torch.empty(nbytes * self.world, dtype=torch.uint8, device="cuda")
        ab.sync()
        host = dev_buf.download(shape=(nbytes,), dtype=np.uint8)
        send.copy_(torch.from_numpy(host))
        for _ in range(2):
            dist.all_gather_into_tensor(recv, send)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        for _ in range(reps):
            dist.all_gather_into_tensor(recv, send)
        e1.record()
        torch.cuda.synchronize()
        ms = self.max(e0.elapsed_time(e1) / reps)
        ok = bool((recv[self.dist.get_rank() * nbytes:(self.dist.get_rank() + 1) * nbytes] == send).all().item())
        return ms, ok

    def close(self):
        if self.torch:
            self.dist.destroy_process_group()


def time_steps(ab, wl, comm, steps, warmup, stream, e2e=False, stream2=None):
    """Times exactly `steps` steps between a barrier + synchronize on both sides; returns the max over ranks (ms).
    The device-resident measurement replays the steps from one CUDA graph, so that the host's launch
    cost (a Python ctypes call per step) does not sit between kernels that last a few microseconds.
    The end-to-end measurement alternates two streams (and two buffer sets), so that the copy-out of one
    step overlaps the copy-in of the next on the full-duplex host link; it is timed on the first stream,
    which waits for the second before the closing event."""
    import ctypes as C
    streams = [stream, stream2 if (e2e and stream2) else stream]

    def fn(i):
        if e2e:
            wl.pin.slot = i % 2
            wl.e2e_step(i, streams[i % 2])
        else:
            wl.step(i, stream)

    for i in range(warmup):
        fn(i)
    ab.sync(stream)
    if streams[1] is not stream:
        ab.sync(streams[1])
    graph = None
    if not e2e:
        graph = ab.Graph(stream, lambda: [fn(warmup + i) for i in range(steps)])
        graph.launch()          # one untimed replay: graph upload
        ab.sync(stream)
    comm.barrier()
    timer = ab.Timer(stream)
    timer.start()
    if graph:
        graph.launch()
    else:
        if streams[1] is not stream:   # the second stream starts after the opening event
            ab.check(ab.lib().ascb200_stream_wait_event(streams[1], timer.e0))
        for i in range(steps):
            fn(warmup + i)
        if streams[1] is not stream:
            ev = C.c_void_p()
            ab.check(ab.lib().ascb200_event_create(C.byref(ev)))
            ab.check(ab.lib().ascb200_event_record(ev, streams[1]))
            ab.check(ab.lib().ascb200_stream_wait_event(stream, ev))
    ms = timer.stop_ms()
    ab.sync(stream)
    if streams[1] is not stream:
        ab.sync(streams[1])
    comm.barrier()
    if graph:
        graph.destroy()
    return comm.max(ms)


def cpu_baseline(wl, target_s):
    import oracle as orc
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
    stream_p = __import__("ctypes").c_void_p()
    ab.check(ab.lib().ascb200_stream_create(__import__("ctypes").byref(stream_p)))
    stream = stream_p.value
    wl = cls(ab, rank, world, sets=2)
    # untimed check that the configuration computes the right thing
    wl.step(0, stream)
    ab.sync(stream)
    import oracle as orc
    verified = wl.verify(orc)

    sampler = ClockSampler(clock_index)
    # keep the GPU busy for a moment so the clock samples describe the loaded state
    t_end = time.time() + 0.3
    sampler.start()
    i = 0
    while time.time() < t_end:
        wl.step(i, stream)
        i += 1
        if i % 16 == 0:
            ab.sync(stream)
    ms = time_steps(ab, wl, comm, args.steps, max(args.warmup, 3), stream)
    clocks = sampler.stop()

    e2e_steps = max(3, min(args.steps, 20))
    bi, bo = wl.e2e_bytes()
    if args.kernel_only:
        ms_e2e, with_cpu = float("nan"), False
    else:
        wl.e2e_setup()
        stream2_p = __import__("ctypes").c_void_p()
        ab.check(ab.lib().ascb200_stream_create(__import__("ctypes").byref(stream2_p)))
        ms_e2e = time_steps(ab, wl, comm, e2e_steps, 4, stream, e2e=True, stream2=stream2_p.value)
        ab.lib().ascb200_stream_destroy(stream2_p.value)

    per_step_s = ms / 1e3 / args.steps
    value = wl.units_total() / per_step_s / wl.unit_scale
    achieved = wl.units_rank() / per_step_s / wl.unit_scale
    peak, punit, pnote = wl.peak(peaks)
    # The timed region is a long back-to-back replay under the power cap: for tensor-bound kernels the same fraction against the
    # SUSTAINED cuBLAS figure (seconds-long loop, same cap) is reported beside the one against the burst figure.
    frac_sustained = None
    if wl.bound == "tensor" and peaks.get("bf16_tflops_sustained"):
        frac_sustained = round(achieved / (peak * peaks["bf16_tflops_sustained"] / peaks["bf16_tflops"]), 4)
    line = {
        "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 6), "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
        "roofline": {"bound": wl.bound, "achieved": round(achieved, 3), "peak": round(peak, 1), "unit": punit,
                     "frac": round(achieved / peak, 4), "traffic": (wl.traffic_1gpu if world == 1 else None),
                     "algorithmic": wl.units_rank() if wl.bound == "hbm" else getattr(wl, "algorithmic_bytes", None),
                     "peak_source": f"{peaks['source']}: {pnote}", "frac_of_sustained_peak": frac_sustained},
        "e2e": {"value": round(wl.units_total() / (ms_e2e / 1e3 / e2e_steps) / wl.unit_scale, 4), "unit": wl.unit, "h2d_bytes_per_step": int(bi),
                "d2h_bytes_per_step": int(bo), "steps": e2e_steps},
        "gpu_launches": args.steps * wl.kernels_per_step, "clocks": clocks, "parity_spot_check": verified,
    }
    if getattr(args, "allgather", False) and world > 1 and hasattr(wl, "n_loc"):
        slab_bytes = wl.c[0].nbytes
        ms_ag, ok_ag = comm.allgather_ms(ab, wl.c[0], slab_bytes)
        line["allgather"] = {"ms": round(ms_ag, 4), "bytes_per_rank": slab_bytes, "layout": "[rank][M][N/ranks]", "ok": ok_ag,
                             "busbw_gbs": round(slab_bytes * (world - 1) / (ms_ag / 1e3) / 1e9, 1)}
    if wl.published:
        line["vs_published_other_hw"] = {"ratio": round(value / wl.published[0], 3), "what": wl.published[1]}
    if with_cpu:
        line["cpu_baseline"] = cpu_baseline(wl, 10.0)
    ab.lib().ascb200_stream_destroy(stream)
    return line


def run_reference_arm(args, rank, world, out):
    """CPU restatement of the reference arithmetic, all host threads, bounded sample per step."""
    if rank != 0:
        return
    import oracle as orc

    class HostOnly:
        """Stands in for the device binding: the reference arm allocates nothing on a GPU."""

        @staticmethod
        def to_dev(a):
            return None

        @staticmethod
        def empty(shape, dtype):
            return None

    wl = WORKLOADS[args.workload](HostOnly, 0, 1, sets=1)
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
        "warmup": args.warmup, "ms_per_step": round(tot_t / args.steps * 1e3, 3), "higher_is_better": True, "scaling": wl.scaling,
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


def main():
    out = OneLineStdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="a8w8", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ascb200", choices=["ascb200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the other baseline configurations at N=1")
    ap.add_argument("--allgather", action="store_true",
                    help="N>1, N-slab workloads: also time the NCCL all-gather that gives every rank all C slabs ([rank][M][N/ranks])")
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
    if world == 1 and not args.no_others and not args.kernel_only:
        others = []
        for name, cls in WORKLOADS.items():
            if name == args.workload:
                continue
            sub = argparse.Namespace(**vars(args))
            sub.steps = min(args.steps, 50)
            o = measure(ab, cls, comm, rank, world, sub, peaks, with_cpu=True, clock_index=local_rank)
            others.append({k: o[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "config", "roofline", "e2e", "cpu_baseline",
                                             "clocks", "parity_spot_check", "gpu_launches", "vs_published_other_hw") if k in o})
        line["others"] = others
    comm.close()
    if rank == 0:
        out.emit(json.dumps(line))


if __name__ == "__main__":
    main()
