#!/usr/bin/env python
"""Benchmark of the matrix-multiply path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one GEMM launch on every GPU.  The headline workload is the bf16 configuration:
M = N = K = 8192 per GPU, N(0,1) operands rounded to bf16, fp32 accumulation, bf16 output.  With N GPUs
the problem is sharded along M with B replicated (each rank owns an 8192-row shard of A and C, so the
global M is 8192 * N: weak scaling) and no collective is on the data path.

The line printed by rank 0 carries:
  value       TFLOP/s of the whole job, operands resident in HBM, CUDA events on the launch stream,
              max over ranks
  e2e         the same metric through the public API with HOST buffers: every step copies A and B from
              pinned host memory, multiplies, and copies C back
  roofline    tensor-pipe roofline of the GEMM kernel against the measured cuBLAS bf16 figure
  cpu_baseline  the CPU restatement of the reference's check loop (oracle/), timed on a row band
  configs     short legs (3 warm-up + 20 timed launches each) of the other configurations the path is specified on:
              the reference example's own f16 4096^3, f32 1024^3, FP8 block-scaled 4096 x 7168 x 7168, int8 8192^3 and
              one GPU's shard of the 2:4-sparse bf16 product, each with its own roofline fractions and its largest
              error against the CPU oracle on sampled rows (checked outside the timed region).  With N > 1 GPUs two
              more: int8 8192^3 with its M split over the ranks (strong scaling), and the sparse configuration's
              16384 rows split over the ranks followed by the all-gather of C, as a kernel plus the NCCL collective
              and as the one fused kernel.

`--impl reference` times that CPU restatement alone, as the reference arm: the reference is Rust and
cannot be built here, and its only host GEMM is the fp64 check loop of examples/matrix_benchmark.rs:36-51.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "GEMM TFLOP/s and % of B200 tensor peak (bf16/FP8/int8) at 1/2/4/8 GPUs"
# dense peaks per GPU; the 2:4-sparse product is scored in dense-equivalent flops against twice the dense bf16 figure
NOMINAL_PEAK = {"bf16": 2250.0, "f16": 2250.0, "i8": 4500.0, "e4m3": 4500.0, "f32": 1125.0, "sparse_bf16": 4500.0}
PEAK_FACTOR = {"bf16": 1.0, "f16": 1.0, "i8": 2.0, "e4m3": 2.0, "f32": 0.5, "sparse_bf16": 2.0}   # of the measured bf16 library GEMM

# name -> (operand kind, output, M per GPU, N, K)
WORKLOADS = {
    "bf16_8192": ("bf16", "bf16", 8192, 8192, 8192),
    "f16_4096_example": ("f16", "f32", 4096, 4096, 4096),
    "int8_8192": ("i8", "i32", 8192, 8192, 8192),
    "int8_shard_1024x8192x8192": ("i8", "i32", 1024, 8192, 8192),      # one GPU's share of int8_8192 split over 8
    "e4m3_unscaled_4096x7168x7168": ("e4m3", "bf16", 4096, 7168, 7168),
    "e4m3_scaled_4096x7168x7168": ("e4m3", "bf16", 4096, 7168, 7168),   # fp32 scales per 1x128 / 128x128 block
    "e4m3_mx_4096x7168x7168": ("e4m3", "bf16", 4096, 7168, 7168),       # power-of-two scales per 1x32, applied by the tensor core
    "f32_1024": ("f32", "f32", 1024, 1024, 1024),
    "f32_4096": ("f32", "f32", 4096, 4096, 4096),
    "f16_skinny_16x4096x4096": ("f16", "f32", 16, 4096, 4096),   # the reference's decode-shaped example, bias included
    "f16_skinny_16x16384x16384": ("f16", "f32", 16, 16384, 16384),   # same shape class with a weight (512 MiB) larger than L2
    "f16_grouped_16384x4096x4096_8e": ("f16", "f16", 16384, 4096, 4096),   # 16384 routed rows over 8 experts (mixture of experts)
    "sparse24_bf16_2048x8192x8192": ("bf16", "bf16", 2048, 8192, 8192),   # one GPU's shard of 16384 x 8192 (2:4) x 8192
    "sparse24_bf16_16384x8192x8192": ("bf16", "bf16", 16384, 8192, 8192),   # the whole sparse configuration on one GPU
}
DEFAULT_WORKLOAD = "bf16_8192"
# The other configurations, run as short legs after the headline workload (name -> tolerance of its check, 0 = bit-exact).
LEGS = {"f16_4096_example": 0.0, "f32_1024": 1e-4, "e4m3_scaled_4096x7168x7168": 2e-2, "int8_8192": 0.0, "sparse24_bf16_2048x8192x8192": 1e-2}
LEG_STEPS, LEG_WARMUP = 20, 3


def peak_kind(workload: str, kind: str) -> str:
    return "sparse_bf16" if workload.startswith("sparse24") else kind


def bf16_bits(values: np.ndarray) -> np.ndarray:
    bits = values.astype(np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def synthetic_operand(kind: str, rows: int, depth: int, seed: int) -> np.ndarray:
    """Seeded synthetic operand with the configuration's value distribution, as storage bits."""
    rng = np.random.default_rng(seed)
    if kind == "bf16":
        return bf16_bits(rng.standard_normal(rows * depth, dtype=np.float32))
    if kind == "f16":
        index = np.arange(rows * depth, dtype=np.int64)
        factor, modulus = (13, 31) if seed % 2 == 1 else (7, 29)  # the reference example's formulas
        return ((index * factor % modulus) / 16.0 - 1.0).astype(np.float16).view(np.uint16)
    if kind == "i8":
        return rng.integers(-128, 128, rows * depth, dtype=np.int8)
    if kind == "f32":
        return rng.uniform(-1.0, 1.0, rows * depth).astype(np.float32)
    if kind == "e4m3":
        import torch

        values = torch.from_numpy(rng.standard_normal(rows * depth, dtype=np.float32)).clamp(-448, 448)
        return values.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    raise ValueError(kind)


class ClockSampler:
    """Polls NVML (read-only) for the SM clock, the power draw and the clock-event reasons while timed regions run.
    NVML refreshes its readings every few tens of milliseconds, so a region of a few milliseconds is seen by a handful of
    samples at most; `under_load` counts the samples taken while the GPU drew more than half of its power limit."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, index: int):
        self.samples, self.loaded, self.reasons, self.max_mhz, self.power_limit = [], [], set(), None, None
        self._stop, self._thread, self._error = threading.Event(), None, None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._device = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._device, pynvml.NVML_CLOCK_SM)
            self.power_limit = pynvml.nvmlDeviceGetEnforcedPowerLimit(self._device) / 1000.0
            self._reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        except Exception as error:  # no NVML: the record says so
            self._nvml, self._error = None, repr(error)

    def _poll(self):
        nvml = self._nvml
        while not self._stop.is_set():
            try:
                clock = nvml.nvmlDeviceGetClockInfo(self._device, nvml.NVML_CLOCK_SM)
                power = nvml.nvmlDeviceGetPowerUsage(self._device) / 1000.0
                mask = self._reasons(self._device)
                self.samples.append(clock)
                if self.power_limit and power > 0.5 * self.power_limit:
                    self.loaded.append(clock)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception as error:
                self._error = repr(error)
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def record(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"], "error": self._error}
        under_load = self.loaded or self.samples
        return {"sm_mhz": float(np.median(under_load)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "samples_under_load": len(self.loaded), "sm_mhz_min": float(min(self.samples)),
                "covers": "the timed steps and the four repetitions that follow them"}


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"bf16": float(data["bf16_tflops"]), "sustained": float(data.get("bf16_tflops_sustained") or 0) or None, "hbm": float(data["hbm_gbs"]),
                "source": "measured (MEASURED_PEAKS.json: cuBLAS bf16 burst, copy bandwidth)"}
    return {"bf16": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback (earlier measurement on this pool)"}


def measured_traffic(workload: str):
    """DRAM bytes one launch of the workload's dominant kernel moves (dram__bytes_read.sum + dram__bytes_write.sum of an
    ncu capture), from the table the profile summaries keep (rows `| workload | bytes | kernel | from |`); None until that
    workload has been captured."""
    path = ROOT / "profiles" / "dram_traffic_per_launch.md"
    if not path.exists():
        return None
    for row in path.read_text().splitlines():
        cells = [cell.strip() for cell in row.strip().strip("|").split("|")]
        if len(cells) >= 2 and cells[0] == workload and cells[1].isdigit():
            return int(cells[1])
    return None


def roofline(workload: str, kind: str, tflops: float, flops: float, algorithmic_bytes: int) -> dict:
    peaks = measured_peaks()
    which = peak_kind(workload, kind)
    peak = peaks["bf16"] * PEAK_FACTOR[which]
    note = {1.0: "", 2.0: " x2 (8-bit operands, or 2:4 sparsity counted in dense-equivalent flops)", 0.5: " /2 (TF32 operands)"}[PEAK_FACTOR[which]]
    line = {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak, "traffic": measured_traffic(workload),
            "peak_source": peaks["source"] + note, "frac_of_nominal": tflops / NOMINAL_PEAK[which], "nominal_peak": NOMINAL_PEAK[which],
            "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": int(algorithmic_bytes)}
    if peaks["sustained"]:
        line["frac_of_sustained_peak"] = tflops / (peaks["sustained"] * PEAK_FACTOR[which])
    return line


# ---- CPU arm ----------------------------------------------------------------------------------------------

def cpu_threads() -> int:
    """All the cores this process may run on, whatever OMP_NUM_THREADS a launcher exported."""
    import oracle as O

    return O.set_threads(O.usable_cores())


def cpu_band(kind: str, n: int, k: int, rows: int, seed: int = 1):
    """Times the oracle's check loop on `rows` complete output rows; returns (seconds, flops, threads)."""
    import oracle as O

    fmt = {"bf16": O.FMT_BF16, "f16": O.FMT_F16, "i8": O.FMT_I8, "e4m3": O.FMT_E4M3, "f32": O.FMT_F32}[kind]
    a = synthetic_operand(kind, rows, k, seed)
    b = synthetic_operand(kind, n, k, seed + 1)
    row_list = np.arange(rows)
    start = time.perf_counter()
    if kind == "i8":
        O.matmul_rows_i8(a, b, n, k, row_list)
    else:
        O.matmul_rows(fmt, a, b, n, k, row_list)
    return time.perf_counter() - start, 2.0 * rows * n * k, O.threads()


def workload_config(workload: str, m: int, n: int, k: int, out: str, world: int, scaling: str) -> dict:
    """The `config` object: the same keys and values from both arms, so that the two lines describe one configuration."""
    kind = WORKLOADS[workload][0]
    element_bytes = {"bf16": 2, "f16": 2, "i8": 1, "e4m3": 1, "f32": 4}[kind]
    out_bytes = {"bf16": 2, "f16": 2, "f32": 4, "i32": 4}[out]
    footprint = ((m * k + n * k) * element_bytes + m * n * out_bytes) >> 20
    return {"workload": workload, "m_per_gpu": m, "global_m": m * world if scaling == "weak" else WORKLOADS[workload][2], "n": n, "k": k, "output": out,
            "operands": "A m x k and B n x k, both K-major (the reference's convention)",
            "parallelism": f"M-sharded x{world}, B replicated, no collective",
            "l2": f"inputs (A+B+C = {footprint} MB per GPU) larger than the 126 MB L2; no flush" if footprint > 126
                  else f"A+B+C = {footprint} MB per GPU fit the 126 MB L2: steps run with a warm L2, as the reference's own back-to-back protocol does"}


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference arm: the CPU restatement of the reference's host check loop, all host threads, each
    step a band of complete output rows of the same workload."""
    if rank != 0:
        return
    kind, out, m, n, k = WORKLOADS[args.workload]
    cpu_threads()
    seconds, flops, threads = cpu_band(kind, n, k, 8)            # calibration, untimed
    rate = flops / seconds
    budget = 150.0                                               # seconds for warm-up + timed steps
    rows = int(max(1, min(m, budget * rate / (2.0 * n * k) / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        cpu_band(kind, n, k, rows)
    total_seconds, total_flops = 0.0, 0.0
    for _ in range(args.steps):
        seconds, flops, threads = cpu_band(kind, n, k, rows)
        total_seconds += seconds
        total_flops += flops
    value = total_flops / total_seconds / 1e12
    sample = f"{rows} complete output rows x N={n} x K={k} per step (of M={m}); fp64 accumulate, k ascending"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total_seconds / max(1, args.steps), "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": kind, "data": "synthetic",
        "config": workload_config(args.workload, m, n, k, out, world, args.scaling),
        "note": "CPU restatement of examples/matrix_benchmark.rs:36-51 (the reference is Rust: no toolchain here), timed on rank 0's host cores",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------------------------

class Prepared:
    """One workload set up on one GPU: operands resident, `launch()` enqueues one step, `check()` compares sampled rows of
    the result with the CPU oracle and returns the largest |d| / max(|ref|, 1)."""

    def __init__(self, G, gpu, stream, workload: str, m: int, rank: int, options, quick_check_rows: int = 4):
        import oracle as O

        kind, out, _, n, k = WORKLOADS[workload]
        self.G, self.gpu, self.stream, self.workload, self.kind, self.out, self.m, self.n, self.k = G, gpu, stream, workload, kind, out, m, n, k
        self.element = {"bf16": G.BF16, "f16": G.F16, "i8": G.I8, "e4m3": G.E4M3, "f32": G.F32}[kind]
        self.out_element = {"bf16": G.BF16, "f16": G.F16, "f32": G.F32, "i32": G.I32}[out]
        self.element_bytes, self.out_bytes = G.host.ELEMENT_BYTES[self.element], G.host.ELEMENT_BYTES[self.out_element]
        self.options = options
        self.shape = [m, n, k]
        self.flops = 2.0 * m * n * k
        self.oracle_scales = (None, None)
        self.dense_for_oracle = None
        fmt = {"bf16": O.FMT_BF16, "f16": O.FMT_F16, "i8": O.FMT_I8, "e4m3": O.FMT_E4M3, "f32": O.FMT_F32}[kind]
        self.fmt = fmt
        scaled = "scaled" in workload and "unscaled" not in workload
        if scaled:
            # the configuration as stated: N(0,1) fp32 sources quantised per 1 x 128 (A) and 128 x 128 (B) block, scale =
            # absmax / 448, by the device quantiser (bit-equal to the oracle's, tests/test_quantize_gpu.py)
            rng = np.random.default_rng(1 + 2 * rank)
            source_a = gpu.upload(rng.standard_normal(m * k, dtype=np.float32))
            source_b = gpu.upload(np.random.default_rng(2).standard_normal(n * k, dtype=np.float32))
            self.a, options.scale_a = G.quantize_e4m3(stream, source_a, m, k, 1)
            self.b, options.scale_b = G.quantize_e4m3(stream, source_b, n, k, 128)
            stream.synchronize()
            del source_a, source_b
            self.a_host, self.b_host = self.a.download(), self.b.download()
            self.oracle_scales = (options.scale_a.download(), options.scale_b.download())
        else:
            # A: this rank's M-shard (its own seed); B: replicated (same seed on every rank).
            self.a_host = synthetic_operand(kind, m, k, 1 + 2 * rank)
            self.b_host = synthetic_operand(kind, n, k, 2)
            self.a, self.b = gpu.upload(self.a_host, self.element), gpu.upload(self.b_host, self.element)
        self.c = gpu.allocate(self.out_element, m * n)
        if "skinny" in workload:
            self.bias_host = (np.arange(n) / 64.0).astype(np.float32)
            options.bias = gpu.upload(self.bias_host)
        if workload.startswith("sparse24"):
            # A becomes 2:4: zero two elements of every group of four (seeded choice), then compress on the device
            rng = np.random.default_rng(5 + rank)
            pairs = np.array([[0, 1], [0, 2], [0, 3], [1, 2], [1, 3], [2, 3]])[rng.integers(0, 6, m * k // 4)]
            groups = self.a_host.reshape(-1, 4).copy()
            keep = np.zeros(groups.shape, bool)
            keep[np.arange(len(groups))[:, None], pairs] = True
            groups[~keep] = 0
            self.dense_for_oracle = groups.reshape(-1)
            dense = gpu.upload(self.dense_for_oracle, self.element)
            self.a, options.metadata, violations = G.compress_24(stream, dense, m, k)
            stream.synchronize()
            assert violations.download()[0] == 0
            del dense
            self.a_host = self.a.download()     # the end-to-end leg copies the compressed operand (its metadata stays resident)
        if "_mx_" in workload:
            # synthetic exponents around the one N(0,1) groups of 32 get (absmax about 2.1: 2^-7 brings it under 448)
            rng = np.random.default_rng(99)
            lib_ = gpu._lib
            options.scale_a = gpu.upload(rng.integers(119, 122, lib_.gpurs_mx_scale_bytes(m, k, 0)).astype(np.int8), G.I8)
            options.scale_b = gpu.upload(rng.integers(119, 122, lib_.gpurs_mx_scale_bytes(n, k, 1)).astype(np.int8), G.I8)
            options.scale_kind = G.SCALES_MX
        self.launch = lambda: G.matmul(stream, self.a, self.b, self.c, self.shape, options)
        self.grouped = "grouped" in workload
        if self.grouped:
            # m routed rows over 8 experts of uneven size; activations = m rows, routing a seeded permutation; B holds the 8 weights
            experts = 8
            rng = np.random.default_rng(11)
            counts = rng.multinomial(m, np.ones(experts) / experts)
            offsets = gpu.upload(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))
            routes = gpu.upload(rng.permutation(m).astype(np.int32))
            self.b_host = synthetic_operand(kind, experts * n, k, 2)
            self.b = gpu.upload(self.b_host, self.element)
            self.launch = lambda: G.matmul_grouped(stream, self.a, routes, offsets, self.b, self.c, m, m, n, k, experts)
        self.algorithmic_bytes = int(self.a_host.nbytes + self.b_host.nbytes + m * n * self.out_bytes +
                                     (options.metadata.nbytes if options.metadata is not None else 0) +
                                     sum(s.nbytes for s in (options.scale_a, options.scale_b) if s is not None))
        self.check_rows = quick_check_rows

    def check(self):
        """Largest |d| / max(|ref|, 1) over a few complete output rows spread over the matrix, against the CPU oracle;
        None for the workloads the bench has no oracle for (mixture-of-experts routing, synthetic MX exponents)."""
        import oracle as O

        if self.grouped or "_mx_" in self.workload:
            return None
        m, n, k = self.m, self.n, self.k
        rows = np.unique(np.linspace(0, m - 1, self.check_rows).astype(np.int64))
        got = self.c.download().reshape(m, n)[rows]
        if self.out == "bf16":
            got = O.bf16_to_f32(got.reshape(-1)).reshape(len(rows), n)
        elif self.out == "f16":
            got = O.f16_to_f32(got.reshape(-1)).reshape(len(rows), n)
        got = got.astype(np.float64)
        if self.kind == "i8":
            expected = O.matmul_rows_i8(self.a_host, self.b_host, n, k, rows).astype(np.float64)
        elif self.dense_for_oracle is not None:
            expected = O.matmul_rows(self.fmt, self.dense_for_oracle, self.b_host, n, k, rows)
        else:
            expected = O.matmul_rows(self.fmt, self.a_host, self.b_host, n, k, rows, *self.oracle_scales)
        if "skinny" in self.workload:
            expected = expected + self.bias_host[None, :].astype(np.float64)
        error = np.abs(got - expected) / np.maximum(np.abs(expected), 1.0)
        return float(np.where(np.isnan(error), np.inf, error).max())

    def timed(self, steps: int) -> float:
        """Milliseconds for `steps` back-to-back launches, CUDA events on the launch stream."""
        start = self.stream.record_timed()
        for _ in range(steps):
            self.launch()
        end = self.stream.record_timed()
        self.stream.synchronize()
        return start.elapsed_ms(end)


def max_over_ranks(dist, value: float) -> float:
    if dist is None:
        return value
    import torch

    worst = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return float(worst.item())


def run_leg(G, gpu, stream, dist, workload: str, m: int, rank: int, world: int, whole_job_flops: float, tolerance: float) -> dict:
    """A short leg of one configuration: LEG_WARMUP + LEG_STEPS launches, then the check against the oracle."""
    kind, out, _, n, k = WORKLOADS[workload]
    prepared = Prepared(G, gpu, stream, workload, m, rank, G.MatmulOptions())
    for _ in range(LEG_WARMUP):
        prepared.launch()
    stream.synchronize()
    if dist is not None:
        dist.barrier()
    launches = gpu.launches
    ms_per_step = max_over_ranks(dist, prepared.timed(LEG_STEPS)) / LEG_STEPS
    launches = (gpu.launches - launches) // LEG_STEPS
    error = prepared.check()
    error = max_over_ranks(dist, error if error is not None else 0.0) if error is not None else None
    tflops = whole_job_flops / (ms_per_step * 1e-3) / 1e12
    per_gpu = tflops / world
    baseline = None
    if workload == "f16_4096_example" and rank == 0:
        baseline = reference_design_leg(gpu, stream, prepared)
    leg = {"value": tflops, "unit": "TFLOP/s" if kind != "i8" else "TOP/s", "ms_per_step": ms_per_step, "steps": LEG_STEPS, "warmup": LEG_WARMUP,
           "m_per_gpu": m, "n": n, "k": k, "dtype": kind, "output": out, "launches_per_step": int(launches),
           "roofline": roofline(workload, kind, per_gpu, prepared.flops, prepared.algorithmic_bytes),
           "max_error_vs_oracle": error, "tolerance": tolerance, "check": f"{prepared.check_rows} complete output rows against the CPU oracle, |d| / max(|ref|, 1)",
           "passed": (error is not None and error <= tolerance)}
    if baseline is not None:
        baseline["product_over_reference_design"] = baseline["ms_per_step"] / ms_per_step if baseline.get("ms_per_step") else None
        leg["reference_design"] = baseline
    return leg, prepared


def reference_design_leg(gpu, stream, prepared: Prepared) -> dict:
    """The reference's own sm_100a kernel DESIGN (one CTA per 128 x 256 tile, one thread issuing copies and products, one
    accumulator, 8-byte stores: examples/blackwell/examples/blackwell_matrix.rs:32-56), restated in CUDA under oracle/ as test
    infrastructure and timed on the same GPU, same inputs, same protocol as the leg beside it.  Not the reference's binary
    (that is Rust compiled by its own toolchain), and no part of the product."""
    try:
        import oracle as O
        from oracle.reference_design import ReferenceDesign

        design = ReferenceDesign(gpu)
    except Exception as error:      # the image is built only where nvcc is installed
        return {"unavailable": repr(error)}
    G = prepared.G
    m, n, k = prepared.shape
    c = gpu.allocate(G.F32, m * n)
    launch = design.prepare(prepared.a, prepared.b, c, m, n, k)
    for _ in range(LEG_WARMUP):
        design.launch(stream, launch)
    stream.synchronize()
    start = stream.record_timed()
    for _ in range(LEG_STEPS):
        design.launch(stream, launch)
    end = stream.record_timed()
    stream.synchronize()
    ms_per_step = start.elapsed_ms(end) / LEG_STEPS
    rows = np.unique(np.linspace(0, m - 1, 4).astype(np.int64))
    exact = bool(np.array_equal(c.download().reshape(m, n)[rows].astype(np.float64), O.matmul_rows(prepared.fmt, prepared.a_host, prepared.b_host, n, k, rows)))
    return {"ms_per_step": ms_per_step, "value": prepared.flops / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s", "bit_exact_vs_oracle": exact,
            "status": [int(x) for x in design.status.download()],
            "what": "CUDA restatement of the reference example's kernel design (128 x 256 x 64 tiles, 4-stage ring, single issuing thread, one accumulator), bounded waits"}


def gather_leg(G, gpu, stream, dist, prepared: Prepared, rank: int, world: int, steps: int) -> dict:
    """The product followed by the all-gather of C, two ways: the kernel and then the NCCL collective (through the C ABI,
    in place, same stream), and the one fused kernel whose epilogue stores every box to all GPUs' copies.  Every rank's
    fused result is compared bit for bit with what the collective gathered."""
    import torch
    from gpurs_b200.sharding import allgather_objects, broadcast_from_rank0

    m, n, k = prepared.shape
    shard_bytes = m * n * prepared.out_bytes
    flops = prepared.flops
    full = gpu.zeros(prepared.out_element, world * m * n)
    mine = full.slice(rank * m * n, (rank + 1) * m * n)
    comm = G.Communicator(gpu, rank, world, broadcast_from_rank0(dist))

    def collective_step():
        G.matmul(stream, prepared.a, prepared.b, mine, prepared.shape, prepared.options)
        comm.allgather(stream, full, shard_bytes)

    def timed(step):
        for _ in range(3):
            step()
        stream.synchronize()
        dist.barrier()
        start = stream.record_timed()
        for _ in range(steps):
            step()
        end = stream.record_timed()
        stream.synchronize()
        elapsed = max_over_ranks(dist, start.elapsed_ms(end)) / steps
        dist.barrier()
        return elapsed

    collective_ms = timed(collective_step)
    gathered_by_nccl = full.download().view(np.uint8)
    result = {"gemm_then_nccl": {"ms_per_step": collective_ms, "value": world * flops / (collective_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                 "bytes_received_per_gpu": int((world - 1) * shard_bytes),
                                 "how": "gpurs_matmul then gpurs_comm_allgather (ncclAllGather, in place) on the same stream"}}
    gathered = G.GatheredMatrix(gpu, prepared.out_element, world * m, n, rank, world, allgather_objects(dist))
    fused_ms = timed(lambda: G.matmul_allgather(stream, prepared.a, prepared.b, gathered, prepared.shape, rank * m, prepared.options))
    same = bool(np.array_equal(gathered.local.download().view(np.uint8), gathered_by_nccl))
    agree = torch.tensor([1 if same else 0], device="cuda")
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    link_bound_ms = (world - 1) * shard_bytes / 770e9 * 1e3        # measured peer bandwidth of this pool, per direction
    result["fused"] = {"ms_per_step": fused_ms, "value": world * flops / (fused_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "bytes_sent_per_gpu": int((world - 1) * shard_bytes), "equals_collective_result": bool(agree.item()),
                       "link_bound_ms": link_bound_ms, "how": "gpurs_matmul_allgather: one kernel per GPU, remote TMA stores from the epilogue"}
    # third way: bands of rows multiplied by the plain kernels, every finished band sent by the copy engines while the next is
    # multiplied.  The gathered matrix is overwritten first, so that the comparison below sees this form's own output.
    dist.barrier()
    gpu._lib.gpurs_fill_u8(stream._handle, gathered.local.pointer, 0x7F, gathered.local.nbytes)
    stream.synchronize()
    dist.barrier()
    import dataclasses
    by_copies = dataclasses.replace(prepared.options, algorithm=prepared.options.algorithm | G.ALGO_GATHER_BY_COPIES)
    copies_ms = timed(lambda: G.matmul_allgather(stream, prepared.a, prepared.b, gathered, prepared.shape, rank * m, by_copies))
    same = bool(np.array_equal(gathered.local.download().view(np.uint8), gathered_by_nccl))
    agree = torch.tensor([1 if same else 0], device="cuda")
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    result["copy_engines"] = {"ms_per_step": copies_ms, "value": world * flops / (copies_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                              "bytes_sent_per_gpu": int((world - 1) * shard_bytes), "equals_collective_result": bool(agree.item()),
                              "link_bound_ms": link_bound_ms,
                              "how": "gpurs_matmul_allgather with GPURS_ALGO_GATHER_BY_COPIES: the block in bands of rows, each sent to every peer by "
                                     "the copy engines (one stream per peer) while the next band is multiplied"}
    dist.barrier()
    gathered.close()
    comm.close()
    return result


def run_gpu_arm(args, rank: int, local_rank: int, world: int) -> None:
    import gpurs_b200 as G

    kind, out, m, n, k = WORKLOADS[args.workload]
    if args.scaling == "strong":
        from gpurs_b200.sharding import row_shard

        m = row_shard(m, world, rank)[1]     # the workload's M split over the ranks, B still replicated

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    gpu = G.Gpu(local_rank)
    stream = gpu.stream()
    options = G.MatmulOptions(algorithm=args.algorithm | (G.ALGO_WHOLE_TILES if args.whole_tiles else 0), raster_rows=args.raster_rows,
                              l2_policy=args.l2_policy)
    prepared = Prepared(G, gpu, stream, args.workload, m, rank, options)
    launch, a, b, c = prepared.launch, prepared.a, prepared.b, prepared.c
    a_host, b_host, out_bytes, shape = prepared.a_host, prepared.b_host, prepared.out_bytes, prepared.shape

    def barrier():
        stream.synchronize()
        if dist is not None:
            dist.barrier()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        launch()
    barrier()
    launches_before = gpu.launches
    with ClockSampler(local_rank) as clocks:
        milliseconds = prepared.timed(args.steps)
        launches = gpu.launches - launches_before
        milliseconds = max_over_ranks(dist, milliseconds)
        if dist is not None:
            dist.barrier()
        flops_per_step = prepared.flops
        ms_per_step = milliseconds / args.steps
        per_gpu_tflops = flops_per_step / (ms_per_step * 1e-3) / 1e12
        value = per_gpu_tflops * world
        # Four more repetitions of the same K steps (this rank's own times), reported beside `value`, which stays the first.
        repetitions = [ms_per_step]
        for _ in range(4):
            repetitions.append(prepared.timed(args.steps) / args.steps)
    headline_error = prepared.check()

    # ---- end to end through the public API with host buffers ------------------------------------
    e2e_steps = max(1, min(args.steps, 8))
    lib = gpu._lib
    import ctypes as C

    pinned = []
    for nbytes in (a_host.nbytes, b_host.nbytes, m * n * out_bytes):
        pointer = C.c_void_p()
        assert lib.gpurs_host_alloc(gpu._handle, nbytes, C.byref(pointer)) == 0
        pinned.append(pointer)
    C.memmove(pinned[0], a_host.ctypes.data, a_host.nbytes)
    C.memmove(pinned[1], b_host.ctypes.data, b_host.nbytes)

    # Dense products go through the host-buffer entry point, which overlaps copy in, product and copy out by blocks of
    # rows; the grouped and the sparse product (operands prepared on the device) copy, launch and copy back in order.
    host_call = "grouped" not in args.workload and not args.workload.startswith("sparse24") and "_mx_" not in args.workload

    def e2e_step():
        if host_call:
            G.matmul_host(stream, pinned[0].value, pinned[1].value, pinned[2].value, a, b, c, shape, options)
            return
        stream.copy_to_device(a, pinned[0].value, a_host.nbytes)
        stream.copy_to_device(b, pinned[1].value, b_host.nbytes)
        launch()
        stream.copy_to_host(pinned[2].value, c, m * n * out_bytes)

    e2e_step()
    barrier()
    start = stream.record_timed()
    for _ in range(e2e_steps):
        e2e_step()
    end = stream.record_timed()
    stream.synchronize()
    e2e_own_ms = start.elapsed_ms(end)
    e2e_ms = max_over_ranks(dist, e2e_own_ms)
    e2e_value = world * flops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
    checksum = int(np.frombuffer(C.string_at(pinned[2], 64), np.uint8).sum())  # the result really arrived on the host
    # what the host link alone allows: the same bytes each way, copies only, both directions at once (this rank)
    link = None
    if host_call:
        copy_in, copy_out = gpu.stream(), gpu.stream()
        def copies():
            copy_in.copy_to_device(a, pinned[0].value, a_host.nbytes)
            copy_in.copy_to_device(b, pinned[1].value, b_host.nbytes)
            copy_out.copy_to_host(pinned[2].value, c, m * n * out_bytes)
        copies()
        copy_in.synchronize(), copy_out.synchronize()
        barrier()
        begin = time.perf_counter()
        for _ in range(2):
            copies()
        copy_in.synchronize(), copy_out.synchronize()
        copies_ms = max_over_ranks(dist, (time.perf_counter() - begin) * 1e3 / 2)
        link = {"copies_only_ms_per_step": copies_ms, "h2d_gbs": (a_host.nbytes + b_host.nbytes) / copies_ms / 1e6,
                "frac_of_copies_only": copies_ms / (e2e_ms / e2e_steps),
                "what": "the step's copies alone (H2D of A and B on one stream, D2H of C on another, no product), max over ranks: the floor the host link sets"}
        del copy_in, copy_out
    for pointer in pinned:
        lib.gpurs_host_free(gpu._handle, pointer)

    # ---- optional: the headline GEMM followed by the all-gather of its C blocks ----------------------------------
    gather = None
    dense_tiles = not any(word in args.workload for word in ("grouped", "skinny", "e4m3_scaled", "_mx_", "f32"))
    if dist is not None and args.allgather and dense_tiles:
        gather = gather_leg(G, gpu, stream, dist, prepared, rank, world, args.steps)
    # Single launches with idle gaps, best of 10: the protocol of the burst figure in MEASURED_PEAKS.json (the timed region
    # above is K back-to-back launches, which run into the power cap like that file's sustained figure when K is large).
    isolated = []
    for _ in range(10):
        time.sleep(0.02)
        isolated.append(prepared.timed(1))
    burst_tflops = flops_per_step / (min(isolated) * 1e-3) / 1e12
    status = gpu.status()
    algorithmic_bytes = prepared.algorithmic_bytes
    del prepared, launch, a, b, c

    # ---- the other configurations, as short legs --------------------------------------------------------------------
    configs = {}
    if args.workload == DEFAULT_WORKLOAD and not args.no_legs:
        for workload, tolerance in LEGS.items():
            leg_m = WORKLOADS[workload][2]
            leg, leg_prepared = run_leg(G, gpu, stream, dist, workload, leg_m, rank, world, world * 2.0 * leg_m * WORKLOADS[workload][3] * WORKLOADS[workload][4], tolerance)
            leg["scaling"] = "weak"
            configs[workload] = leg
            del leg_prepared
        if dist is not None:
            from gpurs_b200.sharding import equal_shards, row_shard

            # int8 8192^3 with its M split over the ranks: the whole job is the one product, whatever the rank count
            _, _, whole_m, n8, k8 = WORKLOADS["int8_8192"]
            leg, leg_prepared = run_leg(G, gpu, stream, dist, "int8_8192", row_shard(whole_m, world, rank)[1], rank, world, 2.0 * whole_m * n8 * k8, 0.0)
            leg["scaling"] = "strong"
            leg["what"] = f"M = {whole_m} split over {world} GPUs, B replicated; value is the whole product's rate"
            configs["int8_8192_strong"] = leg
            del leg_prepared
            # the sparse configuration: 16384 rows split over the ranks, then every GPU receives all of C
            _, _, whole_m, ns, ks = WORKLOADS["sparse24_bf16_16384x8192x8192"]
            if equal_shards(whole_m, world):
                leg, leg_prepared = run_leg(G, gpu, stream, dist, "sparse24_bf16_16384x8192x8192", whole_m // world, rank, world, 2.0 * whole_m * ns * ks, 1e-2)
                leg["scaling"] = "strong"
                leg["what"] = f"M = {whole_m} (2:4 sparse A) split over {world} GPUs, B replicated; value counts dense-equivalent flops of the whole product"
                leg["allgather"] = gather_leg(G, gpu, stream, dist, leg_prepared, rank, world, LEG_STEPS)
                configs["sparse24_bf16_16384x8192x8192_allgather"] = leg
                del leg_prepared

    if rank == 0:
        sustained = measured_peaks()["sustained"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": kind, "data": "synthetic",
            "config": workload_config(args.workload, m, n, k, out, world, args.scaling),
            "options": {"algorithm": args.algorithm, "whole_tiles": args.whole_tiles, "raster_rows": args.raster_rows, "l2_policy": args.l2_policy},
            "clocks": clocks.record(),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(a_host.nbytes + b_host.nbytes),
                    "d2h_bytes_per_step": int(m * n * out_bytes), "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "host_checksum": checksum,
                    "call": "gpurs_matmul_host: pinned host buffers, copies and product overlapped by blocks of rows" if host_call
                            else "copy_to_device x2, product, copy_to_host on one stream",
                    "host_link": link},
            "gpu_launches": int(launches),
            "max_error_vs_oracle": headline_error,
            "repetitions": {"ms_per_step": [round(x, 6) for x in repetitions], "best": min(repetitions), "median": sorted(repetitions)[len(repetitions) // 2],
                            "note": "five times K back-to-back steps on rank 0; `value` and `ms_per_step` are the first (max over ranks)"},
            "roofline": roofline(args.workload, kind, per_gpu_tflops, flops_per_step, algorithmic_bytes),
            "device_status": status,
        }
        line["roofline"]["single_launch"] = {"achieved": burst_tflops, "ms": min(isolated), "frac": burst_tflops / line["roofline"]["peak"],
                                             "protocol": "best of 10 single launches 20 ms apart (the burst protocol of the peak)"}
        if gather is not None:
            line["allgather"] = gather
        if configs:
            line["configs"] = configs
        if "skinny" in args.workload:
            # bound by streaming B once from HBM: report the roofline against the measured copy bandwidth
            peaks = measured_peaks()
            achieved = algorithmic_bytes / (ms_per_step * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                                "traffic": measured_traffic(args.workload), "peak_source": peaks["source"], "algorithmic_bytes_per_launch": int(algorithmic_bytes)}
        if world == 1 and not args.no_cpu_baseline:
            cpu_threads()
            seconds, flops, threads = cpu_band(kind, n, k, 64)          # calibration
            rows = int(max(64, min(m, 20.0 * flops / seconds / (2.0 * n * k))))     # about 20 s of CPU work
            seconds, flops, threads = cpu_band(kind, n, k, rows)
            line["cpu_baseline"] = {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{rows} complete output rows x N={n} x K={k} of the same workload, {seconds:.1f} s"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    gpu.close()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20, help="timed launches; 20 is a burst of about 15 ms, 100 or more settle at the power cap's clock")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    parser.add_argument("--algorithm", type=int, default=0, help="0 auto, 1 single-CTA tiles, 2 CTA-pair tiles")
    parser.add_argument("--whole-tiles", action="store_true", help="never split the last round's tiles along K (no stream-K)")
    parser.add_argument("--raster-rows", type=int, default=0, help="tile rows walked together (0 = library default)")
    parser.add_argument("--l2-policy", type=int, default=0, help="0 default, 1 keep A / stream B, 2 stream A / keep B, 3 keep both, 4 none")
    parser.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                        help="weak: every GPU multiplies a full-size shard (global M grows); strong: the workload's M is split")
    parser.add_argument("--allgather", action="store_true", help="also time the headline GEMM + all-gather of C (N > 1), collective and fused")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-legs", action="store_true", help="skip the short legs of the other configurations")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
    else:
        run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
