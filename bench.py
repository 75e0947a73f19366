#!/usr/bin/env python
"""Benchmark of the matrix-multiply path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one GEMM launch on every GPU.  The default workload is the bf16 configuration:
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
NOMINAL_PEAK = {"bf16": 2250.0, "f16": 2250.0, "i8": 4500.0, "e4m3": 4500.0, "f32": 1125.0}

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
}
DEFAULT_WORKLOAD = "bf16_8192"

# DRAM bytes moved by one launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from
# an ncu capture, see profiles/); None until a capture of that workload has been taken.
MEASURED_TRAFFIC = {"bf16_8192": 1_156_000_000}   # profiles/gemm_bf16_bf16_cg2_8192.md, second capture: 1.024 GB read + 132 MB written


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
    """Polls NVML (read-only) for the SM clock and the throttle reasons while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop, self._thread = [], set(), None, threading.Event(), None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._device = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._device, pynvml.NVML_CLOCK_SM)
        except Exception:  # no NVML: the record says so
            self._nvml = None

    def _poll(self):
        nvml = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(self._device, nvml.NVML_CLOCK_SM))
                mask = nvml.nvmlDeviceGetCurrentClocksEventReasons(self._device)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def measured_peak_tflops() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, cuBLAS burst)"
    return 1590.0, "fallback (earlier measurement on this pool)"


def sustained_peak_tflops(kind: str):
    """The seconds-long cuBLAS bf16 figure of MEASURED_PEAKS.json, scaled like the burst one (x2 for 8-bit, /2 for TF32)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if not path.exists():
        return None
    value = json.loads(path.read_text()).get("bf16_tflops_sustained")
    if not value:
        return None
    return float(value) * (2.0 if kind in ("i8", "e4m3") else 0.5 if kind == "f32" else 1.0)


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


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference arm: the CPU restatement of the reference's host check loop, all host threads, each
    step a band of complete output rows of the same workload."""
    if rank != 0:
        return
    kind, out, m, n, k = WORKLOADS[args.workload]
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
        "ms_per_step": 1e3 * total_seconds / max(1, args.steps), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": kind, "data": "synthetic",
        "config": {"workload": args.workload, "m_per_gpu": m, "n": n, "k": k, "note": "CPU restatement of examples/matrix_benchmark.rs:36-51 (the reference is Rust: no toolchain here)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_gpu_arm(args, rank: int, local_rank: int, world: int) -> None:
    import gpurs_b200 as G

    kind, out, m, n, k = WORKLOADS[args.workload]
    if args.scaling == "strong":
        from gpurs_b200.sharding import row_shard

        m = row_shard(m, world, rank)[1]     # the workload's M split over the ranks, B still replicated
    element = {"bf16": G.BF16, "f16": G.F16, "i8": G.I8, "e4m3": G.E4M3, "f32": G.F32}[kind]
    out_element = {"bf16": G.BF16, "f16": G.F16, "f32": G.F32, "i32": G.I32}[out]
    element_bytes, out_bytes = G.host.ELEMENT_BYTES[element], G.host.ELEMENT_BYTES[out_element]

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    gpu = G.Gpu(local_rank)
    stream = gpu.stream()
    # A: this rank's M-shard (its own seed); B: replicated (same seed on every rank).
    a_host = synthetic_operand(kind, m, k, 1 + 2 * rank)
    b_host = synthetic_operand(kind, n, k, 2)
    a, b = gpu.upload(a_host, element), gpu.upload(b_host, element)
    c = gpu.allocate(out_element, m * n)
    shape = [m, n, k]
    options = G.MatmulOptions(algorithm=args.algorithm | (G.ALGO_WHOLE_TILES if args.whole_tiles else 0), raster_rows=args.raster_rows,
                              l2_policy=args.l2_policy)
    if "skinny" in args.workload:
        options.bias = gpu.upload((np.arange(n) / 64.0).astype(np.float32))
    if args.workload.startswith("sparse24"):
        # A becomes 2:4: zero two elements of every group of four (seeded choice), then compress on the device
        rng = np.random.default_rng(5 + rank)
        pairs = np.array([[0, 1], [0, 2], [0, 3], [1, 2], [1, 3], [2, 3]])[rng.integers(0, 6, m * k // 4)]
        groups = a_host.reshape(-1, 4).copy()
        keep = np.zeros(groups.shape, bool)
        keep[np.arange(len(groups))[:, None], pairs] = True
        groups[~keep] = 0
        dense = gpu.upload(groups.reshape(-1), element)
        a, options.metadata, violations = G.compress_24(stream, dense, m, k)
        stream.synchronize()
        assert violations.download()[0] == 0
        del dense
        a_host = a.download()     # the end-to-end leg copies the compressed operand (its metadata stays resident)
    if "_mx_" in args.workload:
        # synthetic exponents around the one N(0,1) groups of 32 get (absmax about 2.1: 2^-7 brings it under 448)
        rng = np.random.default_rng(99)
        lib_ = gpu._lib
        options.scale_a = gpu.upload(rng.integers(119, 122, lib_.gpurs_mx_scale_bytes(m, k, 0)).astype(np.int8), G.I8)
        options.scale_b = gpu.upload(rng.integers(119, 122, lib_.gpurs_mx_scale_bytes(n, k, 1)).astype(np.int8), G.I8)
        options.scale_kind = G.SCALES_MX
    if "scaled" in args.workload and "unscaled" not in args.workload:
        # synthetic scales with the magnitude absmax/448 has for N(0,1) blocks
        rng = np.random.default_rng(99)
        k_blocks = (k + 127) // 128
        options.scale_a = gpu.upload(rng.uniform(3.0, 4.5, m * k_blocks).astype(np.float32) / np.float32(448.0))
        options.scale_b = gpu.upload(rng.uniform(4.0, 5.0, ((n + 127) // 128) * k_blocks).astype(np.float32) / np.float32(448.0))

    launch = lambda: G.matmul(stream, a, b, c, shape, options)
    if "grouped" in args.workload:
        # m routed rows over 8 experts of uneven size; activations = m rows, routing a seeded permutation; B holds the 8 weights
        experts = 8
        rng = np.random.default_rng(11)
        counts = rng.multinomial(m, np.ones(experts) / experts)
        offsets = gpu.upload(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))
        routes = gpu.upload(rng.permutation(m).astype(np.int32))
        b_host = synthetic_operand(kind, experts * n, k, 2)
        b = gpu.upload(b_host, element)
        launch = lambda: G.matmul_grouped(stream, a, routes, offsets, b, c, m, m, n, k, experts)

    def barrier():
        stream.synchronize()
        if dist is not None:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        launch()
    barrier()
    launches_before = gpu.launches
    with ClockSampler(local_rank) as clocks:
        start = stream.record_timed()
        for _ in range(args.steps):
            launch()
        end = stream.record_timed()
        stream.synchronize()
    milliseconds = start.elapsed_ms(end)
    launches = gpu.launches - launches_before
    if dist is not None:
        import torch

        worst = torch.tensor([milliseconds], device="cuda")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        milliseconds = float(worst.item())
        dist.barrier()
    flops_per_step = 2.0 * m * n * k
    ms_per_step = milliseconds / args.steps
    per_gpu_tflops = flops_per_step / (ms_per_step * 1e-3) / 1e12
    value = per_gpu_tflops * world
    # Four more repetitions of the same K steps (this rank's own times), reported beside `value`, which stays the first.
    repetitions = [ms_per_step]
    for _ in range(4):
        first = stream.record_timed()
        for _ in range(args.steps):
            launch()
        last = stream.record_timed()
        stream.synchronize()
        repetitions.append(first.elapsed_ms(last) / args.steps)

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
    e2e_ms = start.elapsed_ms(end)
    if dist is not None:
        import torch

        worst = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        e2e_ms = float(worst.item())
    e2e_value = world * flops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
    checksum = int(np.frombuffer(C.string_at(pinned[2], 64), np.uint8).sum())  # the result really arrived on the host
    for pointer in pinned:
        lib.gpurs_host_free(gpu._handle, pointer)

    # ---- optional: GEMM followed by the all-gather of the C blocks (NCCL), reported beside `value` ----
    gather = None
    if dist is not None and args.allgather:
        import torch

        shard_bytes = m * n * out_bytes
        full = torch.empty(world * shard_bytes, dtype=torch.uint8, device="cuda")
        mine = full[rank * shard_bytes:(rank + 1) * shard_bytes]
        c_block = gpu.import_allocation(full.data_ptr() + rank * shard_bytes, m * n, out_element)
        torch_stream = torch.cuda.current_stream()
        borrowed = gpu.borrow_stream(torch_stream.cuda_stream)

        def gather_step():
            G.matmul(borrowed, a, b, c_block, shape, options)
            dist.all_gather_into_tensor(full, mine)      # in place: block r of `full` is rank r's C

        for _ in range(3):
            gather_step()
        torch.cuda.synchronize()
        dist.barrier()
        begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(torch_stream)
        for _ in range(args.steps):
            gather_step()
        finish.record(torch_stream)
        torch.cuda.synchronize()
        worst = torch.tensor([begin.elapsed_time(finish)], device="cuda")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        gather_ms = float(worst.item()) / args.steps
        gather = {"ms_per_step": gather_ms, "value": world * flops_per_step / (gather_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                  "bytes_received_per_gpu": int((world - 1) * shard_bytes), "collective": "ncclAllGather, in place, after the GEMM on the same stream"}
        # The same result from ONE kernel per GPU: the epilogue stores every box of C into all GPUs' copies over NVLink.
        dense_tiles = not any(word in args.workload for word in ("grouped", "skinny", "e4m3_scaled", "_mx_"))     # 2:4 sparse bf16 has a push kernel too
        if dense_tiles and (kind, out) in (("bf16", "bf16"), ("i8", "i32"), ("f16", "f32"), ("e4m3", "bf16")):
            def exchange(handle):
                handles = [None] * world
                dist.all_gather_object(handles, handle)
                return handles

            gathered = G.GatheredMatrix(gpu, out_element, world * m, n, rank, world, exchange)
            fused_step = lambda: G.matmul_allgather(stream, a, b, gathered, shape, rank * m, options)
            for _ in range(3):
                fused_step()
            barrier()
            start = stream.record_timed()
            for _ in range(args.steps):
                fused_step()
            end = stream.record_timed()
            stream.synchronize()
            worst = torch.tensor([start.elapsed_ms(end)], device="cuda")
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            dist.barrier()
            fused_ms = float(worst.item()) / args.steps
            # every rank's copy must equal what the collective gathered, bit for bit
            same = bool(np.array_equal(gathered.local.download().view(np.uint8), full.cpu().numpy()))
            agree = torch.tensor([1 if same else 0], device="cuda")
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            gather["fused"] = {"ms_per_step": fused_ms, "value": world * flops_per_step / (fused_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "bytes_sent_per_gpu": int((world - 1) * shard_bytes), "equals_collective_result": bool(agree.item()),
                               "how": "gpurs_matmul_allgather: one kernel per GPU, remote TMA stores from the epilogue"}
            dist.barrier()
            gathered.close()
        del c_block, borrowed
    # Single launches with idle gaps, best of 10: the protocol of the burst figure in MEASURED_PEAKS.json (the timed region
    # above is 100 back-to-back launches, which run into the power cap like that file's sustained figure).
    isolated = []
    for _ in range(10):
        time.sleep(0.02)
        first, _unused = stream.record_timed(), launch()
        last = stream.record_timed()
        stream.synchronize()
        isolated.append(first.elapsed_ms(last))
    burst_tflops = flops_per_step / (min(isolated) * 1e-3) / 1e12
    status = gpu.status()

    if rank == 0:
        peak, peak_source = measured_peak_tflops()
        if kind in ("i8", "e4m3"):
            peak, peak_source = peak * 2.0, peak_source + " x2 for 8-bit operands"
        if kind == "f32":
            peak, peak_source = peak / 2.0, peak_source + " /2 for TF32 operands"
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": kind, "data": "synthetic",
            "config": {"workload": args.workload, "m_per_gpu": m, "global_m": m * world, "n": n, "k": k, "output": out,
                       "operands": "A m x k and B n x k, both K-major (the reference's convention)", "parallelism": f"M-sharded x{world}, B replicated, no collective",
                       "l2": "inputs (A+B+C = %d MB per GPU) larger than the 126 MB L2; no flush" % ((a_host.nbytes + b_host.nbytes + m * n * out_bytes) >> 20),
                       "algorithm": args.algorithm},
            "clocks": clocks.record(),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(a_host.nbytes + b_host.nbytes),
                    "d2h_bytes_per_step": int(m * n * out_bytes), "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "host_checksum": checksum,
                    "call": "gpurs_matmul_host: pinned host buffers, copies and product overlapped by blocks of rows" if host_call
                            else "copy_to_device x2, product, copy_to_host on one stream"},
            "gpu_launches": int(launches),
            "repetitions": {"ms_per_step": [round(x, 6) for x in repetitions], "best": min(repetitions), "median": sorted(repetitions)[len(repetitions) // 2],
                            "note": "five times K back-to-back steps on rank 0; `value` and `ms_per_step` are the first (max over ranks)"},
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu_tflops / peak,
                         "traffic": MEASURED_TRAFFIC.get(args.workload), "peak_source": peak_source,
                         "frac_of_nominal": per_gpu_tflops / NOMINAL_PEAK[kind], "nominal_peak": NOMINAL_PEAK[kind],
                         "algorithmic_flops_per_launch": flops_per_step,
                         "algorithmic_bytes_per_launch": int(a_host.nbytes + b_host.nbytes + m * n * out_bytes),
                         "single_launch": {"achieved": burst_tflops, "ms": min(isolated), "frac": burst_tflops / peak,
                                           "protocol": "best of 10 single launches 20 ms apart (the burst protocol of the peak)"},
                         "frac_of_sustained_peak": (per_gpu_tflops / sustained_peak_tflops(kind)) if sustained_peak_tflops(kind) else None},
            "device_status": status,
        }
        if gather is not None:
            line["allgather"] = gather
        if "skinny" in args.workload:
            # bound by streaming B once from HBM: report the roofline against the measured copy bandwidth
            path = ROOT / "MEASURED_PEAKS.json"
            hbm = float(json.loads(path.read_text())["hbm_gbs"]) if path.exists() else 6650.0
            streamed = float(b_host.nbytes + a_host.nbytes + m * n * out_bytes)
            achieved = streamed / (ms_per_step * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "traffic": None,
                                "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if path.exists() else "fallback",
                                "algorithmic_bytes_per_launch": int(streamed)}
        if world == 1 and not args.no_cpu_baseline:
            rows = 4096
            seconds, flops, threads = cpu_band(kind, n, k, rows)
            line["cpu_baseline"] = {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{rows} complete output rows x N={n} x K={k} of the same workload, {seconds:.1f} s"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    del a, b, c
    gpu.close()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    parser.add_argument("--algorithm", type=int, default=0, help="0 auto, 1 single-CTA tiles, 2 CTA-pair tiles")
    parser.add_argument("--whole-tiles", action="store_true", help="never split the last round's tiles along K (no stream-K)")
    parser.add_argument("--raster-rows", type=int, default=0, help="tile rows walked together (0 = library default)")
    parser.add_argument("--l2-policy", type=int, default=0, help="0 default, 1 keep A / stream B, 2 stream A / keep B, 3 keep both, 4 none")
    parser.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                        help="weak: every GPU multiplies a full-size shard (global M grows); strong: the workload's M is split")
    parser.add_argument("--allgather", action="store_true", help="also time GEMM + NCCL all-gather of C (N > 1)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
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
