"""Benchmark of the FP32 GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). A "step" is one execution of the Plan's
recommended Primitive on inputs resident in HBM. The default workload is the
training-shaped GEMM m=16384 (tokens) k=4096 n=14336, A ~ N(0,1), B ~ N(0,1/k),
alpha=1, beta=0; with N GPUs the rows of A and D are split into N contiguous
blocks, B is replicated and there is no communication (total work fixed:
"strong" scaling). `value` is whole-job TFLOP/s counting 2*m*n*k flops per step
(the three tensor-core products of the 3xTF32 scheme count once).

Timing: CUDA events on the stream the kernels are launched on (torch's current
stream, whose handle is passed to the library), after warm-up, bracketed by a
barrier and a device synchronise, max over ranks. A, B and D together are far
larger than the 126 MB L2, so every step streams its operands from HBM again.

Roofline: the K timed steps last a fraction of a second, so `roofline.frac` is taken against the BURST
tensor peak (measured BF16 dense / 6: TF32 = BF16/2, three products per FP32 product); `sustained` is a
second leg -- the same step repeated for two seconds under the power cap, with the SM clocks sampled --
held against the sustained peak. `tflops_per_gpu_per_ghz` divides by the sampled SM clock so that runs
at different clocks (N = 1 against N = 8) compare.

`e2e` is the same metric through the public Python call
flash_train.torch.HostGemm with HOST inputs: every step copies A and B (and C)
from pinned host memory to the device, runs the GEMM and copies D back to the
host. The call moves A, C and D in bands of rows so that copy-in, kernels and
copy-out of successive bands overlap; all of it is inside the timed region.
With N > 1 every rank uploads 1/N of B's rows and the ranks all-gather the rest over NVLink.

Riding along in the default line (each a few launches, after the timed region):
  `configs`      the other benchmark configurations on this GPU (and one grouped GEMM of eight ragged
                 groups: one persistent tensor-core launch against one launch per group), timed the way the reference's
                 benchmark suite times (warm-up 10, about 200 ms of single event-timed calls clamped to
                 [10, 200], median plus mean / min / p10 / p90; benchmarks/ftrain_bench/timing.py:21-44
                 there): the 128x64x96 default, 4096^3 with addend on the exact-FP32 and on the 3xTF32
                 kernel, the few-rows shapes m = 1 and 17 (A plain and as a transposed view), 1024^3;
  `tiers`        the reference's published tiers at 64^3, 128^3, 256^3 (Python call, one-shot C call,
                 Plan reuse, every Primitive) beside its published medians;
  `plan_reuse`   host microseconds per ftrainPlanExecutePrimitive call, 1000 back-to-back calls;
  `k_split`      (N > 1) the tall-K GEMM m=n=2048, k=262144 sharded along K over the GPUs, reduced by
                 NCCL reduce-scatter and, separately, inside the kernels over peer memory; local GEMM
                 and collective timed apart; every element checked against a float64 product;
  `cpu_baseline` the reference's PyTorch CPU expression on all host cores.

Other workloads (--workload): the 4096^3 GEMM with addend; the default shape with B as a transposed view
(`_bt`); the few-rows shapes m = 1 / 8 / 17 / 32 / 64 with k = n = 4096 (`_fewrows`, HBM-bound, B rotating over four
matrices; `_fewrows_bt` with B as the transposed view of a weight matrix); the tall-K GEMM sharded along K
over the GPUs, reduced by NCCL reduce-scatter (`_ksplit`) or inside the kernel's epilogue over peer memory
(`_ksplit_fused`); and `finder_sweep`, which times every kernel family on a grid of shapes against the
Finder's choice.

`--impl reference` times the reference's own CPU implementation of the path --
its PyTorch reference expression alpha*(a@b)+beta*c on CPU tensors -- on all the
host cores, each step a bounded row-slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "flash-train_b200" / "python"))
sys.path.insert(0, str(REPO))

WORKLOADS = {
    # name: (m, k, n, seed, b_scale, alpha, beta, with_c)
    "gemm_fp32_16384x4096x14336": (16384, 4096, 14336, 3, "rsqrt_k", 1.0, 0.0, False),
    "gemm_fp32_4096x4096x4096_addend": (4096, 4096, 4096, 1, "one", 1.5, 0.5, True),
    # Same product with B stored as the n x k weight of a Linear layer and passed as its transposed view.
    "gemm_fp32_16384x4096x14336_bt": (16384, 4096, 14336, 3, "rsqrt_k", 1.0, 0.0, False),
}
# Tall-K workload: K sharded over the ranks, partial products summed by an NCCL reduce-scatter.
KSPLIT_WORKLOAD = "gemm_fp32_2048x262144x2048_ksplit"
KSPLIT_FUSED_WORKLOAD = KSPLIT_WORKLOAD + "_fused"  # the reduction inside the kernel's epilogue (peer atomics)
KSPLIT_SHAPE = (2048, 262144, 2048)
# Few-rows (memory-bound) shapes of the tail sweep, k = n = 4096, entries U(-1, 1): one GPU streams B once.
FEW_ROWS_WORKLOADS = {"gemm_fp32_1x4096x4096_fewrows": 1, "gemm_fp32_8x4096x4096_fewrows": 8,
                      "gemm_fp32_17x4096x4096_fewrows": 17, "gemm_fp32_32x4096x4096_fewrows": 32,
                      "gemm_fp32_64x4096x4096_fewrows": 64,
                      # B as the transposed view of an n x k weight matrix (x @ W^T)
                      "gemm_fp32_1x4096x4096_fewrows_bt": 1, "gemm_fp32_8x4096x4096_fewrows_bt": 8}
FEW_ROWS_KERNELS = {"Fp32GemmSkinny": "skinnyGemm", "Fp32Gemm3xTf32FewRows": "tensorGemm3xTf32Rows",
                    "Fp32Gemm3xTf32SplitK": "tensorGemm3xTf32 + splitKReduce"}
FEW_ROWS_COPIES = 4  # distinct B matrices visited in turn: 4 x 64 MiB is twice the 126 MB L2
DEFAULT_WORKLOAD = "gemm_fp32_16384x4096x14336"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on one GPU, from the ncu
# captures summarised under profiles/ (a benchmark run cannot profile itself; the source is named in the line).
MEASURED_DRAM_TRAFFIC = {
    ("gemm_fp32_16384x4096x14336", "Fp32Gemm3xTf32", 1): 3226008832 + 925021952,
    ("gemm_fp32_4096x4096x4096_addend", "Fp32Gemm3xTf32", 1): 382524160 + 56027136,
    ("gemm_fp32_1x4096x4096_fewrows", "Fp32GemmSkinny", 1): 67142912 + 49920,
    ("gemm_fp32_8x4096x4096_fewrows", "Fp32GemmSkinny", 1): 67261184 + 69888,
    ("gemm_fp32_17x4096x4096_fewrows", "Fp32GemmSkinny", 1): 67419392 + 43520,
    # dram__bytes.sum.per_second x gpu__time_duration.sum of one launch (reads and writes together)
    ("gemm_fp32_32x4096x4096_fewrows", "Fp32Gemm3xTf32FewRows", 1): 68317000,
}
TRAFFIC_SOURCE = "ncu capture of one launch of this kernel on this workload, summarised under profiles/"
CPU_SAMPLE_ROWS = 2048  # rows of A per CPU-baseline step
SUSTAINED_SECONDS = 2.0
# Medians the reference publishes for its own kernel on its own hardware (Hygon BW1102), in microseconds:
# benchmarks/results/gemm-fp32-20260929T143444.json and gemm-fp32-c-20260929T143454.json there.
PUBLISHED_TIERS_US = {
    64: {"L1_python": 30.88, "L2_one_shot": 27.44, "L3_plan_reuse": 22.4, "torch_matmul": 19.52},
    128: {"L1_python": 48.48, "L2_one_shot": 45.6, "L3_plan_reuse": 40.48, "torch_matmul": 17.92},
    256: {"L1_python": 87.52, "L2_one_shot": 84.96, "L3_plan_reuse": 79.84, "torch_matmul": 18.24},
}


def measured_peaks() -> dict:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        return {"source": "measured", **json.loads(path.read_text())}
    # Earlier measurement on the same pool, used only when the file is absent.
    return {"source": "fallback", "hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def host_cores() -> int:
    """Cores this process may run on (all of the box's unless it was pinned)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.lines: list[str] = []
        self.process = None
        self.thread = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()  # the exact child started above
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self) -> dict:
        clocks, maxima, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxima.append(float(parts[2]))
            except ValueError:
                continue
            try:
                power.append(float(parts[3]))
            except ValueError:
                pass
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "reasons": sorted(reasons),
                "samples": len(clocks), "power_w": statistics.median(power) if power else None}


def clocks_under_load(sampler: "ClockSampler", device_index: int, step, torch, elapsed_ms: float, steps: int) -> dict:
    """The sampler's summary; when the timed region (elapsed_ms, already the maximum over ranks, so every
    rank decides alike) was too short for nvidia-smi to deliver samples, every rank repeats the same
    step for about 0.4 s (untimed, after the measurement) under a second sampler."""
    if elapsed_ms >= 200.0:
        return sampler.summary()
    repeats = max(1, int(400.0 / max(elapsed_ms / max(steps, 1), 1e-3)))
    with ClockSampler(device_index) as extra:
        for _ in range(repeats):
            step()
        torch.cuda.synchronize()
    summary = extra.summary()
    summary["note"] = "timed region shorter than the sampling period: sampled while repeating the step right after it"
    return summary


def per_ghz(tflops_per_gpu: float, clocks: dict):
    mhz = clocks.get("sm_mhz") if clocks else None
    return tflops_per_gpu / (mhz / 1000.0) if mhz else None


def measure_calls(torch, call, warmup: int = 10, target_ms: float = 200.0, fewest: int = 10, most: int = 200) -> dict:
    """The reference suite's timing policy (benchmarks/ftrain_bench/timing.py:21-44 there): `warmup` calls,
    one probe call to size the run, then about `target_ms` of calls, between `fewest` and `most`, each
    bracketed by its own pair of CUDA events on the current stream with a synchronise after it. The median
    is the headline; mean, minimum, 10th and 90th percentile go with it. Microseconds."""
    def one() -> float:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        call()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1e3

    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    probe_us = max(one(), 1.0)
    count = int(min(most, max(fewest, target_ms * 1e3 // probe_us + 1)))
    samples = sorted(one() for _ in range(count))
    pick = lambda fraction: samples[min(count - 1, max(0, int(round(fraction * (count - 1)))))]  # noqa: E731
    return {"median_us": round(statistics.median(samples), 3), "mean_us": round(statistics.fmean(samples), 3),
            "min_us": round(samples[0], 3), "p10_us": round(pick(0.10), 3), "p90_us": round(pick(0.90), 3), "iters": count}


def back_to_back_us(torch, call, calls: int) -> float:
    """Device time per call of `calls` enqueues in a row with one event pair around all of them."""
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(calls):
        call()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) * 1e3 / calls


def make_inputs(workload: str, rank: int, world: int, device):
    """This rank's A rows, all of B and (if any) this rank's C rows, generated on
    the CPU from the workload's seed so that every rank and the CPU baseline see
    the same matrices, then moved to `device`."""
    import torch

    m, k, n, seed, b_scale, alpha, beta, with_c = WORKLOADS[workload]
    rows = m // world
    generator = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=generator)[rank * rows:(rank + 1) * rows].contiguous()
    b = torch.randn(k, n, generator=generator)
    if b_scale == "rsqrt_k":
        b = b / (k ** 0.5)
    c = torch.randn(m, n, generator=generator)[rank * rows:(rank + 1) * rows].contiguous() if with_c else None
    if workload.endswith("_bt"):
        b = b.t().contiguous()  # n x k buffer; the GEMM sees its (k, n) view with strides (1, k)
    if device is not None:
        a, b = a.to(device), b.to(device)
        c = c.to(device) if c is not None else None
    if workload.endswith("_bt"):
        b = b.t()
    return a, b, c, alpha, beta


def workload_shape(workload: str):
    if workload in WORKLOADS:
        return WORKLOADS[workload][:3]
    if workload in (KSPLIT_WORKLOAD, KSPLIT_FUSED_WORKLOAD):
        return KSPLIT_SHAPE
    return FEW_ROWS_WORKLOADS[workload], 4096, 4096


def cpu_inputs(workload: str, rows: int):
    """The first `rows` rows of A (and C), all of B, on the CPU, with the workload's distributions."""
    import torch

    if workload in WORKLOADS:
        a, b, c, alpha, beta = make_inputs(workload, 0, 1, None)  # the GPU run's matrices, same seed
        return a[:rows].contiguous(), b, (c[:rows].contiguous() if c is not None else None), alpha, beta
    m, k, n = workload_shape(workload)
    generator = torch.Generator().manual_seed(2)
    a = torch.rand(min(rows, m), k, generator=generator) * 2 - 1
    b = torch.rand(k, n, generator=generator) * 2 - 1
    return a, b, None, 1.0, 0.0


def cpu_reference_run(workload: str, steps: int, warmup: int) -> dict:
    """The reference's PyTorch expression on CPU tensors, on every core this process may use, timed on a
    row slice. torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the thread count is
    therefore set here, explicitly, and reported."""
    import torch

    m, k, n = workload_shape(workload)
    # Tall K: fewer rows keep a step within seconds.
    rows = min(CPU_SAMPLE_ROWS if k <= 65536 else 256, m)
    cores = host_cores()
    torch.set_num_threads(cores)
    a, b, c, alpha, beta = cpu_inputs(workload, rows)
    threads = torch.get_num_threads()

    def step():
        out = alpha * (a @ b)
        return out + beta * c if c is not None else out

    for _ in range(max(1, warmup)):
        step()
    times = []
    for _ in range(max(1, steps)):
        start = time.perf_counter()
        step()
        times.append(time.perf_counter() - start)
    mean = sum(times) / len(times)
    flops = 2.0 * rows * n * k
    return {"value": flops / mean / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
            "sample": f"first {rows} of {m} rows of A per step (B whole), torch {torch.__version__} CPU float32 "
                      f"alpha*(a@b)+beta*c on {threads} threads ({cores} cores available), mean of {len(times)} steps "
                      f"after {max(1, warmup)} warm-up",
            "ms_per_step": mean * 1e3}


def run_reference_arm(options) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    if options.workload == SWEEP_WORKLOAD:
        print(json.dumps({"impl": "reference", "unavailable": "the Finder sweep compares this library's kernels with one another"}), flush=True)
        return 0
    steps = min(options.steps, 5)
    baseline = cpu_reference_run(options.workload, steps, min(options.warmup, 1))
    m, k, n = workload_shape(options.workload)
    line = {
        "impl": "reference", "metric": "fp32_gemm_tflops", "value": baseline["value"], "unit": "TFLOP/s",
        "n_gpus": options.gpus, "steps": steps, "warmup": min(options.warmup, 1),
        "ms_per_step": baseline["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": options.workload, "m": m, "k": k, "n": n,
                   "note": "reference's PyTorch CPU expression on host cores; each step a bounded row slice"},
        "cpu_baseline": {key: baseline[key] for key in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": baseline["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def plan_reuse_native(device_index: int) -> dict | None:
    """The C++ harness (no binding cost): one Plan for m=n=k=1024, 1000 executes."""
    return native_harness(device_index, 1024, 1024, 1024, 1000)


def plan_reuse_overhead(capi, torch, device) -> dict:
    """Same measurement through the Python ctypes binding (adds the binding's own call cost)."""
    from flash_train.capi import GemmBinding, null_operand, tensor_operand

    a = torch.randn(1024, 1024, device=device)
    b = torch.randn(1024, 1024, device=device)
    d = torch.empty(1024, 1024, device=device)
    plan = GemmBinding().make_plan(tensor_operand(a), tensor_operand(b), null_operand(1024, 1024), tensor_operand(d))
    size = plan.workspace_bytes(0)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
    pointer = workspace.data_ptr() if size else 0
    stream = torch.cuda.current_stream().cuda_stream
    import ctypes

    execute = capi.lib.ftrainPlanExecutePrimitive
    handle, ws, st = plan.handle, ctypes.c_void_p(pointer), ctypes.c_void_p(stream)
    for _ in range(50):
        execute(handle, 0, ws, size, st)
    torch.cuda.synchronize()
    start_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_event.record()
    start = time.perf_counter()
    for _ in range(1000):
        execute(handle, 0, ws, size, st)
    host = time.perf_counter() - start
    end_event.record()
    torch.cuda.synchronize()
    return {"primitive": plan.primitive_name(0), "host_us_per_call": host * 1e3,
            "device_us_per_call": start_event.elapsed_time(end_event),
            "note": "host time of 1000 ftrainPlanExecutePrimitive calls through ctypes (no sync inside), m=n=k=1024"}


def torch_gemm_overhead(ft_torch, torch, device) -> dict:
    """The Python convenience call (Args + Plan per call, output allocated per call), m=n=k=1024."""
    a = torch.randn(1024, 1024, device=device)
    b = torch.randn(1024, 1024, device=device)
    for _ in range(50):
        ft_torch.gemm(a, b)
    torch.cuda.synchronize()
    start_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_event.record()
    start = time.perf_counter()
    for _ in range(1000):
        ft_torch.gemm(a, b)
    host = time.perf_counter() - start
    end_event.record()
    torch.cuda.synchronize()
    return {"host_us_per_call": host * 1e3, "device_us_per_call": start_event.elapsed_time(end_event),
            "note": "1000 calls of flash_train.torch.gemm(a, b), m=n=k=1024, no sync inside"}


# --------------------------------------------------------------------------- ride-along records

class PlanRunner:
    """One Plan with the workspace of one of its primitives: `run()` enqueues it on torch's current stream."""

    def __init__(self, torch, a, b, c, d, alpha=1.0, beta=0.0, primitive=None):
        from flash_train.capi import GemmBinding, null_operand, tensor_operand

        rows, cols = d.shape
        self.plan = GemmBinding().make_plan(tensor_operand(a), tensor_operand(b),
                                            tensor_operand(c) if c is not None else null_operand(rows, cols),
                                            tensor_operand(d), alpha, beta)
        self.names = self.plan.primitive_names()
        self.index = 0 if primitive is None else self.names.index(primitive)
        self.name = self.names[self.index]
        self.size = self.plan.workspace_bytes(self.index)
        self.workspace = torch.empty(max(self.size, 1), dtype=torch.uint8, device=d.device)
        self.pointer = self.workspace.data_ptr() if self.size else 0
        self.stream = torch.cuda.current_stream().cuda_stream
        self.keep = (a, b, c, d)

    def run(self):
        self.plan.execute(self.index, self.pointer, self.size, self.stream)


def tf32_library_probe(torch, device, peaks):
    """cuBLAS TF32 (torch.matmul on FP32 tensors with allow_tf32) on 8192^3: the library's own rate for ONE TF32 product,
    best of 10 (burst) and back to back for two seconds (sustained). A yardstick beside the BF16 / 6 denominators, not a
    code path of this library: a third of it is what three TF32 products per FP32 product could reach."""
    n = 8192
    x = torch.randn(n, n, device=device)
    y = torch.randn(n, n, device=device)
    out = torch.empty(n, n, device=device)
    before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for _ in range(3):
            torch.matmul(x, y, out=out)
        torch.cuda.synchronize(device)
        flops = 2.0 * n * n * n
        best_ms = None
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            torch.matmul(x, y, out=out)
            stop.record()
            torch.cuda.synchronize(device)
            elapsed = start.elapsed_time(stop)
            best_ms = elapsed if best_ms is None else min(best_ms, elapsed)
        repeats = max(10, int(2000.0 / best_ms))
        with ClockSampler(device.index or 0) as sampler:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(repeats):
                torch.matmul(x, y, out=out)
            stop.record()
            torch.cuda.synchronize(device)
        clocks = sampler.summary()
        sustained_ms = start.elapsed_time(stop) / repeats
    finally:
        torch.backends.cuda.matmul.allow_tf32 = before
    burst, sustained = flops / (best_ms * 1e-3) / 1e12, flops / (sustained_ms * 1e-3) / 1e12
    return {"shape": [n, n, n], "burst_tflops": burst, "sustained_tflops": sustained, "sustained_clocks": clocks,
            "fp32_equivalent_burst": burst / 3.0, "fp32_equivalent_sustained": sustained / 3.0,
            "bf16_over_6_burst": peaks["bf16_tflops"] / 6.0, "bf16_over_6_sustained": peaks["bf16_tflops_sustained"] / 6.0,
            "how": "torch.matmul (cuBLAS) on FP32 operands with allow_tf32=True: best of 10 single calls, then back to back for 2 s; "
                   "a third of it is the FP32-equivalent rate of three TF32 products per product; the fractions in this line use "
                   "the driver-measured BF16 / 6 figures"}


def config_records(torch, capi, device, peaks, ffma_tflops) -> dict:
    """The benchmark configurations other than the timed workload, each a few launches on this GPU,
    timed with the reference suite's policy (measure_calls) and, for the short ones, also back to back."""
    records = {}
    burst_tensor = peaks["bf16_tflops"] / 6.0
    # --- 128 x 64 x 96, N(0,1) from seed 0, alpha 1, beta 0, no C (launch-latency bound: microseconds, no fraction)
    generator = torch.Generator().manual_seed(0)
    a = torch.randn(128, 64, generator=generator).to(device)
    b = torch.randn(64, 96, generator=generator).to(device)
    d = torch.empty(128, 96, device=device)
    runner = PlanRunner(torch, a, b, None, d)
    records["config1_128x64x96"] = {"primitive": runner.name, **measure_calls(torch, runner.run),
                                    "back_to_back_us": round(back_to_back_us(torch, runner.run, 200), 3)}
    # --- 4096^3, D = 1.5 A B + 0.5 C, N(0,1) from seed 1: the exact-FP32 kernel and the 3xTF32 kernel
    generator = torch.Generator(device=device).manual_seed(1)
    a, b, c = (torch.randn(4096, 4096, device=device, generator=generator) for _ in range(3))
    d = torch.empty(4096, 4096, device=device)
    flops = 2.0 * 4096 ** 3
    for label, primitive, bound, peak, source in (
            ("config2_4096_cubed_addend_exact_fp32", "Fp32Gemm", "fp32", ffma_tflops, "FFMA probe measured in this run"),
            ("config2_4096_cubed_addend_3xtf32", "Fp32Gemm3xTf32", "tensor", burst_tensor, f"{peaks['source']} bf16_tflops / 6")):
        runner = PlanRunner(torch, a, b, c, d, 1.5, 0.5, primitive)
        stats = measure_calls(torch, runner.run)
        tflops = flops / (stats["median_us"] * 1e-6) / 1e12
        records[label] = {"primitive": runner.name, **stats, "tflops": round(tflops, 2), "bound": bound,
                          "peak_tflops": round(peak, 2) if peak else None, "frac": round(tflops / peak, 4) if peak else None,
                          "peak_source": source}
    del a, b, c, d
    # --- k = n = 4096, m = 1 and 17, U(-1,1) from seed 2, A plain and as the transposed view of a k x m buffer;
    #     B rotates over four matrices (256 MiB, twice the L2) so that every call streams B from HBM.
    generator = torch.Generator(device=device).manual_seed(2)
    copies = [torch.rand(4096, 4096, device=device, generator=generator) * 2 - 1 for _ in range(FEW_ROWS_COPIES)]
    for m in (1, 17):
        plain = torch.rand(m, 4096, device=device, generator=generator) * 2 - 1
        for label, a in (("contiguous", plain), ("transposed_view", plain.t().contiguous().t())):
            d = torch.empty(m, 4096, device=device)
            runners = [PlanRunner(torch, a, b, None, d) for b in copies]
            turn = [0]

            def call():
                runners[turn[0] % FEW_ROWS_COPIES].run()
                turn[0] += 1

            stats = measure_calls(torch, call)
            chained = back_to_back_us(torch, call, 40 * FEW_ROWS_COPIES)
            algorithmic = 4 * (4096 * 4096 + m * 4096 + m * 4096)
            gbs = algorithmic / (chained * 1e-6) / 1e9
            records[f"config3_{m}x4096x4096_{label}"] = {
                "primitive": runners[0].name, **stats, "back_to_back_us": round(chained, 3), "bound": "hbm",
                "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4),
                "peak_source": f"{peaks['source']} hbm_gbs (copy); fraction from the back-to-back time"}
    # ... and the compute-bound members of the same sweep, m = 255 and 4097 (one B is enough: 137 GFLOP and more
    #     per call). The transposed view of a k x m buffer with an odd m has a pitch TMA cannot take: the
    #     tensor-core Primitive stages A in its workspace first (one more small launch).
    for m in (255, 4097):
        plain = torch.rand(m, 4096, device=device, generator=generator) * 2 - 1
        for label, a in (("contiguous", plain), ("transposed_view", plain.t().contiguous().t())):
            d = torch.empty(m, 4096, device=device)
            runner = PlanRunner(torch, a, copies[0], None, d)
            stats = measure_calls(torch, runner.run)
            tflops = 2.0 * m * 4096 * 4096 / (stats["median_us"] * 1e-6) / 1e12
            records[f"config3_{m}x4096x4096_{label}"] = {
                "primitive": runner.name, "workspace_bytes": runner.size, **stats, "bound": "tensor", "tflops": round(tflops, 2),
                "frac": round(tflops / burst_tensor, 4), "peak_source": f"{peaks['source']} bf16_tflops / 6"}
    del copies
    # --- grouped GEMM (GroupedABCDGemm): eight "experts" with ragged token counts, one empty, x @ W_g per group
    from flash_train.capi import GroupedGemmBinding

    counts, hidden, out_features = [1800, 0, 129, 2515, 1024, 64, 2048, 612], 4096, 4096
    tokens = torch.randn(sum(counts), hidden, device=device)
    weights = torch.randn(len(counts), hidden, out_features, device=device) / hidden ** 0.5
    result = torch.empty(sum(counts), out_features, device=device)
    starts = [sum(counts[:g]) for g in range(len(counts))]
    groups = len(counts)
    rows_of = lambda width: {"row_strides": [width] * groups, "col_strides": [1] * groups}  # noqa: E731
    grouped_plan = GroupedGemmBinding().make_plan(
        {"address": tokens.data_ptr(), "rows": counts, "cols": [hidden] * groups, "offsets": [s * hidden for s in starts], **rows_of(hidden)},
        {"address": weights.data_ptr(), "rows": [hidden] * groups, "cols": [out_features] * groups,
         "offsets": [g * hidden * out_features for g in range(groups)], **rows_of(out_features)},
        {"address": 0, "rows": counts, "cols": [out_features] * groups, "offsets": [s * out_features for s in starts], **rows_of(out_features)},
        {"address": result.data_ptr(), "rows": counts, "cols": [out_features] * groups, "offsets": [s * out_features for s in starts],
         **rows_of(out_features)}, 1.0, 0.0)
    grouped_flops = 2.0 * sum(counts) * hidden * out_features
    stream = torch.cuda.current_stream().cuda_stream
    grouped = {"groups": groups, "rows_per_group": counts, "k": hidden, "n": out_features, "plan": grouped_plan.primitive_names()}
    for index, name in enumerate(grouped_plan.primitive_names()):
        size = grouped_plan.workspace_bytes(index)
        workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
        call = lambda: grouped_plan.execute(index, workspace.data_ptr() if size else 0, size, stream)  # noqa: E731
        stats = measure_calls(torch, call)
        tflops = grouped_flops / (stats["median_us"] * 1e-6) / 1e12
        peak, bound = (burst_tensor, "tensor") if "3xTf32" in name else (ffma_tflops, "fp32")
        grouped[name] = {**stats, "tflops": round(tflops, 2), "bound": bound, "frac": round(tflops / peak, 4) if peak else None,
                         "workspace_bytes": size}
    # The same products as separate Plans of the plain Gemm, one launch each, for comparison.
    singles = [PlanRunner(torch, tokens[s:s + count], weights[g], None, result[s:s + count])
               for g, (s, count) in enumerate(zip(starts, counts)) if count]

    def one_by_one():
        for runner in singles:
            runner.run()

    stats = measure_calls(torch, one_by_one)
    grouped["one_plain_gemm_per_group"] = {**stats, "tflops": round(grouped_flops / (stats["median_us"] * 1e-6) / 1e12, 2),
                                           "primitives": sorted({runner.name for runner in singles})}
    records["grouped_gemm_8_ragged_groups_k4096_n4096"] = grouped
    del tokens, weights, result, singles
    # --- 1024^3, the Plan-reuse shape: device time of the selected kernel
    a, b = torch.randn(1024, 1024, device=device), torch.randn(1024, 1024, device=device)
    d = torch.empty(1024, 1024, device=device)
    runner = PlanRunner(torch, a, b, None, d)
    stats = measure_calls(torch, runner.run)
    chained = back_to_back_us(torch, runner.run, 400)
    tflops = 2.0 * 1024 ** 3 / (chained * 1e-6) / 1e12
    records["config5b_1024_cubed"] = {"primitive": runner.name, **stats, "back_to_back_us": round(chained, 3),
                                      "tflops": round(tflops, 2), "bound": "tensor", "frac": round(tflops / burst_tensor, 4),
                                      "peak_source": f"{peaks['source']} bf16_tflops / 6; fraction from the back-to-back time"}
    return records


def native_harness(device_index: int, m: int, k: int, n: int, calls: int) -> dict | None:
    """The C++ harness (no binding in the way) for one shape: Plan-reuse host time and the tiers' medians."""
    binary = REPO / "flash-train_b200" / "python" / "flash_train" / "bin" / "plan_reuse_bench"
    if not binary.exists():
        return None
    environment = dict(os.environ)
    visible = environment.get("CUDA_VISIBLE_DEVICES")
    devices = visible.split(",") if visible else None
    environment["CUDA_VISIBLE_DEVICES"] = devices[device_index] if devices else str(device_index)
    result = subprocess.run([str(binary), str(m), str(k), str(n), str(calls), "0"], capture_output=True, text=True,
                            env=environment, timeout=300)
    if result.returncode != 0:
        return {"error": result.stderr.strip()[-300:]}
    return json.loads(result.stdout.strip().splitlines()[-1])


def tier_records(torch, capi, ft_torch, device) -> dict:
    """The reference's published tiers (its README's L1-L4) at its published shapes, same timing policy,
    alpha 1, beta 0, no C: L1 the Python call (timed here), L2 the one-shot C call, L3 Plan reuse
    (primitive 0) and L4 every primitive of the Plan (timed by the C++ harness, as the reference times them
    from its C harness). `published_us` are the reference's own medians on its own hardware."""
    records = {}
    for size in (64, 128, 256):
        a, b = torch.randn(size, size, device=device), torch.randn(size, size, device=device)
        d = torch.empty(size, size, device=device)
        tiers = {"L1_python": measure_calls(torch, lambda: ft_torch.gemm(a, b))["median_us"],
                 "torch_matmul": measure_calls(torch, lambda: torch.matmul(a, b, out=d))["median_us"]}
        native = native_harness(device.index or 0, size, size, size, 200)
        per_primitive = None
        if native is not None and "tiers" in native:
            tiers["L2_one_shot"] = native["tiers"]["L2_one_shot"]["median_us"]
            tiers["L3_plan_reuse"] = native["tiers"]["L3_plan_reuse"]["median_us"]
            per_primitive = {name: timing["median_us"] for name, timing in native["tiers"]["L4_per_primitive"].items()}
        published = PUBLISHED_TIERS_US[size]
        records[f"{size}x{size}x{size}"] = {
            "median_us": tiers, "L4_per_primitive_us": per_primitive, "published_us": published,
            "published_over_ours": {key: round(published[key] / tiers[key], 2) for key in published if key in tiers}}
    records["note"] = ("published_us: the reference's medians for its kernel on a Hygon BW1102 "
                       "(benchmarks/results/gemm-fp32-*.json there); other hardware, same timing policy "
                       "(every call between its own pair of events, so launch and event overhead are in every figure)")
    return records


def k_split_records(torch, capi, world, rank, device, steps: int, peaks) -> dict | None:
    """m = n = 2048, k = 262144 sharded along K over the ranks: the reduce-scatter form with the local GEMM and
    the collective timed apart, the fused form (reduction inside the kernels over peer memory), and every
    element of both results against a float64 product (scaled error at most twice torch FP32's)."""
    import torch.distributed as dist

    from flash_train import sharded

    m, k, n = KSPLIT_SHAPE
    k_start, k_stop = sharded.k_range(k, world, rank)
    generator = torch.Generator(device=device).manual_seed(4 + rank)
    a = torch.rand(m, k_stop - k_start, device=device, generator=generator) * 2 - 1
    b = torch.rand(k_stop - k_start, n, device=device, generator=generator) * 2 - 1
    flops = 2.0 * m * n * k
    record = {"workload": KSPLIT_WORKLOAD, "m": m, "k": k, "n": n, "k_per_gpu": k_stop - k_start, "steps": steps,
              "bytes_sent_per_rank": (world - 1) * m * n * 4 // world}

    def timed(call, repeats):
        for _ in range(2):
            call()
        dist.barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(repeats):
            call()
        end.record()
        dist.barrier()
        torch.cuda.synchronize()
        slowest = torch.tensor([begin.elapsed_time(end) / repeats], device=device, dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        return float(slowest.item())

    # Exact product and the yardstick (torch FP32 on the same shards, summed over the ranks in FP32).
    rows = slice(*sharded.row_range(m, world, rank))
    exact = a.double() @ b.double()
    dist.all_reduce(exact)
    plain = a @ b
    dist.all_reduce(plain)
    row_squares = (a.double() ** 2).sum(dim=1, keepdim=True)
    col_squares = (b.double() ** 2).sum(dim=0, keepdim=True)
    dist.all_reduce(row_squares)
    dist.all_reduce(col_squares)
    scale = row_squares.sqrt() * col_squares.sqrt() + 1e-300
    torch_error = float(((plain.double() - exact).abs() / scale).max())
    del plain

    def parity(result) -> dict:
        ours = float(((result.double() - exact[rows]).abs() / scale[rows]).max())
        worst = torch.tensor([ours], device=device, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        ours = float(worst.item())
        passed = bool(torch.isfinite(result).all()) and ours <= 2.0 * max(torch_error, 2.0 ** -24)
        flag = torch.tensor([1 if passed else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return {"parity": "pass" if int(flag.item()) == 1 else "FAIL", "scaled_error": ours, "torch_fp32_scaled_error": torch_error,
                "checked": "every element of D against a float64 product"}

    gemm = sharded.KShardedGemm(m, n, k)
    out = torch.empty(m // world, n, device=device)
    partial = torch.empty(m, n, device=device)
    step_ms = timed(lambda: gemm(a, b, None, 1.0, 0.0, out=out), steps)
    local_ms = timed(lambda: gemm.local_gemm(a, b, None, partial, 1.0, 0.0), steps)
    collective_ms = timed(lambda: dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM), steps)
    gemm(a, b, None, 1.0, 0.0, out=out)
    torch.cuda.synchronize()
    record["reduce_scatter"] = {"tflops": flops / (step_ms * 1e-3) / 1e12, "ms_per_step": step_ms, "local_gemm_ms": local_ms,
                                "reduce_scatter_ms": collective_ms, "collective_share": collective_ms / step_ms,
                                "timed": "whole step, local GEMM alone and reduce_scatter_tensor alone, each in its own event-timed loop "
                                         "(maximum over ranks); the loops run one after another, so clocks under the power cap differ a little",
                                "frac_of_burst_tensor_peak_per_gpu": flops / (step_ms * 1e-3) / 1e12 / world / (peaks["bf16_tflops"] / 6.0),
                                **parity(out)}
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings, no NVLink multicast object
        fused = sharded.FusedKShardedGemm(m, n, k)
        fused_ms = timed(lambda: fused(a, b, None, 1.0, 0.0), steps)
        result = fused(a, b, None, 1.0, 0.0)
        torch.cuda.synchronize()
        record["fused"] = {"tflops": flops / (fused_ms * 1e-3) / 1e12, "ms_per_step": fused_ms,
                           "frac_of_burst_tensor_peak_per_gpu": flops / (fused_ms * 1e-3) / 1e12 / world / (peaks["bf16_tflops"] / 6.0),
                           "how": "local K slices combined on this GPU, then added into the owners' rows over NVLink (peer atomics)",
                           **parity(result)}
    except Exception as error:  # noqa: BLE001 - symmetric memory may be unavailable on a box; the record says so
        record["fused"] = {"unavailable": f"{type(error).__name__}: {error}"[:300]}
    record["limited_by"] = ("the local GEMM: the collective moves (N-1)/N of a 16 MiB partial per rank"
                            if collective_ms < 0.25 * step_ms else "local GEMM and collective both count")
    return record if rank == 0 else None


SWEEP_WORKLOAD = "finder_sweep"
# (m, k, n, B given as the transposed view of an n x k buffer)
SWEEP_SHAPES = [(m, k, n, False) for (k, n) in ((4096, 4096), (2048, 2048), (1024, 1024), (256, 4096), (16384, 1024), (65536, 512))
                for m in (1, 8, 12, 16, 17, 32, 33, 64, 128, 256, 1024, 4097)] + \
               [(m, k, n, True) for (k, n) in ((4096, 4096), (16384, 1024), (65536, 512)) for m in (1, 8, 16, 32, 64, 256, 4097)]


def run_finder_sweep(options, torch, capi, rank, device) -> int:
    """Every kernel family that accepts a shape is timed through the platform ABI and compared with the
    Finder's first choice for it: `regret` = time of the choice / time of the fastest family."""
    from flash_train.capi import GemmBinding, null_operand, tensor_operand

    if rank != 0:
        return 0
    stream = torch.cuda.current_stream().cuda_stream
    binding = GemmBinding()
    rows = []
    for m, k, n, b_transposed in SWEEP_SHAPES:
        generator = torch.Generator(device=device).manual_seed(m + k + n)
        a = torch.rand(m, k, device=device, generator=generator) * 2 - 1
        b = torch.rand(k, n, device=device, generator=generator) * 2 - 1
        if b_transposed:
            b = b.t().contiguous().t()
        d = torch.empty(m, n, device=device)
        names = binding.make_plan(tensor_operand(a), tensor_operand(b), null_operand(m, n), tensor_operand(d)).primitive_names()
        operand = lambda t: (t.data_ptr(), tuple(t.shape), None if t.is_contiguous() else tuple(t.stride()))  # noqa: E731
        desc = capi.make_desc(operand(a), operand(b), (0, (m, n), None), operand(d), 1.0, 0.0, device.index or 0)
        times = {}
        for kernel, name in capi.KERNEL_NAMES.items():
            if capi.platform_supports(kernel, desc) is not None:
                continue
            launch = capi.PlatformGemm(kernel, desc)
            workspace = torch.empty(max(launch.workspace_bytes, 1), dtype=torch.uint8, device=device)
            repeats = 3 if 2.0 * m * n * k > 5e10 else 10
            for _ in range(2):
                launch.run(workspace.data_ptr(), launch.workspace_bytes, stream)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(repeats):
                launch.run(workspace.data_ptr(), launch.workspace_bytes, stream)
            end.record()
            torch.cuda.synchronize()
            times[name] = start.elapsed_time(end) / repeats * 1e3
        best = min(times, key=times.get)
        rows.append({"m": m, "k": k, "n": n, "b_transposed": b_transposed, "choice": names[0], "best": best, "regret": times[names[0]] / times[best],
                     "us": {name: round(value, 2) for name, value in times.items()}})
    worst = max(rows, key=lambda row: row["regret"])
    print(json.dumps({"metric": "finder_regret", "value": worst["regret"], "unit": "x", "n_gpus": 1, "higher_is_better": False,
                      "config": {"workload": SWEEP_WORKLOAD, "shapes": len(rows)}, "worst": worst, "rows": rows}), flush=True)
    return 0


def timed_steps(torch, step, steps: int, warmup: int, distributed: bool, device, local_rank: int, capi):
    """W warm-up steps, then exactly K steps between two events on the current stream, a barrier and a
    device synchronise on both sides; returns (ms over the K steps as the maximum over ranks, kernel
    launches counted by the library, the clock sampler that ran beside the region)."""
    if distributed:
        import torch.distributed as dist

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    start_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = capi.launch_count()
    with ClockSampler(local_rank) as sampler:
        start_event.record()
        for _ in range(steps):
            step()
        end_event.record()
        barrier()
        elapsed_ms = start_event.elapsed_time(end_event)
    launches = capi.launch_count() - launches_before
    if distributed:
        slowest = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        elapsed_ms = float(slowest.item())
    return elapsed_ms, launches, sampler


def run_few_rows(options, torch, capi, world, rank, local_rank, device) -> int:
    """m in {1, 8, 17, 32, 64}, k = n = 4096: the selected Primitive is a few-rows kernel (the exact one up
    to 11 rows, the 3xTF32 one with B as the tensor core's 128-row operand from 12 rows on) and the step's
    floor is reading B once from HBM. Every rank runs the same problem on its own GPU (replicas)."""
    from flash_train.capi import GemmBinding, null_operand, tensor_operand

    m, k, n = FEW_ROWS_WORKLOADS[options.workload], 4096, 4096
    generator = torch.Generator(device=device).manual_seed(2)
    a = torch.rand(m, k, device=device, generator=generator) * 2 - 1
    copies = [torch.rand(k, n, device=device, generator=generator) * 2 - 1 for _ in range(FEW_ROWS_COPIES)]
    if options.workload.endswith("_bt"):
        copies = [b.t().contiguous().t() for b in copies]  # n x k buffers seen as (k, n) views
    d = torch.empty(m, n, device=device)
    binding = GemmBinding()
    plans = [binding.make_plan(tensor_operand(a), tensor_operand(b), null_operand(m, n), tensor_operand(d)) for b in copies]
    index = 0 if options.primitive is None else plans[0].index_of(options.primitive)
    primitive = plans[0].primitive_name(index)
    size = plans[0].workspace_bytes(index)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
    pointer = workspace.data_ptr() if size else 0
    stream = torch.cuda.current_stream().cuda_stream
    distributed = world > 1

    def step():  # one step = one GEMM per copy of B
        for plan in plans:
            plan.execute(index, pointer, size, stream)

    elapsed_ms, launches, sampler = timed_steps(torch, step, options.steps, options.warmup, distributed, device, local_rank, capi)
    clocks = clocks_under_load(sampler, local_rank, step, torch, elapsed_ms, options.steps)
    if rank == 0:
        gemms = options.steps * FEW_ROWS_COPIES
        ms_per_gemm = elapsed_ms / gemms
        value = world * 2.0 * m * n * k / (ms_per_gemm * 1e-3) / 1e12
        peaks = measured_peaks()
        algorithmic = 4 * (k * n + m * k + m * n)
        achieved = algorithmic / (ms_per_gemm * 1e-3) / 1e9
        traffic = MEASURED_DRAM_TRAFFIC.get((options.workload, primitive, 1))
        line = {
            "metric": "fp32_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": options.steps,
            "warmup": options.warmup, "ms_per_step": elapsed_ms / options.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": options.workload, "m": m, "k": k, "n": n, "primitive": primitive,
                       "plan": plans[0].primitive_names(), "gemms_per_step": FEW_ROWS_COPIES,
                       "partition": "replicas only: every GPU runs the same problem",
                       "l2": f"{FEW_ROWS_COPIES} B matrices of 64 MiB visited in turn (256 MiB > 126 MB L2)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                         "traffic_source": TRAFFIC_SOURCE if traffic else None,
                         "algorithmic_bytes": algorithmic, "peak_source": f"{peaks['source']} hbm_gbs (copy)",
                         "kernel": FEW_ROWS_KERNELS.get(primitive, primitive), "us_per_launch": ms_per_gemm * 1e3},
            "clocks": clocks, "gpu_launches": launches,
        }
        print(json.dumps(line), flush=True)
    if distributed:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


def run_k_split(options, torch, capi, world, rank, local_rank, device) -> int:
    """m=n=2048, k=262144, U(-1,1): rank r holds A[:, K_r] and B[K_r, :] (contiguous per rank),
    computes a full 2048x2048 partial and the partials are reduce-scattered (rows of D)."""
    import torch.distributed as dist

    from flash_train import sharded

    m, k, n = KSPLIT_SHAPE
    distributed = world > 1
    k_start, k_stop = sharded.k_range(k, world, rank)
    generator = torch.Generator(device=device).manual_seed(4 + rank)
    a = torch.rand(m, k_stop - k_start, device=device, generator=generator) * 2 - 1
    b = torch.rand(k_stop - k_start, n, device=device, generator=generator) * 2 - 1
    if distributed and options.workload == KSPLIT_FUSED_WORKLOAD:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings, no NVLink multicast object
        gemm = sharded.FusedKShardedGemm(m, n, k)

        def step():
            gemm(a, b, None, 1.0, 0.0)
        primitive = "K-sharded: tensor kernel adding into the owners' rows over NVLink (no reduce-scatter)"
    elif distributed:
        gemm = sharded.KShardedGemm(m, n, k)
        out = torch.empty(m // world, n, device=device)

        def step():
            gemm(a, b, None, 1.0, 0.0, out=out)
        primitive = "K-sharded: local Plan + ncclReduceScatter"
    else:
        gemm = sharded.RowShardedGemm(m, 1, 0)
        out = torch.empty(m, n, device=device)

        def step():
            gemm(a, b, None, 1.0, 0.0, out=out)
        primitive = "single GPU"

    elapsed_ms, launches, sampler = timed_steps(torch, step, options.steps, options.warmup, distributed, device, local_rank, capi)
    clocks = clocks_under_load(sampler, local_rank, step, torch, elapsed_ms, options.steps)
    if rank == 0:
        ms_per_step = elapsed_ms / options.steps
        value = 2.0 * m * n * k / (ms_per_step * 1e-3) / 1e12
        peaks = measured_peaks()
        tensor_peak = peaks["bf16_tflops"] / 6.0
        line = {
            "metric": "fp32_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": options.steps,
            "warmup": options.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": options.workload, "m": m, "k": k, "n": n, "k_per_gpu": k_stop - k_start,
                       "partition": "K ranges per GPU; partial D summed over NVLink", "primitive": primitive,
                       "l2": "A and B shards (2 x 2 GiB in total) exceed the 126 MB L2"},
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": value / world / tensor_peak, "traffic": None,
                         "peak_source": f"{peaks['source']} bf16_tflops / 6 (burst: the timed region is well under a second)"},
            "tflops_per_gpu_per_ghz": per_ghz(value / world, clocks),
            "clocks": clocks, "gpu_launches": launches,
        }
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + [KSPLIT_WORKLOAD, KSPLIT_FUSED_WORKLOAD, SWEEP_WORKLOAD] + sorted(FEW_ROWS_WORKLOADS))
    parser.add_argument("--no-extras", action="store_true", help="skip e2e, the sustained leg, the ride-along records and the CPU baseline")
    parser.add_argument("--primitive", default=None,
                        help="run this Primitive of the Plan instead of index 0 (per-primitive tier), e.g. Fp32Gemm")
    options = parser.parse_args()
    options.warmup = max(options.warmup, 3) if options.impl == "ours" else options.warmup

    if options.impl == "reference":
        return run_reference_arm(options)

    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}), flush=True)
        return 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    from flash_train import capi  # fails loudly if libflash_train.so is missing
    import flash_train.torch as ft_torch
    from flash_train.capi import GemmBinding, null_operand, tensor_operand

    if options.workload in (KSPLIT_WORKLOAD, KSPLIT_FUSED_WORKLOAD):
        return run_k_split(options, torch, capi, world, rank, local_rank, device)
    if options.workload in FEW_ROWS_WORKLOADS:
        return run_few_rows(options, torch, capi, world, rank, local_rank, device)
    if options.workload == SWEEP_WORKLOAD:
        return run_finder_sweep(options, torch, capi, rank, device)

    m, k, n, *_ = WORKLOADS[options.workload]
    if m % world != 0:
        raise SystemExit(f"m={m} is not divisible by {world} ranks")
    rows = m // world
    a, b, c, alpha, beta = make_inputs(options.workload, rank, world, device)
    d = torch.empty(rows, n, device=device)
    plan = GemmBinding().make_plan(tensor_operand(a), tensor_operand(b),
                                   tensor_operand(c) if c is not None else null_operand(rows, n),
                                   tensor_operand(d), alpha, beta)
    index = 0 if options.primitive is None else plan.index_of(options.primitive)
    primitive = plan.primitive_name(index)
    size = plan.workspace_bytes(index)
    workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
    pointer = workspace.data_ptr() if size else 0
    stream = torch.cuda.current_stream().cuda_stream

    plan_names, with_c = plan.primitive_names(), c is not None

    def step():
        plan.execute(index, pointer, size, stream)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def slowest_rank(milliseconds: float) -> float:
        if not distributed:
            return milliseconds
        value = torch.tensor([milliseconds], device=device, dtype=torch.float64)
        dist.all_reduce(value, op=dist.ReduceOp.MAX)
        return float(value.item())

    elapsed_ms, launches, sampler = timed_steps(torch, step, options.steps, options.warmup, distributed, device, local_rank, capi)
    clocks = clocks_under_load(sampler, local_rank, step, torch, elapsed_ms, options.steps)
    ms_per_step = elapsed_ms / options.steps
    total_flops = 2.0 * m * n * k
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- what the timed launches computed: a block of this rank's rows against a float64 product ----
    step()
    torch.cuda.synchronize()
    check_rows = min(rows, 512)
    exact = alpha * (a[:check_rows].double() @ b.double())
    plain = alpha * (a[:check_rows] @ b)
    if c is not None:
        exact += beta * c[:check_rows].double()
        plain += beta * c[:check_rows]
    scale = abs(alpha) * a[:check_rows].double().norm(dim=1, keepdim=True) * b.double().norm(dim=0, keepdim=True) + 1e-300
    if c is not None:
        scale += abs(beta) * c[:check_rows].double().abs()
    ours_error = float(((d[:check_rows].double() - exact).abs() / scale).max())
    torch_error = float(((plain.double() - exact).abs() / scale).max())
    passed = bool(torch.isfinite(d[:check_rows]).all()) and ours_error <= 2.0 * max(torch_error, 2.0 ** -24)
    if distributed:
        verdicts = torch.tensor([1.0 if passed else 0.0, -ours_error], device=device, dtype=torch.float64)
        dist.all_reduce(verdicts, op=dist.ReduceOp.MIN)
        passed, ours_error = bool(verdicts[0].item() == 1.0), -float(verdicts[1].item())
    parity = {"result": "pass" if passed else "FAIL", "scaled_error": ours_error, "torch_fp32_scaled_error": torch_error,
              "checked": f"the first {check_rows} rows of every GPU's block of D against a float64 product; "
                         "bar: at most twice torch FP32's scaled error"}
    del exact, plain, scale

    # ---- the same step repeated for about two seconds: the power cap settles, clocks are sampled all along ----
    sustained = None
    if not options.no_extras:
        repeats = max(options.steps, int(SUSTAINED_SECONDS * 1e3 / max(ms_per_step, 1e-3)) + 1)
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as long_sampler:
            begin.record()
            for _ in range(repeats):
                step()
            end.record()
            barrier()
            long_ms = slowest_rank(begin.elapsed_time(end))
        sustained = {"steps": repeats, "seconds": long_ms * 1e-3, "ms_per_step": long_ms / repeats,
                     "value": total_flops / (long_ms / repeats * 1e-3) / 1e12, "clocks": long_sampler.summary()}

    # ---- end to end through the public Python call, host buffers in, host buffer out ----
    e2e = None
    if not options.no_extras and b.is_contiguous():  # HostGemm takes contiguous host matrices
        a_host, b_host = a.cpu().pin_memory(), b.cpu().pin_memory()
        c_host = c.cpu().pin_memory() if c is not None else None
        d_host = torch.empty(rows, n).pin_memory()
        e2e_steps = max(3, min(options.steps, 10))

        # Bands of rows: copy-in, kernels and copy-out of successive bands overlap.
        band_rows = max(128, -(-rows // 16 // 128) * 128)
        shared_b = distributed and k % world == 0
        pipeline = ft_torch.HostGemm(rows, n, k, device=device, band_rows=band_rows, with_c=c_host is not None,
                                     group=dist.group.WORLD if shared_b else None)

        def e2e_step():
            # Consecutive steps pipeline: the next step's copy-in starts while this step's D is still leaving.
            pipeline(a_host, b_host, c_host, alpha=alpha, beta=beta, out=d_host, overlap_calls=True)

        for _ in range(2):
            e2e_step()
        pipeline.join()
        barrier()
        e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record()
        for _ in range(e2e_steps):
            e2e_step()
        pipeline.join()  # the end event comes after the last step's copy-out
        e2e_end.record()
        barrier()
        e2e_ms = slowest_rank(e2e_start.elapsed_time(e2e_end))
        b_bytes = b_host.numel() * 4 // (world if shared_b else 1)
        h2d = (a_host.numel() + (c_host.numel() if c_host is not None else 0)) * 4 + b_bytes
        d2h = d_host.numel() * 4
        e2e = {"value": total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "bytes_are": "per rank", "steps": e2e_steps,
               "ms_per_step": e2e_ms / e2e_steps, "api": "flash_train.torch.HostGemm(..., overlap_calls=True)", "band_rows": band_rows,
               "timed": "events on the current stream around the steps; the stream joins the copy-out stream before the end event, so the last step's copy-out is inside",
               "b_upload": (f"every rank uploads 1/{world} of B's rows, the ranks all-gather the rest over NVLink (NCCL)"
                            if shared_b else "whole B uploaded by this GPU every step"),
               "floor": f"copy-out of D: {d2h / 1e6:.0f} MB per rank per step = {d2h / (e2e_ms / e2e_steps * 1e-3) / 1e9:.1f} GB/s "
                        f"of PCIe device-to-host at the measured step time"}
        del a_host, b_host, c_host, d_host, pipeline

    # ---- the K-sharded tall-K GEMM rides along on every multi-GPU run (all ranks take part) ----
    k_split = None
    if distributed and not options.no_extras:
        del a, b, c, d, plan
        torch.cuda.empty_cache()
        k_split = k_split_records(torch, capi, world, rank, device, max(3, min(options.steps, 10)), measured_peaks())

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return 0

    peaks = measured_peaks()
    # 3xTF32 roofline in FP32-equivalent flops: TF32 dense = BF16 dense / 2, and three tensor-core products
    # per FP32 product. The K timed steps are a burst (well under a second): burst peak. The sustained leg
    # has its own fraction against the sustained peak.
    per_gpu = value / world
    tensor_kernel = primitive.startswith("Fp32Gemm3xTf32")
    ffma_tflops = None
    if not options.no_extras or not tensor_kernel:
        with ClockSampler(local_rank) as ffma_sampler:
            for _ in range(12):  # each call is a few milliseconds of FFMAs; the clock is sampled beside them
                ffma_tflops = max(ffma_tflops or 0.0, capi.measure_ffma_tflops(local_rank))
        ffma_clocks = ffma_sampler.summary()
    if tensor_kernel:
        burst_peak = peaks["bf16_tflops"] / 6.0
        traffic = MEASURED_DRAM_TRAFFIC.get((options.workload, primitive, world))
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": burst_peak, "unit": "TFLOP/s",
                    "frac": per_gpu / burst_peak, "traffic": traffic, "traffic_source": TRAFFIC_SOURCE if traffic else None,
                    "algorithmic_bytes": 4 * (m * k + k * n + m * n * (2 if with_c else 1)),
                    "peak_source": f"{peaks['source']} bf16_tflops / 6 (burst; TF32 = BF16/2; 3 MMAs per product): "
                                   f"{options.steps} steps of {ms_per_step:.2f} ms are a burst",
                    "kernel": "tensorGemm3xTf32", "ms_per_launch": ms_per_step}
        if sustained is not None:
            sustained_peak = peaks["bf16_tflops_sustained"] / 6.0
            sustained.update({"peak": sustained_peak, "frac": sustained["value"] / world / sustained_peak,
                              "peak_source": f"{peaks['source']} bf16_tflops_sustained / 6",
                              "tflops_per_gpu_per_ghz": per_ghz(sustained["value"] / world, sustained["clocks"])})
    else:
        roofline = {"bound": "fp32", "achieved": per_gpu, "peak": ffma_tflops, "unit": "TFLOP/s",
                    "frac": per_gpu / ffma_tflops, "traffic": None,
                    "peak_source": f"FFMA probe kernel measured in this run at {ffma_clocks.get('sm_mhz')} MHz "
                                   "(148 SMs x 128 lanes x 2 x clock is the formula it approaches)",
                    "kernel": primitive, "ms_per_launch": ms_per_step}
        if sustained is not None:
            sustained.update({"peak": ffma_tflops, "frac": sustained["value"] / world / ffma_tflops,
                              "tflops_per_gpu_per_ghz": per_ghz(sustained["value"] / world, sustained["clocks"])})

    line = {
        "metric": "fp32_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": options.steps,
        "warmup": options.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": options.workload, "m": m, "k": k, "n": n, "rows_per_gpu": rows,
                   "partition": "rows of A and D split across GPUs, B replicated, no communication",
                   "primitive": primitive, "plan": plan_names, "workspace_bytes": size,
                   "l2": "operands (A+B+D > 1 GB per GPU at N=1) exceed the 126 MB L2, so each step re-reads HBM"},
        "roofline": roofline, "tflops_per_gpu_per_ghz": per_ghz(per_gpu, clocks), "clocks": clocks, "gpu_launches": launches,
        "parity": parity,
    }
    if sustained is not None:
        line["sustained"] = sustained
    if e2e is not None:
        line["e2e"] = e2e
    if k_split is not None:
        line["k_split"] = k_split
    if not options.no_extras:
        if ffma_tflops is not None:
            line["ffma_probe"] = {"tflops": ffma_tflops, "clocks": ffma_clocks}
        if not distributed:
            line["tf32_probe"] = tf32_library_probe(torch, device, peaks)
            # Beside the official fractions (BF16 / 6): the same values against a third of what the library's own
            # TF32 GEMM reached on this GPU in this run.
            if line.get("roofline", {}).get("bound") == "tensor":
                line["roofline"]["frac_of_library_tf32_over_3"] = line["value"] / line["tf32_probe"]["fp32_equivalent_burst"]
                if "sustained" in line:
                    line["sustained"]["frac_of_library_tf32_over_3"] = (line["sustained"]["value"] /
                                                                         line["tf32_probe"]["fp32_equivalent_sustained"])
        line["plan_reuse"] = {"native": plan_reuse_native(local_rank), "python_ctypes": plan_reuse_overhead(capi, torch, device),
                              "python_torch_gemm": torch_gemm_overhead(ft_torch, torch, device)}
        if not distributed:
            del a, b, c, d
            torch.cuda.empty_cache()
        line["configs"] = config_records(torch, capi, device, peaks, ffma_tflops)
        line["tiers"] = tier_records(torch, capi, ft_torch, device)
        baseline = cpu_reference_run(options.workload, 3, 1)
        line["cpu_baseline"] = {key: baseline[key] for key in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
