"""Benchmark of the fused residual-add + dropout + LayerNorm training step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + one backward of the operator over one batch of
synthetic rows (plus, on N > 1 GPUs, the NCCL all-reduce of the [2, H]
grad_weight/grad_bias buffer), run through ``gfx1010_kernels.sharded`` -- the
package's own row-sharded step, asynchronous all-reduce included.  The headline
workload is H = 768 on 64 Mi fp32 elements (87,381 rows, fp16 branch, dropout
0.1) per GPU; rows are sharded, so N GPUs process N x 87,381 rows of one global
batch (weak scaling) and every rank passes its global row offset so that the
dropout mask is the one of the unsharded call.

Rank 0 prints ONE JSON line.  ``value`` is rows/s with inputs resident in HBM:
the K-step region is timed R times back to back (``regions``) and the median
region is reported, with ``value_min`` / ``value_max``.  ``e2e`` is the same
metric with inputs in pinned host memory and results copied back to the host
inside the timed region; ``roofline`` describes the dominant kernel (the
backward) against the measured HBM peak; ``cpu_baseline`` is the reference's
CPU path (its torch decomposition) timed on this machine's cores.
``strong_c5`` is the second scaling experiment: the fixed [64, 4096, 1024]
batch split by rows over the N GPUs (strong scaling), with the same batch on
one GPU timed in the same run as its baseline.  ``sharded_check`` (N > 1)
verifies, outside the timed regions, the all-reduced gradients against the
fp64 sum of the ranks' unreduced buffers and the ranks' dropout masks against
an unsharded call; a false check makes the run fail.
``--impl reference`` times only the CPU path.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
for _path in (str(REPO), str(REPO / "gfx1010-kernels_b200")):
    if _path not in sys.path:
        sys.path.insert(0, _path)

import torch  # noqa: E402

METRIC = "fwd+bwd rows/s at H=768 (fused residual-add + dropout + LayerNorm)"
UNIT = "rows/s"
HBM_SPEC_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0

WORKLOADS = {
    # name: (rows per GPU, hidden, branch dtype, dropout p)
    "h768_64Mi": (87381, 768, torch.float16, 0.1),
    "c1_8x1024x768": (8192, 768, torch.float16, 0.1),
    "c3_h384": (32768, 384, torch.float16, 0.1),
    "c3_h512": (32768, 512, torch.float16, 0.1),
    "c3_h768": (32768, 768, torch.float16, 0.1),
    "c3_h1024": (32768, 1024, torch.float16, 0.1),
    "c5_64x4096x1024": (262144, 1024, torch.float16, 0.1),
    # the ragged small-hidden parity shapes and two variants of the headline size
    "c2_3x1367x128_fp32": (3 * 1367, 128, torch.float32, 0.15),
    "c2_5x817x256_fp32": (5 * 817, 256, torch.float32, 0.15),
    "h768_64Mi_fp32_branch": (87381, 768, torch.float32, 0.1),
    "h768_64Mi_no_dropout": (87381, 768, torch.float16, 0.0),
    "h768_64Mi_bf16_branch": (87381, 768, torch.bfloat16, 0.1),
    "h128_64Mi": (524288, 128, torch.float16, 0.1),
    "h256_64Mi": (262144, 256, torch.float16, 0.1),
    # `normalized` (and its gradient) in bfloat16: a fifth field, float32 when absent
    "h768_64Mi_bf16_normalized": (87381, 768, torch.float16, 0.1, torch.bfloat16),
    "h768_64Mi_bf16_branch_bf16_normalized": (87381, 768, torch.bfloat16, 0.1, torch.bfloat16),
    "c5_64x4096x1024_bf16_normalized": (262144, 1024, torch.float16, 0.1, torch.bfloat16),
}


def workload(name):
    """(rows per GPU, hidden, branch dtype, dropout p, normalized dtype)."""
    fields = WORKLOADS[name]
    return (*fields[:4], fields[4] if len(fields) > 4 else torch.float32)



# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE backward launch,
# taken from an ncu capture of that workload (two launches, --set full), per workload.
NCU_BACKWARD_TRAFFIC_BYTES = {
    "h768_64Mi": 814_516_480 + 364_516_352,
    "h768_64Mi_bf16_normalized": 680_267_008 + 363_772_160,
}
# the extension's element type codes (False/0 float32, True/1 float16, 2 bfloat16)
BRANCH_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
NORMALIZED_CODES = BRANCH_CODES
CPU_SAMPLE_ROWS = 8192
EPS = 1e-5


def forward_bytes_per_row(hidden, branch_bytes, dropout, normalized_bytes=4):
    """read x 4H + branch sb*H; write updated 4H + normalized sn*H + mean 4 + rstd 4
    (+ mask H/8)."""
    return (8 + branch_bytes + normalized_bytes) * hidden + 8 + (hidden // 8 if dropout else 0)


def backward_bytes_per_row(hidden, branch_bytes, dropout, normalized_bytes=4):
    """read grad_updated 4H, grad_normalized sn*H, updated 4H + mean 4 + rstd 4 (+ mask H/8);
    write grad_x 4H + grad_branch sb*H."""
    return (12 + branch_bytes + normalized_bytes) * hidden + 8 + (hidden // 8 if dropout else 0)


def measured_peak_gbs():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


def draw_inputs(rows, hidden, branch_dtype, seed):
    """Seeded synthetic batch in the distributions of the benchmark configs."""
    generator = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, hidden, generator=generator)
    branch = torch.randn(rows, hidden, generator=generator).to(branch_dtype)
    weight = 1.0 + 0.1 * torch.randn(hidden, generator=generator)
    bias = 0.1 * torch.randn(hidden, generator=generator)
    grad_updated = torch.randn(rows, hidden, generator=generator)
    grad_normalized = torch.randn(rows, hidden, generator=generator)
    return x, branch, weight, bias, grad_updated, grad_normalized


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the benchmark runs
    (read-only NVML queries; nvidia-smi as a fallback)."""

    REASONS = {
        0x1: "gpu_idle",
        0x2: "applications_clocks_setting",
        0x4: "sw_power_cap",
        0x8: "hw_slowdown",
        0x10: "sync_boost",
        0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown",
        0x100: "display_clock_setting",
    }

    def __init__(self, device_index, interval=0.01):
        self.device_index = device_index
        self.interval = interval
        self.samples = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None

    def _physical_index(self):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            entries = [entry.strip() for entry in visible.split(",") if entry.strip()]
            if self.device_index < len(entries) and entries[self.device_index].isdigit():
                return int(entries[self.device_index])
        return self.device_index

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _sample_smi(self):
        query = "clocks.sm,clocks.max.sm,clocks_event_reasons.active"
        out = subprocess.run(
            ["nvidia-smi", f"--query-gpu={query}", "--format=csv,noheader,nounits",
             "-i", str(self._physical_index())],
            capture_output=True, text=True, timeout=5,
        ).stdout.strip().split(",")
        self.max_mhz = int(float(out[1]))
        return int(float(out[0])), int(out[2].strip(), 16)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    mhz = self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM)
                    try:
                        bits = self._nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                    except Exception:
                        bits = self._nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                else:
                    mhz, bits = self._sample_smi()
                self.samples.append((time.perf_counter(), mhz, bits))
            except Exception:
                pass
            self._stop.wait(self.interval)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def summary(self, spans):
        """Median clock and the union of throttle reasons over the first of
        ``spans`` -- (label, begin, end) on the perf_counter clock, narrowest
        first -- that holds at least two samples.  The label of the span that
        was used is always reported as ``window``."""
        for label, begin, end in spans:
            window = [(mhz, bits) for (stamp, mhz, bits) in self.samples if begin <= stamp <= end]
            if len(window) >= 2:
                break
        else:
            label = "all samples of the run"
            window = [(mhz, bits) for (_, mhz, bits) in self.samples]
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "window": "no samples"}
        bits = 0
        for _, sample_bits in window:
            bits |= sample_bits
        reasons = [name for bit, name in self.REASONS.items() if bits & bit and name != "gpu_idle"]
        return {
            "sm_mhz": int(statistics.median(mhz for mhz, _ in window)),
            "sm_max_mhz": self.max_mhz,
            "reasons": reasons,
            "samples": len(window),
            "window": label,
        }


REFERENCE_PACKAGE_DIR = REPO / "oracle" / "_ref"


def reference_public_call():
    """The reference project's own ``residual_layer_norm`` (installed by
    ``oracle/build_ref.py`` into ``oracle/_ref``), or None when it is absent.
    Only for a process that has not imported this repository's package of the
    same name: the reference arm runs in a process of its own."""
    if not (REFERENCE_PACKAGE_DIR / "gfx1010_kernels" / "normalization.py").exists():
        return None
    if "gfx1010_kernels" in sys.modules:
        raise RuntimeError("the reference package must be imported in a fresh process")
    sys.path.insert(0, str(REFERENCE_PACKAGE_DIR))
    try:
        import gfx1010_kernels as reference_package
    finally:
        sys.path.remove(str(REFERENCE_PACKAGE_DIR))
    if not Path(reference_package.__file__).resolve().is_relative_to(REFERENCE_PACKAGE_DIR):
        raise RuntimeError("imported the wrong gfx1010_kernels package")
    return reference_package.residual_layer_norm


def time_cpu_reference(rows, hidden, branch_dtype, dropout_p, steps, warmup,
                       normalized_dtype=torch.float32):
    """The reference's CPU path on all host threads: forward through its public
    call with ``implementation="torch"`` (F.dropout -> add -> F.layer_norm) plus
    ``torch.autograd.grad``.  Returns (times, threads, kind): kind "reference"
    when the reference's own package ran, "port" when only the restatement in
    ``oracle/rln_oracle.py`` was available."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        rows, hidden, branch_dtype, seed=0
    )
    leaves = [t.requires_grad_(True) for t in (x, branch, weight, bias)]
    grad_normalized = grad_normalized.to(normalized_dtype)
    reference_call = reference_public_call()
    if reference_call is not None:
        kind = "reference"

        def forward():
            updated, normalized = reference_call(
                *leaves, dropout_p, EPS, True, implementation="torch"
            )
            # a 16-bit `normalized` is one cast after the reference's float32 result
            return updated, normalized.to(normalized_dtype)
    else:
        from oracle import rln_oracle

        kind = "port"

        def forward():
            return rln_oracle.torch_decomposition(
                *leaves, dropout_p, EPS, True, None, normalized_dtype
            )
    times = []
    for index in range(warmup + steps):
        begin = time.perf_counter()
        outputs = forward()
        torch.autograd.grad(outputs, leaves, (grad_updated, grad_normalized))
        elapsed = time.perf_counter() - begin
        if index >= warmup:
            times.append(elapsed)
    return times, threads, kind


def cpu_sample_description(rows, rows_full, hidden, branch_dtype, dropout_p, kind):
    what = ("the reference package's residual_layer_norm(implementation='torch')"
            if kind == "reference" else "the restated torch decomposition")
    return (
        f"first {rows} rows of the {rows_full}-row workload per step "
        f"(x fp32 [{rows},{hidden}], branch {str(branch_dtype).split('.')[-1]}, p={dropout_p}); "
        f"{what} + torch.autograd.grad"
    )


def run_reference_arm(args, rank):
    if rank != 0:
        return 0
    rows_full, hidden, branch_dtype, dropout_p, normalized_dtype = workload(args.workload)
    rows = min(rows_full, CPU_SAMPLE_ROWS)
    times, threads, kind = time_cpu_reference(
        rows, hidden, branch_dtype, dropout_p, args.steps, args.warmup, normalized_dtype
    )
    total = sum(times)
    value = rows * len(times) / total
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "value_median": rows / statistics.median(times),
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args.workload, args.gpus),
        "cpu_baseline": {
            "value": value, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": cpu_sample_description(rows, rows_full, hidden, branch_dtype, dropout_p, kind),
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def cpu_baseline_record(workload_name):
    """The ``cpu_baseline`` object of the native arm's line: the reference arm run
    as a child process (so that the reference's package, which has this
    package's name, gets an interpreter of its own) on 5 steps after 1 warm-up."""
    completed = subprocess.run(
        [sys.executable, str(Path(__file__).resolve()), "--impl", "reference",
         "--workload", workload_name, "--steps", "5", "--warmup", "1"],
        capture_output=True, text=True, timeout=900,
        env={key: value for key, value in os.environ.items()
             if key not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")},
    )
    lines = [line for line in completed.stdout.splitlines() if line.startswith("{")]
    if completed.returncode != 0 or not lines:
        raise RuntimeError(f"the CPU baseline run failed:\n{completed.stdout}{completed.stderr}")
    record = json.loads(lines[-1])
    baseline = record["cpu_baseline"]
    baseline["value"] = record["value_median"]
    baseline["sample"] += "; median of 5 steps"
    return baseline


def workload_config(name, gpus):
    rows, hidden, branch_dtype, dropout_p, normalized_dtype = workload(name)
    return {
        "workload": name,
        "rows_per_gpu": rows,
        "rows_total": rows * gpus,
        "hidden": hidden,
        "x_dtype": "float32",
        "branch_dtype": str(branch_dtype).split(".")[-1],
        "normalized_dtype": str(normalized_dtype).split(".")[-1],
        "dropout_p": dropout_p,
        "eps": EPS,
        "training": True,
        "parameter_gradients": "atomic (non-deterministic mode)",
        "parallelism": f"rows sharded over {gpus} GPU(s); NCCL all-reduce of the [2,H] grads on a "
                       "high-priority stream, asynchronous (overlaps the next step's forward, "
                       "waited for before that step's backward, inside the timed region)"
        if gpus > 1
        else "1 GPU",
        "l2": "inputs larger than L2 (no flush needed)" if rows * hidden * 4 > 126e6
        else "flushed between steps (256 MB written, then read)",
    }


REGIONS = 11          # back-to-back timed regions of K steps; the median is reported
C5 = "c5_64x4096x1024"


class ShardRunner:
    """This rank's rows of one workload, resident on the device, and the step on
    them: ``gfx1010_kernels.sharded.sharded_forward_backward`` with
    ``async_op=True``, every step handed the previous step's handle (the
    all-reduce overlaps the next forward and is waited for before the next
    backward).  With one rank there is no collective and the handle is inert."""

    def __init__(self, name, rows, row_base, rank_seed, device, world):
        from gfx1010_kernels import sharded

        self.sharded = sharded
        _, self.hidden, self.branch_dtype, self.dropout_p, self.normalized_dtype = workload(name)
        self.rows = rows
        self.row_base = row_base
        self.world = world
        self.device = device
        host = draw_inputs(rows, self.hidden, self.branch_dtype, seed=rank_seed)
        (self.x, self.branch, self.weight, self.bias, self.grad_updated,
         grad_normalized) = (t.to(device) for t in host)
        self.grad_normalized = grad_normalized.to(self.normalized_dtype)
        self.host = host
        if world > 1:
            import torch.distributed as dist

            # replicated parameters: every rank uses rank 0's values
            dist.broadcast(self.weight, 0)
            dist.broadcast(self.bias, 0)
        self.pending = None
        self.flush = None
        if rows * self.hidden * 4 <= 126e6:
            self.flush = torch.zeros(256 << 20, dtype=torch.uint8, device=device)

    def flush_l2(self):
        # Write a buffer twice the size of L2, then read it: the write evicts the
        # workload's lines, the read pushes the write's dirty lines out to HBM, so
        # that the kernel that runs next is not billed for their write-back.
        self.flush.zero_()
        self.flush.sum()

    def step(self, index, after_forward=None):
        self.pending = self.sharded.sharded_forward_backward(
            self.x, self.branch, self.weight, self.bias, self.grad_updated, self.grad_normalized,
            row_base=self.row_base, dropout_p=self.dropout_p, eps=EPS, training=True,
            seed=0, offset=4 * index, async_op=True, previous=self.pending,
            after_forward=after_forward, all_reduce=self.world > 1,
        )
        return self.pending

    def finish(self):
        if self.pending is not None:
            self.pending.wait()
            self.pending = None

    def fence(self):
        self.finish()
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()

    def warm(self, count, first):
        for index in range(count):
            if self.flush is not None:
                self.flush_l2()
            self.step(first + index)
            if index % 50 == 49:
                torch.cuda.synchronize()
        self.finish()
        torch.cuda.synchronize()

    def timed_regions(self, regions, steps, first, run_step=None):
        """``regions`` regions of ``steps`` steps, each bracketed by a fence
        (pending collective, device, barrier) on both sides and timed with CUDA
        events on the launching stream.  Returns the per-region milliseconds of
        this rank and the index after the last step.  Workloads that fit in L2
        are flushed before every step and timed step by step."""
        run_step = run_step or (lambda index: self.step(index))
        elapsed = []
        index = first
        for _ in range(regions):
            self.fence()
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            brackets = []
            start.record()
            for _ in range(steps):
                if self.flush is not None:
                    # the L2 flush is not part of a step: bracket every step on its own
                    self.flush_l2()
                    begin_event = torch.cuda.Event(enable_timing=True)
                    end_event = torch.cuda.Event(enable_timing=True)
                    begin_event.record()
                run_step(index)
                index += 1
                if self.flush is not None:
                    end_event.record()
                    brackets.append((begin_event, end_event))
            self.finish()
            stop.record()
            self.fence()
            if brackets:
                elapsed.append(sum(a.elapsed_time(b) for a, b in brackets))
            else:
                elapsed.append(start.elapsed_time(stop))
        return elapsed, index

    def kernel_pass(self, steps, first):
        """The same steps with CUDA events around the two halves: mean
        milliseconds of (forward + wait for the previous all-reduce) and of
        (zeroing kernel + backward).  Run outside the timed regions: an event
        between two kernels keeps the second from being scheduled while the
        first drains, which slows the step."""
        forward_events, backward_events = [], []
        for index in range(steps):
            if self.flush is not None:
                self.flush_l2()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e2 = torch.cuda.Event(enable_timing=True)
            e0.record()
            self.step(first + index, after_forward=e1.record)
            e2.record()
            forward_events.append((e0, e1))
            backward_events.append((e1, e2))
        self.finish()
        torch.cuda.synchronize()
        forward_ms = statistics.mean(a.elapsed_time(b) for a, b in forward_events)
        backward_ms = statistics.mean(a.elapsed_time(b) for a, b in backward_events)
        return forward_ms, backward_ms


def max_over_ranks(values, device, world):
    """Element-wise maximum of a list of floats over the ranks."""
    if world == 1:
        return list(values)
    import torch.distributed as dist

    tensor = torch.tensor(list(values), device=device, dtype=torch.float64)
    dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
    return tensor.tolist()


def sharded_check(runner, rank, world, rows_total, offset):
    """Correctness of the multi-rank step, outside every timed region.

    1. Every rank runs forward + backward on its shard through the raw entries
       (no collective); the unreduced [2, H] buffers are gathered and summed in
       float64.  The product step (``sharded_forward_backward`` with the same
       Philox state) must return that sum on every rank: <= 1e-4 relative, with
       the absolute floor 1e-5 * sqrt(rows_total) for columns that cancel.
    2. The product step's row-local outputs must be the raw calls' bits.
    3. Rank 0 runs ONE unsharded forward over all rows_total rows (zeros as
       data: the mask depends on the Philox state and the global element index
       only) and compares, bit for bit, the first and last 256 rows of every
       rank's mask with the rows of the unsharded mask they correspond to.
    """
    import torch.distributed as dist

    sharded = runner.sharded
    device = runner.device
    hidden = runner.hidden
    updated, normalized, mean, rstd, mask = sharded._native_forward(
        runner.x, runner.branch, runner.weight, runner.bias, runner.normalized_dtype,
        runner.dropout_p, EPS, True, 0, offset, runner.row_base,
    )
    grad_x, grad_branch, parameters = sharded._native_backward(
        runner.grad_updated, runner.grad_normalized, updated, runner.weight, mean, rstd, mask,
        runner.dropout_p, True, runner.branch_dtype,
    )
    gathered = [torch.empty_like(parameters) for _ in range(world)]
    dist.all_gather(gathered, parameters.contiguous())
    expected = torch.stack(gathered).double().sum(0)
    result = sharded.sharded_forward_backward(
        runner.x, runner.branch, runner.weight, runner.bias, runner.grad_updated,
        runner.grad_normalized, row_base=runner.row_base, dropout_p=runner.dropout_p, eps=EPS,
        training=True, seed=0, offset=offset,
    )
    reduced = torch.stack((result.grad_weight, result.grad_bias)).double()
    scale = float(rows_total) ** 0.5      # typical size of a column sum
    floor = 1e-5 * scale
    difference = (reduced - expected).abs()
    tolerance_used = float((difference / (1e-4 * expected.abs() + floor)).max().item())
    gradients_ok = tolerance_used <= 1.0
    # bare relative error on the columns that are not near-total cancellations
    meaningful = expected.abs() >= 0.01 * scale
    worst_relative = float((difference / expected.abs())[meaningful].max().item())
    row_local_ok = all(
        torch.equal(a, b) for a, b in (
            (result.updated, updated), (result.normalized, normalized), (result.grad_x, grad_x),
            (result.grad_branch, grad_branch), (result.mask, mask))
    )
    # masks: two windows per rank against one unsharded forward on rank 0
    words_per_row = hidden // 32
    window = min(256, runner.rows)
    sample = torch.cat((mask[: window * words_per_row],
                        mask[(runner.rows - window) * words_per_row:])).contiguous()
    layout = torch.tensor([runner.row_base, runner.rows, window], device=device,
                          dtype=torch.int64)
    layouts = [torch.empty_like(layout) for _ in range(world)]
    dist.all_gather(layouts, layout)
    windows = [int(entry[2].item()) for entry in layouts]
    masks_ok = True
    if len(set(windows)) == 1:
        samples = [torch.empty_like(sample) for _ in range(world)]
        dist.all_gather(samples, sample)
        if rank == 0:
            zeros = torch.zeros(rows_total, hidden, device=device)
            whole = sharded._native_forward(
                zeros, zeros.to(runner.branch_dtype), runner.weight, runner.bias,
                torch.float32, runner.dropout_p, EPS, True, 0, offset, 0,
            )[4]
            for entry, got in zip(layouts, samples):
                base, count, width = (int(v) for v in entry.tolist())
                want = torch.cat((
                    whole[base * words_per_row: (base + width) * words_per_row],
                    whole[(base + count - width) * words_per_row: (base + count) * words_per_row],
                ))
                masks_ok = masks_ok and torch.equal(got, want)
            del zeros, whole
    else:
        masks_ok = False
    flags = torch.tensor([gradients_ok, row_local_ok, masks_ok, worst_relative, tolerance_used],
                         device=device, dtype=torch.float64)
    worst = flags.clone()
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    record = {
        "ok": bool(flags[0] > 0 and flags[1] > 0 and flags[2] > 0),
        "all_reduced_equals_fp64_sum_of_rank_buffers": bool(flags[0] > 0),
        "tolerance": "1e-4 relative + 1e-5*sqrt(rows_total) absolute",
        "worst_fraction_of_tolerance": float(worst[4]),
        "worst_relative_error_where_sum_exceeds_1pct_of_sqrt_rows": float(worst[3]),
        "row_local_outputs_bit_identical_to_raw_calls": bool(flags[1] > 0),
        "rank_masks_equal_unsharded_mask": bool(flags[2] > 0),
        "mask_rows_compared_per_rank": 2 * window,
        "ranks": world,
    }
    torch.cuda.synchronize()
    return record


def run_strong_c5(args, rank, world, device):
    """The fixed [64, 4096, 1024] batch (262,144 rows, fp16 branch, p = 0.1) split
    by rows over the ranks: strong scaling.  With more than one rank the same
    batch is then timed on rank 0 alone (the other ranks wait at a barrier), so
    that the speed-up is taken inside one run on one box."""
    from gfx1010_kernels.sharded import shard_bounds

    rows_total, hidden, branch_dtype, dropout_p, normalized_dtype = workload(C5)
    begin, end = shard_bounds(rows_total, world, rank)
    steps = max(3, min(args.steps, 100))
    regions = REGIONS if not args.kernel_only else 3
    branch_bytes = 4 if branch_dtype == torch.float32 else 2
    bytes_per_row = (forward_bytes_per_row(hidden, branch_bytes, True)
                     + backward_bytes_per_row(hidden, branch_bytes, True))

    def measure(runner, ranks):
        runner.warm(max(args.warmup, 3) + 10, 0)
        elapsed, index = runner.timed_regions(regions, steps, 1000)
        elapsed = max_over_ranks(elapsed, device, ranks)
        forward_ms, backward_ms = runner.kernel_pass(min(steps, 50), index)
        forward_ms, backward_ms = max_over_ranks([forward_ms, backward_ms], device, ranks)
        median = statistics.median(elapsed)
        return {
            "rows_s": rows_total * steps / (median * 1e-3),
            "rows_s_min": rows_total * steps / (max(elapsed) * 1e-3),
            "rows_s_max": rows_total * steps / (min(elapsed) * 1e-3),
            "ms_per_step": median / steps,
            "forward_plus_wait_ms": forward_ms,
            "backward_ms": backward_ms,
            "hbm_gbs_per_gpu": rows_total / ranks * bytes_per_row * steps / (median * 1e-3) / 1e9,
        }

    runner = ShardRunner(C5, end - begin, begin, 100 + rank, device, world)
    record = {
        "workload": C5, "scaling": "strong", "rows_total": rows_total,
        "rows_per_gpu": end - begin, "hidden": hidden, "steps": steps, "regions": regions,
        "n_gpus": world,
    }
    record.update(measure(runner, world))
    if world > 1:
        record["sharded_check"] = sharded_check(runner, rank, world, rows_total, 4 * 50000)
    del runner
    torch.cuda.empty_cache()
    if world > 1:
        import torch.distributed as dist

        if rank == 0:
            alone = ShardRunner(C5, rows_total, 0, 100, device, 1)
            record["one_gpu"] = measure(alone, 1)
            record["speedup_vs_one_gpu"] = record["rows_s"] / record["one_gpu"]["rows_s"]
            del alone
            torch.cuda.empty_cache()
        dist.barrier()
        torch.cuda.synchronize()
    return record


def public_api_device_step_ms(runner, steps):
    """Mean milliseconds of the step through the public call --
    ``residual_layer_norm(implementation="gfx1010")`` + ``torch.autograd.grad`` --
    on this rank's device-resident tensors (no collective), CUDA events."""
    from gfx1010_kernels import residual_layer_norm

    leaves = [t.detach().clone().requires_grad_(True)
              for t in (runner.x, runner.branch, runner.weight, runner.bias)]

    def one(index):
        updated, normalized = residual_layer_norm(
            *leaves, runner.dropout_p, EPS, True, implementation="gfx1010",
            normalized_dtype=runner.normalized_dtype,
        )
        return torch.autograd.grad(
            (updated, normalized), leaves, (runner.grad_updated, runner.grad_normalized))

    for index in range(10):
        one(index)
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    brackets = []
    start.record()
    for index in range(steps):
        if runner.flush is not None:
            runner.flush_l2()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
        one(index)
        if runner.flush is not None:
            b.record()
            brackets.append((a, b))
    stop.record()
    torch.cuda.synchronize()
    if brackets:
        return sum(a.elapsed_time(b) for a, b in brackets) / steps
    return start.elapsed_time(stop) / steps


def run_native_arm(args, rank, local_rank, world):
    import torch.distributed as dist

    from gfx1010_kernels import residual_layer_norm, residual_layer_norm_status
    from gfx1010_kernels import sharded

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl native needs a CUDA device (no CPU fallback)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    status = residual_layer_norm_status(device)
    if not status.available:
        raise RuntimeError(f"native backend unavailable: {status.reason}")
    if world > 1:
        # NCCL on a high-priority stream (see sharded.high_priority_nccl_options),
        # and a short timeout: a rank that stops calling collectives must surface
        # as an error within minutes, not hold the GPUs for the default ten.
        sharded.init_sharded_process_group(
            device, timeout=datetime.timedelta(seconds=180),
            high_priority=not args.default_priority_collectives,
        )

    rows, hidden, branch_dtype, dropout_p, normalized_dtype = workload(args.workload)
    branch_bytes = 4 if branch_dtype == torch.float32 else 2
    normalized_bytes = 4 if normalized_dtype == torch.float32 else 2
    runner = ShardRunner(args.workload, rows, rank * rows, rank, device, world)
    regions = 3 if args.kernel_only else args.regions

    sampler = ClockSampler(local_rank)
    sampler.start()

    # warm-up: W steps, then as many more as bring the loaded span to about a second
    # (clock settling + clock samples).  The count is agreed between the ranks --
    # every step contains a collective, so all ranks must run the same number.
    warm_begin = time.perf_counter()
    base = max(args.warmup, 3)
    runner.warm(base, 0)
    warmup_actual = base
    if not args.kernel_only:
        probe_begin = time.perf_counter()
        runner.warm(10, base)    # timed probe (the first steps above carry one-time set-up)
        warmup_actual += 10
        per_step = (time.perf_counter() - probe_begin) / 10
        extra = int(min(5000, 1.0 / max(per_step, 1e-6)))
        if world > 1:
            agreed = torch.tensor([extra], device=device, dtype=torch.int64)
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
            extra = int(agreed.item())
        runner.warm(extra, warmup_actual)
        warmup_actual += extra

    run_step = None
    if args.cuda_graph:
        if world > 1:
            raise RuntimeError("--cuda-graph is a single-GPU mode")
        # One step (forward, zeroing kernel, backward and the allocator's work)
        # recorded once; every replay re-runs it with the recorded Philox offset.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            runner.step(warmup_actual)
        runner.pending = None

        def run_step(index):
            graph.replay()

        for _ in range(10):
            run_step(0)

    timed_begin = time.perf_counter()
    region_ms, next_index = runner.timed_regions(regions, args.steps, warmup_actual, run_step)
    timed_end = time.perf_counter()
    # per-kernel durations: same steps, same buffers, right after the timed regions
    forward_ms, backward_ms = runner.kernel_pass(min(args.steps, 100), next_index)
    next_index += min(args.steps, 100)
    clocks = sampler.summary([
        ("timed regions", timed_begin, timed_end),
        ("warm-up + timed regions (the timed regions hold fewer than two samples)",
         warm_begin, timed_end),
    ])

    check = None
    if world > 1:
        check = sharded_check(runner, rank, world, rows * world, 4 * (next_index + 7))

    public_ms = None
    if not args.kernel_only:
        public_ms = public_api_device_step_ms(runner, min(args.steps, 100))

    # end-to-end: pinned host inputs -> device -> fwd+bwd -> results back to host
    if args.kernel_only:
        e2e = None
    else:
        e2e = run_end_to_end(
            args, device, runner.host, runner.weight, runner.bias, dropout_p, world,
            residual_layer_norm, normalized_dtype,
        )
    sampler.stop()
    del runner
    torch.cuda.empty_cache()

    strong = None
    if (args.workload == "h768_64Mi" and not args.no_strong_c5 and not args.kernel_only
            and not args.cuda_graph):
        strong = run_strong_c5(args, rank, world, device)

    region_ms = max_over_ranks(region_ms, device, world)
    has_public = public_ms is not None
    stats = [forward_ms, backward_ms, public_ms or 0.0]
    if e2e is not None:
        stats += [e2e["ms"], e2e["public_ms"], e2e["copy_ms"], e2e["chunked_copy_ms"]]
    stats = max_over_ranks(stats, device, world)
    forward_ms, backward_ms, public_ms = stats[:3]

    failed = False
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        total_rows = rows * world
        elapsed_ms = statistics.median(region_ms)
        value = total_rows * args.steps / (elapsed_ms * 1e-3)
        fwd_row = forward_bytes_per_row(hidden, branch_bytes, dropout_p > 0, normalized_bytes)
        bwd_row = backward_bytes_per_row(hidden, branch_bytes, dropout_p > 0, normalized_bytes)
        fwd_bytes = fwd_row * rows
        bwd_bytes = bwd_row * rows
        fwd_gbs = fwd_bytes / (forward_ms * 1e-3) / 1e9
        bwd_gbs = bwd_bytes / (backward_ms * 1e-3) / 1e9
        step_gbs = (fwd_bytes + bwd_bytes) * world * args.steps / (elapsed_ms * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.kernel_only:
            cpu = cpu_baseline_record(args.workload)
        line = {
            "metric": METRIC,
            "value": value,
            "value_min": total_rows * args.steps / (max(region_ms) * 1e-3),
            "value_max": total_rows * args.steps / (min(region_ms) * 1e-3),
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "regions": regions,
            "timing": f"median of {regions} back-to-back regions of {args.steps} steps, each "
                      "fenced (pending all-reduce, device, barrier) and timed with CUDA events, "
                      "max over ranks per region",
            "warmup": args.warmup,
            "warmup_actual": warmup_actual,
            "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": workload_config(args.workload, world),
            "launch": "one step recorded into a CUDA graph, replayed (fixed Philox offset)"
            if args.cuda_graph else
            "eager: gfx1010_kernels.sharded.sharded_forward_backward(async_op=True, "
            "previous=...) per step (three kernel launches through the extension)",
            "hbm_gbs_step": step_gbs,
            "hbm_frac_of_8000": step_gbs / (HBM_SPEC_GBS * world),
            "hbm_frac_of_measured": step_gbs / (peak * world),
            "kernels": {
                "forward": {"ms": forward_ms, "gbs": fwd_gbs, "bytes_per_row": fwd_row,
                            "includes": "wait for the previous step's all-reduce (N > 1)"},
                "backward": {"ms": backward_ms, "gbs": bwd_gbs, "bytes_per_row": bwd_row,
                             "includes": "the zeroing kernel of the [2,H] buffer"},
            },
            "roofline": {
                "kernel": "rln_backward_kernel",
                "bound": "hbm",
                "achieved": bwd_gbs,
                "peak": peak,
                "peak_kind": f"{peak_kind} copy bandwidth (burst)",
                "unit": "GB/s",
                "frac": bwd_gbs / peak,
                "frac_of_8000": bwd_gbs / HBM_SPEC_GBS,
                "traffic": NCU_BACKWARD_TRAFFIC_BYTES.get(args.workload),
                "traffic_unit": "bytes per launch (ncu dram read + write)",
                "algorithmic_bytes_per_launch": bwd_bytes,
                "timing": "CUDA events around each backward launch, in a pass of the same "
                          "steps right after the timed regions",
            },
            "cpu_baseline": cpu,
            "public_api_device_value": total_rows / (public_ms * 1e-3) if has_public else None,
            "public_api_device_path": "residual_layer_norm(implementation='gfx1010') + "
                                      "torch.autograd.grad on the same device-resident tensors "
                                      "(C++ autograd node, no collective), CUDA events",
            "e2e": None,
            "sharded_check": check,
            "strong_c5": strong,
            "gpu_launches": 3 * args.steps * regions,  # forward, zeroing kernel, backward
            "gpu_launches_per_step": 3,
            "clocks": clocks,
        }
        if e2e is not None:
            e2e_ms, e2e_public_ms, copy_ms, chunked_copy_ms = stats[3:7]
            line["e2e"] = {
                "value": total_rows * e2e["steps"] / (e2e_ms * 1e-3),
                "unit": UNIT,
                "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"],
                "steps": e2e["steps"],
                "path": "one C-ABI call per step on pinned host buffers "
                        "(rln_sm100_host_forward_backward_enqueue via "
                        "gfx1010_kernels.host_pipeline, wait=False): chunked copy-in / fwd+bwd "
                        "kernels / copy-out on three streams, two output sets, at most two "
                        "steps in flight (rln_sm100_host_pipeline_wait_step before a set is "
                        "reused), every step landed before the host clock stops",
                "public_api_value": total_rows * e2e["steps"] / (e2e_public_ms * 1e-3),
                "public_api_path": "pinned host -> device copies, residual_layer_norm("
                                   "implementation='gfx1010') + torch.autograd.grad, results "
                                   "copied to pinned host, one stream",
                "copy_ceiling_value": total_rows * e2e["steps"] / (copy_ms * 1e-3),
                "copy_ceiling_path": "the step's host->device and device->host bytes only, as "
                                     "whole-tensor pinned copies on two streams, no kernels, "
                                     "all ranks at once",
            }
            line["e2e"]["fraction_of_copy_ceiling"] = (
                line["e2e"]["value"] / line["e2e"]["copy_ceiling_value"])
            line["e2e"]["chunked_copy_ceiling_value"] = (
                total_rows * e2e["steps"] / (chunked_copy_ms * 1e-3))
            line["e2e"]["chunked_copy_ceiling_path"] = (
                "the same bytes in the pipeline's own pattern (8,192-row chunks, four copies "
                "in and four out per chunk, two streams), no kernels, no dependencies: what "
                "chunked bidirectional copies reach on this box")
            line["e2e"]["fraction_of_chunked_copy_ceiling"] = (
                line["e2e"]["value"] / line["e2e"]["chunked_copy_ceiling_value"])
        print(json.dumps(line), flush=True)
        checks = [check] + ([strong.get("sharded_check")] if strong else [])
        failed = any(entry is not None and not entry["ok"] for entry in checks)
    if world > 1:
        flag = torch.tensor([1 if failed else 0], device=device)
        dist.broadcast(flag, 0)
        failed = bool(flag.item())
        dist.barrier()
        dist.destroy_process_group()
    return 3 if failed else 0


def run_end_to_end(args, device, host, weight, bias, dropout_p, world, residual_layer_norm,
                   normalized_dtype=torch.float32):
    """The same step with host buffers on both sides, two ways:

    ``pipeline``    one C-ABI call per step (rln_sm100_host_forward_backward_enqueue
                    through gfx1010_kernels.host_pipeline.HostPipeline): chunked
                    copy-in / kernels / copy-out overlapped on three streams, steps
                    double-buffered so that consecutive steps overlap too;
    ``public_api``  pinned host -> device copies, gfx1010_kernels.residual_layer_norm
                    (implementation='gfx1010') + torch.autograd.grad, results copied
                    back to pinned host, all on one stream.
    Both timed regions contain every host<->device byte of a step.  A third leg
    (``copy``) moves the same bytes and launches nothing: the input tensors as
    whole pinned copies on one stream, the result tensors on another, on all
    ranks at once -- the ceiling the host link sets for this step on this box.
    """
    import torch.distributed as dist

    from gfx1010_kernels.host_pipeline import HostPipeline

    host = list(host)
    host[5] = host[5].to(normalized_dtype)
    x_h, branch_h, weight_h, bias_h, gu_h, gy_h = (t.pin_memory() for t in host)
    rows, hidden = x_h.shape
    pipeline = HostPipeline(hidden, branch_h.dtype, chunk_rows=8192, depth=3, device=device,
                            normalized_dtype=normalized_dtype)
    outputs = pipeline.allocate_outputs(x_h.shape)
    second_outputs = pipeline.allocate_outputs(x_h.shape)
    out_updated, out_normalized, out_grad_x, out_grad_branch, out_grad_params = outputs
    weight_leaf = weight.detach().clone().requires_grad_(True)
    bias_leaf = bias.detach().clone().requires_grad_(True)
    h2d = sum(t.numel() * t.element_size() for t in (x_h, branch_h, gu_h, gy_h, weight_h, bias_h))
    d2h = sum(t.numel() * t.element_size() for t in outputs)
    rank = dist.get_rank() if world > 1 else 0
    counter = [0]

    # Double-buffered consumer: step i fills output set i % 2 while set (i - 1) % 2
    # -- complete once wait(step=...) has returned -- belongs to the caller.  At
    # most two steps are in flight, and the second one's first chunks are copied
    # in while the first one's last chunks are computed and copied out.
    output_sets = (outputs, second_outputs)
    in_flight = []          # (pipeline step number, output set) of enqueued steps

    def land(limit):
        """Wait until at most ``limit`` steps are in flight; reduce what landed."""
        while len(in_flight) > limit:
            number, landed = in_flight.pop(0)
            pipeline.wait(step=number)
            if world > 1:
                parameters = landed[4].to(device, non_blocking=True)
                dist.all_reduce(parameters)
                landed[4].copy_(parameters)

    def pipeline_step():
        counter[0] += 1
        land(1)     # the set about to be refilled was consumed two steps ago
        target = output_sets[counter[0] % 2]
        pipeline.forward_backward(
            x_h, branch_h, weight_h, bias_h, gu_h, gy_h, dropout_p, EPS, True,
            seed=0, offset=4 * counter[0], row_base=rank * rows, out=target, wait=False,
        )
        in_flight.append((pipeline.steps_enqueued(), target))

    def public_api_step():
        x = x_h.to(device, non_blocking=True).requires_grad_(True)
        branch = branch_h.to(device, non_blocking=True).requires_grad_(True)
        grad_updated = gu_h.to(device, non_blocking=True)
        grad_normalized = gy_h.to(device, non_blocking=True)
        updated, normalized = residual_layer_norm(
            x, branch, weight_leaf, bias_leaf, dropout_p, EPS, True, implementation="gfx1010",
            normalized_dtype=normalized_dtype,
        )
        grad_x, grad_branch, grad_weight, grad_bias = torch.autograd.grad(
            (updated, normalized), (x, branch, weight_leaf, bias_leaf),
            (grad_updated, grad_normalized),
        )
        parameters = torch.stack((grad_weight, grad_bias))
        if world > 1:
            dist.all_reduce(parameters)
        out_updated.copy_(updated.detach(), non_blocking=True)
        out_normalized.copy_(normalized.detach(), non_blocking=True)
        out_grad_x.copy_(grad_x, non_blocking=True)
        out_grad_branch.copy_(grad_branch, non_blocking=True)
        out_grad_params.copy_(parameters, non_blocking=True)

    def timed(step, steps):
        for _ in range(2):
            step()
        land(0)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        begin = time.perf_counter()
        for _ in range(steps):
            step()
        land(0)     # every enqueued step has landed in host memory (and is reduced)
        torch.cuda.synchronize()
        elapsed = (time.perf_counter() - begin) * 1e3
        if world > 1:
            dist.barrier()
        return elapsed

    in_stream = torch.cuda.Stream(device)
    out_stream = torch.cuda.Stream(device)
    host_inputs = (x_h, branch_h, gu_h, gy_h)
    device_inputs = [torch.empty_like(t, device=device) for t in host_inputs]
    device_outputs = [torch.empty_like(t, device=device) for t in outputs[:4]]

    def copy_step():
        with torch.cuda.stream(in_stream):
            for target, source in zip(device_inputs, host_inputs):
                target.copy_(source, non_blocking=True)
        with torch.cuda.stream(out_stream):
            for target, source in zip(outputs[:4], device_outputs):
                target.copy_(source, non_blocking=True)

    def chunked_copy_step():
        # the pipeline's own copy pattern -- per 8,192-row chunk four copies in, four
        # out -- with no kernels and no dependency between the two directions
        for begin in range(0, rows, pipeline.chunk_rows):
            end = min(rows, begin + pipeline.chunk_rows)
            with torch.cuda.stream(in_stream):
                for target, source in zip(device_inputs, host_inputs):
                    target[begin:end].copy_(source[begin:end], non_blocking=True)
            with torch.cuda.stream(out_stream):
                for target, source in zip(outputs[:4], device_outputs):
                    target[begin:end].copy_(source[begin:end], non_blocking=True)

    steps = max(2, min(args.steps, 6))
    pipeline_ms = timed(pipeline_step, steps)
    public_ms = timed(public_api_step, steps)
    copy_ms = timed(copy_step, steps)
    chunked_copy_ms = timed(chunked_copy_step, steps)
    pipeline.close()
    return {"ms": pipeline_ms, "public_ms": public_ms, "copy_ms": copy_ms,
            "chunked_copy_ms": chunked_copy_ms, "steps": steps, "h2d": h2d, "d2h": d2h}


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=("native", "reference"), default="native")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default="h768_64Mi")
    parser.add_argument("--regions", type=int, default=REGIONS,
                        help="back-to-back timed regions of K steps; the median is reported")
    parser.add_argument("--no-strong-c5", action="store_true",
                        help="skip the strong-scaling record (the [64,4096,1024] batch split "
                             "over the GPUs), which the headline workload's run appends")
    parser.add_argument("--cuda-graph", action="store_true",
                        help="N = 1: record one step into a CUDA graph and time its replays "
                             "(what a caller does for launch-bound shapes)")
    parser.add_argument("--default-priority-collectives", action="store_true",
                        help="N > 1: run NCCL on a default-priority stream (A/B switch)")
    parser.add_argument(
        "--kernel-only",
        action="store_true",
        help="profiling mode: exactly W warm-up steps, no clock-settling warm-up, three "
             "timed regions, no end-to-end leg and no CPU baseline (few launches, so that "
             "a profiler capture of this command ends quickly)",
    )
    args = parser.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        return run_reference_arm(args, rank)

    if args.gpus > 1 and world == 1:
        # convenience: launch ourselves under torchrun
        command = [
            sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
            f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
            "--master-port", os.environ.get("MASTER_PORT", "29517"),
            str(Path(__file__).resolve()), *sys.argv[1:],
        ]
        return subprocess.call(command)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    return run_native_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    sys.exit(main())
