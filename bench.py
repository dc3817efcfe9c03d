"""Benchmark of the fused residual-add + dropout + LayerNorm training step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + one backward of the operator over one batch of
synthetic rows (plus, on N > 1 GPUs, the NCCL all-reduce of the [2, H]
grad_weight/grad_bias buffer).  The headline workload is H = 768 on 64 Mi fp32
elements (87,381 rows, fp16 branch, dropout 0.1) per GPU; rows are sharded, so
N GPUs process N x 87,381 rows of one global batch (weak scaling) and every
rank passes its global row offset so that the dropout mask is the one of the
unsharded call.

Rank 0 prints ONE JSON line.  ``value`` is rows/s with inputs resident in HBM;
``e2e`` is the same metric with inputs in pinned host memory and results copied
back to the host inside the timed region; ``roofline`` describes the dominant
kernel (the backward) against the measured HBM peak; ``cpu_baseline`` is the
torch decomposition (the reference's CPU path) timed on this machine's cores.
``--impl reference`` times only that CPU path.
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
    "h768_64Mi": 814_518_016 + 363_732_992,
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

    def summary(self, begin, end):
        window = [(mhz, bits) for (stamp, mhz, bits) in self.samples if begin <= stamp <= end]
        if not window:
            window = [(mhz, bits) for (_, mhz, bits) in self.samples]
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for _, sample_bits in window:
            bits |= sample_bits
        reasons = [name for bit, name in self.REASONS.items() if bits & bit and name != "gpu_idle"]
        return {
            "sm_mhz": int(statistics.median(mhz for mhz, _ in window)),
            "sm_max_mhz": self.max_mhz,
            "reasons": reasons,
            "samples": len(window),
        }


def time_cpu_reference(rows, hidden, branch_dtype, dropout_p, steps, warmup,
                       normalized_dtype=torch.float32):
    """The reference's CPU path: its torch decomposition (F.dropout -> add ->
    F.layer_norm) forward plus torch.autograd.grad, on all host threads."""
    from oracle import rln_oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        rows, hidden, branch_dtype, seed=0
    )
    leaves = [t.requires_grad_(True) for t in (x, branch, weight, bias)]
    grad_normalized = grad_normalized.to(normalized_dtype)
    times = []
    for index in range(warmup + steps):
        begin = time.perf_counter()
        outputs = rln_oracle.torch_decomposition(
            *leaves, dropout_p, EPS, True, None, normalized_dtype
        )
        torch.autograd.grad(outputs, leaves, (grad_updated, grad_normalized))
        elapsed = time.perf_counter() - begin
        if index >= warmup:
            times.append(elapsed)
    return times, threads


def run_reference_arm(args, rank):
    if rank != 0:
        return 0
    rows_full, hidden, branch_dtype, dropout_p, normalized_dtype = workload(args.workload)
    rows = min(rows_full, CPU_SAMPLE_ROWS)
    times, threads = time_cpu_reference(
        rows, hidden, branch_dtype, dropout_p, args.steps, args.warmup, normalized_dtype
    )
    total = sum(times)
    value = rows * len(times) / total
    sample = (
        f"first {rows} rows of the {rows_full}-row workload per step "
        f"(x fp32 [{rows},{hidden}], branch {str(branch_dtype).split('.')[-1]}, p={dropout_p})"
    )
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
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
            "value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


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


def run_native_arm(args, rank, local_rank, world):
    import torch.distributed as dist

    from gfx1010_kernels import _C, residual_layer_norm, residual_layer_norm_status

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl native needs a CUDA device (no CPU fallback)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    status = residual_layer_norm_status(device)
    if not status.available:
        raise RuntimeError(f"native backend unavailable: {status.reason}")
    if world > 1:
        # a short timeout: a rank that stops calling collectives must surface as an
        # error within minutes, not hold the GPUs for the default ten
        # NCCL on a high-priority stream: the all-reduce of step i is launched
        # while the forward of step i+1 already fills every SM with short CTAs;
        # at equal priority its CTAs are placed only after the forward's grid has
        # been handed out, i.e. at the forward's tail, and part of its latency
        # shows.  With priority it takes the first slots that free up.
        options = None
        if not args.default_priority_collectives:
            options = dist.ProcessGroupNCCL.Options()
            options.is_high_priority_stream = True
        dist.init_process_group(
            "nccl", device_id=device, timeout=datetime.timedelta(seconds=120),
            pg_options=options,
        )

    rows, hidden, branch_dtype, dropout_p, normalized_dtype = workload(args.workload)
    branch_bytes = 4 if branch_dtype == torch.float32 else 2
    normalized_bytes = 4 if normalized_dtype == torch.float32 else 2
    skip_e2e = args.kernel_only
    host = draw_inputs(rows, hidden, branch_dtype, seed=rank)
    x, branch, weight, bias, grad_updated, grad_normalized = (t.to(device) for t in host)
    grad_normalized = grad_normalized.to(normalized_dtype)
    if world > 1:
        # replicated parameters: every rank uses rank 0's values
        dist.broadcast(weight, 0)
        dist.broadcast(bias, 0)
    row_base = rank * rows
    seed = 0
    flush = None
    if rows * hidden * 4 <= 126e6:
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=device)

    def flush_l2():
        # Write a buffer twice the size of L2, then read it: the write evicts the
        # workload's lines, the read pushes the write's dirty lines out to HBM, so
        # that the kernel that runs next is not billed for their write-back.
        flush.zero_()
        flush.sum()


    forward_events, backward_events = [], []
    pending = []

    def finish_pending():
        while pending:
            work, _buffer = pending.pop()
            work.wait()

    def step(index, record):
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e2 = torch.cuda.Event(enable_timing=True)
            e0.record()
        updated, normalized, mean, rstd, mask = _C.residual_layer_norm_forward_seeded(
            x, branch, weight, bias, dropout_p, EPS, True, 128, seed, 4 * index, row_base,
            NORMALIZED_CODES[normalized_dtype],
        )
        # The backward is a persistent grid that fills every SM exactly once; a
        # communication kernel still resident from the previous step would push
        # part of it into a second wave.  So the previous all-reduce may overlap
        # the forward (dynamically scheduled CTAs) but must be done before this.
        finish_pending()
        if record:
            e1.record()
        gradients = _C.residual_layer_norm_backward(
            grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
            dropout_p, True, BRANCH_CODES[branch_dtype], 128, 64, 256, 1, True,
        )
        if record:
            e2.record()
            forward_events.append((e0, e1))
            backward_events.append((e1, e2))
        if world > 1:
            # grad_weight and grad_bias are views of one [2, H] buffer.  The all-reduce
            # is asynchronous: it runs on NCCL's stream under the NEXT step's forward
            # (which does not depend on it) and is waited for before that step's
            # backward is launched, and once more before the timed region ends.
            buffer = gradients[2]._base if gradients[2]._base is not None else gradients[2]
            pending.append((dist.all_reduce(buffer, async_op=True), buffer))
        return normalized, gradients

    def fence():
        finish_pending()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()

    # warm-up: W steps, then as many more as bring the loaded span to about a second
    # (clock settling + clock samples).  The count is agreed between the ranks --
    # every step contains a collective, so all ranks must run the same number.
    def warm(count, first):
        for index in range(count):
            if flush is not None:
                flush_l2()
            step(first + index, False)
            if index % 50 == 49:
                torch.cuda.synchronize()
        torch.cuda.synchronize()

    warm_begin = time.perf_counter()
    base = max(args.warmup, 3)
    warm(base, 0)
    warmup_actual = base
    if not args.kernel_only:
        probe_begin = time.perf_counter()
        warm(10, base)          # timed probe (the first steps above carry one-time set-up)
        warmup_actual += 10
        per_step = (time.perf_counter() - probe_begin) / 10
        extra = int(min(5000, 1.0 / max(per_step, 1e-6)))
        if world > 1:
            agreed = torch.tensor([extra], device=device, dtype=torch.int64)
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
            extra = int(agreed.item())
        warm(extra, warmup_actual)
        warmup_actual += extra

    run_step = step
    if args.cuda_graph:
        if world > 1:
            raise RuntimeError("--cuda-graph is a single-GPU mode")
        # One step (forward, zeroing kernel, backward and the allocator's work)
        # recorded once; every replay re-runs it with the recorded Philox offset.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_outputs = step(warmup_actual, False)

        def run_step(index, record):
            graph.replay()
            return graph_outputs

        for _ in range(10):
            run_step(0, False)

    fence()
    timed_begin = time.perf_counter()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    step_events = []
    start.record()
    for index in range(args.steps):
        if flush is not None:
            # the L2 flush is not part of a step: bracket every step on its own
            flush_l2()
            begin_event = torch.cuda.Event(enable_timing=True)
            end_event = torch.cuda.Event(enable_timing=True)
            begin_event.record()
        run_step(warmup_actual + index, args.kernel_events_in_loop)
        if flush is not None:
            end_event.record()
            step_events.append((begin_event, end_event))
    finish_pending()
    stop.record()
    fence()
    timed_end = time.perf_counter()
    elapsed_ms = start.elapsed_time(stop)
    if step_events:
        elapsed_ms = sum(a.elapsed_time(b) for a, b in step_events)
    if not args.kernel_events_in_loop:
        # per-kernel durations: same steps, same buffers, right after the timed region
        for index in range(min(args.steps, 100)):
            if flush is not None:
                flush_l2()
            step(warmup_actual + args.steps + index, True)
        finish_pending()
        torch.cuda.synchronize()
    forward_ms = statistics.mean(a.elapsed_time(b) for a, b in forward_events)
    backward_ms = statistics.mean(a.elapsed_time(b) for a, b in backward_events)
    clocks = sampler.summary(timed_begin, timed_end)
    if clocks["samples"] < 2:
        clocks = sampler.summary(warm_begin, timed_end)
        clocks["window"] = "warm-up + timed region (timed region shorter than the sampling interval)"

    # end-to-end: pinned host inputs -> device -> public API fwd+bwd -> results back to host
    if skip_e2e:
        e2e = {"ms": float("nan"), "public_ms": float("nan"), "steps": 0, "h2d": 0, "d2h": 0}
    else:
        e2e = run_end_to_end(
            args, device, host, weight, bias, dropout_p, world, residual_layer_norm,
            normalized_dtype,
        )
    sampler.stop()

    if world > 1:
        stats = torch.tensor(
            [elapsed_ms, e2e["ms"], forward_ms, backward_ms, e2e.get("public_ms", 0.0)],
            device=device, dtype=torch.float64,
        )
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, forward_ms, backward_ms, e2e_public_ms = stats.tolist()
    else:
        e2e_ms = e2e["ms"]
        e2e_public_ms = e2e.get("public_ms", 0.0)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        total_rows = rows * world
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
            sample_rows = min(rows, CPU_SAMPLE_ROWS)
            times, threads = time_cpu_reference(
                sample_rows, hidden, branch_dtype, dropout_p, 5, 1, normalized_dtype
            )
            cpu = {
                "value": sample_rows / statistics.median(times),
                "unit": UNIT,
                "cores": threads,
                "kind": "port",
                "sample": f"first {sample_rows} rows of the workload, median of 5 fwd+bwd runs "
                          "of the torch decomposition (F.dropout + add + F.layer_norm + autograd)",
            }
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
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
            if args.cuda_graph else "eager (three launches per step through the extension)",
            "hbm_gbs_step": step_gbs,
            "hbm_frac_of_8000": step_gbs / (HBM_SPEC_GBS * world),
            "hbm_frac_of_measured": step_gbs / (peak * world),
            "kernels": {
                "forward": {"ms": forward_ms, "gbs": fwd_gbs, "bytes_per_row": fwd_row},
                "backward": {"ms": backward_ms, "gbs": bwd_gbs, "bytes_per_row": bwd_row},
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
                "timing": "CUDA events around each backward launch, "
                          + ("inside the timed steps" if args.kernel_events_in_loop
                             else "in a pass of the same steps right after the timed region"),
            },
            "cpu_baseline": cpu,
            "e2e": None if skip_e2e else {
                "value": total_rows * e2e["steps"] / (e2e_ms * 1e-3),
                "unit": UNIT,
                "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"],
                "steps": e2e["steps"],
                "path": "one C-ABI call per step on pinned host buffers "
                        "(rln_sm100_host_forward_backward via gfx1010_kernels.host_pipeline): "
                        "chunked copy-in / fwd+bwd kernels / copy-out on three streams; timed "
                        "on the host clock around synchronous calls",
                "public_api_value": total_rows * e2e["steps"] / (e2e_public_ms * 1e-3),
                "public_api_path": "pinned host -> device copies, residual_layer_norm("
                                   "implementation='gfx1010') + torch.autograd.grad, results "
                                   "copied to pinned host, one stream",
            },
            "gpu_launches": 3 * args.steps,  # forward, zeroing kernel, backward
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_end_to_end(args, device, host, weight, bias, dropout_p, world, residual_layer_norm,
                   normalized_dtype=torch.float32):
    """The same step with host buffers on both sides, two ways:

    ``pipeline``    one C-ABI call (rln_sm100_host_forward_backward through
                    gfx1010_kernels.host_pipeline.HostPipeline): chunked copy-in /
                    kernels / copy-out overlapped on three streams;
    ``public_api``  pinned host -> device copies, gfx1010_kernels.residual_layer_norm
                    (implementation='gfx1010') + torch.autograd.grad, results copied
                    back to pinned host, all on one stream.
    Both timed regions contain every host<->device byte of a step.
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
    out_updated, out_normalized, out_grad_x, out_grad_branch, out_grad_params = outputs
    weight_leaf = weight.detach().clone().requires_grad_(True)
    bias_leaf = bias.detach().clone().requires_grad_(True)
    h2d = sum(t.numel() * t.element_size() for t in (x_h, branch_h, gu_h, gy_h, weight_h, bias_h))
    d2h = sum(t.numel() * t.element_size() for t in outputs)
    rank = dist.get_rank() if world > 1 else 0
    counter = [0]

    def pipeline_step():
        counter[0] += 1
        pipeline.forward_backward(
            x_h, branch_h, weight_h, bias_h, gu_h, gy_h, dropout_p, EPS, True,
            seed=0, offset=4 * counter[0], row_base=rank * rows, out=outputs,
        )
        if world > 1:
            parameters = out_grad_params.to(device, non_blocking=True)
            dist.all_reduce(parameters)
            out_grad_params.copy_(parameters)

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
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        begin = time.perf_counter()
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
        elapsed = (time.perf_counter() - begin) * 1e3
        if world > 1:
            dist.barrier()
        return elapsed

    steps = max(2, min(args.steps, 5))
    pipeline_ms = timed(pipeline_step, steps)
    public_ms = timed(public_api_step, steps)
    pipeline.close()
    return {"ms": pipeline_ms, "public_ms": public_ms, "steps": steps, "h2d": h2d, "d2h": d2h}


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=("native", "reference"), default="native")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default="h768_64Mi")
    parser.add_argument("--cuda-graph", action="store_true",
                        help="N = 1: record one step into a CUDA graph and time its replays "
                             "(what a caller does for launch-bound shapes)")
    parser.add_argument("--default-priority-collectives", action="store_true",
                        help="N > 1: run NCCL on a default-priority stream (A/B switch)")
    parser.add_argument(
        "--kernel-events-in-loop",
        action="store_true",
        help="record the per-kernel CUDA events inside the K timed steps instead of in a "
             "pass of their own right after them (an event between two kernels keeps the "
             "second from being scheduled while the first drains, which slows the step)",
    )
    parser.add_argument(
        "--kernel-only",
        action="store_true",
        help="profiling mode: exactly W warm-up steps, no clock-settling warm-up, no "
             "end-to-end leg and no CPU baseline (few launches, so that a profiler "
             "capture of this command ends quickly)",
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
