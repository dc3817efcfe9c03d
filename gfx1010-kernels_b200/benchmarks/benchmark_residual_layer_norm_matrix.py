"""Public-API timing matrix: native kernels vs the torch decomposition on the same GPU.

The counterpart of the reference project's
``benchmarks/benchmark_residual_layer_norm_matrix.py`` (:52-69 timing method,
:183-227 matrix): for every (tokens, hidden) cell it times the forward and the
forward+backward of ``residual_layer_norm`` through the public API with
``implementation="gfx1010"`` and with ``implementation="torch"``, using CUDA
events (warm-up, then N measured iterations; median, p20, p80), and prints one
JSON line per cell with the two speed-ups.  The defaults reproduce the setup of
the reference's published table (B=1, H=384, fp32 residual stream, fp16
branch, dropout 0.15, T in 128..4096).

    python benchmarks/benchmark_residual_layer_norm_matrix.py [--hidden 384 768] [--tokens ...]
"""

import argparse
import json
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from gfx1010_kernels import residual_layer_norm, residual_layer_norm_status  # noqa: E402


def percentile(values, fraction):
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, int(fraction * len(ordered)))]


def time_cuda(function, warmup, iterations):
    for _ in range(warmup):
        function()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iterations):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        function()
        stop.record()
        stop.synchronize()
        samples.append(start.elapsed_time(stop))
    return {
        "median_ms": statistics.median(samples),
        "p20_ms": percentile(samples, 0.2),
        "p80_ms": percentile(samples, 0.8),
    }


def make_cell(tokens, hidden, branch_dtype, dropout_p, implementation, normalized_dtype=None):
    x = torch.randn(1, tokens, hidden, device="cuda", requires_grad=True)
    branch = torch.randn(1, tokens, hidden, device="cuda", dtype=branch_dtype, requires_grad=True)
    weight = torch.randn(hidden, device="cuda", requires_grad=True)
    bias = torch.randn(hidden, device="cuda", requires_grad=True)
    grad_updated = torch.randn(1, tokens, hidden, device="cuda")
    grad_normalized = torch.randn(1, tokens, hidden, device="cuda").to(
        normalized_dtype or torch.float32
    )

    def forward():
        with torch.no_grad():
            return residual_layer_norm(
                x, branch, weight, bias, dropout_p, 1e-5, True, implementation=implementation,
                normalized_dtype=normalized_dtype,
            )

    def training():
        outputs = residual_layer_norm(
            x, branch, weight, bias, dropout_p, 1e-5, True, implementation=implementation,
            normalized_dtype=normalized_dtype,
        )
        return torch.autograd.grad(
            outputs, (x, branch, weight, bias), (grad_updated, grad_normalized)
        )

    return forward, training


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--hidden", type=int, nargs="+", default=[384])
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 256, 512, 1024, 2048, 4096])
    parser.add_argument("--dropout", type=float, default=0.15)
    parser.add_argument("--branch-dtype", choices=("float16", "float32", "bfloat16"),
                        default="float16")
    parser.add_argument("--normalized-dtype", choices=("float32", "float16", "bfloat16"),
                        default="float32",
                        help="type of the `normalized` output (float32 = the reference's contract)")
    parser.add_argument("--warmup", type=int, default=100)
    parser.add_argument("--iterations", type=int, default=1000)
    arguments = parser.parse_args()

    status = residual_layer_norm_status()
    if not status.available:
        raise SystemExit(f"native backend unavailable: {status.reason}")
    branch_dtype = getattr(torch, arguments.branch_dtype)
    normalized_dtype = getattr(torch, arguments.normalized_dtype)
    for hidden in arguments.hidden:
        for tokens in arguments.tokens:
            record = {
                "device": status.device, "tokens": tokens, "hidden": hidden,
                "branch_dtype": arguments.branch_dtype,
                "normalized_dtype": arguments.normalized_dtype, "dropout_p": arguments.dropout,
                "warmup": arguments.warmup, "iterations": arguments.iterations,
            }
            for implementation in ("gfx1010", "torch"):
                forward, training = make_cell(
                    tokens, hidden, branch_dtype, arguments.dropout, implementation,
                    normalized_dtype,
                )
                record[f"{implementation}_forward"] = time_cuda(
                    forward, arguments.warmup, arguments.iterations
                )
                record[f"{implementation}_training"] = time_cuda(
                    training, arguments.warmup, arguments.iterations
                )
            record["forward_speedup"] = (
                record["torch_forward"]["median_ms"] / record["gfx1010_forward"]["median_ms"]
            )
            record["training_speedup"] = (
                record["torch_training"]["median_ms"] / record["gfx1010_training"]["median_ms"]
            )
            print(json.dumps(record), flush=True)


if __name__ == "__main__":
    main()
