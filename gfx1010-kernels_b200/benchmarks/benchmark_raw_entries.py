"""Raw-entry timings: vectorised vs scalar kernels, and the parameter-gradient paths.

One script for the questions the reference project answers with three
(``benchmarks/benchmark_forward_vectorization.py``,
``benchmark_backward_vectorization.py`` and ``benchmark_parameter_reduction.py``),
asked of the sm_100a kernels through the same raw ``_C`` entry points:

``forward``    ``_C.residual_layer_norm_forward`` on 16-byte aligned tensors (the
               128-bit-per-lane kernels) against the same call on tensors whose
               storage starts 4 bytes off (the scalar kernels with identical
               results) -- what the alignment predicate of the dispatch buys;
``backward``   the same comparison for ``_C.residual_layer_norm_backward``;
``parameters`` the backward without parameter gradients, with the atomic path,
               and with the fixed-order path of
               ``torch.use_deterministic_algorithms(True)`` (partials + second
               kernel): what grad_weight / grad_bias cost on top of the
               row-local gradients.  In deterministic mode torch also fills
               every fresh output tensor with NaN before the kernels run;
               ``--disable-deterministic-fill`` takes that out of the figure.

Before any timing the scalar and deterministic results are compared with the
vectorised / atomic ones (bit-identical row-local outputs, parameter sums
within 1e-4 relative).  Timing: CUDA events around each call after a warm-up,
median over ``--reps``, the two sides of a comparison alternating from round to
round.  One JSON line per (mode, T, C).

    python benchmarks/benchmark_raw_entries.py --modes forward backward parameters \
        --sequences 2048 32768 --hidden 384 768 1024
"""

import argparse
import json
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from gfx1010_kernels import _C  # noqa: E402

DROPOUT_P = 0.1
EPS = 1e-5
# the launch integers of the reference's entries: range-checked, otherwise unused here
THREADS, BLOCK_ROWS, PARAMETER_THREADS, PARAMETER_GROUPS = 128, 64, 256, 1


def median_ms(call, warmup, reps):
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    samples = []
    for _ in range(reps):
        begin = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        begin.record()
        call()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end))
    return statistics.median(samples)


def alternate(sides, rounds, warmup, reps):
    """``sides``: name -> call.  Every round times all sides, the order rotating;
    returns name -> median over the rounds."""
    names = list(sides)
    collected = {name: [] for name in names}
    for round_index in range(rounds):
        shift = round_index % len(names)
        for name in names[shift:] + names[:shift]:
            collected[name].append(median_ms(sides[name], warmup, reps))
    return {name: statistics.median(values) for name, values in collected.items()}


def off_by_four_bytes(tensor):
    """A contiguous copy of ``tensor`` whose first element sits 4 bytes (fp32) or
    2 bytes (16-bit types) past a 16-byte boundary."""
    storage = torch.empty(tensor.numel() + 8, dtype=tensor.dtype, device=tensor.device)
    shifted = storage[1:1 + tensor.numel()].view(tensor.shape)
    shifted.copy_(tensor)
    assert shifted.data_ptr() % 16 != 0
    return shifted


def make_problem(tokens, hidden):
    generator = torch.Generator(device="cuda").manual_seed(tokens * 7 + hidden)
    def normal(*shape, dtype=torch.float32):
        return torch.randn(*shape, device="cuda", generator=generator).to(dtype)
    return {
        "x": normal(tokens, hidden), "branch": normal(tokens, hidden, dtype=torch.float16),
        "weight": 1.0 + 0.1 * normal(hidden), "bias": 0.1 * normal(hidden),
        "grad_updated": normal(tokens, hidden), "grad_normalized": normal(tokens, hidden),
    }


def forward_seeded(p, seed=3, offset=8):
    return _C.residual_layer_norm_forward_seeded(
        p["x"], p["branch"], p["weight"], p["bias"], DROPOUT_P, EPS, True, THREADS,
        seed, offset, 0, 0)


def backward(p, saved, parameters=True):
    updated, _, mean, rstd, mask = saved
    return _C.residual_layer_norm_backward(
        p["grad_updated"], p["grad_normalized"], updated, p["weight"], mean, rstd, mask,
        DROPOUT_P, True, 1, THREADS, BLOCK_ROWS, PARAMETER_THREADS, PARAMETER_GROUPS, parameters)


def run_forward(tokens, hidden, args):
    aligned = make_problem(tokens, hidden)
    shifted = {key: off_by_four_bytes(value) for key, value in aligned.items()}
    reference = forward_seeded(aligned)
    scalar = forward_seeded(shifted)
    identical = all(torch.equal(a, b) for a, b in zip(reference, scalar))
    times = alternate(
        {"vector": lambda: forward_seeded(aligned), "scalar": lambda: forward_seeded(shifted)},
        args.rounds, args.warmup, args.reps)
    return {"mode": "forward", "T": tokens, "C": hidden, "scalar_equals_vector": identical,
            "vector_ms": times["vector"], "scalar_ms": times["scalar"],
            "speedup": times["scalar"] / times["vector"]}


def run_backward(tokens, hidden, args):
    aligned = make_problem(tokens, hidden)
    saved = forward_seeded(aligned)
    shifted = {key: off_by_four_bytes(value) for key, value in aligned.items()}
    shifted_saved = (off_by_four_bytes(saved[0]), None, saved[2], saved[3], saved[4])
    reference = backward(aligned, saved)
    scalar = backward(shifted, shifted_saved)
    identical = torch.equal(reference[0], scalar[0]) and torch.equal(reference[1], scalar[1])
    sums_close = all(
        torch.allclose(a, b, rtol=1e-4, atol=1e-5 * tokens ** 0.5)
        for a, b in zip(reference[2:], scalar[2:]))
    times = alternate(
        {"vector": lambda: backward(aligned, saved),
         "scalar": lambda: backward(shifted, shifted_saved)},
        args.rounds, args.warmup, args.reps)
    return {"mode": "backward", "T": tokens, "C": hidden,
            "scalar_equals_vector": identical, "parameter_sums_close": sums_close,
            "vector_ms": times["vector"], "scalar_ms": times["scalar"],
            "speedup": times["scalar"] / times["vector"]}


def run_parameters(tokens, hidden, args):
    problem = make_problem(tokens, hidden)
    saved = forward_seeded(problem)

    def deterministic_call():
        torch.use_deterministic_algorithms(True)
        try:
            return backward(problem, saved)
        finally:
            torch.use_deterministic_algorithms(False)

    atomic = backward(problem, saved)
    fixed = deterministic_call()
    again = deterministic_call()
    none = backward(problem, saved, parameters=False)
    row_local = all(torch.equal(atomic[i], other[i]) for other in (fixed, none) for i in (0, 1))
    replay = torch.equal(fixed[2], again[2]) and torch.equal(fixed[3], again[3])
    sums_close = all(
        torch.allclose(a, b, rtol=1e-4, atol=1e-5 * tokens ** 0.5)
        for a, b in zip(atomic[2:], fixed[2:]))
    times = alternate(
        {"without": lambda: backward(problem, saved, parameters=False),
         "atomic": lambda: backward(problem, saved),
         "deterministic": deterministic_call},
        args.rounds, args.warmup, args.reps)
    return {"mode": "parameters", "T": tokens, "C": hidden,
            "row_local_outputs_identical": row_local, "deterministic_replay_bitwise": replay,
            "parameter_sums_close": sums_close,
            "without_ms": times["without"], "atomic_ms": times["atomic"],
            "deterministic_ms": times["deterministic"],
            "atomic_over_without": times["atomic"] / times["without"],
            "deterministic_over_atomic": times["deterministic"] / times["atomic"]}


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--modes", nargs="+", default=("forward", "backward", "parameters"),
                        choices=("forward", "backward", "parameters"))
    parser.add_argument("--sequences", type=int, nargs="+", default=(1024, 8192, 32768))
    parser.add_argument("--hidden", type=int, nargs="+", default=(128, 256, 384, 512, 768, 1024))
    parser.add_argument("--warmup", type=int, default=50)
    parser.add_argument("--reps", type=int, default=200)
    parser.add_argument("--rounds", type=int, default=3)
    parser.add_argument(
        "--disable-deterministic-fill", action="store_true",
        help="switch off torch.utils.deterministic.fill_uninitialized_memory: in deterministic "
             "mode torch fills every freshly allocated output with NaN, which the 'deterministic' "
             "column otherwise includes (the reference's benchmark has the same switch)")
    args = parser.parse_args(argv)
    if args.disable_deterministic_fill:
        torch.utils.deterministic.fill_uninitialized_memory = False
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    runners = {"forward": run_forward, "backward": run_backward, "parameters": run_parameters}
    failed = False
    for mode in args.modes:
        for tokens in args.sequences:
            for hidden in args.hidden:
                line = runners[mode](tokens, hidden, args)
                failed = failed or any(value is False for value in line.values())
                print(json.dumps(line), flush=True)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
