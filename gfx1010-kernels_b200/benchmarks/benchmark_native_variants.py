"""Raw-kernel variant benchmark: arithmetic switches and launch geometry, A/B on one board.

The counterpart of the reference project's ``benchmarks/benchmark_native_variants.py``
and ``benchmark_parameter_reduction.py:87-130``: those sweep the launch knobs
of the HIP kernels (threads, block_rows, parameter_threads, parameter_groups)
through the raw ``_C`` entries.  Here the knobs are template parameters and
compile-time switches, so every variant is a build of its own:
``native_variants/variant_unit.cu`` is compiled once per entry of ``VARIANTS``
(nvcc, sm_100a) into ``native_variants/build/librln_variant_<name>.so`` and all
of them are driven from this process on the same buffers.

Like ``benchmark_residual_layer_norm.py:85-212`` of the reference, every variant
is first CHECKED against the shipped library (``gfx1010_kernels._C``): dropout
mask and ``updated`` bit for bit, the other outputs within the test
tolerances, kept fraction reported.  A variant that fails is not timed.

Timing: the board is warmed for ``--heat`` seconds, then for ``--rounds``
rounds every variant enqueues ``--steps`` steps back to back (forward + zeroing
kernel + backward chained by programmatic dependent launch, fresh Philox offset
per step) between two CUDA events; the median over the rounds is reported per
mode (``step`` = forward + backward, ``forward``, ``backward``).  The variants
take turns inside each round and the order rotates from round to round, so
that slow clock drift under the power cap hits all alike.

    python benchmarks/benchmark_native_variants.py --hidden 768 --rows 87381
    python benchmarks/benchmark_native_variants.py --hidden 1024 --rows 32768 --only shipped bwd_dynamic_tail3
    python benchmarks/benchmark_native_variants.py --build-only      # no GPU needed

One JSON line per variant on stdout.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import statistics
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
PACKAGE_ROOT = HERE.parent
REPO = PACKAGE_ROOT.parent
SOURCE = HERE / "native_variants" / "variant_unit.cu"
BUILD = HERE / "native_variants" / "build"
sys.path.insert(0, str(PACKAGE_ROOT))

# name -> macros.  "shipped" builds the templates exactly as the library does.
VARIANTS = {
    "shipped": {},
    # arithmetic switches
    "packed_math": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1},
    "mask_redux": {"RLN_FWD_MASK_REDUX": 1},
    "packed_redux": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "RLN_FWD_MASK_REDUX": 1},
    "scalar_math": {"VARIANT_PACKED_FWD": 0, "VARIANT_PACKED_BWD": 0},
    "packed_forward": {"VARIANT_PACKED_FWD": 1},
    "packed_backward": {"VARIANT_PACKED_BWD": 1},
    # row hand-out of the backward
    "bwd_static": {"VARIANT_BWD_DYNAMIC": 0},
    "bwd_dynamic_all": {"VARIANT_BWD_DYNAMIC": 1000000000},
    "bwd_dynamic_tail1": {"VARIANT_BWD_DYNAMIC": 1},
    "bwd_dynamic_tail2": {"VARIANT_BWD_DYNAMIC": 2},
    "bwd_dynamic_tail3": {"VARIANT_BWD_DYNAMIC": 3},
    "bwd_dynamic_tail6": {"VARIANT_BWD_DYNAMIC": 6},
    "packed_redux_c16": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "RLN_FWD_MASK_REDUX": 1,
                         "VARIANT_FWD_WARPS": 1, "VARIANT_FWD_MIN_CTAS": 16},
    "packed_redux_c20": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "RLN_FWD_MASK_REDUX": 1,
                         "VARIANT_FWD_WARPS": 1, "VARIANT_FWD_MIN_CTAS": 20},
    # the forward's first CTA clears the [2, H] buffer; no zeroing kernel in the step
    "zero_in_forward": {"VARIANT_ZERO_IN_FORWARD": 1},
    # cache policy
    "stream_hints": {"VARIANT_STREAM_HINTS": 1},
    # forward geometry (wide rows): warps per CTA x resident CTAs per SM
    "fwd_w1_c16": {"VARIANT_FWD_WARPS": 1, "VARIANT_FWD_MIN_CTAS": 16},
    "fwd_w1_c18": {"VARIANT_FWD_WARPS": 1, "VARIANT_FWD_MIN_CTAS": 18},
    "fwd_w1_c20": {"VARIANT_FWD_WARPS": 1, "VARIANT_FWD_MIN_CTAS": 20},
    "fwd_w2_c8": {"VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 8},
    "fwd_w2_c10": {"VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 10},
    "fwd_w2_c12": {"VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 12},
    "fwd_w2_c16": {"VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 16},
    "packed_w2_c10": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 10},
    "packed_w2_c12": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 12},
    "packed_w2_c16": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "VARIANT_FWD_WARPS": 2, "VARIANT_FWD_MIN_CTAS": 16},
    "packed_w4_c6": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "VARIANT_FWD_WARPS": 4, "VARIANT_FWD_MIN_CTAS": 6},
    "packed_w4_c8": {"VARIANT_PACKED_FWD": 1, "VARIANT_PACKED_BWD": 1, "VARIANT_FWD_WARPS": 4, "VARIANT_FWD_MIN_CTAS": 8},
    "fwd_w4_c4": {"VARIANT_FWD_WARPS": 4, "VARIANT_FWD_MIN_CTAS": 4},
    "fwd_w4_c5": {"VARIANT_FWD_WARPS": 4, "VARIANT_FWD_MIN_CTAS": 5},
    # backward geometry: warps per CTA x CTAs per SM
    "bwd_w4_c2": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 2},
    "bwd_w3_c2": {"VARIANT_BWD_WARPS": 3, "VARIANT_BWD_CTAS_PER_SM": 2},
    "bwd_w4_c3": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 3},
    "bwd_w4_c4": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 4},
    "bwd_w8_c2": {"VARIANT_BWD_WARPS": 8, "VARIANT_BWD_CTAS_PER_SM": 2},
    "bwd_w6_c1": {"VARIANT_BWD_WARPS": 6, "VARIANT_BWD_CTAS_PER_SM": 1},
    "bwd_w4_c5": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 5},
    "bwd_w4_c6": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 6},
    "bwd_w2_c8": {"VARIANT_BWD_WARPS": 2, "VARIANT_BWD_CTAS_PER_SM": 8},
    "bwd_w2_c10": {"VARIANT_BWD_WARPS": 2, "VARIANT_BWD_CTAS_PER_SM": 10},
    "bwd_w4_c2_r2": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 2, "VARIANT_BWD_ROWS": 2},
    "bwd_w4_c3_r2": {"VARIANT_BWD_WARPS": 4, "VARIANT_BWD_CTAS_PER_SM": 3, "VARIANT_BWD_ROWS": 2},
    "bwd_w2_c4_r2": {"VARIANT_BWD_WARPS": 2, "VARIANT_BWD_CTAS_PER_SM": 4, "VARIANT_BWD_ROWS": 2},
}
DEFAULT_SET = ("shipped", "scalar_math", "packed_math", "mask_redux", "packed_redux",
               "bwd_static", "bwd_dynamic_all", "bwd_dynamic_tail3")

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
)


def parse_define(text):
    name, _, value = text.partition("=")
    return name, (value if value else "1")


def variant_macros(name, extra):
    macros = dict(VARIANTS[name]) if name in VARIANTS else {}
    macros.update(extra)
    return macros


def library_path(name, hidden_only):
    suffix = f"_h{hidden_only}" if hidden_only else ""
    return BUILD / f"librln_variant_{name}{suffix}.so"


def build_variant(name, macros, hidden_only, force, verbose):
    """nvcc -shared of variant_unit.cu with the variant's macros.  Rebuilt when
    the source or a kernel header is newer than the library."""
    target = library_path(name, hidden_only)
    sources = [SOURCE, *(PACKAGE_ROOT / "csrc").glob("*.cuh"), PACKAGE_ROOT / "csrc" / "rln_launch.h"]
    stamp_file = target.with_suffix(".flags")
    defines = dict(macros)
    if hidden_only:
        defines["VARIANT_HIDDEN"] = hidden_only
    # every variant gets a namespace of its own (the kernels are templates with
    # identical names in every build)
    defines["rln"] = f"rln_variant_{name}"
    flags = " ".join(f"-D{key}={value}" for key, value in sorted(defines.items()))
    if (not force and target.exists() and stamp_file.exists()
            and stamp_file.read_text() == flags
            and all(Path(s).stat().st_mtime <= target.stat().st_mtime for s in sources)):
        return target, None
    BUILD.mkdir(parents=True, exist_ok=True)
    command = [
        "nvcc", *NVCC_FLAGS, "-Xptxas", "-v", f"-I{PACKAGE_ROOT / 'csrc'}", f"-I{REPO / 'include'}",
        *flags.split(), str(SOURCE), "-o", str(target),
    ]
    if verbose:
        print(" ".join(command), file=sys.stderr, flush=True)
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"variant {name} failed to build:\n{result.stdout}{result.stderr}")
    stamp_file.write_text(flags)
    target.with_suffix(".ptxas.log").write_text(result.stderr)
    return target, result.stderr


class VariantArgs(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("branch", ctypes.c_void_p), ("weight", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("updated", ctypes.c_void_p), ("normalized", ctypes.c_void_p),
        ("mean", ctypes.c_void_p), ("rstd", ctypes.c_void_p), ("mask", ctypes.c_void_p),
        ("grad_updated", ctypes.c_void_p), ("grad_normalized", ctypes.c_void_p),
        ("grad_x", ctypes.c_void_p), ("grad_branch", ctypes.c_void_p),
        ("grad_parameters", ctypes.c_void_p), ("partials", ctypes.c_void_p),
        ("row_counter", ctypes.c_void_p),
        ("rows", ctypes.c_int64), ("hidden", ctypes.c_int32), ("deterministic", ctypes.c_int32),
        ("dropout_p", ctypes.c_float), ("eps", ctypes.c_float),
        ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64),
        ("sm_count", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


def load_variant(path):
    library = ctypes.CDLL(str(path))
    library.rln_variant_run.restype = ctypes.c_int
    library.rln_variant_run.argtypes = [ctypes.POINTER(VariantArgs), ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p]
    library.rln_variant_backward_grid.restype = ctypes.c_int
    library.rln_variant_backward_grid.argtypes = [ctypes.POINTER(VariantArgs)]
    library.rln_variant_args_bytes.restype = ctypes.c_int
    if library.rln_variant_args_bytes() != ctypes.sizeof(VariantArgs):
        raise RuntimeError("VariantArgs layout differs between the driver and the library")
    return library


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("-C", "--hidden", type=int, default=768)
    parser.add_argument("--rows", type=int, default=87381)
    parser.add_argument("-p", "--dropout", type=float, default=0.1)
    parser.add_argument("--only", nargs="+", default=None, help="variant names (default: a core set)")
    parser.add_argument("--all", action="store_true", help="every entry of VARIANTS")
    parser.add_argument("-D", dest="defines", action="append", default=[],
                        help="extra macro NAME[=VALUE] for an ad-hoc variant named 'custom'")
    parser.add_argument("--deterministic", action="store_true",
                        help="fixed-order parameter reduction (partials + second kernel)")
    parser.add_argument("--heat", type=float, default=1.5, help="seconds of warm-up load")
    parser.add_argument("--rounds", type=int, default=7)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--flush-l2", action="store_true",
                        help="time single steps with a 256 MB write+read between them (for "
                             "working sets that fit the 126 MB L2)")
    parser.add_argument("--all-widths", action="store_true",
                        help="build every hidden size into each variant (slower build)")
    parser.add_argument("--build-only", action="store_true")
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args(argv)

    names = list(VARIANTS) if args.all else list(args.only or DEFAULT_SET)
    extra = dict(parse_define(text) for text in args.defines)
    if extra:
        names.append("custom")
    unknown = [name for name in names if name not in VARIANTS and name != "custom"]
    if unknown:
        parser.error(f"unknown variants: {unknown}; known: {sorted(VARIANTS)}")
    hidden_only = None if args.all_widths else args.hidden

    with ThreadPoolExecutor(max_workers=8) as pool:
        jobs = {
            name: pool.submit(build_variant, name,
                              variant_macros(name, extra if name == "custom" else {}),
                              hidden_only, args.force, args.verbose)
            for name in names
        }
        paths = {name: job.result()[0] for name, job in jobs.items()}
    if args.build_only:
        for name, path in paths.items():
            print(f"{name}: {path}")
        return 0

    import torch

    from gfx1010_kernels import _C

    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    rows, hidden = args.rows, args.hidden
    generator = torch.Generator(device=device).manual_seed(0)
    x = torch.randn(rows, hidden, device=device, generator=generator)
    branch = torch.randn(rows, hidden, device=device, generator=generator).half()
    weight = 1.0 + 0.1 * torch.randn(hidden, device=device, generator=generator)
    bias = 0.1 * torch.randn(hidden, device=device, generator=generator)
    grad_updated = torch.randn(rows, hidden, device=device, generator=generator)
    grad_normalized = torch.randn(rows, hidden, device=device, generator=generator)
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count

    out = {
        "updated": torch.empty_like(x), "normalized": torch.empty_like(x),
        "mean": torch.empty(rows, device=device), "rstd": torch.empty(rows, device=device),
        "mask": torch.empty(rows * hidden // 32, device=device, dtype=torch.int32),
        "grad_x": torch.empty_like(x), "grad_branch": torch.empty_like(branch),
        "grad_parameters": torch.empty(2, hidden, device=device),
        "partials": torch.empty(sm_count * 32, 2, hidden, device=device),
        "row_counter": torch.zeros(4, device=device, dtype=torch.int32),
    }
    call = VariantArgs(
        x=x.data_ptr(), branch=branch.data_ptr(), weight=weight.data_ptr(), bias=bias.data_ptr(),
        updated=out["updated"].data_ptr(), normalized=out["normalized"].data_ptr(),
        mean=out["mean"].data_ptr(), rstd=out["rstd"].data_ptr(), mask=out["mask"].data_ptr(),
        grad_updated=grad_updated.data_ptr(), grad_normalized=grad_normalized.data_ptr(),
        grad_x=out["grad_x"].data_ptr(), grad_branch=out["grad_branch"].data_ptr(),
        grad_parameters=out["grad_parameters"].data_ptr(), partials=out["partials"].data_ptr(),
        row_counter=out["row_counter"].data_ptr(),
        rows=rows, hidden=hidden, deterministic=int(args.deterministic),
        dropout_p=args.dropout, eps=1e-5, seed=0, offset=0, sm_count=sm_count, reserved=0,
    )
    stream = torch.cuda.current_stream(device).cuda_stream
    libraries = {name: load_variant(path) for name, path in paths.items()}

    def run(name, mode, steps, offset=0):
        call.offset = offset
        status = libraries[name].rln_variant_run(ctypes.byref(call), mode, steps, stream)
        if status != 0:
            raise RuntimeError(f"variant {name}: launch failed with status {status}")

    # ---- numerical check against the shipped library, before any timing ----
    torch.use_deterministic_algorithms(args.deterministic)
    ref_updated, ref_normalized, ref_mean, ref_rstd, ref_mask = \
        _C.residual_layer_norm_forward_seeded(x, branch, weight, bias, args.dropout, 1e-5, True,
                                              128, 0, 0, 0, 0)
    ref_grads = _C.residual_layer_norm_backward(
        grad_updated, grad_normalized, ref_updated, weight, ref_mean, ref_rstd, ref_mask,
        args.dropout, True, 1, 128, 64, 256, 1, True)
    torch.use_deterministic_algorithms(False)
    sample = ref_mask[: 1 << 16].to(torch.int64) & 0xFFFFFFFF
    kept = sum(int(((sample >> bit) & 1).sum()) for bit in range(32))
    kept_fraction = kept / (32 * sample.numel())
    checked = {}
    for name in names:
        for tensor in out.values():
            if tensor.dtype.is_floating_point:
                tensor.fill_(float("nan"))
        run(name, 2, 1)
        torch.cuda.synchronize()
        problems = []
        if not torch.equal(out["mask"], ref_mask):
            problems.append("mask differs")
        if not torch.equal(out["updated"], ref_updated):
            problems.append("updated differs")
        for key, reference, rtol, atol in (
            ("normalized", ref_normalized, 1e-5, 1e-6), ("mean", ref_mean, 1e-5, 1e-6),
            ("rstd", ref_rstd, 1e-5, 1e-6), ("grad_x", ref_grads[0], 1e-5, 1e-5),
            ("grad_branch", ref_grads[1], 2e-3, 1e-5),
        ):
            if not torch.allclose(out[key].float(), reference.float(), rtol=rtol, atol=atol):
                worst = (out[key].float() - reference.float()).abs().max().item()
                problems.append(f"{key} off by {worst:.3g}")
        floor = 1e-5 * rows ** 0.5
        for index, key in enumerate(("grad_weight", "grad_bias")):
            if not torch.allclose(out["grad_parameters"][index], ref_grads[2 + index],
                                  rtol=1e-4, atol=floor):
                worst = (out["grad_parameters"][index] - ref_grads[2 + index]).abs().max().item()
                problems.append(f"{key} off by {worst:.3g}")
        checked[name] = problems

    # ---- timing ----
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=device) if args.flush_l2 else None
    good = [name for name in names if not checked[name]]
    modes = (("step", 2), ("forward", 0), ("backward", 1))
    samples = {name: {mode: [] for mode, _ in modes} for name in good}

    def timed(name, mode_code, steps, offset):
        begin = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        if flush is None:
            begin.record()
            run(name, mode_code, steps, offset)
            end.record()
            end.synchronize()
            return begin.elapsed_time(end) / steps
        total = 0.0
        for index in range(steps):
            flush.zero_()
            flush.sum()
            begin.record()
            run(name, mode_code, 1, offset + 4 * index)
            end.record()
            end.synchronize()
            total += begin.elapsed_time(end)
        return total / steps

    if good:
        heat_until = time.perf_counter() + args.heat
        offset = 8
        while time.perf_counter() < heat_until:
            run(good[0], 2, 50, offset)
            torch.cuda.synchronize()
            offset += 200
        for round_index in range(args.rounds):
            # rotate the order: under the power cap the clock sags over a series
            # of forward-only runs, so a fixed order would favour its first entries
            shift = round_index % len(good)
            order = good[shift:] + good[:shift]
            for mode, code in modes:
                for name in order:
                    samples[name][mode].append(timed(name, code, args.steps, offset))
                    offset += 4 * args.steps

    branch_bytes = 2
    forward_bytes = rows * ((8 + branch_bytes + 4) * hidden + 8 + hidden // 8)
    backward_bytes = rows * ((12 + branch_bytes + 4) * hidden + 8 + hidden // 8)
    volume = {"step": forward_bytes + backward_bytes, "forward": forward_bytes,
              "backward": backward_bytes}
    for name in names:
        line = {
            "variant": name,
            "macros": variant_macros(name, extra if name == "custom" else {}),
            "hidden": hidden, "rows": rows, "dropout_p": args.dropout,
            "deterministic": bool(args.deterministic),
            "check": "ok" if not checked[name] else "; ".join(checked[name]),
            "kept_fraction": kept_fraction,
            "l2": "flushed between steps" if args.flush_l2 else "steps back to back",
        }
        if name in samples:
            for mode, _ in modes:
                values = samples[name][mode]
                median = statistics.median(values)
                line[mode] = {
                    "median_ms": round(median, 5), "min_ms": round(min(values), 5),
                    "max_ms": round(max(values), 5),
                    "gbs": round(volume[mode] / (median * 1e-3) / 1e9, 1),
                }
        print(json.dumps(line), flush=True)
    return 0 if all(not problems for problems in checked.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
