"""The benchmark scripts stay buildable and importable without a GPU."""

import ctypes
import importlib.util
import subprocess
import sys

from conftest import PACKAGE_ROOT

BENCHMARKS = PACKAGE_ROOT / "benchmarks"


def load(name):
    spec = importlib.util.spec_from_file_location(name, BENCHMARKS / f"{name}.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_variant_benchmark_builds_its_kernel_variants(built_libraries):
    """nvcc cross-compiles two variants of the kernel templates (the shipped form and
    one with other template arguments); the libraries export the driver's entry points
    and agree with the driver on the argument structure."""
    completed = subprocess.run(
        [sys.executable, str(BENCHMARKS / "benchmark_native_variants.py"), "--build-only",
         "--hidden", "384", "--only", "shipped", "bwd_dynamic_tail3"],
        capture_output=True, text=True, timeout=900,
    )
    assert completed.returncode == 0, completed.stdout + completed.stderr
    variants = load("benchmark_native_variants")
    for name in ("shipped", "bwd_dynamic_tail3"):
        path = variants.library_path(name, 384)
        assert path.exists(), path
        library = ctypes.CDLL(str(path))
        for symbol in ("rln_variant_run", "rln_variant_backward_grid", "rln_variant_args_bytes"):
            assert hasattr(library, symbol), symbol
        library.rln_variant_args_bytes.restype = ctypes.c_int
        assert library.rln_variant_args_bytes() == ctypes.sizeof(variants.VariantArgs)
    assert set(variants.DEFAULT_SET) <= set(variants.VARIANTS)


def test_raw_entry_benchmark_parses_its_arguments_without_a_gpu(built_libraries):
    completed = subprocess.run(
        [sys.executable, str(BENCHMARKS / "benchmark_raw_entries.py"), "--help"],
        capture_output=True, text=True, timeout=300,
    )
    assert completed.returncode == 0 and "--disable-deterministic-fill" in completed.stdout
