"""In-tree build of the sm_100a residual LayerNorm libraries.

Produces, inside the ``gfx1010_kernels`` package directory:

* ``librln_sm100.so`` -- the CUDA kernels behind the C ABI of
  ``include/rln_sm100.h`` (nvcc, ``-gencode arch=compute_100a,code=sm_100a``).
  It has no dependency on torch or Python.
* ``_C.so`` -- the torch extension ``gfx1010_kernels._C`` (g++), linked
  against ``librln_sm100.so`` through ``$ORIGIN``.

This replaces the reference project's ``setup.py`` (``setup.py:13-35`` of
T-vaccari/gfx1010-kernels), which builds a ``CUDAExtension`` for
``--offload-arch=gfx1010`` and refuses non-ROCm torch.  nvcc cross-compiles
without a GPU, so the build runs on a CPU-only machine.

Usage: ``python build.py [--force] [--verbose]``
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path


ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
INCLUDE = REPO / "include"
PACKAGE = ROOT / "gfx1010_kernels"
OBJECTS = ROOT / "build"

KERNEL_LIBRARY = PACKAGE / "librln_sm100.so"
EXTENSION = PACKAGE / "_C.so"

CUDA_SOURCES = (
    "rln_api.cu",
    "rln_forward.cu",
    "rln_forward_narrow.cu",
    "rln_backward.cu",
    "rln_backward_narrow.cu",
    "rln_host_pipeline.cu",
    "rln_backward_static.cu",
)
CUDA_HEADERS = (
    "rln_kernels.cuh",
    "rln_launch.h",
    "rln_forward_dispatch.cuh",
    "rln_backward_dispatch.cuh",
)
NVCC_FLAGS = (
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
)


def _cuda_home() -> Path:
    for candidate in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if candidate and (Path(candidate) / "bin" / "nvcc").exists():
            return Path(candidate)
    nvcc = shutil.which("nvcc")
    if nvcc is None:
        raise RuntimeError("nvcc was not found; set CUDA_HOME")
    return Path(nvcc).resolve().parent.parent


def _host_compiler() -> str:
    """The system g++ (the one nvcc also uses as its host compiler).

    ``$CXX`` is deliberately not consulted: a wrapper that links libstdc++
    statically gives the extension a second, uninitialised copy of the iostream
    locale machinery next to the one torch uses, and formatting a number into an
    error message then crashes.  ``RLN_CXX`` overrides for unusual setups.
    """
    override = os.environ.get("RLN_CXX")
    if override:
        return override
    for candidate in ("/usr/bin/g++", shutil.which("g++")):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("g++ was not found")


def _digest(sources) -> str:
    digest = hashlib.sha256()
    for source in sources:
        digest.update(str(Path(source).name).encode())
        digest.update(Path(source).read_bytes())
    return digest.hexdigest()


def _stamp_path(target: Path) -> Path:
    return OBJECTS / (target.name + ".sha256")


def _newer(target: Path, sources) -> bool:
    """True when ``target`` was built from exactly these ``sources``.  Decided by
    a content hash recorded at build time, not by timestamps: a copy of the tree
    (to another machine, out of an archive) keeps its binaries valid and a
    source edit always invalidates them, whatever the copy did to the mtimes."""
    stamp = _stamp_path(target)
    if not target.exists() or not stamp.exists():
        return False
    return stamp.read_text().strip() == _digest(sources)


def _record(target: Path, sources) -> None:
    OBJECTS.mkdir(exist_ok=True)
    _stamp_path(target).write_text(_digest(sources) + "\n")


def _run(command, verbose):
    if verbose:
        print(" ".join(str(part) for part in command), flush=True)
    result = subprocess.run(
        [str(part) for part in command], capture_output=True, text=True
    )
    if result.returncode != 0:
        raise RuntimeError(
            "build step failed:\n"
            + " ".join(str(part) for part in command)
            + "\n"
            + result.stdout
            + result.stderr
        )
    if verbose and (result.stdout or result.stderr):
        print(result.stdout + result.stderr, flush=True)


def build_kernel_library(force=False, verbose=False) -> Path:
    cuda = _cuda_home()
    nvcc = cuda / "bin" / "nvcc"
    OBJECTS.mkdir(exist_ok=True)
    sources = [CSRC / name for name in CUDA_SOURCES if (CSRC / name).exists()]
    headers = [CSRC / name for name in CUDA_HEADERS] + [INCLUDE / "rln_sm100.h", Path(__file__)]
    if not force and _newer(KERNEL_LIBRARY, sources + headers):
        return KERNEL_LIBRARY

    def compile_one(source):
        target = OBJECTS / (source.stem + ".o")
        if not force and _newer(target, [source] + headers):
            return target
        _run([nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", source, "-o", target], verbose)
        _record(target, [source] + headers)
        return target

    with ThreadPoolExecutor(max_workers=len(sources)) as pool:
        objects = list(pool.map(compile_one, sources))
    _run(
        [
            nvcc,
            "-shared",
            "-gencode",
            "arch=compute_100a,code=sm_100a",
            "-cudart",
            "static",
            "-o",
            KERNEL_LIBRARY,
            *objects,
        ],
        verbose,
    )
    _record(KERNEL_LIBRARY, sources + headers)
    return KERNEL_LIBRARY


def build_extension(force=False, verbose=False) -> Path:
    import torch
    from torch.utils import cpp_extension

    cuda = _cuda_home()
    source = CSRC / "rln_bindings.cpp"
    # (the extension links the kernel library by name and calls it through the
    # C ABI of the header, so the library's content is not a dependency)
    dependencies = [source, INCLUDE / "rln_sm100.h", Path(__file__)]
    if not force and KERNEL_LIBRARY.exists() and _newer(EXTENSION, dependencies):
        return EXTENSION
    torch_library = Path(torch.__file__).resolve().parent / "lib"
    includes = []
    for path in cpp_extension.include_paths():
        includes += ["-isystem", path]
    includes += ["-isystem", sysconfig.get_paths()["include"], "-isystem", cuda / "include"]
    command = [
        _host_compiler(),
        "-O2",
        "-std=c++17",
        "-fPIC",
        "-shared",
        "-fvisibility=hidden",
        "-DTORCH_EXTENSION_NAME=_C",
        "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        "-I",
        INCLUDE,
        *includes,
        source,
        "-o",
        EXTENSION,
        f"-L{PACKAGE}",
        "-lrln_sm100",
        f"-L{torch_library}",
        "-lc10",
        "-lc10_cuda",
        "-ltorch_cpu",
        "-ltorch_cuda",
        "-ltorch",
        "-ltorch_python",
        "-Wl,-rpath,$ORIGIN",
        f"-Wl,-rpath,{torch_library}",
    ]
    _run(command, verbose)
    _check_dynamic_libstdcxx(EXTENSION)
    _record(EXTENSION, dependencies)
    return EXTENSION


def _check_dynamic_libstdcxx(library: Path) -> None:
    """Refuse an extension that carries its own copy of libstdc++."""
    listing = subprocess.run(
        ["nm", "-D", "--defined-only", str(library)], capture_output=True, text=True
    ).stdout
    if "_ZNSt6locale5facet" in listing:
        library.unlink()
        raise RuntimeError(
            f"{library.name} was linked with a static libstdc++; "
            "set RLN_CXX to a compiler that links it dynamically"
        )


def build_all(force=False, verbose=False):
    library = build_kernel_library(force=force, verbose=verbose)
    extension = build_extension(force=force, verbose=verbose)
    return library, extension


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true", help="rebuild everything")
    parser.add_argument("--verbose", action="store_true", help="print every command")
    arguments = parser.parse_args(argv)
    library, extension = build_all(force=arguments.force, verbose=arguments.verbose)
    print(f"built {library}")
    print(f"built {extension}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
