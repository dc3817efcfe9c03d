"""Packaging of the sm_100a build of ``gfx1010_kernels``.

Counterpart of the reference project's ``setup.py`` (``setup.py:1-35`` of
T-vaccari/gfx1010-kernels), which compiles a ROCm ``CUDAExtension`` and refuses
non-ROCm torch.  Here the native pieces are produced by ``build.py`` (nvcc for
``librln_sm100.so``, g++ for ``_C.so``) before the package is collected, so that

    pip install --no-build-isolation -e gfx1010-kernels_b200

gives an importable ``gfx1010_kernels`` with both libraries inside the package
directory.  The C-ABI header is installed next to them as package data.
"""

import shutil
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


class BuildNativeThenPython(build_py):
    def run(self):
        import build as rln_build

        rln_build.build_all()
        header = ROOT.parent / "include" / "rln_sm100.h"
        if header.exists():
            shutil.copy2(header, ROOT / "gfx1010_kernels" / "rln_sm100.h")
        super().run()


setup(
    name="gfx1010-kernels-b200",
    version="0.4.0",
    description="sm_100a (B200) build of the gfx1010_kernels fused residual-add + dropout + "
                "LayerNorm operator",
    packages=["gfx1010_kernels"],
    package_data={"gfx1010_kernels": ["*.so", "rln_sm100.h"]},
    python_requires=">=3.10",
    cmdclass={"build_py": BuildNativeThenPython},
    zip_safe=False,
)
