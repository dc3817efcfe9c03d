"""Test configuration: import paths, the ``gpu`` marker and shared fixtures."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
PACKAGE_ROOT = REPO / "gfx1010-kernels_b200"
for path in (str(REPO), str(PACKAGE_ROOT), str(Path(__file__).resolve().parent)):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line(
        "markers", "gpu: needs a CUDA device of compute capability 10.x (B200)"
    )


def pytest_collection_modifyitems(config, items):
    """GPU tests fail (not skip) on a GPU box whose native backend is broken;
    without any CUDA device they are skipped."""
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def built_libraries():
    """Build the in-tree libraries (nvcc cross-compiles without a GPU).  The
    build is incremental: objects newer than their sources are kept, anything
    stale is rebuilt, so the tests never run against binaries of older sources."""
    import build as rln_build

    rln_build.build_all()
    return rln_build.KERNEL_LIBRARY, rln_build.EXTENSION


@pytest.fixture(scope="session")
def golden_cases():
    """name -> dict of numpy arrays + the case's metadata."""
    directory = REPO / "tests" / "golden"
    meta = json.loads((directory / "rln_cases.json").read_text())["cases"]
    arrays = np.load(directory / "rln_cases.npz")
    cases = {}
    for entry in meta:
        name = entry["name"]
        record = {
            key.split("/", 1)[1]: arrays[key]
            for key in arrays.files
            if key.startswith(name + "/")
        }
        record["meta"] = entry
        cases[name] = record
    return cases


def golden_tensors(case, device="cpu"):
    """The arrays of one golden case as torch tensors, with ``branch`` and
    ``grad_branch`` in the case's branch dtype and ``normalized`` /
    ``grad_normalized`` in its normalized dtype (16-bit values are stored
    widened to float32, which represents them exactly)."""
    import torch

    dtype = getattr(torch, case["meta"]["branch_dtype"])
    normalized_dtype = getattr(torch, case["meta"].get("normalized_dtype", "float32"))
    tensors = {}
    for key, value in case.items():
        if key in ("meta", "config"):
            continue
        tensor = torch.from_numpy(value)
        if key in ("branch", "grad_branch"):
            tensor = tensor.to(dtype)
        elif key in ("normalized", "grad_normalized"):
            tensor = tensor.to(normalized_dtype)
        tensors[key] = tensor.to(device)
    return tensors


@pytest.fixture(scope="session")
def philox_kat():
    return json.loads((REPO / "tests" / "golden" / "philox_kat.json").read_text())
