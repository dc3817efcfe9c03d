"""Installs the reference project's pure-Python package into ``oracle/_ref/``.

Test and benchmark infrastructure only: nothing in the product imports it.

The reference's CPU path for this operator is plain Python over torch ops
(``gfx1010_kernels/normalization.py:15-33`` reached through
``residual_layer_norm(..., implementation="torch")``, ``:164-173``).  Its
``setup.py`` (:7-8) refuses a torch that was not built for ROCm, so ``pip
install`` cannot produce the package here; the package directory is copied as
``pip`` would lay it out instead, unmodified, ``.py`` files only.  The output
directory is git-ignored (it is an installed third-party package, not source
of this repository) and travels to the GPU box with the working tree, where
``bench.py --impl reference`` and the ``cpu_baseline`` leg import it in a
process of its own and time the reference's public call.

    python oracle/build_ref.py [--reference /path/to/gfx1010-kernels]

(default: ``$RLN_REFERENCE``, else a directory ``reference`` beside this repository).

Without a reference checkout nothing is written and ``bench.py`` falls back to
the restatement in ``oracle/rln_oracle.py`` (``cpu_baseline.kind`` "port").
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
PACKAGE = "gfx1010_kernels"
# a checkout of the reference project: $RLN_REFERENCE, else a directory named
# "reference" next to this repository
DEFAULT_REFERENCE = Path(os.environ.get("RLN_REFERENCE") or HERE.parent.parent / "reference")


def build(reference: Path = DEFAULT_REFERENCE):
    """Returns the installed package directory, or None without a reference."""
    source = Path(reference) / PACKAGE
    if not (source / "normalization.py").exists():
        return None
    destination = TARGET / PACKAGE
    if destination.exists():
        shutil.rmtree(destination)
    destination.mkdir(parents=True)
    manifest = {"source": str(source), "files": {}}
    for path in sorted(source.glob("*.py")):
        shutil.copyfile(path, destination / path.name)
        manifest["files"][path.name] = hashlib.sha256(path.read_bytes()).hexdigest()
    (TARGET / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")
    return destination


def installed():
    """The installed package directory, or None."""
    destination = TARGET / PACKAGE
    return destination if (destination / "normalization.py").exists() else None


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    result = build(parser.parse_args().reference)
    print(result if result else "no reference checkout: nothing installed")
    sys.exit(0)
