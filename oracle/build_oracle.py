"""Compile the scalar C oracle (oracle/rln_oracle.c) into oracle/_build/librln_oracle.so.

Test infrastructure only.  ``build()`` is called by ``__graft_entry__.build()``
and, when the library is missing, by the tests that use it.
"""

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "rln_oracle.c"
OUTPUT = HERE / "_build" / "librln_oracle.so"


def build(force=False):
    if not force and OUTPUT.exists() and OUTPUT.stat().st_mtime >= SOURCE.stat().st_mtime:
        return OUTPUT
    OUTPUT.parent.mkdir(exist_ok=True)
    command = [
        "gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off",
        str(SOURCE), "-o", str(OUTPUT), "-lm",
    ]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("building the C oracle failed:\n" + result.stdout + result.stderr)
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True))
