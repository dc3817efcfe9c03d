"""The C-ABI library loads without a GPU and exports every symbol that
``include/rln_sm100.h`` declares; argument validation that precedes any CUDA
call behaves as documented."""

import ctypes
import re
from pathlib import Path

import cabi

HEADER = Path(__file__).resolve().parent.parent / "include" / "rln_sm100.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"RLN_API[^;(]*?\b(rln_sm100_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    symbols = declared_symbols()
    for required in (
        "rln_sm100_forward",
        "rln_sm100_backward",
        "rln_sm100_backward_workspace_bytes",
        "rln_sm100_status_string",
        "rln_sm100_last_cuda_error",
        "rln_sm100_abi_version",
    ):
        assert required in symbols


def test_library_exports_every_declared_symbol(built_libraries):
    lib = ctypes.CDLL(str(built_libraries[0]))
    for symbol in declared_symbols():
        assert hasattr(lib, symbol), symbol


def test_abi_version_matches_header(built_libraries):
    version = int(re.search(r"#define RLN_SM100_ABI_VERSION (\d+)", HEADER.read_text()).group(1))
    assert cabi.library().rln_sm100_abi_version() == version


def test_status_strings_cover_every_code(built_libraries):
    codes = re.findall(r"#define (RLN_(?:OK|ERR_\w+)) \(?(-?\d+)\)?", HEADER.read_text())
    assert len(codes) >= 10
    seen = set()
    for _, value in codes:
        text = cabi.status_text(int(value))
        assert text and text != "unknown status"
        seen.add(text)
    assert len(seen) == len(codes)
    assert cabi.status_text(-999) == "unknown status"
    # texts the reference's callers match on
    assert "empty tensors are unsupported" in cabi.status_text(-3)
    assert "dropout_p must be in [0, 1)" in cabi.status_text(-4)


def test_argument_validation_precedes_any_cuda_call(built_libraries):
    lib = cabi.library()
    null = ctypes.c_void_p(None)
    fake = ctypes.c_void_p(0x1000)

    def forward(rows=4, hidden=128, p=0.1, eps=1e-5, x=fake, branch_dtype=1, normalized_dtype=0,
                normalized=fake):
        return lib.rln_sm100_forward(
            x, fake, fake, fake, fake, normalized, fake, fake, fake,
            rows, hidden, branch_dtype, normalized_dtype, 1, p, eps, 0, 0, 0, null,
        )

    assert forward(hidden=160) == -2
    assert forward(rows=0) == -3
    assert forward(p=1.0) == -4
    assert forward(p=-0.1) == -4
    assert forward(eps=0.0) == -5
    assert forward(x=null) == -1
    assert forward(x=ctypes.c_void_p(0x1002)) == -6
    assert forward(branch_dtype=3) == -11
    assert forward(normalized_dtype=3) == -12
    assert forward(normalized_dtype=-1) == -12
    # a 16-bit `normalized` has no scalar-access kernel: 8-byte alignment or nothing
    assert forward(normalized_dtype=2, normalized=ctypes.c_void_p(0x1004)) == -6
    assert forward(normalized_dtype=0, normalized=ctypes.c_void_p(0x1002)) == -6
    assert lib.rln_sm100_backward_workspace_bytes(0, 128, 1) == -3
    assert lib.rln_sm100_backward_workspace_bytes(16, 100, 1) == -2
    assert lib.rln_sm100_backward_workspace_bytes(16, 128, 0) == 0
