"""ctypes view of ``librln_sm100.so`` for the tests: the same binding a
non-torch host would write against ``include/rln_sm100.h``.  Tensors are only
used as device-memory holders; what crosses the boundary is raw addresses."""

import ctypes
from pathlib import Path

import torch

LIBRARY_PATH = (
    Path(__file__).resolve().parent.parent
    / "gfx1010-kernels_b200"
    / "gfx1010_kernels"
    / "librln_sm100.so"
)

_p = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64
_u64 = ctypes.c_uint64
_f32 = ctypes.c_float

_library = None
# RLN_DTYPE_* of include/rln_sm100.h (branch and normalized element types)
DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
BRANCH_CODES = DTYPE_CODES


def library():
    global _library
    if _library is None:
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        lib.rln_sm100_abi_version.restype = ctypes.c_int
        lib.rln_sm100_status_string.restype = ctypes.c_char_p
        lib.rln_sm100_status_string.argtypes = [ctypes.c_int]
        lib.rln_sm100_last_cuda_error.restype = ctypes.c_int
        lib.rln_sm100_forward.restype = ctypes.c_int
        lib.rln_sm100_forward.argtypes = [
            _p, _p, _p, _p, _p, _p, _p, _p, _p,
            _i64, _i32, _i32, _i32, _i32, _f32, _f32, _u64, _u64, _i64, _p,
        ]
        lib.rln_sm100_forward_device_rng.restype = ctypes.c_int
        lib.rln_sm100_forward_device_rng.argtypes = [
            _p, _p, _p, _p, _p, _p, _p, _p, _p,
            _i64, _i32, _i32, _i32, _i32, _f32, _f32, _p, _p, _u64, _i64, _p,
        ]
        lib.rln_sm100_backward_workspace_bytes.restype = _i64
        lib.rln_sm100_backward_workspace_bytes.argtypes = [_i64, _i32, _i32]
        lib.rln_sm100_backward.restype = ctypes.c_int
        lib.rln_sm100_backward.argtypes = [
            _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p,
            _i64, _i64, _i32, _i32, _i32, _i32, _f32, _i32, _p,
        ]
        _library = lib
    return _library


def _ptr(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_text(status):
    return library().rln_sm100_status_string(status).decode()


def forward(x, branch, weight, bias, dropout_p, eps, training, seed=0, offset=0, row_base=0,
            outputs=None, normalized_dtype=torch.float32):
    """Returns (status, updated, normalized, mean, rstd, mask)."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    active = bool(training and dropout_p > 0.0)
    if outputs is None:
        updated = torch.empty_like(x)
        normalized = torch.empty(x.shape, dtype=normalized_dtype, device=x.device)
        mean = torch.empty(rows, device=x.device)
        rstd = torch.empty(rows, device=x.device)
        mask = torch.empty(
            rows * (hidden // 32) if active else 0, dtype=torch.int32, device=x.device
        )
    else:
        updated, normalized, mean, rstd, mask = outputs
    status = library().rln_sm100_forward(
        _ptr(x), _ptr(branch), _ptr(weight), _ptr(bias),
        _ptr(updated), _ptr(normalized), _ptr(mean), _ptr(rstd),
        _ptr(mask) if active else None,
        rows, hidden, DTYPE_CODES[branch.dtype], DTYPE_CODES[normalized.dtype], int(active),
        dropout_p, eps, seed, offset, row_base, _stream(),
    )
    return status, updated, normalized, mean, rstd, mask


def forward_device_rng(x, branch, weight, bias, dropout_p, eps, training, device_seed,
                       device_offset, offset_extra=0, row_base=0,
                       normalized_dtype=torch.float32):
    """``rln_sm100_forward_device_rng``: the Philox seed and offset are read by the
    kernel from two int64 words in device memory (``device_seed``, ``device_offset``:
    one-element int64 CUDA tensors).  Returns (status, updated, normalized, mean,
    rstd, mask)."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    active = bool(training and dropout_p > 0.0)
    updated = torch.empty_like(x)
    normalized = torch.empty(x.shape, dtype=normalized_dtype, device=x.device)
    mean = torch.empty(rows, device=x.device)
    rstd = torch.empty(rows, device=x.device)
    mask = torch.empty(rows * (hidden // 32) if active else 0, dtype=torch.int32, device=x.device)
    status = library().rln_sm100_forward_device_rng(
        _ptr(x), _ptr(branch), _ptr(weight), _ptr(bias),
        _ptr(updated), _ptr(normalized), _ptr(mean), _ptr(rstd),
        _ptr(mask) if active else None,
        rows, hidden, DTYPE_CODES[branch.dtype], DTYPE_CODES[normalized.dtype], int(active),
        dropout_p, eps, _ptr(device_seed), _ptr(device_offset), offset_extra, row_base, _stream(),
    )
    return status, updated, normalized, mean, rstd, mask


def backward(grad_updated, grad_normalized, updated, weight, mean, rstd, mask, dropout_p,
             training, branch_dtype, deterministic, parameters=True, grad_x=None):
    """Returns (status, grad_x, grad_branch, grad_parameters[2,H] or None)."""
    hidden = updated.shape[-1]
    rows = updated.numel() // hidden
    active = bool(training and dropout_p > 0.0)
    device = updated.device
    if grad_x is None:
        grad_x = torch.empty_like(updated)
    grad_branch = torch.empty(updated.shape, dtype=branch_dtype, device=device)
    grad_parameters = torch.empty(2, hidden, device=device) if parameters else None
    workspace = None
    workspace_bytes = 0
    if parameters:
        workspace_bytes = library().rln_sm100_backward_workspace_bytes(
            rows, hidden, int(deterministic)
        )
        assert workspace_bytes >= 0, status_text(workspace_bytes)
        if workspace_bytes:
            # non-zero garbage: the call itself has to clear what it needs cleared
            workspace = torch.full((workspace_bytes // 4,), 123.0, device=device)
    status = library().rln_sm100_backward(
        _ptr(grad_updated), _ptr(grad_normalized), _ptr(updated), _ptr(weight),
        _ptr(mean), _ptr(rstd), _ptr(mask) if active else None,
        _ptr(grad_x), _ptr(grad_branch), _ptr(grad_parameters), _ptr(workspace),
        workspace_bytes, rows, hidden, DTYPE_CODES[branch_dtype],
        DTYPE_CODES[grad_normalized.dtype], int(active),
        dropout_p, int(deterministic), _stream(),
    )
    return status, grad_x, grad_branch, grad_parameters
