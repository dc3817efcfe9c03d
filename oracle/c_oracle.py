"""numpy front-end of the scalar C oracle (``oracle/rln_oracle.c``).

Test infrastructure only.  The C code restates the reference kernels'
arithmetic one element at a time; this module builds it on demand and exposes
it on numpy arrays.  Half-precision branches are passed widened to float32 and
come back as float32 values that are exactly representable in the branch type.
"""

import ctypes

import numpy as np

from . import build_oracle

_library = None


def _lib():
    global _library
    if _library is None:
        _library = ctypes.CDLL(str(build_oracle.build()))
    return _library


def _p(array):
    return array.ctypes.data_as(ctypes.c_void_p)


def philox(counter, key):
    counter = np.ascontiguousarray(counter, dtype=np.uint32)
    key = np.ascontiguousarray(key, dtype=np.uint32)
    out = np.empty(4, dtype=np.uint32)
    _lib().rln_oracle_philox(_p(counter), _p(key), _p(out))
    return out


def keep_mask(rows, hidden, dropout_p, seed, offset, row_base=0):
    keep = np.empty((rows, hidden), dtype=np.uint8)
    words = np.empty(rows * hidden // 32, dtype=np.uint32)
    _lib().rln_oracle_keep_mask(
        ctypes.c_int64(rows), ctypes.c_int32(hidden), ctypes.c_float(dropout_p),
        ctypes.c_uint64(seed), ctypes.c_uint64(offset), ctypes.c_int64(row_base),
        _p(keep), _p(words),
    )
    return keep.astype(bool), words.view(np.int32)


def forward(x, branch, weight, bias, keep, dropout_p, eps, branch_kind, normalized_kind=0):
    """``branch_kind`` / ``normalized_kind``: 0/False float32, 1/True float16, 2 bfloat16.

    ``normalized`` is returned as float32 values that are exactly representable
    in the ``normalized_kind`` type (rounded once from the float32 result).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, hidden = x.shape
    branch = np.ascontiguousarray(branch, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    keep_bytes = None if keep is None else np.ascontiguousarray(keep, dtype=np.uint8)
    updated = np.empty_like(x)
    normalized = np.empty_like(x)
    mean = np.empty(rows, dtype=np.float32)
    rstd = np.empty(rows, dtype=np.float32)
    _lib().rln_oracle_forward(
        _p(x), _p(branch), _p(weight), _p(bias),
        None if keep_bytes is None else _p(keep_bytes),
        ctypes.c_float(dropout_p), ctypes.c_float(eps), ctypes.c_int32(int(branch_kind)),
        ctypes.c_int64(rows), ctypes.c_int32(hidden),
        _p(updated), _p(normalized), _p(mean), _p(rstd),
    )
    if int(normalized_kind) != 0:
        _lib().rln_oracle_round(
            _p(normalized), ctypes.c_int64(normalized.size), ctypes.c_int32(int(normalized_kind))
        )
    return updated, normalized, mean, rstd


def backward(grad_updated, grad_normalized, updated, weight, mean, rstd, keep, dropout_p,
             branch_kind):
    updated = np.ascontiguousarray(updated, dtype=np.float32)
    rows, hidden = updated.shape
    grad_updated = np.ascontiguousarray(grad_updated, dtype=np.float32)
    grad_normalized = np.ascontiguousarray(grad_normalized, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    mean = np.ascontiguousarray(mean, dtype=np.float32)
    rstd = np.ascontiguousarray(rstd, dtype=np.float32)
    keep_bytes = None if keep is None else np.ascontiguousarray(keep, dtype=np.uint8)
    grad_x = np.empty_like(updated)
    grad_branch = np.empty_like(updated)
    grad_weight = np.empty(hidden, dtype=np.float32)
    grad_bias = np.empty(hidden, dtype=np.float32)
    _lib().rln_oracle_backward(
        _p(grad_updated), _p(grad_normalized), _p(updated), _p(weight), _p(mean), _p(rstd),
        None if keep_bytes is None else _p(keep_bytes),
        ctypes.c_float(dropout_p), ctypes.c_int32(int(branch_kind)),
        ctypes.c_int64(rows), ctypes.c_int32(hidden),
        _p(grad_x), _p(grad_branch), _p(grad_weight), _p(grad_bias),
    )
    return grad_x, grad_branch, grad_weight, grad_bias
