"""Native route: lazy import of the ``_C`` extension and the launch-policy ints.

Mirrors ``gfx1010_kernels/_normalization_native.py`` of the reference
(T-vaccari/gfx1010-kernels): ``native_residual_layer_norm`` (:71-99),
``native_extension_status`` (:66-68) and the policy helpers
``_block_rows`` / ``_parameter_threads`` / ``_parameter_groups`` (:5-54).

The four integers the policy produces are gfx1010 tuning knobs.  The sm_100a
kernels fix their launch geometry per hidden size, so the extension only
range-checks them; they are still computed with the reference's tuned values
because (a) the ``_C`` entry points keep the reference's positional signature
and validation and (b) ``threads`` determines how far the torch generator's
Philox offset advances per dropout call, which keeps the RNG stream seen by
later random ops identical to the reference's.
"""

from bisect import bisect_left
from functools import lru_cache

import torch


NATIVE_HIDDEN_SIZES = (128, 256, 384, 512, 768, 1024)

# threads per row-CTA of the reference kernels (:5-12)
_THREADS = {128: 128, 256: 128, 384: 128, 512: 128, 768: 128, 1024: 192}

# row-count buckets: rows <= 128, <= 256, <= 512, <= 1024, <= 2048, larger (:35-54)
_ROW_BUCKET_LIMITS = (128, 256, 512, 1024, 2048)
_PARAMETER_GROUPS = {
    128: (80, 12, 48, 80, 96, 128),
    256: (48, 32, 12, 64, 80, 80),
    384: (8, 16, 64, 64, 80, 80),
    512: (48, 48, 48, 64, 48, 48),
    768: (32, 48, 48, 48, 48, 32),
    1024: (32, 32, 32, 24, 24, 24),
}
_WIDE_PARAMETER_THREADS = 256
_NARROW_PARAMETER_THREADS = 64


def _block_rows(hidden_size, row_count):
    """Rows per deterministic partial group in the reference (:23-28)."""
    if row_count > 2048:
        return 64
    if row_count > 512 and hidden_size not in (512, 1024):
        return 32
    return 16


def _parameter_threads(hidden_size, row_count):
    """Threads of the reference's parameter-gradient kernels (:31-38)."""
    tuned_wide = (
        (hidden_size, row_count) in ((512, 256), (256, 512))
        or (hidden_size in (768, 1024) and row_count >= 4096)
    )
    return _WIDE_PARAMETER_THREADS if tuned_wide else _NARROW_PARAMETER_THREADS


def _parameter_groups(hidden_size, row_count):
    """Row groups of the reference's atomic parameter kernels (:41-54)."""
    bucket = bisect_left(_ROW_BUCKET_LIMITS, row_count)
    return min(row_count, _PARAMETER_GROUPS[hidden_size][bucket])


@lru_cache(maxsize=1)
def _extension():
    """Import ``gfx1010_kernels._C`` once; failure becomes a reason string (:57-63)."""
    try:
        from . import _C
    except ImportError as error:
        return None, str(error)
    return _C, ""


def native_extension_status():
    extension, reason = _extension()
    return extension is not None, reason


# extension codes of the ``normalized`` element type (RLN_DTYPE_* of the C header)
NORMALIZED_DTYPE_CODES = {None: 0, torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def normalized_dtype_code(normalized_dtype):
    """Extension code of ``normalized_dtype`` (None = float32); ValueError otherwise."""
    try:
        return NORMALIZED_DTYPE_CODES[normalized_dtype]
    except (KeyError, TypeError):
        raise ValueError(
            "normalized_dtype must be None, torch.float32, torch.float16 or torch.bfloat16"
        ) from None


def native_residual_layer_norm(x, branch, weight, bias, dropout_p, eps, training,
                               normalized_dtype=None):
    """Call the autograd-connected extension entry; no Python-side validation.

    There is deliberately no fallback here: a missing extension raises.
    """
    extension, reason = _extension()
    if extension is None:
        raise RuntimeError(f"gfx1010 native extension is unavailable: {reason}")
    hidden_size = x.shape[-1]
    row_count = x.numel() // hidden_size
    outputs = extension.residual_layer_norm(
        x,
        branch,
        weight,
        bias,
        float(dropout_p),
        float(eps),
        bool(training),
        _THREADS[hidden_size],
        _block_rows(hidden_size, row_count),
        _parameter_threads(hidden_size, row_count),
        _parameter_groups(hidden_size, row_count),
        normalized_dtype_code(normalized_dtype),
    )
    return tuple(outputs)
