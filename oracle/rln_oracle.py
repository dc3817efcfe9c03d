"""CPU oracle for the fused residual-add + dropout + LayerNorm operator.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
it is the checker used by the tests, by the smoke entry and by the CPU-baseline
leg of the benchmark.  It never stands in for the CUDA path.

What it restates, and from where (paths are relative to the reference project
T-vaccari/gfx1010-kernels):

* ``torch_decomposition``  follows ``gfx1010_kernels/normalization.py:15-33``
  (dropout -> residual add -> ``F.layer_norm``).  The reference's ``F.dropout``
  draws its own mask, so the oracle takes the keep mask as an argument and
  applies it with the native kernel's rounding rule,
  ``csrc/residual_layer_norm_kernel.hip:491-497``: the branch value is widened
  to fp32, multiplied by keep and by the fp32 scale, rounded ONCE to the branch
  dtype, and only then added to x.
* ``dropout_threshold`` / ``dropout_scale`` follow
  ``csrc/residual_layer_norm_kernel.hip:896-899``.
* ``pack_mask`` / ``unpack_mask`` follow the ballot layout of
  ``csrc/residual_layer_norm_kernel.hip:500-511`` (write) and ``:607-612``
  (read): one uint32 word per 32 columns, word ``row*(H/32) + col/32``,
  bit ``col & 31``.
* ``kernel_backward`` restates the arithmetic of the backward-input kernel
  (``csrc/residual_layer_norm_kernel.hip:548-618``) and of the parameter
  reductions (``:727-786``) in the dtype it is given (use float64 as arbiter).
* ``philox4x32_10`` is the published Philox4x32-10 generator (Salmon, Moraes,
  Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11; Random123).
  The reference obtains it from hipRAND (``hiprand_init``/``hiprand4``,
  ``csrc/residual_layer_norm_kernel.hip:451-481``), a dependency that is not
  vendored in the reference tree; its subsequence layout is not pinned by any
  stored vector in the reference, which only demands replay with the same
  (seed, offset), a kept fraction near 1-p and no overlap between consecutive
  calls.  ``dropout_keep`` therefore states THIS implementation's counter
  layout (the one the sm_100a kernel uses) and is pinned by the Random123
  known-answer vectors in ``tests/golden``.

Parity pin: the decomposition is checked against outputs of the reference's own
``_torch_residual_layer_norm`` (imported from the reference tree when the
fixtures in ``tests/golden`` were generated; the generating script is
``tests/golden/make_golden.py``).
"""

from __future__ import annotations

import numpy as np
import torch
from torch.nn import functional as F


PHILOX_M0 = 0xD2511F53
PHILOX_M1 = 0xCD9E8D57
PHILOX_W0 = 0x9E3779B9
PHILOX_W1 = 0xBB67AE85
_U32 = np.uint64(0xFFFFFFFF)
_SHIFT32 = np.uint64(32)


def philox4x32_10(counter, key):
    """Philox4x32-10 over an array of counters.

    ``counter``: integer array ``[..., 4]`` of 32-bit words; ``key``: two
    32-bit words.  Returns ``uint32[..., 4]``.
    """
    c = np.asarray(counter, dtype=np.uint64)
    c0, c1, c2, c3 = (c[..., i].copy() for i in range(4))
    k0 = int(key[0]) & 0xFFFFFFFF
    k1 = int(key[1]) & 0xFFFFFFFF
    m0 = np.uint64(PHILOX_M0)
    m1 = np.uint64(PHILOX_M1)
    for _ in range(10):
        p0 = m0 * c0
        p1 = m1 * c2
        hi0, lo0 = p0 >> _SHIFT32, p0 & _U32
        hi1, lo1 = p1 >> _SHIFT32, p1 & _U32
        c0, c1, c2, c3 = (
            hi1 ^ c1 ^ np.uint64(k0),
            lo1,
            hi0 ^ c3 ^ np.uint64(k1),
            lo0,
        )
        k0 = (k0 + PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + PHILOX_W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def dropout_threshold(dropout_p):
    """uint32(double(float32(p)) * 2**32); keep <=> random >= threshold."""
    return int(float(np.float32(dropout_p)) * 4294967296.0) & 0xFFFFFFFF


def dropout_scale(dropout_p):
    """fp32 1/(1-p) computed in fp32."""
    return np.float32(1.0) / (np.float32(1.0) - np.float32(dropout_p))


def dropout_random_words(rows, hidden, seed, offset, row_base=0):
    """The 32-bit random word of every element, ``uint32[rows, hidden]``.

    Counter layout of the sm_100a kernel: one Philox call serves the four
    consecutive columns ``4g .. 4g+3`` of element group
    ``g = ((row_base + row) * hidden + col) / 4``; ``offset`` counts 32-bit
    words of the generator's stream and a call yields four, so the counter holds
    the block index ``b = offset // 4``: counter =
    ``(lo32(b), hi32(b), lo32(g), hi32(g))``, key =
    ``(lo32(seed), hi32(seed))``; output word ``j`` belongs to column
    ``4g + j``.  ``row_base`` is the global index of the first row, so a row
    shard reproduces the mask of the unsharded call.
    """
    groups_per_row = hidden // 4
    group = (
        (np.arange(rows, dtype=np.uint64)[:, None] + np.uint64(row_base))
        * np.uint64(groups_per_row)
        + np.arange(groups_per_row, dtype=np.uint64)[None, :]
    )
    counter = np.empty((rows, groups_per_row, 4), dtype=np.uint64)
    block = int(offset) >> 2
    counter[..., 0] = np.uint64(block & 0xFFFFFFFF)
    counter[..., 1] = np.uint64((block >> 32) & 0xFFFFFFFF)
    counter[..., 2] = group & _U32
    counter[..., 3] = group >> _SHIFT32
    key = (int(seed) & 0xFFFFFFFF, (int(seed) >> 32) & 0xFFFFFFFF)
    return philox4x32_10(counter, key).reshape(rows, hidden)


def dropout_keep(rows, hidden, dropout_p, seed, offset, row_base=0):
    """Boolean keep mask ``[rows, hidden]`` of the sm_100a kernel."""
    words = dropout_random_words(rows, hidden, seed, offset, row_base)
    return words >= np.uint32(dropout_threshold(dropout_p))


def pack_mask(keep):
    """bool ``[rows, H]`` -> int32 words ``[rows * H/32]`` (bit = col & 31)."""
    keep = np.asarray(keep, dtype=bool)
    rows, hidden = keep.shape
    bits = keep.reshape(rows, hidden // 32, 32).astype(np.uint64)
    weights = np.uint64(1) << np.arange(32, dtype=np.uint64)
    words = (bits * weights).sum(axis=-1).astype(np.uint32)
    return words.reshape(-1).view(np.int32)


def unpack_mask(words, rows, hidden):
    """int32 words ``[rows * H/32]`` -> bool ``[rows, H]``."""
    words = np.asarray(words).reshape(-1).view(np.uint32).reshape(rows, hidden // 32)
    bits = (words[..., None] >> np.arange(32, dtype=np.uint32)) & np.uint32(1)
    return bits.reshape(rows, hidden).astype(bool)


def masked_dropout(branch, keep, dropout_p):
    """Dropout with a given keep mask and the native kernel's rounding.

    ``round_to_branch_dtype(float32(branch) * keep * float32_scale)``
    (``csrc/residual_layer_norm_kernel.hip:491-497``).  Differentiable with
    respect to ``branch``.
    """
    scale = float(dropout_scale(dropout_p))
    keep = torch.as_tensor(keep, device=branch.device)
    wide = branch.to(torch.float32) * keep.to(torch.float32)
    wide = wide * torch.tensor(scale, dtype=torch.float32, device=branch.device)
    return wide.to(branch.dtype)


def torch_decomposition(
    x,
    branch,
    weight,
    bias,
    dropout_p=0.0,
    eps=1e-5,
    training=True,
    keep=None,
    normalized_dtype=None,
):
    """``normalization.py:15-33`` with the dropout mask supplied by the caller.

    ``keep=None`` with active dropout falls back to ``F.dropout`` exactly as the
    reference does (used only for timing the CPU baseline, where the mask values
    do not matter).  ``normalized_dtype`` (float16 / bfloat16; not part of the
    reference) rounds ``normalized`` once at the end, as the native kernels do
    on store; autograd then widens the incoming gradient.
    """
    active = training and dropout_p > 0.0
    if active and keep is not None:
        dropped = masked_dropout(branch, keep.reshape(branch.shape), dropout_p)
    elif training:
        dropped = F.dropout(branch, dropout_p, True)
    else:
        dropped = branch
    updated = x + dropped
    normalized = F.layer_norm(updated, (updated.shape[-1],), weight, bias, eps)
    if normalized_dtype is not None and normalized_dtype != normalized.dtype:
        normalized = normalized.to(normalized_dtype)
    return updated, normalized


def row_statistics(updated, eps):
    """Per-row mean and rstd in the two-pass centred form
    (``csrc/residual_layer_norm_kernel.hip:516-528``)."""
    mean = updated.mean(dim=-1)
    centered = updated - mean[..., None]
    variance = (centered * centered).mean(dim=-1)
    return mean, torch.rsqrt(variance + eps)


def decomposition_gradients(
    x,
    branch,
    weight,
    bias,
    grad_updated,
    grad_normalized,
    dropout_p=0.0,
    eps=1e-5,
    training=True,
    keep=None,
    dtype=None,
    normalized_dtype=None,
):
    """Forward + autograd through ``torch_decomposition``.

    ``dtype=torch.float64`` gives the arbiter copy: all tensors are widened
    AFTER the branch-dtype rounding of the dropped branch, so the arbiter sees
    the same ``updated`` values as the fp32 path.  With ``normalized_dtype``
    the fp32 path returns ``normalized`` in that type and expects
    ``grad_normalized`` in it; the arbiter keeps ``normalized`` unrounded.
    Returns ``(updated, normalized, grad_x, grad_branch, grad_weight, grad_bias)``.
    """
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, branch, weight, bias)]
    lx, lb, lw, lbias = leaves
    if dtype is None:
        updated, normalized = torch_decomposition(
            lx, lb, lw, lbias, dropout_p, eps, training, keep, normalized_dtype
        )
    else:
        active = training and dropout_p > 0.0
        if active:
            dropped = masked_dropout(lb, torch.as_tensor(keep).reshape(lb.shape), dropout_p)
        else:
            dropped = lb
        updated = lx.to(dtype) + dropped.to(dtype)
        normalized = F.layer_norm(
            updated, (updated.shape[-1],), lw.to(dtype), lbias.to(dtype), eps
        )
        grad_updated = grad_updated.to(dtype)
        grad_normalized = grad_normalized.to(dtype)
    grads = torch.autograd.grad(
        (updated, normalized), leaves, (grad_updated, grad_normalized)
    )
    return (updated.detach(), normalized.detach(), *grads)


def kernel_backward(
    grad_updated,
    grad_normalized,
    updated,
    weight,
    mean,
    rstd,
    keep,
    dropout_p,
    dropout_active,
    branch_dtype,
    dtype=torch.float64,
):
    """The native backward's formulas, evaluated in ``dtype``.

    ``csrc/residual_layer_norm_kernel.hip:548-618``:
    ``xhat = (u - mean) * rstd``; ``q = g_y * gamma``;
    ``g = g_u + rstd * (q - mean(q) - xhat * mean(q * xhat))``;
    ``grad_x = g``; ``grad_branch = round(g * keep * scale)``.
    ``:727-786``: ``grad_weight = sum_rows g_y * xhat``; ``grad_bias = sum_rows g_y``.
    """
    hidden = updated.shape[-1]
    u = updated.reshape(-1, hidden).to(dtype)
    gu = grad_updated.reshape(-1, hidden).to(dtype)
    gy = grad_normalized.reshape(-1, hidden).to(dtype)
    xhat = (u - mean.reshape(-1, 1).to(dtype)) * rstd.reshape(-1, 1).to(dtype)
    q = gy * weight.to(dtype)
    mean_q = q.mean(dim=-1, keepdim=True)
    mean_qx = (q * xhat).mean(dim=-1, keepdim=True)
    g = gu + rstd.reshape(-1, 1).to(dtype) * (q - mean_q - xhat * mean_qx)
    grad_branch = g
    if dropout_active:
        scale = float(dropout_scale(dropout_p))
        grad_branch = g * torch.as_tensor(keep).reshape(g.shape).to(dtype) * scale
    grad_weight = (gy * xhat).sum(dim=0)
    grad_bias = gy.sum(dim=0)
    return (
        g.reshape(updated.shape),
        grad_branch.to(branch_dtype).reshape(updated.shape),
        grad_weight,
        grad_bias,
    )
