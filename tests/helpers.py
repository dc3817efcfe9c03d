"""Shared helpers of the GPU parity tests: seeded inputs in the distributions
the benchmark configurations name, mask unpacking on the device, and the
tolerances the parity claims are made at."""

import numpy as np
import torch

from oracle import rln_oracle

# Tolerances (|actual - expected| <= atol + rtol * |expected|).
# `updated` is compared with torch.equal: one fp32 add of identical operands is exact.
NORMALIZED_TOL = dict(rtol=1e-5, atol=1e-6)      # vs the torch decomposition with the kernel's mask
GRAD_X_TOL = dict(rtol=1e-5, atol=1e-5)
GRAD_BRANCH_HALF_TOL = dict(rtol=2e-3, atol=1e-5)  # one fp16 rounding of an fp32-close value
GRAD_BRANCH_BF16_TOL = dict(rtol=1.6e-2, atol=1e-5)  # one bfloat16 rounding (8 significant bits)


def grad_branch_tolerance(branch_dtype):
    import torch as _torch

    if branch_dtype == _torch.float16:
        return GRAD_BRANCH_HALF_TOL
    if branch_dtype == _torch.bfloat16:
        return GRAD_BRANCH_BF16_TOL
    return GRAD_X_TOL


def assert_narrow_normalized(actual, reference64, what="normalized"):
    """``actual`` (float16 / bfloat16) is the single rounding of a float32 value
    within NORMALIZED_TOL of ``reference64``.

    Rounding to nearest is monotonic, so a float32 result in
    ``[r - tol, r + tol]`` must round into ``[round(r - tol), round(r + tol)]``:
    the check is exact, with no extra slack for the 16-bit type.
    """
    reference64 = reference64.double().reshape(actual.shape)
    tolerance = NORMALIZED_TOL["atol"] + NORMALIZED_TOL["rtol"] * reference64.abs()
    low = (reference64 - tolerance).float().to(actual.dtype).double()
    high = (reference64 + tolerance).float().to(actual.dtype).double()
    value = actual.double()
    inside = (value >= low) & (value <= high)
    assert bool(inside.all()), (
        f"{what}: {int((~inside).sum())} of {inside.numel()} elements are not the rounding "
        f"of a float32-close value"
    )


PARAM_RTOL = 1e-4                                 # grad_weight / grad_bias, relative


def draw_inputs(shape, hidden, branch_dtype, seed, device="cuda"):
    """x ~ N(0,1) fp32, branch ~ N(0,1) in its dtype, weight = 1 + 0.1 N(0,1),
    bias = 0.1 N(0,1), both upstream gradients ~ N(0,1); drawn on the CPU in a
    fixed order so that CPU and GPU runs see identical values."""
    generator = torch.Generator().manual_seed(seed)
    if isinstance(shape, int):
        shape = (shape,)
    full = (*shape, hidden)
    x = torch.randn(full, generator=generator)
    branch = torch.randn(full, generator=generator).to(branch_dtype)
    weight = 1.0 + 0.1 * torch.randn(hidden, generator=generator)
    bias = 0.1 * torch.randn(hidden, generator=generator)
    grad_updated = torch.randn(full, generator=generator)
    grad_normalized = torch.randn(full, generator=generator)
    return tuple(
        t.to(device) for t in (x, branch, weight, bias, grad_updated, grad_normalized)
    )


def unpack_mask_device(mask, rows, hidden):
    """int32 words on the device -> bool [rows, hidden] on the device."""
    words = mask.view(rows, hidden // 32, 1)
    shifts = torch.arange(32, device=mask.device, dtype=torch.int32).view(1, 1, 32)
    return ((words >> shifts) & 1).bool().view(rows, hidden)


def oracle_keep(rows, hidden, dropout_p, seed, offset, row_base=0, device="cuda"):
    keep = rln_oracle.dropout_keep(rows, hidden, dropout_p, seed, offset, row_base)
    return torch.from_numpy(keep).to(device)


def assert_parameters_close(actual, expected64, rows, what):
    """<= 1e-4 relative, with an absolute floor of 1e-5 * sqrt(rows) (the sums
    have magnitude ~sqrt(rows); entries that cancel to near zero are compared
    on that scale)."""
    torch.testing.assert_close(
        actual.double(),
        expected64.double(),
        rtol=PARAM_RTOL,
        atol=1e-5 * float(np.sqrt(rows)),
        msg=lambda text: f"{what}: {text}",
    )
