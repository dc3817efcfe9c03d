"""The benchmark configurations at their full sizes, through the C ABI.

At these sizes the checks are size-independent properties of the operator plus
a direct comparison with the torch decomposition evaluated on the same device
(the decomposition is cheap on a GPU even at 268 M elements):

* replay with the same (seed, offset) is bit-exact, another offset is not;
* ``updated - x`` is exactly the rounded, scaled branch where the returned mask
  keeps and 0 where it drops; the kept fraction is within 4 sigma of 1 - p;
* ``normalized`` equals LayerNorm(updated) to 1e-5 / 1e-6;
* the backward is linear: doubling both upstream gradients doubles every
  output bit for bit (a power-of-two scale is exact in binary floating point);
* per row, ``grad_x - grad_updated`` has zero mean and is orthogonal to xhat;
* ``grad_bias`` is the column sum of ``grad_normalized`` (a checksum of
  checksums) and ``grad_weight`` the column sum of ``grad_normalized * xhat``;
* deterministic mode replays bit for bit; row shards reproduce the unsharded
  call.
"""

import numpy as np
import pytest
import torch
from torch.nn import functional as F

import cabi
from helpers import (
    NORMALIZED_TOL,
    assert_parameters_close,
    grad_branch_tolerance,
    unpack_mask_device,
)

pytestmark = pytest.mark.gpu

CONFIGS = {
    # name: (rows, hidden, branch dtype, p)
    "transformer_width_384": (16 * 2048, 384, torch.float16, 0.1),
    "transformer_width_512": (16 * 2048, 512, torch.float16, 0.1),
    "transformer_width_768": (16 * 2048, 768, torch.float16, 0.1),
    "transformer_width_1024": (16 * 2048, 1024, torch.float16, 0.1),
    "headline_64Mi_h768": (87381, 768, torch.float16, 0.1),
    "headline_64Mi_h768_bf16": (87381, 768, torch.bfloat16, 0.1),
    "ragged_h128_fp32": (3 * 1367, 128, torch.float32, 0.15),
    "ragged_h256_fp32": (5 * 817, 256, torch.float32, 0.15),
}


def device_inputs(rows, hidden, branch_dtype, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, hidden, device="cuda", generator=generator)
    branch = torch.randn(rows, hidden, device="cuda", generator=generator).to(branch_dtype)
    weight = 1.0 + 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    bias = 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    grad_updated = torch.randn(rows, hidden, device="cuda", generator=generator)
    grad_normalized = torch.randn(rows, hidden, device="cuda", generator=generator)
    return x, branch, weight, bias, grad_updated, grad_normalized


def check_forward_properties(x, branch, weight, bias, p, outputs):
    _, updated, normalized, mean, rstd, mask = outputs
    rows, hidden = x.shape
    keep = unpack_mask_device(mask, rows, hidden)
    p32 = np.float32(p)
    scale = float(np.float32(1.0) / (np.float32(1.0) - p32))
    dropped = (branch.float() * keep.float() * scale).to(branch.dtype).float()
    assert torch.equal(updated, x + dropped)
    sigma = (float(p32) * (1 - float(p32)) / keep.numel()) ** 0.5
    assert abs(keep.float().mean().item() - (1 - float(p32))) < 4 * sigma
    torch.testing.assert_close(
        normalized, F.layer_norm(updated, (hidden,), weight, bias, 1e-5), **NORMALIZED_TOL
    )
    torch.testing.assert_close(mean, updated.mean(dim=-1), rtol=1e-5, atol=1e-6)
    variance = updated.double().var(dim=-1, unbiased=False)
    torch.testing.assert_close(rstd.double(), torch.rsqrt(variance + 1e-5), rtol=1e-5, atol=0)
    return keep


@pytest.mark.parametrize("name", list(CONFIGS))
def test_full_size_forward_and_backward_properties(name):
    rows, hidden, branch_dtype, p = CONFIGS[name]
    x, branch, weight, bias, grad_updated, grad_normalized = device_inputs(
        rows, hidden, branch_dtype, seed=len(name)
    )
    first = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=0, offset=0)
    again = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=0, offset=0)
    other = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=0, offset=4)
    assert first[0] == again[0] == other[0] == 0
    for a, b in zip(first[1:], again[1:]):
        assert torch.equal(a, b)
    assert not torch.equal(first[5], other[5])
    keep = check_forward_properties(x, branch, weight, bias, p, first)
    del again, other

    _, updated, _, mean, rstd, mask = first
    args = (updated, weight, mean, rstd, mask, p, True, branch_dtype)
    once = cabi.backward(grad_updated, grad_normalized, *args, True)
    twice = cabi.backward(grad_updated, grad_normalized, *args, True)
    doubled = cabi.backward(2 * grad_updated, 2 * grad_normalized, *args, True)
    atomic = cabi.backward(grad_updated, grad_normalized, *args, False)
    assert once[0] == twice[0] == doubled[0] == atomic[0] == 0
    torch.cuda.synchronize()
    for a, b in zip(once[1:], twice[1:]):
        assert torch.equal(a, b)                      # deterministic replay
    for a, b in zip(once[1:], doubled[1:]):
        expected = 2 * a.float()
        if a.dtype == torch.bfloat16:
            assert torch.equal(expected, b.float())       # bfloat16 has float32's exponent range
        elif a.dtype == torch.float16:
            # doubling commutes with rounding except among fp16 subnormals,
            # where the grid spacing (2**-24) does not scale with the value
            normal = a.float().abs() >= 2.0 ** -13
            assert torch.equal(expected[normal], b.float()[normal])
            assert (expected - b.float()).abs().max().item() <= 2.0 ** -23
        else:
            assert torch.equal(expected, b)               # linearity, exact
    assert torch.equal(once[1], atomic[1]) and torch.equal(once[2], atomic[2])

    grad_x, grad_branch, grad_parameters = once[1], once[2], once[3]
    xhat = (updated - mean[:, None]) * rstd[:, None]
    delta = grad_x - grad_updated
    assert delta.mean(dim=-1).abs().max().item() < 1e-4
    assert (delta * xhat).mean(dim=-1).abs().max().item() < 1e-4
    expected_bias = grad_normalized.double().sum(dim=0)
    expected_weight = (grad_normalized.double() * xhat.double()).sum(dim=0)
    for parameters in (grad_parameters, atomic[3]):
        assert_parameters_close(parameters[0], expected_weight, rows, "grad_weight")
        assert_parameters_close(parameters[1], expected_bias, rows, "grad_bias")
    scale = float(np.float32(1.0) / (np.float32(1.0) - np.float32(p)))
    assert torch.equal(grad_branch, (grad_x * keep.float() * scale).to(branch_dtype))

    # direct comparison with autograd through the decomposition, same device
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, branch, weight, bias)]
    dropped = (leaves[1].float() * keep.float() * scale).to(branch_dtype)
    reference_updated = leaves[0] + dropped
    reference_normalized = F.layer_norm(reference_updated, (hidden,), leaves[2], leaves[3], 1e-5)
    reference = torch.autograd.grad(
        (reference_updated, reference_normalized), leaves, (grad_updated, grad_normalized)
    )
    torch.testing.assert_close(grad_x, reference[0], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(
        grad_branch.float(), reference[1].float(), **grad_branch_tolerance(branch_dtype)
    )
    assert_parameters_close(grad_parameters[0], reference[2], rows, "grad_weight vs autograd")
    assert_parameters_close(grad_parameters[1], reference[3], rows, "grad_bias vs autograd")


def test_deterministic_mode_at_32x4096x1024():
    """x fp32 [32, 4096, 1024], fp16 branch, p 0.15: two full runs with the same
    seed/offset give bitwise-identical outputs, mask and gradients."""
    rows, hidden, p = 32 * 4096, 1024, 0.15
    x, branch, weight, bias, grad_updated, grad_normalized = device_inputs(
        rows, hidden, torch.float16, seed=4
    )
    runs = []
    for _ in range(2):
        forward = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=3, offset=20)
        assert forward[0] == 0
        backward = cabi.backward(
            grad_updated, grad_normalized, forward[1], weight, forward[3], forward[4],
            forward[5], p, True, torch.float16, True,
        )
        assert backward[0] == 0
        runs.append((*forward[1:], *backward[1:]))
    torch.cuda.synchronize()
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    check_forward_properties(x, branch, weight, bias, p, (0, *runs[0][:5]))


def test_row_sharded_64x4096x1024_reproduces_unsharded_rows():
    """x fp32 [64, 4096, 1024] (268 M elements) cut into 8 row shards: every
    shard's mask and row-local outputs equal the unsharded call's rows."""
    rows, hidden, p, world = 64 * 4096, 1024, 0.1, 8
    x, branch, weight, bias, grad_updated, grad_normalized = device_inputs(
        rows, hidden, torch.float16, seed=5
    )
    whole = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=1, offset=0)
    assert whole[0] == 0
    whole_back = cabi.backward(
        grad_updated, grad_normalized, whole[1], weight, whole[3], whole[4], whole[5],
        p, True, torch.float16, True,
    )
    assert whole_back[0] == 0
    total = torch.zeros(2, hidden, device="cuda", dtype=torch.float64)
    for rank in range(world):
        begin, end = rows * rank // world, rows * (rank + 1) // world
        piece = cabi.forward(
            x[begin:end], branch[begin:end], weight, bias, p, 1e-5, True,
            seed=1, offset=0, row_base=begin,
        )
        assert piece[0] == 0
        words = hidden // 32
        assert torch.equal(piece[1], whole[1][begin:end])
        assert torch.equal(piece[2], whole[2][begin:end])
        assert torch.equal(piece[5], whole[5][begin * words:end * words])
        back = cabi.backward(
            grad_updated[begin:end], grad_normalized[begin:end], piece[1], weight, piece[3],
            piece[4], piece[5], p, True, torch.float16, False,
        )
        assert back[0] == 0
        assert torch.equal(back[1], whole_back[1][begin:end])
        assert torch.equal(back[2], whole_back[2][begin:end])
        total += back[3].double()
    assert_parameters_close(whole_back[3][0], total[0], rows, "grad_weight")
    assert_parameters_close(whole_back[3][1], total[1], rows, "grad_bias")


def test_more_than_2_to_the_31_elements_is_indexed_with_64_bits():
    """2,100,000 x 1,024 = 2.15e9 elements per tensor: element offsets no longer
    fit in 32 bits.  The last rows of the big call must equal a small call on
    those rows alone (given the same global row offset), forward and backward."""
    rows, hidden, p, tail = 2_100_000, 1024, 0.1, 96
    free_bytes = torch.cuda.mem_get_info()[0]
    if free_bytes < 80 * (1 << 30):
        pytest.skip("needs about 70 GB of free device memory")
    generator = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(rows, hidden, device="cuda", generator=generator)
    branch = torch.randn(rows, hidden, device="cuda", generator=generator, dtype=torch.float16)
    weight = 1.0 + 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    bias = 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    assert x.numel() > 2 ** 31
    big = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=2, offset=8)
    assert big[0] == 0, cabi.status_text(big[0])
    begin = rows - tail
    small = cabi.forward(
        x[begin:], branch[begin:], weight, bias, p, 1e-5, True, seed=2, offset=8, row_base=begin
    )
    assert small[0] == 0
    words = hidden // 32
    assert torch.equal(big[1][begin:], small[1])
    assert torch.equal(big[2][begin:], small[2])
    assert torch.equal(big[3][begin:], small[3])
    assert torch.equal(big[4][begin:], small[4])
    assert torch.equal(big[5][begin * words:], small[5])
    # rows just below the 2**31-element boundary and the very first rows too
    boundary = (2 ** 31) // hidden
    for lo in (0, boundary - 8):
        piece = cabi.forward(
            x[lo:lo + 16], branch[lo:lo + 16], weight, bias, p, 1e-5, True,
            seed=2, offset=8, row_base=lo,
        )
        assert torch.equal(big[1][lo:lo + 16], piece[1])
        assert torch.equal(big[5][lo * words:(lo + 16) * words], piece[5])
    keep_fraction = unpack_mask_device(big[5][-words * 4096:], 4096, hidden).float().mean().item()
    assert abs(keep_fraction - 0.9) < 4 * (0.09 / (4096 * hidden)) ** 0.5

    _, updated, _, mean, rstd, mask = big
    del x, branch, big, small, piece
    torch.cuda.empty_cache()
    grad_updated = torch.randn(rows, hidden, device="cuda", generator=generator)
    grad_normalized = torch.randn(rows, hidden, device="cuda", generator=generator)
    whole = cabi.backward(grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
                          p, True, torch.float16, True)
    assert whole[0] == 0, cabi.status_text(whole[0])
    part = cabi.backward(
        grad_updated[begin:], grad_normalized[begin:], updated[begin:], weight, mean[begin:],
        rstd[begin:], mask[begin * words:], p, True, torch.float16, True,
    )
    assert part[0] == 0
    torch.cuda.synchronize()
    assert torch.equal(whole[1][begin:], part[1])
    assert torch.equal(whole[2][begin:], part[2])
    expected_bias = grad_normalized.sum(dim=0, dtype=torch.float64)
    assert_parameters_close(whole[3][1], expected_bias, rows, "grad_bias")


@pytest.mark.parametrize(
    "rows,hidden,branch_dtype,normalized_dtype",
    [
        (87381, 768, torch.float16, torch.bfloat16),
        (87381, 768, torch.bfloat16, torch.float16),
        (64 * 4096, 1024, torch.float16, torch.bfloat16),
        (5 * 817, 256, torch.float32, torch.bfloat16),
    ],
)
def test_full_size_16_bit_normalized_is_the_cast_of_the_float32_path(
        rows, hidden, branch_dtype, normalized_dtype):
    """The 16-bit `normalized` path is the float32 path with one rounding on
    store and one widening on load, so at any size: every other forward output
    is bit-identical, `normalized` is bit-identical to the cast of the float32
    output, and the backward fed the 16-bit gradient is bit-identical to the
    float32 backward fed the widened gradient (fixed-order mode)."""
    x, branch, weight, bias, grad_updated, grad_normalized = device_inputs(
        rows, hidden, branch_dtype, seed=rows % 97
    )
    p = 0.1
    wide = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=3, offset=8)
    narrow = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=3, offset=8,
                          normalized_dtype=normalized_dtype)
    assert wide[0] == narrow[0] == 0
    for index in (1, 3, 4, 5):                       # updated, mean, rstd, mask
        assert torch.equal(wide[index], narrow[index])
    assert narrow[2].dtype == normalized_dtype
    assert torch.equal(narrow[2], wide[2].to(normalized_dtype))

    narrow_gradient = grad_normalized.to(normalized_dtype)
    _, updated, _, mean, rstd, mask = wide
    args = (updated, weight, mean, rstd, mask, p, True, branch_dtype, True)
    from_narrow = cabi.backward(grad_updated, narrow_gradient, *args)
    from_wide = cabi.backward(grad_updated, narrow_gradient.float(), *args)
    assert from_narrow[0] == from_wide[0] == 0
    torch.cuda.synchronize()
    for a, b in zip(from_narrow[1:], from_wide[1:]):
        assert torch.equal(a, b)


@pytest.mark.parametrize(
    "rows,hidden", [(8 * 1024, 768), (64 * 4096, 1024)], ids=["8x1024x768", "64x4096x1024"]
)
def test_parameter_gradients_meet_the_relative_bound_without_the_floor(rows, hidden):
    """grad_weight / grad_bias against float64 column sums with the bare 1e-4
    relative bound (no absolute floor), on every column whose exact sum is not a
    near-total cancellation (|sum| >= 1 % of the sqrt(rows) scale of such sums);
    both the atomic and the fixed-order path."""
    x, branch, weight, bias, grad_updated, grad_normalized = device_inputs(
        rows, hidden, torch.float16, seed=rows % 97
    )
    _, updated, _, mean, rstd, mask = cabi.forward(x, branch, weight, bias, 0.1, 1e-5, True)
    xhat = (updated.double() - mean.double()[:, None]) * rstd.double()[:, None]
    exact = torch.stack(((grad_normalized.double() * xhat).sum(0), grad_normalized.double().sum(0)))
    del xhat
    for deterministic in (False, True):
        status, _, _, parameters = cabi.backward(
            grad_updated, grad_normalized, updated, weight, mean, rstd, mask, 0.1, True,
            torch.float16, deterministic,
        )
        assert status == 0
        relative = (parameters.double() - exact).abs() / exact.abs()
        meaningful = exact.abs() >= 0.01 * rows ** 0.5
        assert meaningful.float().mean().item() > 0.95
        worst = relative[meaningful].max().item()
        assert worst <= 1e-4, f"worst relative error {worst:.3g} (deterministic={deterministic})"
