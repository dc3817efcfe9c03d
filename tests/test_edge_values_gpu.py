"""Edge values and edge probabilities through the C ABI: non-finite inputs,
fp16 overflow in the dropped branch, extreme dropout probabilities, zero
affine parameters, and tensors on a device other than the current one."""

import numpy as np
import pytest
import torch
from torch.nn import functional as F

import cabi
from helpers import NORMALIZED_TOL, draw_inputs, oracle_keep, unpack_mask_device
from oracle import rln_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dropout_p", [1e-7, 2.0 ** -20, 0.5, 0.999, 1.0 - 2.0 ** -20])
def test_extreme_dropout_probabilities_follow_the_threshold_rule(dropout_p):
    rows, hidden = 512, 256
    x, branch, weight, bias, _, _ = draw_inputs((rows,), hidden, torch.float32, 2)
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, dropout_p, 1e-5, True, seed=3, offset=0
    )
    assert status == 0, cabi.status_text(status)
    keep = unpack_mask_device(mask, rows, hidden)
    assert torch.equal(keep, oracle_keep(rows, hidden, dropout_p, 3, 0))
    expected = rln_oracle.torch_decomposition(x, branch, weight, bias, dropout_p, 1e-5, True, keep)
    assert torch.equal(updated, expected[0])
    assert torch.isfinite(normalized).all()
    torch.testing.assert_close(normalized, expected[1], **NORMALIZED_TOL)
    threshold = rln_oracle.dropout_threshold(dropout_p)
    kept = keep.float().mean().item()
    assert abs(kept - (1 - threshold / 2.0 ** 32)) < 5 * (0.25 / keep.numel()) ** 0.5 + 1e-9


def test_non_finite_inputs_propagate_like_the_decomposition():
    rows, hidden = 9, 384
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, torch.float16, 4
    )
    x[1, 5] = float("inf")
    x[3, 7] = float("nan")
    branch[5, 11] = float("-inf")
    status, updated, normalized, mean, rstd, _ = cabi.forward(
        x, branch, weight, bias, 0.0, 1e-5, True
    )
    assert status == 0
    expected = rln_oracle.torch_decomposition(x, branch, weight, bias, 0.0, 1e-5, True)
    assert torch.equal(torch.isnan(updated), torch.isnan(expected[0]))
    assert torch.equal(updated[~torch.isnan(updated)], expected[0][~torch.isnan(expected[0])])
    # a row that holds inf or nan has no finite statistics; the other rows are untouched
    poisoned = torch.tensor([1, 3, 5], device="cuda")
    clean = torch.tensor([0, 2, 4, 6, 7, 8], device="cuda")
    assert torch.isnan(normalized[poisoned]).all()
    torch.testing.assert_close(normalized[clean], expected[1][clean], **NORMALIZED_TOL)
    status, grad_x, grad_branch, grad_parameters = cabi.backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, None, 0.0, True,
        torch.float16, True,
    )
    assert status == 0
    torch.cuda.synchronize()
    assert torch.isfinite(grad_x[clean]).all() and torch.isfinite(grad_branch[clean]).all()


def test_fp16_overflow_of_the_scaled_branch_rounds_to_infinity_like_the_oracle():
    rows, hidden, p = 4, 128, 0.5
    x = torch.zeros(rows, hidden, device="cuda")
    branch = torch.full((rows, hidden), 60000.0, device="cuda", dtype=torch.float16)
    weight = torch.ones(hidden, device="cuda")
    bias = torch.zeros(hidden, device="cuda")
    status, updated, _, _, _, mask = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=1)
    assert status == 0
    keep = unpack_mask_device(mask, rows, hidden)
    expected = rln_oracle.masked_dropout(branch, keep, p).float()   # 120000 -> inf in fp16
    assert torch.isinf(expected[keep]).all()
    assert torch.equal(updated, x + expected)


def test_zero_weight_and_bias_and_large_magnitudes():
    rows, hidden = 33, 512
    x, branch, _, _, grad_updated, grad_normalized = draw_inputs((rows,), hidden, torch.float32, 6)
    x = x * 1e4
    weight = torch.zeros(hidden, device="cuda")
    bias = torch.zeros(hidden, device="cuda")
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, 0.1, 1e-5, True, seed=2
    )
    assert status == 0
    assert torch.equal(normalized, torch.zeros_like(normalized))
    status, grad_x, grad_branch, grad_parameters = cabi.backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, mask, 0.1, True,
        torch.float32, True,
    )
    assert status == 0
    # gamma = 0 removes the LayerNorm term: the residual gradient passes through
    assert torch.equal(grad_x, grad_updated)
    xhat = (updated.double() - mean.double()[:, None]) * rstd.double()[:, None]
    torch.testing.assert_close(
        grad_parameters[0].double(), (grad_normalized.double() * xhat).sum(0), rtol=1e-4, atol=1e-4
    )
    reference = F.layer_norm(updated, (hidden,), torch.ones_like(weight), bias, 1e-5)
    torch.testing.assert_close(xhat.float(), reference, rtol=1e-4, atol=1e-4)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensors_on_a_device_other_than_the_current_one():
    from gfx1010_kernels import residual_layer_norm

    torch.cuda.set_device(0)
    device = torch.device("cuda", 1)
    torch.manual_seed(3)
    x = torch.randn(17, 768, device=device, requires_grad=True)
    branch = torch.randn(17, 768, device=device, dtype=torch.float16, requires_grad=True)
    weight = torch.randn(768, device=device, requires_grad=True)
    bias = torch.randn(768, device=device, requires_grad=True)
    for implementation in ("gfx1010", "auto"):
        updated, normalized = residual_layer_norm(x, branch, weight, bias,
                                                  implementation=implementation)
        assert updated.device == device and torch.cuda.current_device() == 0
        assert torch.equal(updated, x + branch.float())
        torch.testing.assert_close(
            normalized, F.layer_norm(updated, (768,), weight, bias), **NORMALIZED_TOL
        )
        gradients = torch.autograd.grad(
            (updated, normalized), (x, branch, weight, bias),
            (torch.ones_like(updated), torch.ones_like(normalized)),
        )
        assert all(g.device == device and torch.isfinite(g).all() for g in gradients)
