"""``ResidualLayerNorm``: LayerNorm-compatible state, decomposition semantics
on CPU, native kernels on a B200."""

import warnings

import pytest
import torch
from torch import nn
from torch.nn import functional as F

from gfx1010_kernels.modules import ResidualLayerNorm


def test_state_dict_is_interchangeable_with_layer_norm():
    reference = nn.LayerNorm(256, eps=1e-3)
    with torch.no_grad():
        reference.weight.normal_()
        reference.bias.normal_()
    module = ResidualLayerNorm(256, dropout_p=0.1, eps=1e-3)
    assert set(module.state_dict()) == set(reference.state_dict()) == {"weight", "bias"}
    module.load_state_dict(reference.state_dict())
    reference.load_state_dict(module.state_dict())
    assert module.native_width and not ResidualLayerNorm(160).native_width
    with pytest.raises(ValueError):
        ResidualLayerNorm(128, dropout_p=1.0)
    assert "dropout_p=0.1" in repr(module)


def test_cpu_module_matches_the_decomposition_in_eval_and_training():
    torch.manual_seed(0)
    module = ResidualLayerNorm(128, dropout_p=0.5, implementation="torch")
    x = torch.randn(3, 5, 128)
    branch = torch.randn(3, 5, 128)
    module.eval()
    updated, normalized = module(x, branch)
    assert torch.equal(updated, x + branch)
    torch.testing.assert_close(
        normalized, F.layer_norm(x + branch, (128,), module.weight, module.bias, module.eps)
    )
    module.train()
    updated, normalized = module(x, branch)
    kept = ((updated - x) != 0).float().mean().item()
    assert 0.3 < kept < 0.7
    (updated.sum() + normalized.sum()).backward()
    assert module.weight.grad is not None and module.bias.grad is not None


def test_auto_on_cpu_warns_and_still_works():
    module = ResidualLayerNorm(128)
    with pytest.warns(RuntimeWarning, match="was not used"):
        module(torch.randn(2, 128), torch.randn(2, 128))


@pytest.mark.gpu
def test_module_runs_the_native_kernels_on_gpu():
    torch.manual_seed(1)
    module = ResidualLayerNorm(768, dropout_p=0.0, implementation="gfx1010").cuda()
    x = torch.randn(4, 9, 768, device="cuda", requires_grad=True)
    branch = torch.randn(4, 9, 768, device="cuda", dtype=torch.float16, requires_grad=True)
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        updated, normalized = module(x, branch)
    assert torch.equal(updated, x + branch.float())
    torch.testing.assert_close(
        normalized, F.layer_norm(updated, (768,), module.weight, module.bias, module.eps),
        rtol=1e-5, atol=1e-6,
    )
    (updated.square().sum() + normalized.sum()).backward()
    assert module.weight.grad.shape == (768,) and x.grad is not None and branch.grad is not None


def test_module_passes_normalized_dtype_through():
    module = ResidualLayerNorm(128, implementation="torch", normalized_dtype=torch.bfloat16)
    updated, normalized = module(torch.randn(3, 128), torch.randn(3, 128))
    assert updated.dtype == torch.float32 and normalized.dtype == torch.bfloat16
    assert "normalized_dtype=torch.bfloat16" in repr(module)
    assert "normalized_dtype" not in repr(ResidualLayerNorm(128))


def test_from_layer_norm_shares_the_parameters_of_the_wrapped_module():
    torch.manual_seed(0)
    original = torch.nn.LayerNorm(128, eps=3e-5)
    with torch.no_grad():
        original.weight.normal_()
        original.bias.normal_()
    original.eval()
    wrapped = ResidualLayerNorm.from_layer_norm(original, dropout_p=0.25, implementation="torch")
    assert wrapped.weight is original.weight and wrapped.bias is original.bias
    assert wrapped.eps == original.eps and wrapped.dropout_p == 0.25 and not wrapped.training
    x, branch = torch.randn(5, 128), torch.randn(5, 128)
    updated, normalized = wrapped(x, branch)
    torch.testing.assert_close(updated, x + branch)
    torch.testing.assert_close(normalized, original(x + branch))
    # gradients land in the original module's parameters
    wrapped.train()
    wrapped(x, branch)[1].sum().backward()
    assert original.weight.grad is not None and original.bias.grad is not None
    with pytest.raises(ValueError):
        ResidualLayerNorm.from_layer_norm(torch.nn.LayerNorm((4, 128)))
    with pytest.raises(ValueError):
        ResidualLayerNorm.from_layer_norm(torch.nn.LayerNorm(128, elementwise_affine=False))
    with pytest.raises(TypeError):
        ResidualLayerNorm.from_layer_norm(torch.nn.Linear(4, 4))
