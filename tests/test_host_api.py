"""Host-side behaviour of the public API that needs no GPU.  These follow the
CPU-runnable checks of the reference's own test-suite
(tests/test_residual_layer_norm.py:34-99, 274-287; tests/test_api.py:43-48;
tests/test_residual_layer_norm_edge_cases.py:77-95, 382-396)."""

import pytest
import torch
from torch.nn import functional as F

import gfx1010_kernels
from gfx1010_kernels import (
    BackendStatus,
    can_use_residual_layer_norm,
    residual_layer_norm,
    residual_layer_norm_status,
)
import gfx1010_kernels.normalization as normalization


def decomposition(x, branch, weight, bias, dropout_p=0.0, eps=1e-5, training=True):
    if training:
        branch = F.dropout(branch, dropout_p, True)
    updated = x + branch
    return updated, F.layer_norm(updated, (updated.shape[-1],), weight, bias, eps)


def test_public_surface():
    assert gfx1010_kernels.__version__ == "0.4.0"
    assert callable(gfx1010_kernels.residual_layer_norm_status)
    status = residual_layer_norm_status()
    assert isinstance(status, BackendStatus)
    with pytest.raises(Exception):
        status.available = True  # frozen record


def test_status_without_cuda_or_for_a_cpu_device():
    if not torch.cuda.is_available():
        status = residual_layer_norm_status()
        assert not status.available
        assert status.reason == "PyTorch CUDA/HIP is unavailable"
    else:
        status = residual_layer_norm_status("cpu")
        assert not status.available
        assert status.reason == "the device must be a HIP GPU"


def test_auto_on_cpu_warns_and_uses_the_decomposition():
    x = torch.randn(2, 4, 16)
    branch = torch.randn_like(x)
    weight = torch.randn(16)
    bias = torch.randn(16)
    with pytest.warns(RuntimeWarning, match="was not used"):
        actual = residual_layer_norm(x, branch, weight, bias)
    expected = decomposition(x, branch, weight, bias)
    torch.testing.assert_close(actual[0], expected[0])
    torch.testing.assert_close(actual[1], expected[1])
    assert not can_use_residual_layer_norm(x, branch, weight, bias)


def test_torch_route_is_differentiable_and_matches():
    torch.manual_seed(3)
    x = torch.randn(3, 128, requires_grad=True)
    branch = torch.randn(3, 128, requires_grad=True)
    weight = torch.randn(128, requires_grad=True)
    bias = torch.randn(128, requires_grad=True)
    updated, normalized = residual_layer_norm(x, branch, weight, bias, implementation="torch")
    (updated.sum() + normalized.square().sum()).backward()
    assert all(t.grad is not None for t in (x, branch, weight, bias))


def test_eval_mode_on_torch_route_consumes_no_rng():
    torch.manual_seed(101)
    x = torch.randn(7, 384)
    branch = torch.randn(7, 384)
    weight = torch.randn(384)
    bias = torch.randn(384)
    state = torch.random.get_rng_state()
    actual = residual_layer_norm(
        x, branch, weight, bias, dropout_p=0.8, training=False, implementation="torch"
    )
    expected = decomposition(x, branch, weight, bias, 0.8, training=False)
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=1e-6)
    torch.testing.assert_close(actual[1], expected[1], rtol=5e-4, atol=5e-4)
    assert torch.equal(torch.random.get_rng_state(), state)


def test_forced_route_reports_cpu_input_before_backend_lookup(monkeypatch):
    def fail(*args, **kwargs):
        raise AssertionError("forced CPU input reached backend lookup")

    monkeypatch.setattr(normalization, "residual_layer_norm_status", fail)
    x = torch.randn(2, 4, 128)
    with pytest.raises(RuntimeError, match="x must be a HIP tensor"):
        residual_layer_norm(x, x, torch.ones(128), torch.zeros(128), implementation="gfx1010")


def test_forced_route_reports_hidden_size_before_backend_lookup(monkeypatch):
    class FakeCudaTensor:
        is_cuda = True
        ndim = 2
        shape = (4, 160)

    def fail(*args, **kwargs):
        raise AssertionError("invalid hidden size reached backend lookup")

    monkeypatch.setattr(normalization, "residual_layer_norm_status", fail)
    tensor = FakeCudaTensor()
    with pytest.raises(RuntimeError, match="native hidden size must be one of"):
        residual_layer_norm(tensor, tensor, tensor, tensor, implementation="gfx1010")


def test_forced_route_reports_scalar_input():
    class FakeScalar:
        is_cuda = True
        ndim = 0
        shape = ()

    tensor = FakeScalar()
    with pytest.raises(RuntimeError, match="at least two dimensions"):
        residual_layer_norm(tensor, tensor, tensor, tensor, implementation="gfx1010")


def test_forced_route_reports_backend_reason(monkeypatch):
    class FakeCudaTensor:
        is_cuda = True
        ndim = 2
        shape = (4, 128)
        device = "cuda:0"

    monkeypatch.setattr(
        normalization,
        "residual_layer_norm_status",
        lambda device=None: BackendStatus(False, "x", "sm_90", "the native extension targets sm_100 (B200)"),
    )
    tensor = FakeCudaTensor()
    with pytest.raises(RuntimeError, match="targets sm_100"):
        residual_layer_norm(tensor, tensor, tensor, tensor, implementation="gfx1010")


def test_unknown_implementation_is_a_value_error():
    x = torch.randn(2, 128)
    with pytest.raises(ValueError, match="implementation must be"):
        residual_layer_norm(x, x, torch.ones(128), torch.zeros(128), implementation="hip")


def test_triton_route_is_unavailable():
    x = torch.randn(2, 128)
    with pytest.raises(RuntimeError, match="unavailable"):
        residual_layer_norm(x, x, torch.ones(128), torch.zeros(128), implementation="triton")


@pytest.mark.parametrize(
    "mutate,reason",
    [
        (lambda a: a.update(x=torch.randn(128)), "x must be a HIP tensor"),
    ],
)
def test_input_reason_first_check(mutate, reason):
    arguments = dict(
        x=torch.randn(2, 128), branch=torch.randn(2, 128),
        weight=torch.ones(128), bias=torch.zeros(128), dropout_p=0.0, eps=1e-5,
    )
    mutate(arguments)
    assert normalization._input_reason(**arguments) == reason


def test_input_reason_ladder_with_fake_device_tensors():
    """The ladder past the device checks, driven with duck-typed tensors."""

    class Fake:
        def __init__(self, shape, dtype=torch.float32, contiguous=True, device="cuda:0"):
            self.shape = torch.Size(shape)
            self.dtype = dtype
            self.is_cuda = True
            self.device = device
            self.ndim = len(shape)
            self._contiguous = contiguous

        def is_contiguous(self):
            return self._contiguous

        def numel(self):
            total = 1
            for extent in self.shape:
                total *= extent
            return total

    def reason(x, branch=None, weight=None, bias=None, p=0.0, eps=1e-5):
        hidden = x.shape[-1] if x.ndim else 0
        branch = branch if branch is not None else Fake(x.shape)
        weight = weight if weight is not None else Fake((hidden,))
        bias = bias if bias is not None else Fake((hidden,))
        return normalization._input_reason(x, branch, weight, bias, p, eps)

    ok = Fake((4, 256))
    assert reason(ok) is None
    assert "same device" in reason(ok, branch=Fake((4, 256), device="cuda:1"))
    assert "same shape" in reason(Fake((256,)))
    assert "same shape" in reason(ok, branch=Fake((2, 256)))
    assert "between 128 and 1024" in reason(Fake((4, 64)))
    assert "between 128 and 1024" in reason(Fake((4, 2048)))
    assert "divisible by 8" in reason(Fake((4, 132)))
    assert "final tensor dimension" in reason(ok, weight=Fake((128,)))
    assert "float32 x" in reason(Fake((4, 256), dtype=torch.float16))
    assert "float16 or float32" in reason(ok, branch=Fake((4, 256), dtype=torch.float64))
    assert reason(ok, branch=Fake((4, 256), dtype=torch.bfloat16)) is None
    assert "weight and bias must use float32" in reason(ok, bias=Fake((256,), dtype=torch.float16))
    assert "contiguous" in reason(ok, branch=Fake((4, 256), contiguous=False))
    assert "dropout_p must be in [0, 1)" in reason(ok, p=1.0)
    assert "eps must be positive" in reason(ok, eps=0.0)
    assert "empty tensors" in reason(Fake((0, 256)))
    # a supported-range width that has no native kernel is eligible for the
    # generic routes but not for the native one
    assert reason(Fake((4, 640))) is None


def test_launch_policy_matches_tuned_profiles():
    from gfx1010_kernels._normalization_native import (
        _block_rows,
        _parameter_groups,
        _parameter_threads,
        _THREADS,
    )

    assert _parameter_threads(384, 1024) == 64
    assert _parameter_threads(512, 256) == 256
    assert _parameter_threads(256, 512) == 256
    assert _parameter_threads(1024, 4096) == 256
    assert _parameter_groups(384, 128) == 8
    assert _parameter_groups(384, 1024) == 64
    assert _parameter_groups(128, 4096) == 128
    assert _parameter_groups(1024, 4096) == 24
    assert _parameter_groups(768, 5) == 5
    assert _THREADS[768] == 128 and _THREADS[1024] == 192
    assert _block_rows(768, 8192) == 64
    assert _block_rows(512, 1024) == 16 and _block_rows(384, 1024) == 32
    assert _block_rows(128, 512) == 16


def test_raw_extension_rejects_cpu_tensors(built_libraries):
    from gfx1010_kernels import _C

    x = torch.zeros(2, 128)
    with pytest.raises(RuntimeError, match="x must be a HIP tensor"):
        _C.residual_layer_norm_forward(x, x, torch.ones(128), torch.zeros(128), 0.0, 1e-5, True, 128)
    stats = torch.zeros(2)
    with pytest.raises(RuntimeError, match="updated must be a HIP tensor"):
        _C.residual_layer_norm_backward(
            x, x, x, torch.ones(128), stats, stats, torch.empty(0, dtype=torch.int32),
            0.0, True, True, 128, 16, 64, 1, True,
        )


def test_extension_keeps_the_reference_entry_points(built_libraries):
    from gfx1010_kernels import _C

    for name in (
        "residual_layer_norm",
        "residual_layer_norm_forward",
        "residual_layer_norm_backward",
    ):
        assert callable(getattr(_C, name))


@pytest.mark.parametrize("normalized_dtype", [torch.float16, torch.bfloat16])
def test_torch_route_casts_normalized_once_and_stays_differentiable(normalized_dtype):
    torch.manual_seed(7)
    tensors = [torch.randn(5, 256), torch.randn(5, 256), torch.randn(256), torch.randn(256)]
    plain = residual_layer_norm(*tensors, implementation="torch")
    leaves = [t.clone().requires_grad_(True) for t in tensors]
    updated, normalized = residual_layer_norm(
        *leaves, implementation="torch", normalized_dtype=normalized_dtype
    )
    assert updated.dtype == torch.float32 and normalized.dtype == normalized_dtype
    assert torch.equal(updated, plain[0])
    assert torch.equal(normalized, plain[1].to(normalized_dtype))
    grads = torch.autograd.grad(
        (updated, normalized), leaves,
        (torch.ones_like(updated), torch.ones_like(normalized)),
    )
    assert [g.dtype for g in grads] == [torch.float32] * 4
    # float32 is the default spelled out
    same = residual_layer_norm(*tensors, implementation="torch", normalized_dtype=torch.float32)
    assert same[1].dtype == torch.float32 and torch.equal(same[1], plain[1])


def test_auto_fallback_honours_normalized_dtype():
    tensors = [torch.randn(2, 128), torch.randn(2, 128), torch.ones(128), torch.zeros(128)]
    with pytest.warns(RuntimeWarning, match="was not used"):
        _, normalized = residual_layer_norm(*tensors, normalized_dtype=torch.bfloat16)
    assert normalized.dtype == torch.bfloat16


@pytest.mark.parametrize("bad", [torch.float64, torch.int32, "bfloat16"])
def test_unsupported_normalized_dtype_is_a_value_error(bad):
    tensors = [torch.randn(2, 128), torch.randn(2, 128), torch.ones(128), torch.zeros(128)]
    for implementation in ("torch", "auto", "gfx1010"):
        with pytest.raises(ValueError, match="normalized_dtype"):
            residual_layer_norm(*tensors, implementation=implementation, normalized_dtype=bad)


def test_extension_signatures_keep_the_reference_arity_with_an_optional_tail(built_libraries):
    """The reference's positional calls still bind; `normalized_dtype` is a
    trailing optional argument of the three forward-side entries."""
    from gfx1010_kernels import _C

    doc = _C.residual_layer_norm.__doc__
    assert "parameter_groups: typing.SupportsInt" in doc or "parameter_groups: int" in doc
    assert "normalized_dtype" in doc and "= 0" in doc
    assert "normalized_dtype" in _C.residual_layer_norm_forward.__doc__
    assert "normalized_dtype" in _C.residual_layer_norm_forward_seeded.__doc__
    assert "normalized_dtype" not in _C.residual_layer_norm_backward.__doc__
    x = torch.randn(2, 128)
    with pytest.raises(RuntimeError, match="x must be a HIP tensor"):
        _C.residual_layer_norm_forward(x, x, x[0], x[0], 0.0, 1e-5, True, 128, 2)


def test_host_pipeline_output_tensors_are_checked_before_the_native_call():
    """Shape, type, layout and residency of caller-supplied result tensors: the
    native call writes rows * hidden elements into them unchecked."""
    from gfx1010_kernels.host_pipeline import check_output_tensors

    shape, hidden = (6, 128), 128

    def outputs(**replace):
        tensors = {
            "updated": torch.empty(shape), "normalized": torch.empty(shape, dtype=torch.bfloat16),
            "grad_x": torch.empty(shape), "grad_branch": torch.empty(shape, dtype=torch.float16),
            "grad_parameters": torch.empty(2, hidden),
        }
        tensors.update(replace)
        return tuple(tensors.values())

    check_output_tensors(outputs(), shape, hidden, torch.bfloat16, torch.float16)
    cases = {
        "updated must have shape": outputs(updated=torch.empty(5, 128)),
        "grad_x must use": outputs(grad_x=torch.empty(shape, dtype=torch.float64)),
        "normalized must use": outputs(normalized=torch.empty(shape)),
        "grad_branch must be contiguous": outputs(
            grad_branch=torch.empty(128, 6, dtype=torch.float16).t()),
        "grad_parameters must have shape": outputs(grad_parameters=torch.empty(2 * hidden)),
        "updated must be a host tensor": outputs(updated=None),
    }
    for message, out in cases.items():
        with pytest.raises(RuntimeError, match=message):
            check_output_tensors(out, shape, hidden, torch.bfloat16, torch.float16)
    with pytest.raises(RuntimeError, match="out must be"):
        check_output_tensors(outputs()[:4], shape, hidden, torch.bfloat16, torch.float16)
