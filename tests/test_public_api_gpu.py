"""The public Python API and the raw ``_C`` entry points on a B200.

These restate, against the sm_100a kernels, the GPU-gated checks of the
reference project's own suite (T-vaccari/gfx1010-kernels):
tests/test_residual_layer_norm.py:102-271,
tests/test_residual_layer_norm_edge_cases.py (gpu-gfx1010 parametrisation),
tests/test_residual_layer_norm_native_matrix.py and
tests/test_residual_layer_norm_vectorized.py -- same scenarios and seeds, with
tolerances at least as tight as the reference's."""

import pytest
import torch
from torch.nn import functional as F

import gfx1010_kernels.normalization as normalization
from gfx1010_kernels import (
    can_use_residual_layer_norm,
    residual_layer_norm,
    residual_layer_norm_status,
)

pytestmark = pytest.mark.gpu

HIDDEN_SIZES = (128, 256, 384, 512, 768, 1024)
DEVICE = "cuda"


def decomposition(x, branch, weight, bias, dropout_p=0.0, eps=1e-5, training=True):
    if training:
        branch = F.dropout(branch, dropout_p, True)
    updated = x + branch
    return updated, F.layer_norm(updated, (updated.shape[-1],), weight, bias, eps)


def leaves(tensors):
    return tuple(t.detach().clone().requires_grad_(True) for t in tensors)


def random_inputs(rows, hidden, branch_dtype=torch.float16, leading=()):
    return (
        torch.randn(*leading, rows, hidden, device=DEVICE),
        torch.randn(*leading, rows, hidden, device=DEVICE, dtype=branch_dtype),
        torch.randn(hidden, device=DEVICE),
        torch.randn(hidden, device=DEVICE),
    )


def test_backend_is_available_on_this_device():
    status = residual_layer_norm_status()
    assert status.available, status.reason
    assert status.architecture == "sm_100"
    assert residual_layer_norm_status("cuda:0").available
    assert not residual_layer_norm_status("cpu").available
    inputs = random_inputs(4, 256)
    assert can_use_residual_layer_norm(*inputs)
    assert not can_use_residual_layer_norm(inputs[0][:, :160].contiguous(),
                                           inputs[1][:, :160].contiguous(),
                                           inputs[2][:160].contiguous(),
                                           inputs[3][:160].contiguous())


def test_auto_route_uses_the_native_kernels_without_warning(recwarn):
    torch.manual_seed(5)
    inputs = random_inputs(9, 512)
    actual = residual_layer_norm(*inputs)
    expected = decomposition(*inputs)
    assert not [w for w in recwarn.list if issubclass(w.category, RuntimeWarning)]
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)


def test_auto_route_falls_back_with_warning_for_unsupported_width():
    inputs = random_inputs(4, 640)
    with pytest.warns(RuntimeWarning, match="was not used: native hidden size"):
        actual = residual_layer_norm(*inputs)
    expected = decomposition(*inputs)
    torch.testing.assert_close(actual[1], expected[1])


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
def test_forward_matches_pytorch(hidden):
    torch.manual_seed(17)
    inputs = random_inputs(37, hidden, leading=(1,))
    actual = residual_layer_norm(*inputs, implementation="gfx1010")
    expected = decomposition(*inputs)
    assert actual[0].dtype == actual[1].dtype == torch.float32
    assert actual[0].shape == inputs[0].shape
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
def test_backward_matches_pytorch(hidden):
    torch.manual_seed(23)
    data = random_inputs(41, hidden, leading=(1,))
    actual_inputs = leaves(data)
    expected_inputs = leaves(data)
    actual = residual_layer_norm(*actual_inputs, implementation="gfx1010")
    grad_updated = torch.randn_like(actual[0])
    grad_normalized = torch.randn_like(actual[1])
    torch.autograd.backward(actual, (grad_updated, grad_normalized))
    torch.autograd.backward(decomposition(*expected_inputs), (grad_updated, grad_normalized))
    for mine, theirs in zip(actual_inputs, expected_inputs):
        assert mine.grad.dtype == theirs.grad.dtype
        torch.testing.assert_close(mine.grad, theirs.grad, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
@pytest.mark.parametrize("dropout_p", [0.15, 0.2])
def test_dropout_forward_and_backward_are_consistent(hidden, dropout_p):
    torch.manual_seed(29)
    x = torch.randn(1, 43, hidden, device=DEVICE)
    branch = torch.ones(1, 43, hidden, device=DEVICE, dtype=torch.float16)
    weight = torch.randn(hidden, device=DEVICE)
    bias = torch.randn(hidden, device=DEVICE)
    actual_inputs = leaves((x, branch, weight, bias))
    expected_inputs = leaves((x, branch, weight, bias))
    actual = residual_layer_norm(*actual_inputs, dropout_p=dropout_p, implementation="gfx1010")
    mask_scale = ((actual[0] - actual_inputs[0]) / actual_inputs[1].float()).detach()
    scales = torch.tensor([0.0, 1.0 / (1.0 - dropout_p)], device=DEVICE)
    assert (mask_scale[..., None] - scales).abs().amin(dim=-1).max().item() < 2e-3
    kept = (mask_scale > 0).float().mean().item()
    sigma = (dropout_p * (1 - dropout_p) / mask_scale.numel()) ** 0.5
    assert abs(kept - (1 - dropout_p)) < 4 * sigma

    torch.testing.assert_close(
        actual[1], F.layer_norm(actual[0], (hidden,), weight, bias), rtol=1e-5, atol=1e-6
    )
    grad_updated = torch.randn_like(actual[0])
    grad_normalized = torch.randn_like(actual[1])
    torch.autograd.backward(actual, (grad_updated, grad_normalized))
    expected_updated = expected_inputs[0] + expected_inputs[1] * mask_scale
    expected_normalized = F.layer_norm(
        expected_updated, (hidden,), expected_inputs[2], expected_inputs[3]
    )
    torch.autograd.backward(
        (expected_updated, expected_normalized), (grad_updated, grad_normalized)
    )
    for mine, theirs in zip(actual_inputs, expected_inputs):
        torch.testing.assert_close(mine.grad, theirs.grad, rtol=2e-3, atol=2e-3)


def test_eval_bypasses_dropout_without_consuming_rng():
    torch.manual_seed(101)
    inputs = random_inputs(7, 384)
    cpu_state = torch.random.get_rng_state()
    gpu_state = torch.cuda.get_rng_state(DEVICE)
    actual = residual_layer_norm(
        *inputs, dropout_p=0.8, training=False, implementation="gfx1010"
    )
    expected = decomposition(*inputs, dropout_p=0.8, training=False)
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)
    assert torch.equal(torch.random.get_rng_state(), cpu_state)
    assert torch.equal(torch.cuda.get_rng_state(DEVICE), gpu_state)
    # p == 0 in training mode consumes nothing either
    residual_layer_norm(*inputs, dropout_p=0.0, training=True, implementation="gfx1010")
    assert torch.equal(torch.cuda.get_rng_state(DEVICE), gpu_state)
    # active dropout does advance the generator
    residual_layer_norm(*inputs, dropout_p=0.5, training=True, implementation="gfx1010")
    assert not torch.equal(torch.cuda.get_rng_state(DEVICE), gpu_state)


@pytest.mark.parametrize("used_output", [0, 1], ids=["updated-only", "normalized-only"])
def test_each_output_can_drive_backward_alone(used_output):
    torch.manual_seed(103)
    data = random_inputs(7, 384)
    actual_inputs = leaves(data)
    expected_inputs = leaves(data)
    actual = residual_layer_norm(*actual_inputs, implementation="gfx1010")
    expected = decomposition(*expected_inputs)
    upstream = torch.randn_like(actual[used_output])
    actual_gradients = torch.autograd.grad(
        actual[used_output], actual_inputs, upstream, allow_unused=True
    )
    expected_gradients = torch.autograd.grad(
        expected[used_output], expected_inputs, upstream, allow_unused=True
    )
    for mine, theirs, like in zip(actual_gradients, expected_gradients, actual_inputs):
        if theirs is None:
            if mine is not None:
                torch.testing.assert_close(mine, torch.zeros_like(like))
            continue
        assert mine is not None
        torch.testing.assert_close(mine, theirs, rtol=3e-3, atol=3e-3)


@pytest.mark.parametrize("eps", [1e-5, 1e-3])
def test_nearly_constant_rows_respect_eps(eps):
    hidden = 384
    columns = torch.linspace(-1.0, 1.0, hidden, device=DEVICE)
    centers = torch.tensor([-3.0, 0.25, 4.0], device=DEVICE)[:, None]
    x = centers + columns[None, :] * 2e-4
    branch = (-columns[None, :] * 5e-5).expand_as(x).contiguous().half()
    weight = torch.linspace(0.75, 1.25, hidden, device=DEVICE)
    bias = torch.linspace(-0.1, 0.1, hidden, device=DEVICE)
    actual_inputs = leaves((x, branch, weight, bias))
    expected_inputs = leaves((x, branch, weight, bias))
    actual = residual_layer_norm(*actual_inputs, eps=eps, implementation="gfx1010")
    expected = decomposition(*expected_inputs, eps=eps)
    upstream = torch.sin(columns)[None, :].expand_as(actual[1]).contiguous()
    actual_gradients = torch.autograd.grad(actual[1], actual_inputs, upstream)
    expected_gradients = torch.autograd.grad(expected[1], expected_inputs, upstream)
    assert all(torch.isfinite(v).all() for v in (*actual, *actual_gradients))
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=1e-6)
    torch.testing.assert_close(actual[1], expected[1], rtol=8e-3, atol=8e-3)
    for mine, theirs in zip(actual_gradients, expected_gradients):
        torch.testing.assert_close(mine, theirs, rtol=1e-2, atol=1e-2)


def test_dropout_replays_after_rng_state_restore():
    torch.manual_seed(109)
    data = random_inputs(11, 384)
    first_inputs = leaves(data)
    second_inputs = leaves(data)
    grad_updated = torch.linspace(
        -0.5, 0.5, data[0].numel(), device=DEVICE
    ).reshape_as(data[0])
    grad_normalized = torch.cos(grad_updated)
    state = torch.cuda.get_rng_state(DEVICE)
    was_enabled = torch.are_deterministic_algorithms_enabled()
    warn_only = torch.is_deterministic_algorithms_warn_only_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        first = residual_layer_norm(
            *first_inputs, dropout_p=0.25, training=True, implementation="gfx1010"
        )
        torch.cuda.set_rng_state(state, DEVICE)
        second = residual_layer_norm(
            *second_inputs, dropout_p=0.25, training=True, implementation="gfx1010"
        )
        first_gradients = torch.autograd.grad(first, first_inputs, (grad_updated, grad_normalized))
        second_gradients = torch.autograd.grad(
            second, second_inputs, (grad_updated, grad_normalized)
        )
        for a, b in zip((*first, *first_gradients), (*second, *second_gradients)):
            assert torch.equal(a, b)
    finally:
        torch.use_deterministic_algorithms(was_enabled, warn_only=warn_only)


def test_native_route_does_not_consult_triton(monkeypatch):
    def fail(*args, **kwargs):
        raise AssertionError("native dispatch queried Triton")

    monkeypatch.setattr(normalization, "_triton_is_usable", fail)
    residual_layer_norm(*random_inputs(7, 384), implementation="gfx1010")


def test_forced_hot_path_skips_python_validation_and_device_guard(monkeypatch):
    inputs = random_inputs(7, 384)

    def fail(*args, **kwargs):
        raise AssertionError("forced native hot path used Python dispatch work")

    monkeypatch.setattr(normalization, "_input_reason", fail)
    monkeypatch.setattr(torch.cuda, "device", fail)
    residual_layer_norm(*inputs, implementation="gfx1010")


def test_consecutive_dropout_calls_do_not_overlap_philox_subsequences():
    hidden, rows = 768, 3
    x = torch.zeros(rows, hidden, device=DEVICE)
    branch = torch.ones(rows, hidden, device=DEVICE, dtype=torch.float16)
    weight = torch.ones(hidden, device=DEVICE)
    bias = torch.zeros(hidden, device=DEVICE)
    torch.manual_seed(127)
    first = residual_layer_norm(x, branch, weight, bias, dropout_p=0.5, implementation="gfx1010")[0]
    second = residual_layer_norm(x, branch, weight, bias, dropout_p=0.5, implementation="gfx1010")[0]
    assert not torch.equal(first, second)
    assert not torch.equal(first[:, 512:768], second[:, :256])


def test_generator_offset_advances_like_the_reference():
    """increment = 4 * ceil(ceil(H / threads) / 4) per dropout call
    (csrc/residual_layer_norm_kernel.hip:1767-1774): 4 for H <= 512, 8 for
    H = 768 (threads 128) and H = 1024 (threads 192)."""
    generator = torch.cuda.default_generators[0]
    for hidden, expected in ((128, 4), (512, 4), (768, 8), (1024, 8)):
        inputs = random_inputs(3, hidden)
        before = generator.get_offset()
        residual_layer_norm(*inputs, dropout_p=0.1, implementation="gfx1010")
        assert generator.get_offset() - before == expected


def test_raw_extension_rejects_invalid_inputs():
    from gfx1010_kernels import _C

    cpu = torch.zeros(2, 128)
    with pytest.raises(RuntimeError, match="x must be a HIP tensor"):
        _C.residual_layer_norm_forward(cpu, cpu, torch.ones(128), torch.zeros(128), 0.0, 1e-5, True, 128)
    x, branch, weight, bias = random_inputs(2, 128)
    with pytest.raises(RuntimeError, match="threads must be 128, 192 or 256"):
        _C.residual_layer_norm_forward(x, branch, weight, bias, 0.0, 1e-5, True, 64)
    with pytest.raises(RuntimeError, match=r"dropout_p must be in \[0, 1\)"):
        _C.residual_layer_norm_forward(x, branch, weight, bias, 1.0, 1e-5, True, 128)
    with pytest.raises(RuntimeError, match="eps must be positive"):
        _C.residual_layer_norm_forward(x, branch, weight, bias, 0.0, 0.0, True, 128)
    with pytest.raises(RuntimeError, match="branch must match x"):
        _C.residual_layer_norm_forward(x, branch[:1], weight, bias, 0.0, 1e-5, True, 128)
    with pytest.raises(RuntimeError, match="all tensors must be contiguous"):
        strided = torch.randn(2, 256, device=DEVICE)[:, ::2]
        _C.residual_layer_norm_forward(strided, branch, weight, bias, 0.0, 1e-5, True, 128)
    with pytest.raises(RuntimeError, match="unsupported native hidden size"):
        wide = torch.randn(2, 160, device=DEVICE)
        _C.residual_layer_norm_forward(
            wide, wide.half(), torch.ones(160, device=DEVICE), torch.zeros(160, device=DEVICE),
            0.0, 1e-5, True, 128,
        )
    with pytest.raises(RuntimeError, match="x must use float32"):
        _C.residual_layer_norm_forward(x.half(), branch, weight, bias, 0.0, 1e-5, True, 128)


def test_float32_branch_forward_and_backward():
    torch.manual_seed(211)
    data = random_inputs(37, 384, branch_dtype=torch.float32)
    _assert_forward_backward_close(data)


def _assert_forward_backward_close(data, upstream_scale=1.0):
    actual_inputs = leaves(data)
    expected_inputs = leaves(data)
    actual = residual_layer_norm(*actual_inputs, implementation="gfx1010")
    expected = decomposition(*expected_inputs)
    grad_updated = torch.randn_like(actual[0]) * upstream_scale
    grad_normalized = torch.randn_like(actual[1]) * upstream_scale
    actual_gradients = torch.autograd.grad(actual, actual_inputs, (grad_updated, grad_normalized))
    expected_gradients = torch.autograd.grad(
        expected, expected_inputs, (grad_updated, grad_normalized)
    )
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)
    for mine, theirs in zip(actual_gradients, expected_gradients):
        torch.testing.assert_close(mine, theirs, rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize("rows", [1, 15, 16, 17, 511, 512, 513, 2047, 2048, 2049])
def test_row_count_boundaries(rows):
    torch.manual_seed(227 + rows)
    _assert_forward_backward_close(random_inputs(rows, 128), upstream_scale=rows ** -0.5)


def test_updated_only_backward_leaves_layer_norm_parameters_unused():
    torch.manual_seed(229)
    actual_inputs = leaves(random_inputs(13, 384))
    expected_inputs = leaves(tuple(v.detach() for v in actual_inputs))
    actual_updated = residual_layer_norm(*actual_inputs, implementation="gfx1010")[0]
    expected_updated = decomposition(*expected_inputs)[0]
    upstream = torch.randn_like(actual_updated)
    actual_gradients = torch.autograd.grad(
        actual_updated, actual_inputs, upstream, allow_unused=True, materialize_grads=False
    )
    expected_gradients = torch.autograd.grad(
        expected_updated, expected_inputs, upstream, allow_unused=True, materialize_grads=False
    )
    assert torch.equal(actual_gradients[0], expected_gradients[0])
    assert torch.equal(actual_gradients[1], expected_gradients[1])
    assert actual_gradients[2:] == expected_gradients[2:] == (None, None)


def test_raw_backward_rejects_cpu_and_empty_inputs():
    from gfx1010_kernels import _C

    cpu = torch.zeros(2, 128)
    stats = torch.zeros(2)
    with pytest.raises(RuntimeError, match="updated must be a HIP tensor"):
        _C.residual_layer_norm_backward(
            cpu, cpu, cpu, torch.ones(128), stats, stats, torch.empty(0, dtype=torch.int32),
            0.0, True, True, 128, 16, 64, 1, True,
        )
    empty = torch.empty(0, 128, device=DEVICE)
    no_stats = torch.empty(0, device=DEVICE)
    with pytest.raises(RuntimeError, match="empty tensors are unsupported"):
        _C.residual_layer_norm_backward(
            empty, empty, empty, torch.ones(128, device=DEVICE), no_stats, no_stats,
            torch.empty(0, device=DEVICE, dtype=torch.int32),
            0.0, True, True, 128, 16, 64, 1, True,
        )


def test_raw_parameter_gradient_reduction_modes():
    from gfx1010_kernels import _C

    torch.manual_seed(233)
    rows, hidden = 257, 384
    x, branch, weight, bias = random_inputs(rows, hidden)
    outputs = _C.residual_layer_norm_forward(x, branch, weight, bias, 0.0, 1e-5, True, 128)
    assert outputs[4].numel() == 0 and outputs[4].dtype == torch.int32
    grad_updated = torch.randn_like(outputs[0])
    grad_normalized = torch.randn_like(outputs[1])

    def backward(parameter_groups):
        return _C.residual_layer_norm_backward(
            grad_updated, grad_normalized, outputs[0], weight, outputs[2], outputs[3],
            outputs[4], 0.0, True, True, 128, 32, 64, parameter_groups, True,
        )

    with pytest.raises(RuntimeError, match=r"parameter_groups must be in \[1, row_count\]"):
        backward(0)
    with pytest.raises(RuntimeError, match=r"parameter_groups must be in \[1, row_count\]"):
        backward(rows + 1)
    was_enabled = torch.are_deterministic_algorithms_enabled()
    warn_only = torch.is_deterministic_algorithms_warn_only_enabled()
    try:
        torch.use_deterministic_algorithms(False)
        atomic_one = backward(1)
        atomic_twelve = backward(12)
        torch.use_deterministic_algorithms(True)
        deterministic_one = backward(1)
        deterministic_twelve = backward(12)
    finally:
        torch.use_deterministic_algorithms(was_enabled, warn_only=warn_only)
    xhat = (outputs[0].double() - outputs[2].double()[:, None]) * outputs[3].double()[:, None]
    expected_weight = (grad_normalized.double() * xhat).sum(dim=0).float()
    expected_bias = grad_normalized.double().sum(dim=0).float()
    for gradients in (atomic_one, atomic_twelve, deterministic_one, deterministic_twelve):
        torch.testing.assert_close(gradients[2], expected_weight, rtol=1e-4, atol=2e-4)
        torch.testing.assert_close(gradients[3], expected_bias, rtol=1e-4, atol=2e-4)
        # one [2, H] allocation, as in the reference
        assert gradients[2].data_ptr() + hidden * 4 == gradients[3].data_ptr()
    assert torch.equal(deterministic_one[2], deterministic_twelve[2])
    assert torch.equal(deterministic_one[3], deterministic_twelve[3])


@pytest.mark.parametrize("hidden", [256, 384, 512, 768, 1024])
@pytest.mark.parametrize("dropout_p", [0.0, 0.15])
@pytest.mark.parametrize("branch_dtype", [torch.float16, torch.float32], ids=["half", "float"])
def test_backward_with_unit_branch(hidden, dropout_p, branch_dtype):
    torch.manual_seed(401 + hidden)
    rows = 19
    inputs = (
        torch.randn(rows, hidden, device=DEVICE),
        torch.ones(rows, hidden, device=DEVICE, dtype=branch_dtype),
        torch.randn(hidden, device=DEVICE),
        torch.randn(hidden, device=DEVICE),
    )
    actual_inputs = leaves(inputs)
    expected_inputs = leaves(inputs)
    actual = residual_layer_norm(
        *actual_inputs, dropout_p=dropout_p, training=True, implementation="gfx1010"
    )
    if dropout_p:
        mask_scale = actual[0].detach() - actual_inputs[0].detach()
    else:
        mask_scale = torch.ones_like(actual_inputs[0])
    expected_updated = expected_inputs[0] + expected_inputs[1].float() * mask_scale
    expected_normalized = F.layer_norm(
        expected_updated, (hidden,), expected_inputs[2], expected_inputs[3]
    )
    gradients = (torch.randn_like(actual[0]), torch.randn_like(actual[1]))
    actual_gradients = torch.autograd.grad(actual, actual_inputs, gradients)
    expected_gradients = torch.autograd.grad(
        (expected_updated, expected_normalized), expected_inputs, gradients
    )
    for mine, theirs in zip(actual_gradients, expected_gradients):
        torch.testing.assert_close(mine, theirs, rtol=5e-3, atol=5e-3)


def test_misaligned_contiguous_gradient_agrees_with_aligned():
    from gfx1010_kernels import _C

    torch.manual_seed(409)
    rows, hidden = 23, 384
    x, branch, weight, bias = random_inputs(rows, hidden)
    outputs = _C.residual_layer_norm_forward(x, branch, weight, bias, 0.15, 1e-5, True, 128)
    storage = torch.randn(rows * hidden + 1, device=DEVICE)
    misaligned = storage[1:].view(rows, hidden)
    aligned = misaligned.clone()
    grad_normalized = torch.randn_like(x)
    assert misaligned.is_contiguous() and misaligned.data_ptr() % 16 != 0

    def backward(grad_updated):
        return _C.residual_layer_norm_backward(
            grad_updated, grad_normalized, outputs[0], weight, outputs[2], outputs[3],
            outputs[4], 0.15, True, True, 128, 16, 64, 1, False,
        )

    vectorized = backward(aligned)
    scalar = backward(misaligned)
    assert torch.equal(vectorized[0], scalar[0])
    assert torch.equal(vectorized[1], scalar[1])
    assert vectorized[2] is None and vectorized[3] is None


def test_deterministic_raw_backward_replay_is_bitwise_exact():
    from gfx1010_kernels import _C

    torch.manual_seed(419)
    rows, hidden = 31, 768
    x, branch, weight, bias = random_inputs(rows, hidden)
    outputs = _C.residual_layer_norm_forward(x, branch, weight, bias, 0.15, 1e-5, True, 128)
    grad_updated = torch.randn_like(x)
    grad_normalized = torch.randn_like(x)

    def backward():
        return _C.residual_layer_norm_backward(
            grad_updated, grad_normalized, outputs[0], weight, outputs[2], outputs[3],
            outputs[4], 0.15, True, True, 128, 16, 64, 1, True,
        )

    was_enabled = torch.are_deterministic_algorithms_enabled()
    warn_only = torch.is_deterministic_algorithms_warn_only_enabled()
    try:
        torch.use_deterministic_algorithms(True)
        first = backward()
        second = backward()
    finally:
        torch.use_deterministic_algorithms(was_enabled, warn_only=warn_only)
    for a, b in zip(first, second):
        assert torch.equal(a, b)


def test_dropout_refuses_stream_capture():
    inputs = random_inputs(4, 128)
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        with pytest.raises(RuntimeError, match="does not support HIP graph capture"):
            with torch.cuda.graph(graph, stream=stream):
                residual_layer_norm(*inputs, dropout_p=0.1, implementation="gfx1010")
    torch.cuda.synchronize()


def test_work_is_enqueued_on_the_current_stream():
    inputs = random_inputs(64, 768)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        actual = residual_layer_norm(*inputs, implementation="gfx1010")
    side.synchronize()
    expected = decomposition(*inputs)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)


def test_bfloat16_branch_forward_and_backward():
    """bfloat16 is accepted in addition to the reference's float16 / float32."""
    torch.manual_seed(251)
    data = random_inputs(37, 768, branch_dtype=torch.bfloat16)
    assert can_use_residual_layer_norm(*data)
    actual_inputs = leaves(data)
    expected_inputs = leaves(data)
    actual = residual_layer_norm(*actual_inputs, implementation="gfx1010")
    expected = decomposition(*expected_inputs)
    grad_updated = torch.randn_like(actual[0])
    grad_normalized = torch.randn_like(actual[1])
    actual_gradients = torch.autograd.grad(actual, actual_inputs, (grad_updated, grad_normalized))
    expected_gradients = torch.autograd.grad(
        expected, expected_inputs, (grad_updated, grad_normalized)
    )
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    torch.testing.assert_close(actual[1], expected[1], rtol=1e-5, atol=1e-6)
    assert actual_gradients[1].dtype == torch.bfloat16
    torch.testing.assert_close(actual_gradients[0], expected_gradients[0], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(
        actual_gradients[1].float(), expected_gradients[1].float(), rtol=1.6e-2, atol=1e-5
    )
    for mine, theirs in zip(actual_gradients[2:], expected_gradients[2:]):
        torch.testing.assert_close(mine, theirs, rtol=1e-4, atol=2e-4)
    # dropout on a unit branch: updated - x is 0 or bfloat16(1 / (1 - p))
    ones = torch.ones(64, 768, device=DEVICE, dtype=torch.bfloat16)
    zeros = torch.zeros(64, 768, device=DEVICE)
    updated = residual_layer_norm(zeros, ones, data[2], data[3], dropout_p=0.3,
                                  implementation="gfx1010")[0]
    kept_value = torch.tensor(1.0 / (1.0 - 0.3), dtype=torch.float32).to(torch.bfloat16).float()
    assert set(updated.unique().tolist()) <= {0.0, kept_value.item()}


@pytest.mark.parametrize("normalized_dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("hidden", [128, 768, 1024])
def test_narrow_normalized_output_through_autograd(hidden, normalized_dtype):
    """`normalized_dtype=`: the native route returns `normalized` in a 16-bit
    type and takes its gradient in that type; compared with the decomposition
    followed by one cast (torch autograd widens the gradient through the cast)."""
    torch.manual_seed(263 + hidden)
    data = random_inputs(41, hidden, leading=(2,))
    actual_inputs = leaves(data)
    expected_inputs = leaves(data)
    actual = residual_layer_norm(
        *actual_inputs, implementation="gfx1010", normalized_dtype=normalized_dtype
    )
    expected = decomposition(*expected_inputs)
    expected = (expected[0], expected[1].to(normalized_dtype))
    assert actual[0].dtype == torch.float32 and actual[1].dtype == normalized_dtype
    torch.testing.assert_close(actual[0], expected[0], rtol=0, atol=0)
    # one rounding of float32 values that agree to 1e-5: neighbours at worst
    tolerance = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[normalized_dtype]
    torch.testing.assert_close(actual[1].float(), expected[1].float(), rtol=tolerance, atol=1e-4)
    assert (actual[1] == expected[1]).float().mean().item() > 0.99
    grad_updated = torch.randn_like(actual[0])
    grad_normalized = torch.randn_like(actual[1])
    assert grad_normalized.dtype == normalized_dtype
    actual_gradients = torch.autograd.grad(actual, actual_inputs, (grad_updated, grad_normalized))
    expected_gradients = torch.autograd.grad(
        expected, expected_inputs, (grad_updated, grad_normalized)
    )
    torch.testing.assert_close(actual_gradients[0], expected_gradients[0], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(
        actual_gradients[1].float(), expected_gradients[1].float(), rtol=2e-3, atol=1e-5
    )
    for mine, theirs in zip(actual_gradients[2:], expected_gradients[2:]):
        torch.testing.assert_close(mine, theirs, rtol=1e-4, atol=2e-4)


def test_narrow_normalized_with_dropout_only_normalized_used_and_auto_route(recwarn):
    torch.manual_seed(269)
    x, branch, weight, bias = random_inputs(33, 512, branch_dtype=torch.bfloat16)
    inputs = leaves((x, branch, weight, bias))
    state = torch.cuda.get_rng_state()
    updated, normalized = residual_layer_norm(
        *inputs, dropout_p=0.2, normalized_dtype=torch.bfloat16
    )
    assert not [w for w in recwarn.list if issubclass(w.category, RuntimeWarning)]
    torch.cuda.set_rng_state(state)
    reference = residual_layer_norm(x, branch, weight, bias, dropout_p=0.2)
    # same mask, same float32 arithmetic: the 16-bit output is the cast of the float32 one
    assert torch.equal(updated, reference[0])
    assert torch.equal(normalized, reference[1].to(torch.bfloat16))
    gradients = torch.autograd.grad(normalized.float().square().sum(), inputs)
    assert gradients[1].dtype == torch.bfloat16
    assert all(torch.isfinite(g.float()).all() for g in gradients)


def test_narrow_normalized_in_the_module():
    from gfx1010_kernels.modules import ResidualLayerNorm

    module = ResidualLayerNorm(
        768, dropout_p=0.1, implementation="gfx1010", normalized_dtype=torch.bfloat16
    ).cuda()
    x = torch.randn(4, 9, 768, device=DEVICE, requires_grad=True)
    branch = torch.randn(4, 9, 768, device=DEVICE, dtype=torch.bfloat16, requires_grad=True)
    updated, normalized = module(x, branch)
    assert normalized.dtype == torch.bfloat16
    projection = torch.randn(768, 64, device=DEVICE, dtype=torch.bfloat16)
    ((normalized @ projection).float().square().mean() + updated.mean()).backward()
    assert module.weight.grad is not None and module.weight.grad.dtype == torch.float32
    assert branch.grad.dtype == torch.bfloat16 and x.grad.dtype == torch.float32
