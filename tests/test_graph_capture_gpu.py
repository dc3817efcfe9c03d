"""Opt-in CUDA-graph capture of the native dropout path.

Default behaviour (refusal, as in the reference) is covered in
``test_public_api_gpu.py``; here the switch is on: the captured forward reads
the generator's seed/offset from device memory at replay time."""

import pytest
import torch

from gfx1010_kernels import allow_graph_capture, residual_layer_norm

pytestmark = pytest.mark.gpu


@pytest.fixture
def capture_allowed():
    previous = allow_graph_capture(True)
    yield
    allow_graph_capture(previous)


def _inputs(rows, hidden, requires_grad=False):
    generator = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, hidden, device="cuda", generator=generator)
    branch = torch.randn(rows, hidden, device="cuda", generator=generator).half()
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    bias = 0.1 * torch.randn(hidden, device="cuda", generator=generator)
    tensors = (x, branch, weight, bias)
    if requires_grad:
        tensors = tuple(t.requires_grad_(True) for t in tensors)
    return tensors


def _warm_up(function):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            function()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()


@pytest.mark.parametrize(
    "hidden,normalized_dtype",
    [(128, None), (768, None), (256, torch.bfloat16), (1024, torch.float16)],
)
def test_captured_forward_draws_the_mask_of_the_generator_state_at_replay(
        capture_allowed, hidden, normalized_dtype):
    inputs = _inputs(64, hidden)

    def forward():
        return residual_layer_norm(*inputs, dropout_p=0.5, implementation="gfx1010",
                                   normalized_dtype=normalized_dtype)

    _warm_up(forward)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        updated, normalized = forward()
    torch.cuda.manual_seed(123)
    graph.replay()
    first = (updated.clone(), normalized.clone())
    graph.replay()
    second = updated.clone()
    torch.cuda.manual_seed(123)
    graph.replay()
    third = updated.clone()
    torch.cuda.manual_seed(123)
    eager = forward()
    torch.cuda.synchronize()
    assert not torch.equal(first[0], second)      # the offset advanced between replays
    assert torch.equal(first[0], third)           # same generator state, same mask
    assert torch.equal(first[0], eager[0])        # and the same as an eager call
    assert torch.equal(first[1], eager[1])


def test_captured_training_step_matches_eager(capture_allowed):
    inputs = _inputs(48, 384, requires_grad=True)
    grad_updated = torch.randn(48, 384, device="cuda")
    grad_normalized = torch.randn(48, 384, device="cuda")

    def step():
        outputs = residual_layer_norm(*inputs, dropout_p=0.1, implementation="gfx1010")
        return outputs, torch.autograd.grad(outputs, inputs, (grad_updated, grad_normalized))

    was_enabled = torch.are_deterministic_algorithms_enabled()
    warn_only = torch.is_deterministic_algorithms_warn_only_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        _warm_up(step)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outputs, gradients = step()
        torch.cuda.manual_seed(7)
        graph.replay()
        captured = [t.clone() for t in (*outputs, *gradients)]
        torch.cuda.manual_seed(7)
        eager_outputs, eager_gradients = step()
        torch.cuda.synchronize()
        for a, b in zip(captured, (*eager_outputs, *eager_gradients)):
            assert torch.equal(a, b)
    finally:
        torch.use_deterministic_algorithms(was_enabled, warn_only=warn_only)


def test_switch_restores_the_refusal():
    previous = allow_graph_capture(False)
    assert allow_graph_capture(previous) is False
