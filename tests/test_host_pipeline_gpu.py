"""Host-buffer pipeline (``rln_sm100_host_*`` through
``gfx1010_kernels.host_pipeline``) against the device-buffer C-ABI calls on the
same rows: row-local outputs bit for bit, parameter gradients to 1e-4."""

import pytest
import torch

import cabi
from helpers import assert_parameters_close, draw_inputs
from gfx1010_kernels.host_pipeline import HostPipeline

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize(
    "rows,hidden,branch_dtype,chunk_rows,depth,deterministic,normalized_dtype",
    [
        (1000, 768, torch.float16, 128, 2, False, torch.float32),
        (1000, 768, torch.float16, 128, 3, True, torch.float32),
        (257, 128, torch.float32, 100, 2, True, torch.float32),
        (64, 1024, torch.float16, 4096, 2, False, torch.float32),   # single partial chunk
        (4101, 256, torch.float32, 512, 4, False, torch.float32),
        (777, 512, torch.bfloat16, 256, 3, True, torch.float32),
        (1000, 768, torch.float16, 128, 3, False, torch.bfloat16),
        (515, 384, torch.bfloat16, 200, 2, True, torch.float16),
    ],
)
def test_host_pipeline_matches_device_calls(rows, hidden, branch_dtype, chunk_rows, depth,
                                            deterministic, normalized_dtype):
    host = list(draw_inputs((rows,), hidden, branch_dtype, seed=rows, device="cpu"))
    host[5] = host[5].to(normalized_dtype)
    x, branch, weight, bias, grad_updated, grad_normalized = (t.pin_memory() for t in host)
    dropout_p, eps, seed, offset, row_base = 0.1, 1e-5, 77, 12, 5000
    with HostPipeline(hidden, branch_dtype, chunk_rows=chunk_rows, depth=depth,
                      normalized_dtype=normalized_dtype) as pipeline:
        out = pipeline.forward_backward(
            x, branch, weight, bias, grad_updated, grad_normalized, dropout_p, eps, True,
            seed=seed, offset=offset, row_base=row_base, deterministic=deterministic,
        )
        again = pipeline.forward_backward(
            x, branch, weight, bias, grad_updated, grad_normalized, dropout_p, eps, True,
            seed=seed, offset=offset, row_base=row_base, deterministic=deterministic,
        )
    device = [t.cuda() for t in host]
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        device[0], device[1], device[2], device[3], dropout_p, eps, True,
        seed=seed, offset=offset, row_base=row_base, normalized_dtype=normalized_dtype,
    )
    assert status == 0
    status, grad_x, grad_branch, grad_parameters = cabi.backward(
        device[4], device[5], updated, device[2], mean, rstd, mask, dropout_p, True,
        branch_dtype, deterministic,
    )
    assert status == 0
    torch.cuda.synchronize()
    assert out[1].dtype == normalized_dtype
    assert torch.equal(out[0], updated.cpu())
    assert torch.equal(out[1], normalized.cpu())
    assert torch.equal(out[2], grad_x.cpu())
    assert torch.equal(out[3], grad_branch.cpu())
    assert_parameters_close(out[4][0], grad_parameters[0].cpu(), rows, "grad_weight")
    assert_parameters_close(out[4][1], grad_parameters[1].cpu(), rows, "grad_bias")
    for a, b in zip(out[:4], again[:4]):
        assert torch.equal(a, b)
    if deterministic:
        assert torch.equal(out[4], again[4])


def test_host_pipeline_without_dropout_and_with_pageable_memory():
    rows, hidden = 300, 384
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, torch.float16, seed=3, device="cpu"
    )
    with HostPipeline(hidden, torch.float16, chunk_rows=64, depth=2) as pipeline:
        out = pipeline.forward_backward(
            x, branch, weight, bias, grad_updated, grad_normalized, 0.0, 1e-5, True,
            out=pipeline.allocate_outputs(x.shape, pinned=False),
        )
    assert torch.equal(out[0], x + branch.float())
    expected = torch.nn.functional.layer_norm(out[0].cuda(), (hidden,), weight.cuda(), bias.cuda())
    torch.testing.assert_close(out[1].cuda(), expected, rtol=1e-5, atol=1e-6)


def test_host_pipeline_rejects_bad_arguments():
    with pytest.raises(RuntimeError, match="unsupported native hidden size"):
        HostPipeline(160)
    with pytest.raises(RuntimeError, match="host-buffer pipeline"):
        HostPipeline(128, depth=1)
    with HostPipeline(128, torch.float16, chunk_rows=16, depth=2) as pipeline:
        x = torch.zeros(4, 128)
        with pytest.raises(RuntimeError, match="branch must use"):
            pipeline.forward_backward(x, x, torch.ones(128), torch.zeros(128), x, x)
        with pytest.raises(RuntimeError, match="grad_normalized must use"):
            pipeline.forward_backward(
                x, x.half(), torch.ones(128), torch.zeros(128), x, x.bfloat16())
        with pytest.raises(RuntimeError, match="host tensors"):
            pipeline.forward_backward(x.cuda(), x.half(), torch.ones(128), torch.zeros(128), x, x)
        with pytest.raises(RuntimeError, match=r"dropout_p must be in \[0, 1\)"):
            pipeline.forward_backward(x, x.half(), torch.ones(128), torch.zeros(128), x, x, 1.0)
        short = list(pipeline.allocate_outputs((4, 128)))
        short[2] = torch.empty(3, 128)
        with pytest.raises(RuntimeError, match="grad_x must have shape"):
            pipeline.forward_backward(
                x, x.half(), torch.ones(128), torch.zeros(128), x, x, out=tuple(short))


@pytest.mark.parametrize("depth", [2, 3])
def test_enqueued_steps_overlap_and_match_synchronous_calls(depth):
    """Four steps enqueued back to back (different Philox offsets, two sets of
    inputs, separate output tensors, chunk counts that do not divide the slot
    ring evenly) against the same four steps run one at a time, in deterministic
    mode: every output bit for bit."""
    rows, hidden, chunk_rows = 1100, 256, 256          # 5 chunks per step
    first = [t.pin_memory() for t in draw_inputs((rows,), hidden, torch.float16, 3, device="cpu")]
    second = [t.pin_memory() for t in draw_inputs((rows,), hidden, torch.float16, 4, device="cpu")]
    steps = [(first, 0), (second, 4), (first, 8), (second, 12)]
    with HostPipeline(hidden, torch.float16, chunk_rows=chunk_rows, depth=depth) as pipeline:
        expected = [
            [t.clone() for t in pipeline.forward_backward(
                *inputs, 0.1, 1e-5, True, seed=9, offset=offset, row_base=70, deterministic=True)]
            for inputs, offset in steps
        ]
        outputs = [pipeline.allocate_outputs((rows, hidden)) for _ in steps]
        for out in outputs:
            for tensor in out:
                tensor.fill_(float("nan"))
        already = pipeline.steps_enqueued()
        for (inputs, offset), out in zip(steps, outputs):
            returned = pipeline.forward_backward(
                *inputs, 0.1, 1e-5, True, seed=9, offset=offset, row_base=70,
                deterministic=True, out=out, wait=False,
            )
            assert returned is out
        assert pipeline.steps_enqueued() == already + len(steps)
        # the first enqueued step alone: its outputs are complete after this wait
        pipeline.wait(step=already + 1)
        for a, b in zip(outputs[0], expected[0]):
            assert torch.equal(a, b)
        with pytest.raises(RuntimeError, match="host-buffer pipeline"):
            pipeline.wait(step=already + len(steps) + 1)
        pipeline.wait()
        pipeline.wait()      # nothing left: returns at once
        # a synchronous call after enqueued ones still works
        after = pipeline.forward_backward(
            *first, 0.1, 1e-5, True, seed=9, offset=0, row_base=70, deterministic=True)
    for got, want in zip(outputs, expected):
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    for a, b in zip(after, expected[0]):
        assert torch.equal(a, b)
    assert not torch.equal(expected[0][0], expected[2][0])   # the offsets matter
