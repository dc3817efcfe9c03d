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
