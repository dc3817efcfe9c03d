"""``gfx1010_kernels.sharded`` with the native kernels: shards processed one
after the other on one GPU reproduce the unsharded step (the multi-process
collective itself is covered on CPU ranks and by the multi-GPU benchmark)."""

import pytest
import torch

from helpers import assert_parameters_close, draw_inputs
from gfx1010_kernels.sharded import shard_bounds, sharded_forward_backward

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize(
    "world,normalized_dtype",
    [(2, torch.float32), (3, torch.float32), (8, torch.float32), (3, torch.bfloat16)],
)
def test_native_shards_reproduce_the_unsharded_step(world, normalized_dtype):
    rows, hidden = 1001, 768
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, torch.float16, 21
    )
    # `normalized` comes back in the type its gradient is given in
    grad_normalized = grad_normalized.to(normalized_dtype)
    arguments = dict(dropout_p=0.1, eps=1e-5, training=True, seed=5, offset=16)
    whole = sharded_forward_backward(
        x, branch, weight, bias, grad_updated, grad_normalized, row_base=0, **arguments
    )
    total_weight = torch.zeros(hidden, device="cuda", dtype=torch.float64)
    total_bias = torch.zeros(hidden, device="cuda", dtype=torch.float64)
    pieces = []
    for rank in range(world):
        begin, end = shard_bounds(rows, world, rank)
        piece = sharded_forward_backward(
            x[begin:end], branch[begin:end], weight, bias,
            grad_updated[begin:end], grad_normalized[begin:end], row_base=begin, **arguments
        )
        total_weight += piece.grad_weight.double()
        total_bias += piece.grad_bias.double()
        pieces.append(piece)
    assert whole.normalized.dtype == normalized_dtype
    for name in ("updated", "normalized", "grad_x", "grad_branch", "mask"):
        joined = torch.cat([getattr(piece, name) for piece in pieces])
        assert torch.equal(joined, getattr(whole, name)), name
    assert_parameters_close(whole.grad_weight, total_weight, rows, "grad_weight")
    assert_parameters_close(whole.grad_bias, total_bias, rows, "grad_bias")
