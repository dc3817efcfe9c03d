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


# ---------------------------------------------------------------------------
# Real ranks: one child process per GPU, NCCL, native kernels, checked against
# the CPU oracle.  Needs at least two GPUs (skipped on a single-GPU box).
# ---------------------------------------------------------------------------
def _nccl_worker(rank, world, port, out_dir):
    import datetime
    import os
    from pathlib import Path

    import torch.distributed as dist

    from gfx1010_kernels import sharded

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    sharded.init_sharded_process_group(
        torch.device("cuda", rank), timeout=datetime.timedelta(seconds=60),
        rank=rank, world_size=world,
    )
    try:
        rows, hidden, p, seed = 4099, 512, 0.1, 11
        x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
            (rows,), hidden, torch.float16, 77, device=torch.device("cuda", rank)
        )
        begin, end = shard_bounds(rows, world, rank)
        shard = (x[begin:end], branch[begin:end], weight, bias,
                 grad_updated[begin:end], grad_normalized[begin:end])
        sharded.check_replicated_parameters(weight, bias)
        pending, handles = None, []
        for step in range(3):
            pending = sharded_forward_backward(
                *shard, row_base=begin, dropout_p=p, seed=seed, offset=4 * step,
                async_op=True, previous=pending,
            )
            handles.append(pending)
        results = [handle.wait() for handle in handles]
        # a second NCCL group made by the module's helper gives the same sums
        group = sharded.new_high_priority_group()
        regrouped = sharded_forward_backward(
            *shard, row_base=begin, dropout_p=p, seed=seed, offset=8, group=group)
        assert torch.equal(regrouped.mask, results[2].mask)
        torch.testing.assert_close(regrouped.grad_weight, results[2].grad_weight,
                                   rtol=1e-4, atol=1e-3)
        torch.cuda.synchronize()
        torch.save(
            {"begin": begin, "end": end,
             "steps": [
                 {name: getattr(result, name).cpu() for name in
                  ("updated", "normalized", "grad_x", "grad_branch", "grad_weight", "grad_bias",
                   "mask")}
                 for result in results]},
            Path(out_dir) / f"rank{rank}.pt",
        )
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_ranks_reproduce_the_oracle_of_the_unsharded_step(tmp_path):
    import socket

    import torch.multiprocessing as mp

    from helpers import oracle_keep
    from oracle import rln_oracle

    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    mp.spawn(_nccl_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    pieces = [torch.load(tmp_path / f"rank{rank}.pt") for rank in range(world)]
    rows, hidden, p, seed = 4099, 512, 0.1, 11
    x, branch, weight, bias, grad_updated, grad_normalized = (
        t.cpu() for t in draw_inputs((rows,), hidden, torch.float16, 77)
    )
    for step in range(3):
        keep = oracle_keep(rows, hidden, p, seed, 4 * step).cpu()
        expected = rln_oracle.decomposition_gradients(
            x, branch, weight, bias, grad_updated, grad_normalized, p, 1e-5, True, keep,
            dtype=torch.float64,
        )
        mask = torch.cat([piece["steps"][step]["mask"] for piece in pieces])
        assert torch.equal(mask, torch.from_numpy(rln_oracle.pack_mask(keep.numpy()))), \
            "a rank's dropout mask differs from the Philox oracle of the unsharded call"
        updated = torch.cat([piece["steps"][step]["updated"] for piece in pieces])
        assert torch.equal(updated, expected[0].float())
        grad_x = torch.cat([piece["steps"][step]["grad_x"] for piece in pieces])
        torch.testing.assert_close(grad_x.double(), expected[2].double(), rtol=1e-5, atol=1e-5)
        for piece in pieces:
            # every rank holds the all-reduced sums, and they are the oracle's
            assert_parameters_close(piece["steps"][step]["grad_weight"], expected[4], rows,
                                    "grad_weight")
            assert_parameters_close(piece["steps"][step]["grad_bias"], expected[5], rows,
                                    "grad_bias")
            assert torch.equal(piece["steps"][step]["grad_weight"],
                               pieces[0]["steps"][step]["grad_weight"])
