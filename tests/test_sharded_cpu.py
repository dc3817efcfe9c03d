"""Row-sharded step on CPU ranks (gloo, world_size 2 and 3).

The native forward+backward is replaced by the CPU oracle through the
``compute`` hook, so what is exercised here is the host logic that is new with
respect to the single-device reference: the row partition, the global row
offset that keeps the dropout mask shard-invariant, and the all-reduce of the
``[2, hidden]`` parameter gradients -- plus what happens when a rank fails
before the collective (the failure is made on the host; no GPU is involved).
"""

import datetime
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent
for path in (str(REPO), str(REPO / "gfx1010-kernels_b200")):
    if path not in sys.path:
        sys.path.insert(0, path)

from gfx1010_kernels.sharded import (  # noqa: E402
    check_replicated_parameters,
    shard_bounds,
    sharded_forward_backward,
)
from oracle import rln_oracle  # noqa: E402

ROWS, HIDDEN, P, EPS, SEED, OFFSET = 53, 128, 0.2, 1e-5, 99, 8


def global_problem(branch_dtype=torch.float16):
    generator = torch.Generator().manual_seed(7)
    x = torch.randn(ROWS, HIDDEN, generator=generator)
    branch = torch.randn(ROWS, HIDDEN, generator=generator).to(branch_dtype)
    weight = 1.0 + 0.1 * torch.randn(HIDDEN, generator=generator)
    bias = 0.1 * torch.randn(HIDDEN, generator=generator)
    grad_updated = torch.randn(ROWS, HIDDEN, generator=generator)
    grad_normalized = torch.randn(ROWS, HIDDEN, generator=generator)
    return x, branch, weight, bias, grad_updated, grad_normalized


def oracle_compute(x, branch, weight, bias, grad_updated, grad_normalized,
                   dropout_p, eps, training, seed, offset, row_base):
    rows = x.shape[0]
    keep = rln_oracle.dropout_keep(rows, HIDDEN, dropout_p, seed, offset, row_base)
    updated, normalized, grad_x, grad_branch, grad_weight, grad_bias = (
        rln_oracle.decomposition_gradients(
            x, branch, weight, bias, grad_updated, grad_normalized,
            dropout_p, eps, training, torch.from_numpy(keep),
        )
    )
    mask = torch.from_numpy(rln_oracle.pack_mask(keep))
    return updated, normalized, grad_x, grad_branch, torch.stack((grad_weight, grad_bias)), mask


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def init(rank, world, port, timeout=30):
    dist.init_process_group(
        "gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
        timeout=datetime.timedelta(seconds=timeout),
    )


def worker_parity(rank, world, port, out_dir):
    init(rank, world, port)
    try:
        x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
        begin, end = shard_bounds(ROWS, world, rank)
        check_replicated_parameters(weight, bias)
        result = sharded_forward_backward(
            x[begin:end], branch[begin:end], weight, bias,
            grad_updated[begin:end], grad_normalized[begin:end],
            row_base=begin, dropout_p=P, eps=EPS, training=True, seed=SEED, offset=OFFSET,
            compute=oracle_compute,
        )
        torch.save(
            {
                "begin": begin, "end": end, "updated": result.updated,
                "normalized": result.normalized, "grad_x": result.grad_x,
                "grad_branch": result.grad_branch, "grad_weight": result.grad_weight,
                "grad_bias": result.grad_bias, "mask": result.mask,
            },
            Path(out_dir) / f"rank{rank}.pt",
        )
    finally:
        dist.destroy_process_group()


def worker_mismatch(rank, world, port, out_dir):
    init(rank, world, port)
    try:
        _, _, weight, bias, _, _ = global_problem()
        if rank == 1:
            weight = weight + 1.0
        try:
            check_replicated_parameters(weight, bias)
            outcome = "no error"
        except RuntimeError as error:
            outcome = str(error)
        (Path(out_dir) / f"rank{rank}.txt").write_text(outcome)
    finally:
        dist.destroy_process_group()


def worker_failing_rank(rank, world, port, out_dir):
    """Rank 1 fails on the host before the collective; rank 0 must get an error
    from its all-reduce within the process-group timeout instead of hanging."""
    init(rank, world, port, timeout=4)
    x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
    begin, end = shard_bounds(ROWS, world, rank)
    if rank == 1:
        (Path(out_dir) / "rank1.txt").write_text("left before the collective")
        return  # exits without joining the all-reduce
    try:
        sharded_forward_backward(
            x[begin:end], branch[begin:end], weight, bias,
            grad_updated[begin:end], grad_normalized[begin:end],
            row_base=begin, dropout_p=P, seed=SEED, offset=OFFSET, compute=oracle_compute,
        )
        outcome = "no error"
    except Exception as error:  # gloo reports a timeout or a closed connection
        outcome = f"error: {type(error).__name__}"
    (Path(out_dir) / "rank0.txt").write_text(outcome)


def test_shard_bounds_partition_every_row_once():
    for rows in (0, 1, 7, 53, 87381, 262144):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for rank in range(world):
                begin, end = shard_bounds(rows, world, rank)
                assert 0 <= begin <= end <= rows
                covered.append((begin, end))
            assert covered[0][0] == 0 and covered[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
            sizes = [end - begin for begin, end in covered]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_step_reproduces_the_unsharded_step(world, tmp_path):
    mp.spawn(worker_parity, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    pieces = [torch.load(tmp_path / f"rank{rank}.pt") for rank in range(world)]
    x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
    whole = oracle_compute(x, branch, weight, bias, grad_updated, grad_normalized,
                           P, EPS, True, SEED, OFFSET, 0)
    names = ("updated", "normalized", "grad_x", "grad_branch")
    for index, name in enumerate(names):
        joined = torch.cat([piece[name] for piece in pieces])
        assert torch.equal(joined, whole[index]), name
    assert torch.equal(torch.cat([piece["mask"] for piece in pieces]), whole[5])
    for piece in pieces:
        # every rank holds the global sums after the all-reduce
        torch.testing.assert_close(piece["grad_weight"], whole[4][0], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(piece["grad_bias"], whole[4][1], rtol=1e-5, atol=1e-5)
        assert torch.equal(piece["grad_weight"], pieces[0]["grad_weight"])


def test_replicated_parameter_check_fails_on_every_rank(tmp_path):
    mp.spawn(worker_mismatch, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert "differ between ranks" in (tmp_path / f"rank{rank}.txt").read_text()


def test_rank_that_leaves_before_the_collective_is_reported_not_waited_for(tmp_path):
    mp.spawn(worker_failing_rank, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "rank1.txt").read_text() == "left before the collective"
    assert (tmp_path / "rank0.txt").read_text().startswith("error:")


def test_single_process_step_needs_no_process_group():
    x, branch, weight, bias, grad_updated, grad_normalized = global_problem(torch.float32)
    result = sharded_forward_backward(
        x, branch, weight, bias, grad_updated, grad_normalized,
        row_base=0, dropout_p=P, seed=SEED, offset=OFFSET, compute=oracle_compute,
    )
    keep = rln_oracle.dropout_keep(ROWS, HIDDEN, P, SEED, OFFSET)
    assert np.array_equal(result.mask.numpy(), rln_oracle.pack_mask(keep))
    with pytest.raises(ValueError):
        sharded_forward_backward(x, branch[:3], weight, bias, grad_updated, grad_normalized,
                                 row_base=0, compute=oracle_compute)


def worker_fewer_rows_than_ranks(rank, world, port, out_dir):
    """Two rows over three ranks: one rank owns nothing, skips the compute,
    contributes zeros and still joins the all-reduce (nobody waits for it)."""
    init(rank, world, port, timeout=20)
    try:
        x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
        rows = 2
        begin, end = shard_bounds(rows, world, rank)
        calls = []

        def counting_compute(*args):
            calls.append(1)
            return oracle_compute(*args)

        result = sharded_forward_backward(
            x[begin:end], branch[begin:end], weight, bias,
            grad_updated[begin:end], grad_normalized[begin:end],
            row_base=begin, dropout_p=P, eps=EPS, training=True, seed=SEED, offset=OFFSET,
            compute=counting_compute,
        )
        torch.save(
            {"begin": begin, "end": end, "calls": len(calls), "updated": result.updated,
             "mask": result.mask, "grad_weight": result.grad_weight,
             "grad_bias": result.grad_bias},
            Path(out_dir) / f"rank{rank}.pt",
        )
    finally:
        dist.destroy_process_group()


def test_rank_without_rows_still_joins_the_all_reduce(tmp_path):
    world = 3
    mp.spawn(worker_fewer_rows_than_ranks, args=(world, free_port(), str(tmp_path)),
             nprocs=world, join=True)
    pieces = [torch.load(tmp_path / f"rank{rank}.pt") for rank in range(world)]
    empty = [piece for piece in pieces if piece["begin"] == piece["end"]]
    assert len(empty) == 1 and empty[0]["calls"] == 0
    assert empty[0]["updated"].shape == (0, HIDDEN) and empty[0]["mask"].numel() == 0
    x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
    whole = oracle_compute(x[:2], branch[:2], weight, bias, grad_updated[:2], grad_normalized[:2],
                           P, EPS, True, SEED, OFFSET, 0)
    for piece in pieces:
        torch.testing.assert_close(piece["grad_weight"], whole[4][0], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(piece["grad_bias"], whole[4][1], rtol=1e-5, atol=1e-5)


def worker_async_chain(rank, world, port, out_dir):
    """Three steps with async_op=True, each handed the previous step's handle:
    the sums of every step must be the synchronous ones."""
    init(rank, world, port)
    try:
        x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
        begin, end = shard_bounds(ROWS, world, rank)
        shard = (x[begin:end], branch[begin:end], weight, bias,
                 grad_updated[begin:end], grad_normalized[begin:end])
        pending, handles = None, []
        for step in range(3):
            pending = sharded_forward_backward(
                *shard, row_base=begin, dropout_p=P, eps=EPS, seed=SEED, offset=OFFSET + 4 * step,
                compute=oracle_compute, async_op=True, previous=pending,
            )
            handles.append(pending)
        results = [handle.wait() for handle in handles]
        assert all(handle.is_completed() for handle in handles)
        reference = [
            sharded_forward_backward(
                *shard, row_base=begin, dropout_p=P, eps=EPS, seed=SEED, offset=OFFSET + 4 * step,
                compute=oracle_compute,
            )
            for step in range(3)
        ]
        same = all(
            torch.equal(a.grad_weight, b.grad_weight) and torch.equal(a.grad_bias, b.grad_bias)
            and torch.equal(a.mask, b.mask)
            for a, b in zip(results, reference)
        )
        distinct = not torch.equal(results[0].mask, results[1].mask)
        (Path(out_dir) / f"rank{rank}.txt").write_text(f"{same} {distinct}")
    finally:
        dist.destroy_process_group()


def test_async_steps_chained_through_previous_give_the_synchronous_sums(tmp_path):
    mp.spawn(worker_async_chain, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert (tmp_path / f"rank{rank}.txt").read_text() == "True True"


def worker_local_sums(rank, world, port, out_dir):
    """all_reduce=False: a rank that works alone while a process group exists
    (gradient accumulation) issues no collective -- rank 1 does not call at all,
    so a collective here would time out -- and keeps its own sums."""
    init(rank, world, port, timeout=10)
    try:
        outcome = "idle"
        if rank == 0:
            x, branch, weight, bias, grad_updated, grad_normalized = global_problem()
            result = sharded_forward_backward(
                x, branch, weight, bias, grad_updated, grad_normalized,
                row_base=0, dropout_p=P, eps=EPS, seed=SEED, offset=OFFSET,
                compute=oracle_compute, all_reduce=False,
            )
            whole = oracle_compute(x, branch, weight, bias, grad_updated, grad_normalized,
                                   P, EPS, True, SEED, OFFSET, 0)
            outcome = str(torch.equal(result.grad_weight, whole[4][0])
                          and torch.equal(result.grad_bias, whole[4][1]))
        (Path(out_dir) / f"rank{rank}.txt").write_text(outcome)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_all_reduce_can_be_skipped_for_local_accumulation(tmp_path):
    mp.spawn(worker_local_sums, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "rank0.txt").read_text() == "True"
    assert (tmp_path / "rank1.txt").read_text() == "idle"
