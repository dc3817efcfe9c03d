"""``ResidualLayerNorm`` under ``DistributedDataParallel`` (gloo, two CPU ranks).

The module's weight and bias are ordinary parameters reached through autograd,
so DDP's bucketed all-reduce is the "hook" that combines the parameter
gradients of data-parallel ranks: each rank feeds its half of the batch through
a small pre-norm block (the integration pattern of the reference's
``docs/residual_layer_norm.md:51-83``) and after ``backward`` every rank must
hold the gradients of the whole batch.  On CPU tensors ``implementation="auto"``
takes the torch decomposition with its pinned ``RuntimeWarning``; dropout is
off so that the two ranks and the single-process run see the same function.
"""

import datetime
import socket
import sys
import warnings
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn
from torch.nn.parallel import DistributedDataParallel

REPO = Path(__file__).resolve().parent.parent
for path in (str(REPO), str(REPO / "gfx1010-kernels_b200")):
    if path not in sys.path:
        sys.path.insert(0, path)

from gfx1010_kernels.modules import ResidualLayerNorm  # noqa: E402

HIDDEN, ROWS = 128, 12


class Block(nn.Module):
    """x -> x + branch(x) fused with the next LayerNorm, then a projection."""

    def __init__(self):
        super().__init__()
        self.branch = nn.Linear(HIDDEN, HIDDEN)
        self.norm = ResidualLayerNorm(HIDDEN, dropout_p=0.0, implementation="auto")
        self.head = nn.Linear(HIDDEN, 4)

    def forward(self, x):
        updated, normalized = self.norm(x, self.branch(x))
        return self.head(normalized).sum() + 0.01 * updated.square().sum()


def make_block():
    torch.manual_seed(3)
    return Block()


def batch():
    return torch.randn(ROWS, HIDDEN, generator=torch.Generator().manual_seed(5))


def worker(rank, world, port, out_dir):
    dist.init_process_group(
        "gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
        timeout=datetime.timedelta(seconds=60),
    )
    try:
        model = DistributedDataParallel(make_block())
        shard = batch()[rank * ROWS // world: (rank + 1) * ROWS // world]
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            # DDP averages gradients over the ranks; scale so that the sum of the
            # two ranks' losses is the whole batch's loss
            (model(shard) * world).backward()
        fell_back = any("was not used" in str(w.message) for w in caught)
        torch.save(
            {"fell_back": fell_back,
             "grads": {name: p.grad.clone() for name, p in model.module.named_parameters()}},
            Path(out_dir) / f"rank{rank}.pt",
        )
    finally:
        dist.destroy_process_group()


def test_ddp_reduces_the_module_parameter_gradients(tmp_path):
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    world = 2
    mp.spawn(worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    model = make_block()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        model(batch()).backward()
    pieces = [torch.load(tmp_path / f"rank{rank}.pt") for rank in range(world)]
    for piece in pieces:
        assert piece["fell_back"], "auto on CPU tensors must warn and use the decomposition"
        assert set(piece["grads"]) == {name for name, _ in model.named_parameters()}
        for name, parameter in model.named_parameters():
            torch.testing.assert_close(piece["grads"][name], parameter.grad, rtol=1e-5, atol=1e-5)
    # the module's own parameters are among them, identical on both ranks
    for name in ("norm.weight", "norm.bias"):
        assert torch.equal(pieces[0]["grads"][name], pieces[1]["grads"][name])
        assert pieces[0]["grads"][name].abs().sum() > 0
