"""Row-sharded residual LayerNorm step for data-parallel ranks (one process per GPU).

The operator is row-local except for ``grad_weight`` / ``grad_bias``, which are
sums over all rows.  A rank that owns a contiguous slice of the rows therefore
needs exactly two things beyond the single-GPU calls:

* the global index of its first row, so that the Philox counter of every
  element -- and with it the dropout mask, ``updated``, ``normalized``,
  ``grad_x`` and ``grad_branch`` -- is the one of the unsharded call;
* one all-reduce (sum) of the contiguous ``[2, hidden]`` parameter-gradient
  buffer after the backward.

Overlap: the all-reduce may run under the NEXT step's forward but should be
finished before that step's backward is launched (the backward's persistent
grid fills every SM exactly once; a resident communication kernel splits it
into two waves).  Create the NCCL group with a high-priority stream
(``ProcessGroupNCCL.Options.is_high_priority_stream = True``), otherwise the
collective is scheduled behind the forward's queued CTAs and its latency shows
(measured on 8 GPUs: 7.41x -> 7.91x of one GPU).

The reference project is single-device and has no counterpart of this module;
it sits on the caller side of the path.  The collective goes through
``torch.distributed`` (NCCL over NVLink/NVSwitch between GPUs; any backend
works -- the CPU tests use gloo with an injected compute function).
"""

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch


# the extension's element type codes (branch and normalized): False/0 float32,
# True/1 float16, 2 bfloat16
_BRANCH_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def shard_bounds(row_count: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Rows ``[begin, end)`` of ``rank``: contiguous, ordered by rank, sizes differ by at most 1."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    if row_count < 0:
        raise ValueError("row_count must be non-negative")
    begin = (row_count * rank) // world_size
    end = (row_count * (rank + 1)) // world_size
    return begin, end


@dataclass
class ShardedStepResult:
    updated: torch.Tensor
    normalized: torch.Tensor
    grad_x: torch.Tensor
    grad_branch: torch.Tensor
    grad_weight: torch.Tensor   # summed over all ranks
    grad_bias: torch.Tensor     # summed over all ranks
    mask: torch.Tensor
    row_base: int


def _native_forward_backward(x, branch, weight, bias, grad_updated, grad_normalized,
                             dropout_p, eps, training, seed, offset, row_base):
    """Forward + backward of one shard through the raw extension entries.

    ``normalized`` is produced in the type of ``grad_normalized`` (float32, or
    float16 / bfloat16 for a consumer that takes it in half precision).
    """
    from ._normalization_native import _extension

    extension, reason = _extension()
    if extension is None:
        raise RuntimeError(f"gfx1010 native extension is unavailable: {reason}")
    updated, normalized, mean, rstd, mask = extension.residual_layer_norm_forward_seeded(
        x, branch, weight, bias, float(dropout_p), float(eps), bool(training), 128,
        int(seed), int(offset), int(row_base), _BRANCH_CODES[grad_normalized.dtype],
    )
    grad_x, grad_branch, grad_weight, grad_bias = extension.residual_layer_norm_backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
        float(dropout_p), bool(training), _BRANCH_CODES[branch.dtype],
        128, 16, 64, 1, True,
    )
    # grad_weight / grad_bias are views of one [2, hidden] allocation
    parameters = grad_weight._base if grad_weight._base is not None else torch.stack(
        (grad_weight, grad_bias)
    )
    return updated, normalized, grad_x, grad_branch, parameters, mask


def sharded_forward_backward(
    x_shard: torch.Tensor,
    branch_shard: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    grad_updated_shard: torch.Tensor,
    grad_normalized_shard: torch.Tensor,
    *,
    row_base: int,
    dropout_p: float = 0.0,
    eps: float = 1e-5,
    training: bool = True,
    seed: int = 0,
    offset: int = 0,
    group=None,
    compute: Optional[Callable] = None,
) -> ShardedStepResult:
    """One training step of the operator on this rank's rows.

    ``row_base`` is the global index of the shard's first row (see
    ``shard_bounds``).  All ranks must pass the same ``seed``/``offset`` and
    identical ``weight``/``bias``.  ``compute`` replaces the native
    forward+backward (same signature as ``_native_forward_backward``); it exists
    so that the partition and the collective can be exercised without a GPU.
    """
    import torch.distributed as dist

    if row_base < 0:
        raise ValueError("row_base must be non-negative")
    if x_shard.shape != branch_shard.shape or x_shard.shape != grad_updated_shard.shape \
            or x_shard.shape != grad_normalized_shard.shape:
        raise ValueError("the shard's tensors must have the same shape")
    if grad_normalized_shard.dtype not in _BRANCH_CODES:
        raise ValueError("grad_normalized must use float32, float16 or bfloat16")
    compute = compute or _native_forward_backward
    updated, normalized, grad_x, grad_branch, parameters, mask = compute(
        x_shard, branch_shard, weight, bias, grad_updated_shard, grad_normalized_shard,
        dropout_p, eps, training, seed, offset, row_base,
    )
    if parameters.shape != (2, weight.shape[0]) or not parameters.is_contiguous():
        raise RuntimeError("parameter gradients must be one contiguous [2, hidden] buffer")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(parameters, op=dist.ReduceOp.SUM, group=group)
    return ShardedStepResult(
        updated=updated,
        normalized=normalized,
        grad_x=grad_x,
        grad_branch=grad_branch,
        grad_weight=parameters[0],
        grad_bias=parameters[1],
        mask=mask,
        row_base=row_base,
    )


def check_replicated_parameters(weight: torch.Tensor, bias: torch.Tensor, group=None) -> None:
    """Raise on every rank when ``weight``/``bias`` differ between ranks
    (shape or values).  A debugging aid for data-parallel set-ups; costs two
    small all-reduces."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return
    world = dist.get_world_size(group)
    if world == 1:
        return
    size = torch.tensor([float(weight.numel()), float(bias.numel())], device=weight.device)
    low, high = size.clone(), size.clone()
    dist.all_reduce(low, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(high, op=dist.ReduceOp.MAX, group=group)
    if not torch.equal(low, high):
        raise RuntimeError("weight/bias have different sizes on different ranks")
    stacked = torch.cat((weight.detach().reshape(-1), bias.detach().reshape(-1))).to(torch.float32)
    low, high = stacked.clone(), stacked.clone()
    dist.all_reduce(low, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(high, op=dist.ReduceOp.MAX, group=group)
    if not torch.equal(low, high):
        raise RuntimeError("weight/bias differ between ranks")
