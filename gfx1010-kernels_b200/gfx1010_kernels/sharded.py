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


class PendingShardedStep:
    """A step whose all-reduce is still in flight (``async_op=True``).

    ``result`` is usable at once for everything row-local (``updated``,
    ``normalized``, ``grad_x``, ``grad_branch``, ``mask``: ordinary stream-ordered
    tensors); ``grad_weight`` / ``grad_bias`` hold the all-rank sums only after
    ``wait()``, which makes the current stream wait for the collective (it does
    not block the host for NCCL) and returns ``result``.  Waiting twice is fine.
    """

    def __init__(self, result: ShardedStepResult, work=None):
        self.result = result
        self._work = work

    def wait(self) -> ShardedStepResult:
        if self._work is not None:
            self._work.wait()
            self._work = None
        return self.result

    def is_completed(self) -> bool:
        return self._work is None or self._work.is_completed()


def high_priority_nccl_options():
    """``ProcessGroupNCCL.Options`` that put the group's collectives on a
    high-priority CUDA stream.  The all-reduce of a step is issued while the next
    forward's short CTAs are already queued on every SM; at equal priority its
    CTAs are placed only once that queue has been handed out and its latency
    shows at the forward's tail, with priority it takes the first slots that
    free up (measured on 8 GPUs: 7.41x -> 7.91x of one GPU)."""
    import torch.distributed as dist

    options = dist.ProcessGroupNCCL.Options()
    options.is_high_priority_stream = True
    return options


def init_sharded_process_group(device=None, *, timeout=None, high_priority=True, **kwargs):
    """``torch.distributed.init_process_group("nccl", ...)`` for one process per
    GPU with the options this module's overlap is measured with: a
    high-priority NCCL stream and eager initialisation on ``device``.  Rank,
    world size and rendezvous come from the environment (torchrun) unless given
    in ``kwargs``.  Returns the default group."""
    import torch.distributed as dist

    if high_priority:
        kwargs.setdefault("pg_options", high_priority_nccl_options())
    if device is not None:
        kwargs.setdefault("device_id", torch.device(device))
    if timeout is not None:
        kwargs["timeout"] = timeout
    dist.init_process_group("nccl", **kwargs)
    return dist.group.WORLD


def new_high_priority_group(ranks=None, *, timeout=None):
    """A NCCL group over ``ranks`` (default: all) with a high-priority stream,
    for programs whose default group already exists with other options.  Must be
    called by every rank, like ``torch.distributed.new_group``."""
    import torch.distributed as dist

    return dist.new_group(
        ranks=ranks, timeout=timeout, backend="nccl", pg_options=high_priority_nccl_options()
    )


def _extension_or_raise():
    from ._normalization_native import _extension

    extension, reason = _extension()
    if extension is None:
        raise RuntimeError(f"gfx1010 native extension is unavailable: {reason}")
    return extension


def _native_forward(x, branch, weight, bias, normalized_dtype, dropout_p, eps, training, seed,
                    offset, row_base):
    return _extension_or_raise().residual_layer_norm_forward_seeded(
        x, branch, weight, bias, float(dropout_p), float(eps), bool(training), 128,
        int(seed), int(offset), int(row_base), _BRANCH_CODES[normalized_dtype],
    )


def _native_backward(grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
                     dropout_p, training, branch_dtype):
    grad_x, grad_branch, grad_weight, grad_bias = \
        _extension_or_raise().residual_layer_norm_backward(
            grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
            float(dropout_p), bool(training), _BRANCH_CODES[branch_dtype],
            128, 16, 64, 1, True,
        )
    # grad_weight / grad_bias are views of one [2, hidden] allocation
    parameters = grad_weight._base if grad_weight._base is not None else torch.stack(
        (grad_weight, grad_bias)
    )
    return grad_x, grad_branch, parameters


def _native_forward_backward(x, branch, weight, bias, grad_updated, grad_normalized,
                             dropout_p, eps, training, seed, offset, row_base):
    """Forward + backward of one shard through the raw extension entries.

    ``normalized`` is produced in the type of ``grad_normalized`` (float32, or
    float16 / bfloat16 for a consumer that takes it in half precision).
    """
    updated, normalized, mean, rstd, mask = _native_forward(
        x, branch, weight, bias, grad_normalized.dtype, dropout_p, eps, training, seed, offset,
        row_base,
    )
    grad_x, grad_branch, parameters = _native_backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, mask, dropout_p, training,
        branch.dtype,
    )
    return updated, normalized, grad_x, grad_branch, parameters, mask


def _empty_shard(x, branch, weight, grad_normalized):
    """What a rank without rows contributes: empty row-local tensors (the mask
    of zero rows is empty whether or not dropout is on) and a zero
    ``[2, hidden]`` buffer for the sum."""
    updated = torch.empty_like(x)
    normalized = torch.empty_like(x, dtype=grad_normalized.dtype)
    mask = torch.empty(0, dtype=torch.int32, device=x.device)
    parameters = torch.zeros(2, weight.shape[0], dtype=torch.float32, device=weight.device)
    return updated, normalized, torch.empty_like(x), torch.empty_like(branch), parameters, mask


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
    async_op: bool = False,
    previous: Optional[PendingShardedStep] = None,
    after_forward: Optional[Callable[[], None]] = None,
    all_reduce: bool = True,
):
    """One training step of the operator on this rank's rows.

    ``row_base`` is the global index of the shard's first row (see
    ``shard_bounds``).  All ranks must pass the same ``seed``/``offset`` and
    identical ``weight``/``bias``.  A rank whose shard is empty (fewer rows than
    ranks) computes nothing, contributes zeros and still joins the all-reduce.

    ``async_op=True`` returns a ``PendingShardedStep`` right after the all-reduce
    has been issued.  Pass it as ``previous`` to the next call: that call runs its
    forward, then makes the stream wait for the previous step's all-reduce, then
    launches its backward -- the collective overlaps the forward (short CTAs,
    scheduled dynamically) and is gone before the backward's persistent grid
    needs every SM.  Wait on the last step's handle yourself.

    ``compute`` replaces the native forward+backward (same signature as
    ``_native_forward_backward``); it exists so that the partition and the
    collective can be exercised without a GPU.  With it, ``previous`` is waited
    for before ``compute`` runs.

    ``all_reduce=False`` leaves ``grad_weight`` / ``grad_bias`` as this rank's own
    sums (no collective is issued): for gradient accumulation over micro-batches,
    where only the last one reduces, and for a rank that works alone while a
    process group exists.

    ``after_forward`` (a profiling aid) is called with no arguments between the
    forward (plus the wait for ``previous``) and the backward of the native
    path, e.g. to record a CUDA event there.
    """
    import torch.distributed as dist

    if row_base < 0:
        raise ValueError("row_base must be non-negative")
    if x_shard.shape != branch_shard.shape or x_shard.shape != grad_updated_shard.shape \
            or x_shard.shape != grad_normalized_shard.shape:
        raise ValueError("the shard's tensors must have the same shape")
    if grad_normalized_shard.dtype not in _BRANCH_CODES:
        raise ValueError("grad_normalized must use float32, float16 or bfloat16")

    if x_shard.numel() == 0:
        if previous is not None:
            previous.wait()
        updated, normalized, grad_x, grad_branch, parameters, mask = _empty_shard(
            x_shard, branch_shard, weight, grad_normalized_shard
        )
    elif compute is not None:
        if previous is not None:
            previous.wait()
        updated, normalized, grad_x, grad_branch, parameters, mask = compute(
            x_shard, branch_shard, weight, bias, grad_updated_shard, grad_normalized_shard,
            dropout_p, eps, training, seed, offset, row_base,
        )
    else:
        updated, normalized, mean, rstd, mask = _native_forward(
            x_shard, branch_shard, weight, bias, grad_normalized_shard.dtype, dropout_p, eps,
            training, seed, offset, row_base,
        )
        # The backward is a persistent grid that fills every SM exactly once; a
        # communication kernel still resident from the previous step would push
        # part of it into a second wave.  So the previous all-reduce may overlap
        # the forward above but has to be done before the backward below.
        if previous is not None:
            previous.wait()
        if after_forward is not None:
            after_forward()
        grad_x, grad_branch, parameters = _native_backward(
            grad_updated_shard, grad_normalized_shard, updated, weight, mean, rstd, mask,
            dropout_p, training, branch_shard.dtype,
        )
    if parameters.shape != (2, weight.shape[0]) or not parameters.is_contiguous():
        raise RuntimeError("parameter gradients must be one contiguous [2, hidden] buffer")
    work = None
    if all_reduce and dist.is_available() and dist.is_initialized() \
            and dist.get_world_size(group) > 1:
        work = dist.all_reduce(parameters, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
    result = ShardedStepResult(
        updated=updated,
        normalized=normalized,
        grad_x=grad_x,
        grad_branch=grad_branch,
        grad_weight=parameters[0],
        grad_bias=parameters[1],
        mask=mask,
        row_base=row_base,
    )
    if async_op:
        return PendingShardedStep(result, work)
    return result


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
