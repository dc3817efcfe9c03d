"""The allocation-free backward entry point, ``rln_sm100_backward_static_scratch``.

Some hosts of this library may not allocate device memory while an operator
runs: a runtime that gave the whole GPU to its own memory pool, a plugin
interface whose run step must not call an allocator, a loop that cannot take
the device-wide stall of a cudaMalloc.  For them the deterministic backward
keeps its per-CTA partial sums in a 4 MiB array that ships inside the library's
device image, instead of a workspace the caller would have to allocate.

This file checks, through the C ABI, that the entry point returns exactly what
``rln_sm100_backward(..., deterministic=1)`` returns, on two calls in a row
that share the scratch array (the second one smaller than the first, so stale
partials from the first call sit right behind the ones it reads), and that the
calls leave the amount of free device memory unchanged.

The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

import ctypes

import pytest
import torch

import cabi
from helpers import draw_inputs

pytestmark = pytest.mark.gpu

_P = ctypes.c_void_p


def _entry():
    lib = cabi.library()
    function = lib.rln_sm100_backward_static_scratch
    function.restype = ctypes.c_int
    function.argtypes = [_P] * 10 + [
        ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, _P,
    ]
    return function


def _outputs(updated, branch_dtype):
    hidden = updated.shape[-1]
    return (
        torch.empty_like(updated),
        torch.empty(updated.shape, dtype=branch_dtype, device=updated.device),
        torch.empty(2, hidden, device=updated.device),
    )


def _static_backward(grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
                     dropout_p, branch_dtype, outputs=None):
    hidden = updated.shape[-1]
    rows = updated.numel() // hidden
    active = dropout_p > 0.0
    grad_x, grad_branch, grad_parameters = outputs or _outputs(updated, branch_dtype)
    status = _entry()(
        grad_updated.data_ptr(), grad_normalized.data_ptr(), updated.data_ptr(),
        weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
        mask.data_ptr() if active else None,
        grad_x.data_ptr(), grad_branch.data_ptr(), grad_parameters.data_ptr(),
        rows, hidden, cabi.BRANCH_CODES[branch_dtype], int(active), dropout_p,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    return status, grad_x, grad_branch, grad_parameters


def _case(rows, hidden, branch_dtype, dropout_p, seed):
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, branch_dtype, seed
    )
    status, updated, _, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, dropout_p, 1e-5, True, seed=seed, offset=0
    )
    assert status == 0, cabi.status_text(status)
    return grad_updated, grad_normalized, updated, weight, mean, rstd, mask


@pytest.mark.parametrize("hidden,branch_dtype", [(768, torch.float16), (128, torch.float32),
                                                 (1024, torch.float16), (384, torch.bfloat16)])
def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row(hidden, branch_dtype):
    dropout_p = 0.1
    # first call fills the whole persistent grid, second call uses a few CTAs only
    calls = [_case(5000, hidden, branch_dtype, dropout_p, seed=11),
             _case(37, hidden, branch_dtype, dropout_p, seed=12)]
    torch.cuda.synchronize()
    for tensors in calls:
        status, grad_x, grad_branch, grad_parameters = _static_backward(
            *tensors, dropout_p, branch_dtype
        )
        assert status == 0, cabi.status_text(status)
        reference = cabi.backward(*tensors, dropout_p, True, branch_dtype, True)
        assert reference[0] == 0, cabi.status_text(reference[0])
        torch.cuda.synchronize()
        # same kernels, same grid, same summation order: bit for bit
        assert torch.equal(grad_x, reference[1])
        assert torch.equal(grad_branch, reference[2])
        assert torch.equal(grad_parameters, reference[3])
    # The one-time address look-up is behind us.  With the output buffers made
    # beforehand (so that this test's own allocator stays out of the picture),
    # a call must not lower the free memory of the device.
    outputs = _outputs(calls[0][2], branch_dtype)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status, *_ = _static_backward(*calls[0], dropout_p, branch_dtype, outputs=outputs)
    assert status == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before


def test_static_scratch_backward_without_dropout_and_argument_checks():
    tensors = _case(300, 384, torch.float16, 0.0, seed=5)
    status, grad_x, grad_branch, grad_parameters = _static_backward(*tensors, 0.0, torch.float16)
    assert status == 0, cabi.status_text(status)
    reference = cabi.backward(*tensors, 0.0, True, torch.float16, True)
    torch.cuda.synchronize()
    assert torch.equal(grad_x, reference[1])
    assert torch.equal(grad_branch, reference[2])
    assert torch.equal(grad_parameters, reference[3])

    entry = _entry()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g_u, g_y, updated, weight, mean, rstd, _ = tensors
    pointers = [t.data_ptr() for t in (g_u, g_y, updated, weight, mean, rstd)]
    outs = [torch.empty_like(updated), torch.empty_like(updated, dtype=torch.float16),
            torch.empty(2, 384, device="cuda")]

    def call(rows=300, hidden=384, p=0.0, parameters=outs[2].data_ptr()):
        return entry(*pointers, None, outs[0].data_ptr(), outs[1].data_ptr(), parameters,
                     rows, hidden, 1, 0, p, stream)

    assert call(hidden=160) == -2
    assert call(rows=0) == -3
    assert call(p=1.0) == -4
    assert call(parameters=None) == -1
    assert "fixed maximum" in cabi.status_text(-10)
    # every supported width fits the 4 MiB scratch on this device at any row count
    lib = cabi.library()
    for hidden in (128, 256, 384, 512, 768, 1024):
        assert lib.rln_sm100_backward_workspace_bytes(1 << 30, hidden, 1) <= (4 << 20)
