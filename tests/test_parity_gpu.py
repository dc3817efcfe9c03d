"""CUDA path vs the oracle, through the C ABI (``include/rln_sm100.h``).

Every test drives ``librln_sm100.so`` with raw device addresses via ctypes and
checks against ``oracle/rln_oracle.py`` evaluated on the same seeded inputs:
the dropout mask bit for bit against the Philox oracle, ``updated`` bit for bit
and ``normalized`` to 1e-5 relative / 1e-6 absolute against the torch
decomposition fed the kernel's mask, gradients against autograd through that
decomposition (fp32 on the device, fp64 as arbiter)."""

import numpy as np
import pytest
import torch

import cabi
from conftest import golden_tensors
from helpers import (
    GRAD_X_TOL,
    grad_branch_tolerance,
    NORMALIZED_TOL,
    assert_narrow_normalized,
    assert_parameters_close,
    draw_inputs,
    oracle_keep,
    unpack_mask_device,
)
from oracle import rln_oracle

pytestmark = pytest.mark.gpu

HIDDEN_SIZES = (128, 256, 384, 512, 768, 1024)


def run_and_check(shape, hidden, branch_dtype, dropout_p, seed, *, training=True, eps=1e-5,
                  philox=(0, 0), deterministic=False, check_mask_with_oracle=True,
                  normalized_dtype=torch.float32):
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        shape, hidden, branch_dtype, seed
    )
    narrow = normalized_dtype != torch.float32
    # the gradient of a 16-bit `normalized` arrives in that type
    grad_normalized = grad_normalized.to(normalized_dtype)
    rows = x.numel() // hidden
    active = training and dropout_p > 0
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, dropout_p, eps, training, seed=philox[0], offset=philox[1],
        normalized_dtype=normalized_dtype,
    )
    assert status == 0, cabi.status_text(status)
    keep = None
    if active:
        keep = unpack_mask_device(mask, rows, hidden)
        if check_mask_with_oracle:
            expected_keep = oracle_keep(rows, hidden, dropout_p, *philox)
            assert torch.equal(keep, expected_keep), "dropout mask differs from the Philox oracle"
    expected = rln_oracle.decomposition_gradients(
        x, branch, weight, bias, grad_updated, grad_normalized,
        dropout_p, eps, training, keep,
        normalized_dtype=normalized_dtype if narrow else None,
    )
    arbiter = rln_oracle.decomposition_gradients(
        x, branch, weight, bias, grad_updated, grad_normalized,
        dropout_p, eps, training, keep, dtype=torch.float64,
    )
    assert torch.equal(updated, expected[0]), "updated is not bit-identical"
    assert normalized.dtype == normalized_dtype
    if narrow:
        # one rounding of the float32 result: exact bracket against the fp64
        # arbiter, and the same 16-bit number as the torch oracle except where
        # the two float32 values straddle a rounding boundary
        assert_narrow_normalized(normalized, arbiter[1])
        same = (normalized == expected[1]).float().mean().item()
        assert same > 0.99, same
    else:
        torch.testing.assert_close(normalized, expected[1], **NORMALIZED_TOL)
        torch.testing.assert_close(normalized.double(), arbiter[1], **NORMALIZED_TOL)
    mean64, rstd64 = rln_oracle.row_statistics(updated.double().view(rows, hidden), eps)
    torch.testing.assert_close(mean.double(), mean64, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(rstd.double(), rstd64, rtol=1e-5, atol=0)

    status, grad_x, grad_branch, grad_parameters = cabi.backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, mask,
        dropout_p, training, branch_dtype, deterministic,
    )
    assert status == 0, cabi.status_text(status)
    torch.cuda.synchronize()
    torch.testing.assert_close(grad_x, expected[2], **GRAD_X_TOL)
    torch.testing.assert_close(grad_x.double(), arbiter[2].double(), **GRAD_X_TOL)
    torch.testing.assert_close(
        grad_branch.float(), expected[3].float(), **grad_branch_tolerance(branch_dtype)
    )
    assert_parameters_close(grad_parameters[0], arbiter[4], rows, "grad_weight")
    assert_parameters_close(grad_parameters[1], arbiter[5], rows, "grad_bias")
    return dict(
        x=x, branch=branch, weight=weight, bias=bias, updated=updated, normalized=normalized,
        mean=mean, rstd=rstd, mask=mask, grad_x=grad_x, grad_branch=grad_branch,
        grad_parameters=grad_parameters, grad_updated=grad_updated,
        grad_normalized=grad_normalized,
    )


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
@pytest.mark.parametrize(
    "branch_dtype", [torch.float16, torch.float32, torch.bfloat16], ids=["half", "float", "bf16"]
)
@pytest.mark.parametrize("dropout_p", [0.0, 0.1])
def test_forward_backward_parity_all_widths(hidden, branch_dtype, dropout_p):
    run_and_check((1, 37), hidden, branch_dtype, dropout_p, seed=17 + hidden,
                  philox=(5, 12))


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
@pytest.mark.parametrize(
    "branch_dtype", [torch.float16, torch.float32, torch.bfloat16], ids=["half", "float", "bf16"]
)
@pytest.mark.parametrize("normalized_dtype", [torch.float16, torch.bfloat16], ids=["f16n", "bf16n"])
@pytest.mark.parametrize("dropout_p", [0.0, 0.1])
def test_narrow_normalized_parity_all_widths(hidden, branch_dtype, normalized_dtype, dropout_p):
    """`normalized` stored as float16 / bfloat16 and its gradient read in that
    type; everything else as in the float32 case."""
    run_and_check((1, 37), hidden, branch_dtype, dropout_p, seed=19 + hidden,
                  philox=(5, 12), normalized_dtype=normalized_dtype)


@pytest.mark.parametrize("hidden", [128, 768, 1024])
def test_narrow_normalized_deterministic_and_ragged(hidden):
    run_and_check((513,), hidden, torch.float16, 0.15, seed=29, deterministic=True,
                  normalized_dtype=torch.bfloat16)


def test_narrow_normalized_needs_vector_alignment():
    """A 16-bit `normalized` / `grad_normalized` that is not 8-byte aligned is
    refused (there is no scalar-access kernel for it), never mis-read."""
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (9,), 256, torch.float16, 3
    )
    rows, hidden = 9, 256
    storage = torch.empty(rows * hidden + 8, dtype=torch.bfloat16, device="cuda")
    shifted = storage[1:1 + rows * hidden].view(rows, hidden)   # 2-byte aligned only
    outputs = (torch.empty_like(x), shifted, torch.empty(rows, device="cuda"),
               torch.empty(rows, device="cuda"), torch.empty(0, dtype=torch.int32, device="cuda"))
    status, *_ = cabi.forward(x, branch, weight, bias, 0.0, 1e-5, True, outputs=outputs)
    assert status == -6
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, 0.0, 1e-5, True, normalized_dtype=torch.bfloat16
    )
    assert status == 0
    shifted.copy_(grad_normalized)
    status, *_ = cabi.backward(
        grad_updated, shifted, updated, weight, mean, rstd, mask, 0.0, True, torch.float16, False
    )
    assert status == -6


@pytest.mark.parametrize("hidden", HIDDEN_SIZES)
def test_deterministic_path_parity(hidden):
    run_and_check((41,), hidden, torch.float16, 0.15, seed=23, deterministic=True)


@pytest.mark.parametrize("rows", [1, 2, 3, 15, 16, 17, 511, 512, 513, 2047, 2048, 2049])
def test_row_count_boundaries_at_h128(rows):
    run_and_check((rows,), 128, torch.float16, 0.15, seed=227 + rows)


@pytest.mark.parametrize("hidden", HIDDEN_SIZES[1:])
@pytest.mark.parametrize("rows", [1, 5, 33])
def test_fewer_rows_than_warps(hidden, rows):
    run_and_check((rows,), hidden, torch.float32, 0.2, seed=31 + rows)


def test_config_cpu_runnable_reference_case():
    # x fp32 [8,1024,768], branch fp16, p 0.1, seed 0
    run_and_check((8, 1024), 768, torch.float16, 0.1, seed=0)


@pytest.mark.parametrize("shape,hidden", [((3, 1367), 128), ((5, 817), 256)])
def test_config_small_hidden_ragged_rows_fp32_branch(shape, hidden):
    run_and_check(shape, hidden, torch.float32, 0.15, seed=1)


def test_eval_mode_ignores_dropout_and_mask():
    run_and_check((7,), 384, torch.float16, 0.8, seed=101, training=False)


def test_large_eps_and_nearly_constant_rows():
    hidden = 384
    columns = torch.linspace(-1.0, 1.0, hidden, device="cuda")
    centers = torch.tensor([-3.0, 0.25, 4.0], device="cuda")[:, None]
    x = (centers + columns[None, :] * 2e-4).contiguous()
    branch = (-columns[None, :] * 5e-5).expand_as(x).contiguous().half()
    weight = torch.linspace(0.75, 1.25, hidden, device="cuda")
    bias = torch.linspace(-0.1, 0.1, hidden, device="cuda")
    for eps in (1e-5, 1e-3):
        status, updated, normalized, mean, rstd, _ = cabi.forward(
            x, branch, weight, bias, 0.0, eps, True
        )
        assert status == 0
        expected = rln_oracle.torch_decomposition(
            x.double(), branch.double(), weight.double(), bias.double(), 0.0, eps, True
        )
        assert torch.isfinite(normalized).all()
        assert torch.equal(updated, x + branch.float())
        # rows are nearly constant: cancellation amplifies fp32 rounding of
        # `updated` itself, so compare on the scale the reference's test uses
        torch.testing.assert_close(normalized.double(), expected[1], rtol=8e-3, atol=8e-3)


@pytest.mark.parametrize(
    "name",
    ["h128_half_p10", "h256_float_p15", "h384_half_eval", "h512_half_p0", "h768_half_p10",
     "h1024_float_p25", "h768_bfloat16_p10", "h768_half_p10_bf16norm",
     "h256_bfloat16_p20_f16norm", "h1024_float_eval_bf16norm"],
)
def test_golden_fixtures_from_the_reference(golden_cases, name):
    case = golden_cases[name]
    meta = case["meta"]
    t = golden_tensors(case, device="cuda")
    hidden = meta["hidden"]
    branch_dtype = t["branch"].dtype
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        t["x"], t["branch"], t["weight"], t["bias"], meta["dropout_p"], meta["eps"],
        meta["training"], seed=meta["philox_seed"], offset=meta["philox_offset"],
        normalized_dtype=t["normalized"].dtype,
    )
    assert status == 0, cabi.status_text(status)
    active = meta["training"] and meta["dropout_p"] > 0
    if active:
        assert torch.equal(mask, t["mask"]), "mask differs from the fixture"
    assert torch.equal(updated, t["updated"])
    if t["normalized"].dtype == torch.float32:
        torch.testing.assert_close(normalized, t["normalized"], **NORMALIZED_TOL)
    else:
        # both are one rounding of float32-close values: neighbours at worst,
        # identical almost everywhere
        tolerance = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[normalized.dtype]
        torch.testing.assert_close(
            normalized.float(), t["normalized"].float(), rtol=tolerance, atol=1e-4)
        assert (normalized == t["normalized"]).float().mean().item() > 0.99
    torch.testing.assert_close(mean.double(), t["mean64"].reshape(-1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(rstd.double(), t["rstd64"].reshape(-1), rtol=1e-5, atol=0)
    rows = t["x"].numel() // hidden
    for deterministic in (False, True):
        status, grad_x, grad_branch, grad_parameters = cabi.backward(
            t["grad_updated"], t["grad_normalized"], updated, t["weight"], mean, rstd, mask,
            meta["dropout_p"], meta["training"], branch_dtype, deterministic,
        )
        assert status == 0, cabi.status_text(status)
        torch.testing.assert_close(grad_x, t["grad_x"], **GRAD_X_TOL)
        torch.testing.assert_close(
            grad_branch.float(), t["grad_branch"].float(), **grad_branch_tolerance(branch_dtype)
        )
        assert_parameters_close(grad_parameters[0], t["grad_weight"], rows, "grad_weight")
        assert_parameters_close(grad_parameters[1], t["grad_bias"], rows, "grad_bias")


def test_mask_replay_is_bit_exact_and_offsets_do_not_overlap():
    x, branch, weight, bias, _, _ = draw_inputs((64,), 768, torch.float16, 3)
    first = cabi.forward(x, branch, weight, bias, 0.5, 1e-5, True, seed=127, offset=0)
    again = cabi.forward(x, branch, weight, bias, 0.5, 1e-5, True, seed=127, offset=0)
    later = cabi.forward(x, branch, weight, bias, 0.5, 1e-5, True, seed=127, offset=8)
    other = cabi.forward(x, branch, weight, bias, 0.5, 1e-5, True, seed=128, offset=0)
    for a, b in zip(first[1:], again[1:]):
        assert torch.equal(a, b)
    assert not torch.equal(first[5], later[5])
    assert not torch.equal(first[5], other[5])
    # no shifted reuse of the stream either: compare column windows
    keep_first = unpack_mask_device(first[5], 64, 768)
    keep_later = unpack_mask_device(later[5], 64, 768)
    assert not torch.equal(keep_first[:, 512:768], keep_later[:, :256])


@pytest.mark.parametrize("dropout_p", [0.1, 0.15, 0.5, 0.9])
def test_kept_fraction_within_four_sigma(dropout_p):
    rows, hidden = 4096, 768
    x, branch, weight, bias, _, _ = draw_inputs((rows,), hidden, torch.float16, 5)
    status, *_, mask = cabi.forward(x, branch, weight, bias, dropout_p, 1e-5, True, seed=0, offset=0)
    assert status == 0
    keep = unpack_mask_device(mask, rows, hidden)
    n = rows * hidden
    p32 = float(np.float32(dropout_p))
    sigma = (p32 * (1 - p32) / n) ** 0.5
    assert abs(keep.float().mean().item() - (1 - p32)) < 4 * sigma


def test_row_shards_reproduce_the_unsharded_call_bit_for_bit():
    rows, hidden = 1000, 512
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, torch.float16, 7
    )
    full = cabi.forward(x, branch, weight, bias, 0.1, 1e-5, True, seed=11, offset=4)
    assert full[0] == 0
    bounds = [0, 333, 334, 777, rows]
    pieces = []
    for begin, end in zip(bounds[:-1], bounds[1:]):
        piece = cabi.forward(
            x[begin:end], branch[begin:end], weight, bias, 0.1, 1e-5, True,
            seed=11, offset=4, row_base=begin,
        )
        assert piece[0] == 0
        pieces.append(piece)
    for index in range(1, 6):
        joined = torch.cat([piece[index] for piece in pieces])
        assert torch.equal(joined, full[index]), index
    # backward: row-local outputs identical, parameter sums add up across shards
    whole = cabi.backward(grad_updated, grad_normalized, full[1], weight, full[3], full[4],
                          full[5], 0.1, True, torch.float16, True)
    total = torch.zeros(2, hidden, device="cuda", dtype=torch.float64)
    for (begin, end), piece in zip(zip(bounds[:-1], bounds[1:]), pieces):
        part = cabi.backward(
            grad_updated[begin:end], grad_normalized[begin:end], piece[1], weight, piece[3],
            piece[4], piece[5], 0.1, True, torch.float16, True,
        )
        assert part[0] == 0
        assert torch.equal(part[1], whole[1][begin:end])
        assert torch.equal(part[2], whole[2][begin:end])
        total += part[3].double()
    assert_parameters_close(whole[3][0], total[0], rows, "grad_weight")
    assert_parameters_close(whole[3][1], total[1], rows, "grad_bias")


def test_deterministic_replay_is_bitwise_and_close_to_atomic_path():
    result = run_and_check((257,), 384, torch.float16, 0.0, seed=233)
    args = (result["grad_updated"], result["grad_normalized"], result["updated"],
            result["weight"], result["mean"], result["rstd"], result["mask"],
            0.0, True, torch.float16)
    first = cabi.backward(*args, True)
    second = cabi.backward(*args, True)
    atomic = cabi.backward(*args, False)
    torch.cuda.synchronize()
    for a, b in zip(first[1:], second[1:]):
        assert torch.equal(a, b)
    torch.testing.assert_close(first[3], atomic[3], rtol=5e-4, atol=5e-4)
    assert torch.equal(first[1], atomic[1]) and torch.equal(first[2], atomic[2])


@pytest.mark.parametrize("hidden", [128, 256, 768, 1024])
@pytest.mark.parametrize("seed,offset,extra", [(0, 0, 0), (1234, 8, 4), (2 ** 40 + 5, 2 ** 33, 12)])
def test_device_resident_philox_state_gives_the_oracle_mask(hidden, seed, offset, extra):
    """The kernels that read (seed, offset) from device memory -- the ones a CUDA
    graph records -- checked directly against the Philox oracle for
    (seed, offset + offset_extra), and bit for bit against the immediate-state
    kernels on every output.  No graph is involved: the two words are plain
    int64 device tensors."""
    rows, p = 301, 0.1
    x, branch, weight, bias, _, _ = draw_inputs((rows,), hidden, torch.float16, 41)
    device_seed = torch.tensor([seed], dtype=torch.int64, device="cuda")
    device_offset = torch.tensor([offset], dtype=torch.int64, device="cuda")
    from_device = cabi.forward_device_rng(
        x, branch, weight, bias, p, 1e-5, True, device_seed, device_offset, offset_extra=extra,
        row_base=17,
    )
    immediate = cabi.forward(x, branch, weight, bias, p, 1e-5, True, seed=seed,
                             offset=offset + extra, row_base=17)
    torch.cuda.synchronize()
    assert from_device[0] == 0 and immediate[0] == 0, cabi.status_text(from_device[0])
    keep = unpack_mask_device(from_device[5], rows, hidden)
    expected = oracle_keep(rows, hidden, p, seed, offset + extra, row_base=17)
    assert torch.equal(keep, expected), "device-state mask differs from the Philox oracle"
    for a, b in zip(from_device[1:], immediate[1:]):
        assert torch.equal(a, b)
    # the state is read at run time: changing the words changes the next launch
    device_offset.add_(4)
    moved = cabi.forward_device_rng(
        x, branch, weight, bias, p, 1e-5, True, device_seed, device_offset, offset_extra=extra,
        row_base=17,
    )
    assert torch.equal(
        unpack_mask_device(moved[5], rows, hidden),
        oracle_keep(rows, hidden, p, seed, offset + extra + 4, row_base=17),
    )


def test_parameter_gradients_can_be_skipped():
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (19,), 256, torch.float16, 9
    )
    _, updated, _, mean, rstd, mask = cabi.forward(x, branch, weight, bias, 0.15, 1e-5, True)
    with_parameters = cabi.backward(grad_updated, grad_normalized, updated, weight, mean, rstd,
                                    mask, 0.15, True, torch.float16, False)
    without = cabi.backward(grad_updated, grad_normalized, updated, weight, mean, rstd,
                            mask, 0.15, True, torch.float16, False, parameters=False)
    assert without[0] == 0 and without[3] is None
    assert torch.equal(with_parameters[1], without[1])
    assert torch.equal(with_parameters[2], without[2])


def test_updated_only_gradient_passes_through_exactly():
    x, branch, weight, bias, grad_updated, _ = draw_inputs((13,), 384, torch.float16, 229)
    _, updated, _, mean, rstd, mask = cabi.forward(x, branch, weight, bias, 0.0, 1e-5, True)
    zeros = torch.zeros_like(grad_updated)
    status, grad_x, grad_branch, _ = cabi.backward(
        grad_updated, zeros, updated, weight, mean, rstd, mask, 0.0, True, torch.float16,
        False, parameters=False,
    )
    assert status == 0
    assert torch.equal(grad_x, grad_updated)
    assert torch.equal(grad_branch, grad_updated.half())


@pytest.mark.parametrize("hidden", [128, 384, 1024])
@pytest.mark.parametrize(
    "branch_dtype", [torch.float16, torch.float32, torch.bfloat16], ids=["half", "float", "bf16"]
)
def test_misaligned_pointers_take_the_scalar_kernels_with_identical_results(hidden, branch_dtype):
    rows = 23
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, branch_dtype, 409
    )

    def shifted(tensor):
        storage = torch.empty(tensor.numel() + 1, dtype=tensor.dtype, device=tensor.device)
        view = storage[1:].view(tensor.shape)
        view.copy_(tensor)
        assert view.data_ptr() % 16 != 0
        return view

    aligned = cabi.forward(x, branch, weight, bias, 0.15, 1e-5, True, seed=1, offset=0)
    outputs = tuple(
        shifted(t) for t in (aligned[1], aligned[2])
    ) + (torch.empty_like(aligned[3]), torch.empty_like(aligned[4]), torch.empty_like(aligned[5]))
    misaligned = cabi.forward(
        shifted(x), shifted(branch), shifted(weight), shifted(bias), 0.15, 1e-5, True,
        seed=1, offset=0, outputs=outputs,
    )
    assert aligned[0] == 0 and misaligned[0] == 0
    for a, b in zip(aligned[1:], misaligned[1:]):
        assert torch.equal(a, b)

    fast = cabi.backward(grad_updated, grad_normalized, aligned[1], weight, aligned[3],
                         aligned[4], aligned[5], 0.15, True, branch_dtype, True)
    slow = cabi.backward(shifted(grad_updated), grad_normalized, aligned[1], weight, aligned[3],
                         aligned[4], aligned[5], 0.15, True, branch_dtype, True)
    assert fast[0] == 0 and slow[0] == 0
    for a, b in zip(fast[1:], slow[1:]):
        assert torch.equal(a, b)


def test_outputs_do_not_write_outside_their_extent():
    rows, hidden = 45, 768
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, torch.float16, 13
    )
    pad = 256
    sentinel = 1234.5

    def guarded(count, dtype=torch.float32):
        storage = torch.full((count + 2 * pad,), sentinel, dtype=dtype, device="cuda")
        return storage, storage[pad:pad + count]

    stores = [guarded(rows * hidden), guarded(rows * hidden), guarded(rows), guarded(rows)]
    mask_store = torch.full((rows * hidden // 32 + 2 * pad,), 0x5A5A5A5A, dtype=torch.int32,
                            device="cuda")
    outputs = (
        stores[0][1].view(rows, hidden), stores[1][1].view(rows, hidden), stores[2][1],
        stores[3][1], mask_store[pad:pad + rows * hidden // 32],
    )
    status, *_ = cabi.forward(x, branch, weight, bias, 0.1, 1e-5, True, outputs=outputs)
    assert status == 0
    torch.cuda.synchronize()
    for storage, _ in stores:
        assert (storage[:pad] == sentinel).all() and (storage[-pad:] == sentinel).all()
    assert (mask_store[:pad] == 0x5A5A5A5A).all() and (mask_store[-pad:] == 0x5A5A5A5A).all()


def test_c_abi_rejects_bad_arguments_on_device():
    x, branch, weight, bias, _, _ = draw_inputs((4,), 128, torch.float16, 1)
    status, *_ = cabi.forward(x, branch, weight, bias, 1.0, 1e-5, True)
    assert status == -4
    status, *_ = cabi.forward(x, branch, weight, bias, 0.1, 0.0, True)
    assert status == -5
    _, updated, _, mean, rstd, mask = cabi.forward(x, branch, weight, bias, 0.0, 1e-5, True)
    lib = cabi.library()
    needed = lib.rln_sm100_backward_workspace_bytes(4, 128, 1)
    assert needed > 0
    import ctypes
    status = lib.rln_sm100_backward(
        updated.data_ptr(), updated.data_ptr(), updated.data_ptr(), weight.data_ptr(),
        mean.data_ptr(), rstd.data_ptr(), None, torch.empty_like(updated).data_ptr(),
        torch.empty_like(branch).data_ptr(), torch.empty(2, 128, device="cuda").data_ptr(),
        None, 0, 4, 128, 1, 0, 0, 0.0, 1,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert status == -7


@pytest.mark.parametrize("hidden,branch_dtype", [(128, torch.float32), (768, torch.float16),
                                                 (1024, torch.float16), (256, torch.bfloat16),
                                                 (768, torch.bfloat16)])
def test_cuda_path_matches_the_scalar_c_oracle(hidden, branch_dtype):
    """Independent second oracle: ``oracle/rln_oracle.c`` walks the reference
    kernels' formulas one element at a time."""
    from oracle import c_oracle

    rows, p, eps, seed, offset, row_base = 29, 0.15, 1e-5, 21, 4, 1 << 33
    x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
        (rows,), hidden, branch_dtype, 31
    )
    half = cabi.BRANCH_CODES[branch_dtype]   # the C oracle's branch kind
    status, updated, normalized, mean, rstd, mask = cabi.forward(
        x, branch, weight, bias, p, eps, True, seed=seed, offset=offset, row_base=row_base
    )
    assert status == 0
    keep, words = c_oracle.keep_mask(rows, hidden, p, seed, offset, row_base)
    assert np.array_equal(mask.cpu().numpy(), words)
    expected = c_oracle.forward(
        x.cpu().numpy(), branch.float().cpu().numpy(), weight.cpu().numpy(), bias.cpu().numpy(),
        keep, p, eps, half,
    )
    assert np.array_equal(updated.cpu().numpy(), expected[0])
    np.testing.assert_allclose(normalized.cpu().numpy(), expected[1], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(mean.cpu().numpy(), expected[2], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(rstd.cpu().numpy(), expected[3], rtol=1e-5, atol=0)
    status, grad_x, grad_branch, grad_parameters = cabi.backward(
        grad_updated, grad_normalized, updated, weight, mean, rstd, mask, p, True,
        branch_dtype, True,
    )
    assert status == 0
    reference = c_oracle.backward(
        grad_updated.cpu().numpy(), grad_normalized.cpu().numpy(), updated.cpu().numpy(),
        weight.cpu().numpy(), mean.cpu().numpy(), rstd.cpu().numpy(), keep, p, half,
    )
    np.testing.assert_allclose(grad_x.cpu().numpy(), reference[0], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(
        grad_branch.float().cpu().numpy(), reference[1],
        rtol=grad_branch_tolerance(branch_dtype)["rtol"], atol=1e-5,
    )
    np.testing.assert_allclose(grad_parameters[0].cpu().numpy(), reference[2], rtol=1e-4, atol=5e-5)
    np.testing.assert_allclose(grad_parameters[1].cpu().numpy(), reference[3], rtol=1e-4, atol=5e-5)
