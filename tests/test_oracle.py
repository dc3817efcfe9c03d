"""The oracle against its pins: Random123 known-answer vectors for the
generator, and the golden fixtures produced by the reference's own
``_torch_residual_layer_norm`` (see ``tests/golden/make_golden.py``)."""

import numpy as np
import pytest
import torch

from conftest import golden_tensors
from oracle import rln_oracle


def test_philox_matches_random123_known_answers(philox_kat):
    for vector in philox_kat:
        actual = rln_oracle.philox4x32_10(
            np.array(vector["counter"], dtype=np.uint64), vector["key"]
        )
        assert [int(word) for word in actual] == vector["output"]


def test_philox_is_vectorised_consistently():
    counters = np.arange(64, dtype=np.uint64).reshape(16, 4) * np.uint64(0x01234567)
    counters &= np.uint64(0xFFFFFFFF)
    batched = rln_oracle.philox4x32_10(counters, (3, 5))
    for index in range(16):
        single = rln_oracle.philox4x32_10(counters[index], (3, 5))
        assert np.array_equal(batched[index], single)


def test_threshold_and_scale_follow_the_reference_rule():
    # uint32(double(float32(p)) * 2**32) and fp32 1/(1-p)
    assert rln_oracle.dropout_threshold(0.0) == 0
    assert rln_oracle.dropout_threshold(0.5) == 1 << 31
    assert rln_oracle.dropout_threshold(0.1) == int(float(np.float32(0.1)) * 2.0**32)
    assert rln_oracle.dropout_scale(0.5) == np.float32(2.0)
    assert rln_oracle.dropout_scale(0.1).dtype == np.float32


def test_mask_pack_layout_and_round_trip():
    rng = np.random.default_rng(0)
    keep = rng.random((7, 256)) < 0.8
    words = rln_oracle.pack_mask(keep)
    assert words.dtype == np.int32 and words.shape == (7 * 8,)
    # bit (col & 31) of word row*(H/32) + col/32
    unsigned = words.view(np.uint32)
    for row, col in ((0, 0), (3, 31), (3, 32), (6, 255), (5, 100)):
        bit = (unsigned[row * 8 + col // 32] >> (col & 31)) & 1
        assert bool(bit) == bool(keep[row, col])
    assert np.array_equal(rln_oracle.unpack_mask(words, 7, 256), keep)


def test_keep_mask_is_shard_invariant_and_offset_sensitive():
    full = rln_oracle.dropout_keep(12, 128, 0.3, seed=9, offset=4)
    tail = rln_oracle.dropout_keep(5, 128, 0.3, seed=9, offset=4, row_base=7)
    assert np.array_equal(full[7:], tail)
    other = rln_oracle.dropout_keep(12, 128, 0.3, seed=9, offset=8)
    assert not np.array_equal(full, other)
    big = rln_oracle.dropout_keep(1, 128, 0.3, seed=9, offset=4, row_base=(1 << 40))
    assert big.shape == (1, 128)


def test_offset_counts_words_and_one_call_uses_one_philox_block():
    """The offset is in 32-bit words (torch's generator convention); a Philox call
    yields four, so the counter holds offset // 4: offsets inside one block give
    the same words, the next block gives others, and the words of element group
    g at offset o are exactly Philox(counter = (o // 4, g), key = seed) -- the
    block a later consumer starting at o + 4 can never produce again."""
    rows, hidden, seed = 3, 128, 77
    base = rln_oracle.dropout_random_words(rows, hidden, seed, 8)
    assert np.array_equal(base, rln_oracle.dropout_random_words(rows, hidden, seed, 11))
    assert not np.array_equal(base, rln_oracle.dropout_random_words(rows, hidden, seed, 12))
    big = (1 << 35) + 40
    words = rln_oracle.dropout_random_words(rows, hidden, seed, big, row_base=5)
    group = 5 * (hidden // 4) + 7                      # row 0, columns 28..31
    counter = np.array([[(big >> 2) & 0xFFFFFFFF, (big >> 2) >> 32, group, 0]], dtype=np.uint64)
    expected = rln_oracle.philox4x32_10(counter, (seed, 0)).reshape(-1)
    assert np.array_equal(words[0, 28:32], expected.astype(words.dtype))


def test_kept_fraction_is_within_four_sigma():
    p = 0.1
    keep = rln_oracle.dropout_keep(512, 768, p, seed=0, offset=0)
    n = keep.size
    sigma = (p * (1 - p) / n) ** 0.5
    assert abs(keep.mean() - (1 - p)) < 4 * sigma


@pytest.mark.parametrize(
    "name",
    [
        "h128_half_p10",
        "h256_float_p15",
        "h384_half_eval",
        "h512_half_p0",
        "h768_half_p10",
        "h1024_float_p25",
        "h768_bfloat16_p10",
        "h768_half_p10_bf16norm",
        "h256_bfloat16_p20_f16norm",
        "h1024_float_eval_bf16norm",
    ],
)
def test_oracle_reproduces_reference_fixtures(golden_cases, name):
    case = golden_cases[name]
    meta = case["meta"]
    tensors = golden_tensors(case)
    hidden = meta["hidden"]
    rows = tensors["x"].numel() // hidden
    active = meta["training"] and meta["dropout_p"] > 0
    keep = None
    if active:
        keep = rln_oracle.dropout_keep(
            rows, hidden, meta["dropout_p"], meta["philox_seed"], meta["philox_offset"]
        )
        assert np.array_equal(rln_oracle.pack_mask(keep), case["mask"])
        keep = torch.from_numpy(keep)
    result = rln_oracle.decomposition_gradients(
        tensors["x"], tensors["branch"], tensors["weight"], tensors["bias"],
        tensors["grad_updated"], tensors["grad_normalized"],
        meta["dropout_p"], meta["eps"], meta["training"], keep,
        normalized_dtype=tensors["normalized"].dtype,
    )
    names = ("updated", "normalized", "grad_x", "grad_branch", "grad_weight", "grad_bias")
    for key, actual in zip(names, result):
        # same torch ops on the same machine class: bit-exact
        assert torch.equal(actual, tensors[key]), key

    # the explicit restatement of the native backward formulas, in fp64,
    # agrees with autograd through the reference decomposition
    mean, rstd = rln_oracle.row_statistics(tensors["updated"].double(), meta["eps"])
    assert torch.allclose(mean, tensors["mean64"], rtol=1e-12, atol=1e-12)
    grad_x, grad_branch, grad_weight, grad_bias = rln_oracle.kernel_backward(
        tensors["grad_updated"], tensors["grad_normalized"], tensors["updated"],
        tensors["weight"], mean, rstd, keep, meta["dropout_p"], active,
        tensors["branch"].dtype,
    )
    arbiter = rln_oracle.decomposition_gradients(
        tensors["x"], tensors["branch"], tensors["weight"], tensors["bias"],
        tensors["grad_updated"], tensors["grad_normalized"],
        meta["dropout_p"], meta["eps"], meta["training"], keep, dtype=torch.float64,
    )
    # the arbiter keeps `updated` unrounded and returns fp32-rounded gradients:
    # agreement is to a few fp32 ulps of the data, not to fp64 precision
    torch.testing.assert_close(grad_x.reshape(arbiter[2].shape), arbiter[2].double(),
                               rtol=2e-6, atol=2e-6)
    torch.testing.assert_close(grad_weight, arbiter[4].double(), rtol=2e-6, atol=2e-6)
    torch.testing.assert_close(grad_bias, arbiter[5].double(), rtol=2e-6, atol=2e-6)
    # one rounding of an fp32-close value to the branch type
    rounding = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2, torch.float32: 1e-5}
    tolerance = rounding[tensors["branch"].dtype]
    torch.testing.assert_close(
        grad_branch.float(), tensors["grad_branch"].float(), rtol=tolerance, atol=tolerance
    )


def test_fp16_rounding_rule_differs_from_stock_cpu_dropout():
    """Why the oracle carries its own masked dropout: rounding once from fp32
    is not what stock fp16 dropout does, so the mask AND the rounding rule must
    both be injected to compare against the kernel."""
    generator = torch.Generator().manual_seed(0)
    branch = torch.randn(64, 128, generator=generator).half()
    keep = torch.ones(64, 128, dtype=torch.bool)
    once = rln_oracle.masked_dropout(branch, keep, 0.1)
    twice = branch * torch.tensor(1.0 / 0.9).half()
    assert (once != twice).any()
    torch.testing.assert_close(once.float(), twice.float(), rtol=2e-3, atol=0)
