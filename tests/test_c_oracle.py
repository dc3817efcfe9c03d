"""The scalar C restatement (``oracle/rln_oracle.c``) against the same pins as
the numpy/torch oracle: Random123 known answers and the fixtures generated
from the reference's own torch decomposition."""

import numpy as np
import pytest

from oracle import c_oracle, rln_oracle

CASES = ["h128_half_p10", "h256_float_p15", "h384_half_eval", "h512_half_p0",
         "h768_half_p10", "h1024_float_p25", "h768_bfloat16_p10",
         "h768_half_p10_bf16norm", "h256_bfloat16_p20_f16norm", "h1024_float_eval_bf16norm"]
BRANCH_KIND = {"float32": 0, "float16": 1, "bfloat16": 2}
ROUNDING = {"float32": 1e-5, "float16": 2e-3, "bfloat16": 1.6e-2}


def test_c_philox_matches_known_answers(philox_kat):
    for vector in philox_kat:
        out = c_oracle.philox(vector["counter"], vector["key"])
        assert [int(word) for word in out] == vector["output"]


def test_c_mask_equals_numpy_mask_including_64_bit_counters():
    for seed, offset, row_base in ((0, 0, 0), (0xDEADBEEFCAFE, 1 << 33, 0), (7, 4, 1 << 36)):
        keep_c, words_c = c_oracle.keep_mask(9, 256, 0.3, seed, offset, row_base)
        keep_np = rln_oracle.dropout_keep(9, 256, 0.3, seed, offset, row_base)
        assert np.array_equal(keep_c, keep_np)
        assert np.array_equal(words_c, rln_oracle.pack_mask(keep_np))


@pytest.mark.parametrize("name", CASES)
def test_c_oracle_reproduces_reference_fixtures(golden_cases, name):
    case = golden_cases[name]
    meta = case["meta"]
    hidden = meta["hidden"]
    kind = BRANCH_KIND[meta["branch_dtype"]]
    normalized_dtype = meta.get("normalized_dtype", "float32")
    x = case["x"].reshape(-1, hidden)
    rows = x.shape[0]
    active = meta["training"] and meta["dropout_p"] > 0
    keep = None
    if active:
        keep, words = c_oracle.keep_mask(
            rows, hidden, meta["dropout_p"], meta["philox_seed"], meta["philox_offset"]
        )
        assert np.array_equal(words, case["mask"])
    updated, normalized, mean, rstd = c_oracle.forward(
        x, case["branch"].reshape(-1, hidden).astype(np.float32), case["weight"], case["bias"],
        keep, meta["dropout_p"], meta["eps"], kind, BRANCH_KIND[normalized_dtype],
    )
    assert np.array_equal(updated, case["updated"].reshape(-1, hidden))
    # float32: the parity tolerance; 16-bit: two roundings of float32-close
    # values may land on neighbouring representable numbers
    np.testing.assert_allclose(
        normalized, case["normalized"].reshape(-1, hidden),
        rtol=ROUNDING[normalized_dtype], atol=1e-6 if normalized_dtype == "float32" else 1e-4,
    )
    if normalized_dtype != "float32":
        exact = np.mean(normalized == case["normalized"].reshape(-1, hidden))
        assert exact > 0.995, exact
    np.testing.assert_allclose(mean, case["mean64"].reshape(-1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(rstd, case["rstd64"].reshape(-1), rtol=1e-5, atol=0)
    grad_x, grad_branch, grad_weight, grad_bias = c_oracle.backward(
        case["grad_updated"].reshape(-1, hidden), case["grad_normalized"].reshape(-1, hidden),
        updated, case["weight"], mean, rstd, keep, meta["dropout_p"], kind,
    )
    np.testing.assert_allclose(grad_x, case["grad_x"].reshape(-1, hidden), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(
        grad_branch, case["grad_branch"].reshape(-1, hidden).astype(np.float32),
        rtol=ROUNDING[meta["branch_dtype"]], atol=1e-5,
    )
    np.testing.assert_allclose(grad_weight, case["grad_weight"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(grad_bias, case["grad_bias"], rtol=1e-4, atol=1e-5)
