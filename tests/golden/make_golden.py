"""Generate the golden fixtures of this directory from the reference project.

Run where the reference tree (T-vaccari/gfx1010-kernels) is available:

    python tests/golden/make_golden.py --reference /path/to/reference

What is recorded, per case, in ``rln_cases.npz``:

* the inputs (x, branch, weight, bias, upstream gradients), drawn from
  ``torch.Generator().manual_seed(seed)`` in the order x, branch, weight, bias,
  grad_updated, grad_normalized;
* the packed keep mask for the case's Philox (seed, offset), produced by the
  oracle's statement of the kernel's counter layout;
* the outputs of the REFERENCE's own ``_torch_residual_layer_norm``
  (``gfx1010_kernels/normalization.py:15-33``) on CPU, with its ``F.dropout``
  replaced by a dropout that applies that mask and rounds once to the branch
  dtype (the native kernel's rule, ``csrc/residual_layer_norm_kernel.hip:491-497``),
  and the gradients torch autograd derives through that function.

``philox_kat.json`` holds the Random123 known-answer vectors for
Philox4x32-10 (counter, key -> output), which pin the generator itself.

The fixtures are read by the CPU tests (oracle vs fixtures) and by the GPU
tests (CUDA path vs fixtures); nothing at test time needs the reference tree.
"""

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import rln_oracle  # noqa: E402


CASES = (
    # name, rows-shape, hidden, branch dtype, p, eps, training, seed, philox seed, philox offset
    ("h128_half_p10", (5,), 128, "float16", 0.10, 1e-5, True, 0, 0, 0),
    ("h256_float_p15", (2, 3), 256, "float32", 0.15, 1e-5, True, 1, 1234, 8),
    ("h384_half_eval", (7,), 384, "float16", 0.80, 1e-5, False, 2, 0, 0),
    ("h512_half_p0", (3,), 512, "float16", 0.0, 1e-3, True, 3, 0, 0),
    ("h768_half_p10", (2, 2), 768, "float16", 0.10, 1e-5, True, 4, 0xDEADBEEFCAFE, 4),
    ("h1024_float_p25", (3,), 1024, "float32", 0.25, 1e-5, True, 5, 7, 1 << 33),
    # bfloat16 branch (an addition of the sm_100a build; the reference's own
    # decomposition handles it through torch's type promotion)
    ("h768_bfloat16_p10", (4,), 768, "bfloat16", 0.10, 1e-5, True, 6, 99, 12),
    # `normalized` stored in a 16-bit type (another addition; trailing field).
    # The reference function runs unchanged; this script casts its float32
    # `normalized` once and sends the 16-bit upstream gradient back through
    # that cast, which is what the native kernels do on store / load.
    ("h768_half_p10_bf16norm", (6,), 768, "float16", 0.10, 1e-5, True, 7, 5, 16, "bfloat16"),
    ("h256_bfloat16_p20_f16norm", (3,), 256, "bfloat16", 0.20, 1e-5, True, 8, 11, 0, "float16"),
    ("h1024_float_eval_bf16norm", (5,), 1024, "float32", 0.30, 1e-5, False, 9, 0, 0, "bfloat16"),
)


def unpack_case(case):
    """The ten base fields plus the optional ``normalized`` dtype name."""
    base = case[:10]
    normalized_dtype = case[10] if len(case) > 10 else "float32"
    return (*base, normalized_dtype)

PHILOX_KAT = (
    # Random123 kat_vectors, philox4x32 with 10 rounds
    {"counter": [0, 0, 0, 0], "key": [0, 0],
     "output": [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]},
    {"counter": [0xFFFFFFFF] * 4, "key": [0xFFFFFFFF] * 2,
     "output": [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]},
    {"counter": [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344],
     "key": [0xA4093822, 0x299F31D0],
     "output": [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]},
)


def draw_inputs(shape, hidden, branch_dtype, seed):
    generator = torch.Generator().manual_seed(seed)
    full = (*shape, hidden)
    x = torch.randn(full, generator=generator)
    branch = torch.randn(full, generator=generator).to(getattr(torch, branch_dtype))
    weight = 1.0 + 0.1 * torch.randn(hidden, generator=generator)
    bias = 0.1 * torch.randn(hidden, generator=generator)
    grad_updated = torch.randn(full, generator=generator)
    grad_normalized = torch.randn(full, generator=generator)
    return x, branch, weight, bias, grad_updated, grad_normalized


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference project")
    arguments = parser.parse_args()
    sys.path.insert(0, arguments.reference)
    import gfx1010_kernels.normalization as reference  # the reference package

    arrays = {}
    names = []
    for case in CASES:
        (name, shape, hidden, branch_dtype, p, eps, training, seed, pseed, poffset,
         normalized_dtype) = unpack_case(case)
        x, branch, weight, bias, grad_updated, grad_normalized = draw_inputs(
            shape, hidden, branch_dtype, seed
        )
        rows = x.numel() // hidden
        active = training and p > 0.0
        keep = rln_oracle.dropout_keep(rows, hidden, p, pseed, poffset) if active else None

        def masked(tensor, probability, train):
            assert train and active
            return rln_oracle.masked_dropout(
                tensor, torch.from_numpy(keep).reshape(tensor.shape), probability
            )

        original = reference.F.dropout
        reference.F.dropout = masked if active else original
        try:
            leaves = [
                t.detach().clone().requires_grad_(True) for t in (x, branch, weight, bias)
            ]
            updated, normalized = reference._torch_residual_layer_norm(
                *leaves, p, eps, training
            )
            if normalized_dtype != "float32":
                normalized = normalized.to(getattr(torch, normalized_dtype))
                grad_normalized = grad_normalized.to(normalized.dtype)
            grads = torch.autograd.grad(
                (updated, normalized), leaves, (grad_updated, grad_normalized)
            )
        finally:
            reference.F.dropout = original
        mean, rstd = rln_oracle.row_statistics(updated.detach().double(), eps)
        record = {
            "x": x, "branch": branch, "weight": weight, "bias": bias,
            "grad_updated": grad_updated, "grad_normalized": grad_normalized,
            "updated": updated.detach(), "normalized": normalized.detach(),
            "mean64": mean, "rstd64": rstd,
            "grad_x": grads[0], "grad_branch": grads[1],
            "grad_weight": grads[2], "grad_bias": grads[3],
        }
        for key, tensor in record.items():
            if tensor.dtype == torch.bfloat16 or (
                    key in ("normalized", "grad_normalized") and tensor.dtype == torch.float16):
                tensor = tensor.float()  # exact in fp32; numpy has no bfloat16
            arrays[f"{name}/{key}"] = tensor.numpy()
        arrays[f"{name}/mask"] = (
            rln_oracle.pack_mask(keep) if active else np.zeros(0, dtype=np.int32)
        )
        arrays[f"{name}/config"] = np.array(
            [hidden, rows, p, eps, float(training), float(pseed), float(poffset)],
            dtype=np.float64,
        )
        names.append(name)
    np.savez_compressed(HERE / "rln_cases.npz", **arrays)
    meta = {
        "cases": [
            {
                "name": name, "shape": list(shape), "hidden": hidden,
                "branch_dtype": branch_dtype, "dropout_p": p, "eps": eps,
                "training": training, "input_seed": seed,
                "philox_seed": pseed, "philox_offset": poffset,
                "normalized_dtype": normalized_dtype,
            }
            for (name, shape, hidden, branch_dtype, p, eps, training, seed, pseed, poffset,
                 normalized_dtype) in map(unpack_case, CASES)
        ],
        "torch_version": torch.__version__,
        "reference": "T-vaccari/gfx1010-kernels 0.4.0, "
                     "gfx1010_kernels/normalization.py:_torch_residual_layer_norm on CPU",
    }
    (HERE / "rln_cases.json").write_text(json.dumps(meta, indent=1) + "\n")
    (HERE / "philox_kat.json").write_text(json.dumps(PHILOX_KAT, indent=1) + "\n")
    print("wrote", len(names), "cases")


if __name__ == "__main__":
    main()
