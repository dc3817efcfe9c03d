"""Module form of the operator for pre-norm transformer blocks.

The reference documents the integration pattern (``docs/residual_layer_norm.md:51-83``
of T-vaccari/gfx1010-kernels): keep the block's ``nn.LayerNorm`` module, so that
``state_dict`` keys do not change, and replace

    x = x + dropout(branch); h = ln(x)

by ``x, h = residual_layer_norm(x, branch, ln.weight, ln.bias, p, ln.eps, training)``.
``ResidualLayerNorm`` packages exactly that: it *is* an ``nn.LayerNorm`` (same
parameters, same ``state_dict`` keys ``weight`` / ``bias``, loadable from and
into a plain LayerNorm checkpoint) whose ``forward`` takes the residual stream
and the branch output and returns ``(updated, normalized)``.  Because weight and
bias are ordinary parameters reached through autograd, ``DistributedDataParallel``
buckets their gradients with the rest of the model and all-reduces them in its
own backward hook; that hook is the data-parallel exchange of this module and
nothing extra is needed (checked on two gloo ranks against the single-process
gradients in ``tests/test_modules_ddp_cpu.py``).  Callers that drive the raw
step themselves use ``gfx1010_kernels.sharded`` instead.
"""

import torch
from torch import nn

from .normalization import NATIVE_HIDDEN_SIZES, residual_layer_norm


class ResidualLayerNorm(nn.LayerNorm):
    """``updated = x + dropout(branch)``; ``normalized = LayerNorm(updated)``.

    ``hidden_size`` must be the size of the last dimension; the native kernels
    cover ``NATIVE_HIDDEN_SIZES`` and ``implementation="auto"`` falls back to
    the torch decomposition (with a warning) elsewhere.
    """

    def __init__(self, hidden_size, dropout_p=0.0, eps=1e-5, implementation="auto",
                 device=None, dtype=torch.float32, normalized_dtype=None):
        if isinstance(hidden_size, (tuple, list, torch.Size)):
            if len(hidden_size) != 1:
                raise ValueError("ResidualLayerNorm normalises over the last dimension only")
            hidden_size = hidden_size[0]
        super().__init__(int(hidden_size), eps=eps, elementwise_affine=True, bias=True,
                         device=device, dtype=dtype)
        if not 0.0 <= dropout_p < 1.0:
            raise ValueError("dropout_p must be in [0, 1)")
        self.dropout_p = float(dropout_p)
        self.implementation = implementation
        # None = float32; torch.bfloat16 / torch.float16 hand the following GEMM
        # a half-precision activation without a separate cast kernel
        self.normalized_dtype = normalized_dtype

    @classmethod
    def from_layer_norm(cls, layer_norm, dropout_p=0.0, implementation="auto",
                        normalized_dtype=None):
        """Wrap an existing ``nn.LayerNorm`` of a model: the new module SHARES its
        ``weight`` and ``bias`` parameters (same tensors, so the optimiser state,
        the checkpoint keys of the original module and tied references stay
        valid) and takes over its ``eps``.  The layer must normalise over the
        last dimension only and have an affine weight and bias."""
        if not isinstance(layer_norm, nn.LayerNorm):
            raise TypeError("from_layer_norm expects an nn.LayerNorm")
        if len(layer_norm.normalized_shape) != 1:
            raise ValueError("ResidualLayerNorm normalises over the last dimension only")
        if layer_norm.weight is None or layer_norm.bias is None:
            raise ValueError("the LayerNorm must have an affine weight and bias")
        module = cls(layer_norm.normalized_shape[0], dropout_p=dropout_p, eps=layer_norm.eps,
                     implementation=implementation, device=layer_norm.weight.device,
                     dtype=layer_norm.weight.dtype, normalized_dtype=normalized_dtype)
        module.weight = layer_norm.weight
        module.bias = layer_norm.bias
        module.train(layer_norm.training)
        return module

    @property
    def native_width(self):
        return self.normalized_shape[0] in NATIVE_HIDDEN_SIZES

    def forward(self, x, branch):  # noqa: D102 - see the class docstring
        return residual_layer_norm(
            x, branch, self.weight, self.bias, self.dropout_p, self.eps, self.training,
            implementation=self.implementation, normalized_dtype=self.normalized_dtype,
        )

    def extra_repr(self):
        text = (f"{self.normalized_shape[0]}, eps={self.eps}, dropout_p={self.dropout_p}, "
                f"implementation={self.implementation!r}")
        if self.normalized_dtype is not None:
            text += f", normalized_dtype={self.normalized_dtype}"
        return text
