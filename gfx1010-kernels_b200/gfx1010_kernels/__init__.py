"""B200 (sm_100a) build of the gfx1010_kernels residual LayerNorm path.

Drop-in for the residual-add + dropout + LayerNorm surface of
T-vaccari/gfx1010-kernels (``gfx1010_kernels/__init__.py:15-19``): the same
three public callables and the ``BackendStatus`` record, backed by hand-written
sm_100a CUDA kernels instead of the gfx1010 HIP extension.  The reference's
attention, patching and linear helpers are separate operators and are not
provided here.
"""

from ._status import BackendStatus
from .normalization import (
    allow_graph_capture,
    can_use_residual_layer_norm,
    residual_layer_norm,
    residual_layer_norm_status,
)

__version__ = "0.4.0"

__all__ = [
    "__version__",
    "BackendStatus",
    "allow_graph_capture",
    "can_use_residual_layer_norm",
    "residual_layer_norm",
    "residual_layer_norm_status",
]
