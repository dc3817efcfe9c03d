"""Public residual-add + dropout + LayerNorm operator, eligibility and status.

Host-side mirror of ``gfx1010_kernels/normalization.py`` of the reference
(T-vaccari/gfx1010-kernels): ``residual_layer_norm`` (:149-298),
``can_use_residual_layer_norm`` (:135-146), ``residual_layer_norm_status``
(:75-94), ``_input_reason`` (:97-132), ``_native_status`` (:41-72) and the torch
decomposition ``_torch_residual_layer_norm`` (:15-33).  Call signatures, return
values, warning and error texts are kept; the route name ``"gfx1010"`` still
selects the native kernels, which are now sm_100a CUDA.

Differences, all forced by the hardware change:

* the capability gate asks for a CUDA device of compute capability 10.x and an
  importable ``_C`` extension instead of ROCm + gfx1010;
* a bfloat16 branch is accepted in addition to float16 / float32;
* ``normalized_dtype`` (keyword-only, default ``None`` = float32, the
  reference's output type) lets ``normalized`` be stored as float16 or bfloat16
  for a consumer that feeds it to a half-precision GEMM;
* ``implementation="triton"`` is always reported unavailable (there is no
  Triton route in this build);
* in ``"auto"`` mode, eligible tensors on an sm_100 device never fall back to
  the torch decomposition when the extension cannot be imported -- that is an
  installation error and raises.  Other fallbacks of ``"auto"`` (CPU tensors,
  unsupported shapes or dtypes, a GPU that is not sm_100) warn and use the
  torch decomposition exactly as the reference does.
"""

from functools import lru_cache
import warnings

import torch
from torch.nn import functional as F

from ._status import BackendStatus


MIN_HIDDEN_SIZE = 128
MAX_HIDDEN_SIZE = 1024
NATIVE_HIDDEN_SIZES = (128, 256, 384, 512, 768, 1024)
# The build emits sm_100a code only, and architecture-specific ("a") targets run
# on exactly that compute capability: 10.0 (B200), not on other 10.x parts.
NATIVE_COMPUTE_CAPABILITY = (10, 0)
NATIVE_COMPUTE_CAPABILITY_MAJOR = NATIVE_COMPUTE_CAPABILITY[0]
# float16 / float32 are the reference's branch types; bfloat16 is accepted in
# addition (the sm_100a kernels have it, the gfx1010 ones could not).
NATIVE_BRANCH_DTYPES = (torch.float16, torch.float32, torch.bfloat16)

_IMPLEMENTATIONS = ("auto", "gfx1010", "triton", "torch")
_NO_CUDA = "PyTorch CUDA/HIP is unavailable"
_FORCED_PREFIX = "gfx1010 native residual LayerNorm is unavailable: "


def _torch_residual_layer_norm(x, branch, weight, bias, dropout_p, eps, training,
                               normalized_dtype=None):
    """dropout -> residual add -> LayerNorm with stock torch ops (reference :15-33).

    ``normalized_dtype`` (not in the reference) casts ``normalized`` at the end,
    which is what the native kernels do on store.
    """
    if training:
        branch = F.dropout(branch, dropout_p, True)
    updated = x + branch
    normalized = F.layer_norm(updated, updated.shape[-1:], weight, bias, eps)
    if normalized_dtype is not None and normalized.dtype != normalized_dtype:
        normalized = normalized.to(normalized_dtype)
    return updated, normalized


@lru_cache(maxsize=None)
def _triton_is_usable(device_index):
    """Status of the Triton route (reference :36-38); never available here."""
    return BackendStatus(
        False,
        None,
        None,
        "the Triton implementation is not part of the sm_100a build",
    )


@lru_cache(maxsize=None)
def _native_status(device_index):
    """Capability probe for one CUDA device, cached (reference :41-72)."""
    if not torch.cuda.is_available():
        return BackendStatus(False, None, None, _NO_CUDA)
    name = torch.cuda.get_device_name(device_index)
    major, minor = torch.cuda.get_device_capability(device_index)
    architecture = f"sm_{major}{minor}"
    if (major, minor) != NATIVE_COMPUTE_CAPABILITY:
        return BackendStatus(
            False,
            name,
            architecture,
            "the native extension targets sm_100 (B200)",
        )
    from ._normalization_native import native_extension_status

    available, reason = native_extension_status()
    if available:
        reason = "sm_100 native normalization backend is ready"
    return BackendStatus(available, name, architecture, reason)


def residual_layer_norm_status(device=None):
    """Whether the native kernels can run on ``device`` (default: current device)."""
    if not torch.cuda.is_available():
        return BackendStatus(False, None, None, _NO_CUDA)
    if device is None:
        return _native_status(torch.cuda.current_device())
    resolved = torch.device(device)
    if resolved.type != "cuda":
        return BackendStatus(False, str(resolved), None, "the device must be a HIP GPU")
    if resolved.index is None:
        return _native_status(torch.cuda.current_device())
    return _native_status(resolved.index)


def allow_graph_capture(enabled=True):
    """Let the native dropout be recorded into a CUDA graph.

    Off by default: like the reference (``csrc/residual_layer_norm_kernel.hip:1758-1777``)
    the native route then raises "... does not support HIP graph capture" when
    called with active dropout while a stream is capturing.  When enabled, the
    forward takes torch's graph-safe generator state by pointer, so every
    replay draws the mask for the generator's state at replay time (replaying
    after ``torch.cuda.manual_seed(s)`` gives the mask an eager call with the
    same seed gives).  Returns the previous setting.
    """
    from ._normalization_native import _extension

    extension, reason = _extension()
    if extension is None:
        raise RuntimeError(f"gfx1010 native extension is unavailable: {reason}")
    previous = extension.graph_capture_allowed()
    extension.set_graph_capture_allowed(bool(enabled))
    return previous


def _input_reason(x, branch, weight, bias, dropout_p, eps):
    """First reason the optimised routes cannot take these inputs, else None.

    Same checks, order and texts as the reference (:97-132).
    """
    if not x.is_cuda:
        return "x must be a HIP tensor"
    others = (branch, weight, bias)
    if not all(tensor.is_cuda for tensor in others):
        return "x, branch, weight and bias must be HIP tensors"
    if any(tensor.device != x.device for tensor in others):
        return "x, branch, weight and bias must be on the same device"
    if x.ndim < 2 or branch.shape != x.shape:
        return "x and branch must have the same shape with at least two dimensions"
    hidden_size = x.shape[-1]
    if hidden_size < MIN_HIDDEN_SIZE or hidden_size > MAX_HIDDEN_SIZE:
        return f"hidden size must be between {MIN_HIDDEN_SIZE} and {MAX_HIDDEN_SIZE}"
    if hidden_size % 8:
        return "hidden size must be divisible by 8"
    if tuple(weight.shape) != (hidden_size,) or tuple(bias.shape) != (hidden_size,):
        return "weight and bias must match the final tensor dimension"
    if x.dtype != torch.float32:
        return "the optimized residual stream requires float32 x"
    if branch.dtype not in NATIVE_BRANCH_DTYPES:
        return "branch must use float16 or float32"
    if weight.dtype != torch.float32 or bias.dtype != torch.float32:
        return "weight and bias must use float32"
    if not (
        x.is_contiguous()
        and branch.is_contiguous()
        and weight.is_contiguous()
        and bias.is_contiguous()
    ):
        return "x, branch, weight and bias must be contiguous"
    if not 0.0 <= dropout_p < 1.0:
        return "dropout_p must be in [0, 1)"
    if eps <= 0.0:
        return "eps must be positive"
    if x.numel() == 0:
        return "empty tensors use the PyTorch fallback"
    return None


def can_use_residual_layer_norm(x, branch, weight, bias, dropout_p=0.0, eps=1e-5):
    """True when ``residual_layer_norm(..., implementation="auto")`` runs natively."""
    if _input_reason(x, branch, weight, bias, dropout_p, eps) is not None:
        return False
    if x.shape[-1] not in NATIVE_HIDDEN_SIZES:
        return False
    return residual_layer_norm_status(x.device).available


def _warn_and_decompose(message, x, branch, weight, bias, dropout_p, eps, training,
                        normalized_dtype=None):
    warnings.warn(message, RuntimeWarning, stacklevel=3)
    return _torch_residual_layer_norm(
        x, branch, weight, bias, dropout_p, eps, training, normalized_dtype
    )


def residual_layer_norm(
    x,
    branch,
    weight,
    bias,
    dropout_p=0.0,
    eps=1e-5,
    training=True,
    *,
    implementation="auto",
    normalized_dtype=None,
):
    """``updated = x + dropout(branch)``; ``normalized = LayerNorm(updated)``.

    Returns ``(updated, normalized)``, both float32 with the shape of ``x``,
    differentiable to first order with respect to ``x``, ``branch``, ``weight``
    and ``bias``.

    ``normalized_dtype`` (an addition to the reference's signature): ``None`` or
    ``torch.float32`` keeps the contract above; ``torch.float16`` /
    ``torch.bfloat16`` return ``normalized`` in that type -- the float32 result
    rounded once -- and its gradient arrives in that type, so the operator
    moves 4 bytes less per element over forward + backward.  On the native
    route this needs 16-byte aligned tensors (what torch allocates).

    ``implementation``:
      ``"torch"``    the decomposition with stock torch ops (any device);
      ``"gfx1010"``  the native kernels, or ``RuntimeError`` saying why not.
                     Only ``x.is_cuda``, ``x.ndim`` and ``x.shape[-1]`` are
                     inspected in Python, and before any backend lookup; the
                     extension validates everything else;
      ``"auto"``     the native kernels when inputs and device qualify, else a
                     ``RuntimeWarning`` ("... was not used: <reason>") and the
                     decomposition;
      ``"triton"``   unavailable in this build (``RuntimeError``).
    """
    if implementation not in _IMPLEMENTATIONS:
        raise ValueError("implementation must be 'auto', 'gfx1010', 'triton' or 'torch'")
    if normalized_dtype is not None:
        from ._normalization_native import normalized_dtype_code

        normalized_dtype_code(normalized_dtype)  # ValueError for anything else

    if implementation == "torch":
        return _torch_residual_layer_norm(
            x, branch, weight, bias, dropout_p, eps, training, normalized_dtype
        )

    if implementation == "gfx1010":
        # Forced hot path: three duck-typed checks, then straight to the extension.
        if not x.is_cuda:
            raise RuntimeError(_FORCED_PREFIX + "x must be a HIP tensor")
        if x.ndim == 0:
            raise RuntimeError(_FORCED_PREFIX + "x must have at least two dimensions")
        if x.shape[-1] not in NATIVE_HIDDEN_SIZES:
            raise RuntimeError(
                _FORCED_PREFIX + f"native hidden size must be one of {NATIVE_HIDDEN_SIZES}"
            )
        status = residual_layer_norm_status(x.device)
        if not status.available:
            raise RuntimeError(_FORCED_PREFIX + status.reason)
        from ._normalization_native import native_residual_layer_norm

        return native_residual_layer_norm(
            x, branch, weight, bias, float(dropout_p), float(eps), bool(training),
            normalized_dtype,
        )

    reason = _input_reason(x, branch, weight, bias, dropout_p, eps)

    if implementation == "triton":
        if reason is None:
            index = x.device.index
            if index is None:
                index = torch.cuda.current_device()
            reason = _triton_is_usable(index).reason
        raise RuntimeError(f"gfx1010 residual LayerNorm is unavailable: {reason}")

    # implementation == "auto"
    if reason is not None:
        return _warn_and_decompose(
            f"gfx1010 optimized residual LayerNorm was not used: {reason}",
            x, branch, weight, bias, dropout_p, eps, training, normalized_dtype,
        )
    if x.shape[-1] not in NATIVE_HIDDEN_SIZES:
        native_reason = f"native hidden size must be one of {NATIVE_HIDDEN_SIZES}"
    else:
        status = residual_layer_norm_status(x.device)
        if status.available:
            from ._normalization_native import native_residual_layer_norm

            with torch.cuda.device(x.device):
                return native_residual_layer_norm(
                    x, branch, weight, bias, float(dropout_p), float(eps), bool(training),
                    normalized_dtype,
                )
        if status.architecture == f"sm_{NATIVE_COMPUTE_CAPABILITY_MAJOR}0":
            # An sm_100 device without a loadable extension is a broken
            # installation, not a reason to run something else silently.
            raise RuntimeError(_FORCED_PREFIX + status.reason)
        native_reason = status.reason
    return _warn_and_decompose(
        f"gfx1010 native residual LayerNorm was not used: {native_reason}",
        x, branch, weight, bias, dropout_p, eps, training, normalized_dtype,
    )
