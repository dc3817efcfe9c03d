"""Training step over HOST-resident rows: chunked copy-in / compute / copy-out.

``HostPipeline`` drives the ``rln_sm100_host_*`` entry points of
``librln_sm100.so`` (declared in ``include/rln_sm100.h``) through ctypes.  It is
the call to use when activations live in host memory (offloaded or produced on
the CPU): instead of one copy in, the kernels, and one copy out, rows are cut
into chunks and the three stages overlap on separate streams.

The reference project has no host-buffer entry; this module is an addition on
the caller side of the path.  Its results are those of
``_C.residual_layer_norm_forward`` + ``_C.residual_layer_norm_backward`` on the
same rows with the same Philox ``(seed, offset)``.

There is no CPU fallback: without a CUDA device or without the native library
the constructor raises.
"""

import ctypes
from pathlib import Path

import torch

_LIBRARY_PATH = Path(__file__).resolve().parent / "librln_sm100.so"
_library = None

_ptr = ctypes.c_void_p
# RLN_DTYPE_FLOAT32 / FLOAT16 / BFLOAT16 of include/rln_sm100.h (branch and normalized)
_BRANCH_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _load():
    global _library
    if _library is None:
        if not _LIBRARY_PATH.exists():
            raise RuntimeError(f"native kernel library is missing: {_LIBRARY_PATH}")
        lib = ctypes.CDLL(str(_LIBRARY_PATH))
        lib.rln_sm100_status_string.restype = ctypes.c_char_p
        lib.rln_sm100_status_string.argtypes = [ctypes.c_int]
        lib.rln_sm100_host_pipeline_create.restype = ctypes.c_int
        lib.rln_sm100_host_pipeline_create.argtypes = [
            ctypes.POINTER(_ptr), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
            ctypes.c_int64, ctypes.c_int32,
        ]
        lib.rln_sm100_host_pipeline_destroy.restype = ctypes.c_int
        lib.rln_sm100_host_pipeline_destroy.argtypes = [_ptr]
        lib.rln_sm100_host_forward_backward.restype = ctypes.c_int
        lib.rln_sm100_host_forward_backward.argtypes = (
            [_ptr] * 12
            + [ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_float,
               ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int32]
        )
        lib.rln_sm100_host_forward_backward_enqueue.restype = ctypes.c_int
        lib.rln_sm100_host_forward_backward_enqueue.argtypes = \
            lib.rln_sm100_host_forward_backward.argtypes
        lib.rln_sm100_host_pipeline_wait.restype = ctypes.c_int
        lib.rln_sm100_host_pipeline_wait.argtypes = [_ptr]
        lib.rln_sm100_host_pipeline_steps_enqueued.restype = ctypes.c_int64
        lib.rln_sm100_host_pipeline_steps_enqueued.argtypes = [_ptr]
        lib.rln_sm100_host_pipeline_wait_step.restype = ctypes.c_int
        lib.rln_sm100_host_pipeline_wait_step.argtypes = [_ptr, ctypes.c_int64]
        _library = lib
    return _library


def _check(status, what):
    if status != 0:
        text = _load().rln_sm100_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {text}")


def check_output_tensors(out, shape, hidden, normalized_dtype, branch_dtype):
    """Raises unless ``out`` is ``(updated, normalized, grad_x, grad_branch,
    grad_parameters)`` as contiguous HOST tensors of exactly the shapes and types
    the native call fills.  That call copies ``rows * hidden`` elements straight
    into the five pointers, so anything else would be written out of bounds."""
    if not isinstance(out, (tuple, list)) or len(out) != 5:
        raise RuntimeError(
            "out must be (updated, normalized, grad_x, grad_branch, grad_parameters)")
    expected = (
        ("updated", shape, torch.float32),
        ("normalized", shape, normalized_dtype),
        ("grad_x", shape, torch.float32),
        ("grad_branch", shape, branch_dtype),
        ("grad_parameters", (2, hidden), torch.float32),
    )
    for tensor, (name, wanted_shape, dtype) in zip(out, expected):
        if not isinstance(tensor, torch.Tensor) or tensor.is_cuda:
            raise RuntimeError(f"out: {name} must be a host tensor")
        if tensor.dtype != dtype:
            raise RuntimeError(f"out: {name} must use {dtype}")
        if tuple(tensor.shape) != tuple(wanted_shape):
            raise RuntimeError(f"out: {name} must have shape {tuple(wanted_shape)}")
        if not tensor.is_contiguous():
            raise RuntimeError(f"out: {name} must be contiguous")


class HostPipeline:
    """Device staging buffers, streams and events for one (hidden, branch dtype,
    normalized dtype).

    ``chunk_rows`` rows are in flight per stage and ``depth`` chunks are
    buffered (device memory: about ``depth * chunk_rows * hidden * 30`` bytes).
    ``normalized_dtype`` is the type of ``normalized`` and ``grad_normalized``
    (float32 by default; float16 / bfloat16 move 2 bytes less per element in
    each direction over the PCIe link that bounds this step).
    One call at a time per pipeline.
    """

    def __init__(self, hidden, branch_dtype=torch.float16, chunk_rows=8192, depth=3, device=None,
                 normalized_dtype=torch.float32):
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device; there is no CPU fallback")
        if branch_dtype not in _BRANCH_CODES:
            raise ValueError("branch must use float16, bfloat16 or float32")
        if normalized_dtype not in _BRANCH_CODES:
            raise ValueError("normalized must use float16, bfloat16 or float32")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.hidden = int(hidden)
        self.branch_dtype = branch_dtype
        self.normalized_dtype = normalized_dtype
        self.chunk_rows = int(chunk_rows)
        self.depth = int(depth)
        self._handle = _ptr()
        self._in_flight = []
        with torch.cuda.device(self.device):
            torch.cuda.current_stream()  # make sure the device's context exists
            status = _load().rln_sm100_host_pipeline_create(
                ctypes.byref(self._handle), self.hidden,
                _BRANCH_CODES[branch_dtype], _BRANCH_CODES[normalized_dtype],
                self.chunk_rows, self.depth,
            )
        _check(status, "rln_sm100_host_pipeline_create")

    def close(self):
        if getattr(self, "_handle", None):
            with torch.cuda.device(self.device):
                _load().rln_sm100_host_pipeline_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def allocate_outputs(self, shape, pinned=True):
        """Host tensors for ``(updated, normalized, grad_x, grad_branch, grad_parameters)``."""
        def host(size, dtype):
            return torch.empty(size, dtype=dtype, pin_memory=pinned)

        return (
            host(shape, torch.float32),
            host(shape, self.normalized_dtype),
            host(shape, torch.float32),
            host(shape, self.branch_dtype),
            host((2, self.hidden), torch.float32),
        )

    def forward_backward(
        self,
        x,
        branch,
        weight,
        bias,
        grad_updated,
        grad_normalized,
        dropout_p=0.0,
        eps=1e-5,
        training=True,
        *,
        seed=0,
        offset=0,
        row_base=0,
        deterministic=False,
        out=None,
        wait=True,
    ):
        """One forward + backward over host tensors.

        Returns ``(updated, normalized, grad_x, grad_branch, grad_parameters)``
        as host tensors (``out`` is filled and returned when given);
        ``grad_parameters[0]`` is grad_weight and ``[1]`` is grad_bias.

        ``wait=False`` only enqueues the step and returns the (not yet filled)
        output tensors; ``wait()`` returns once every enqueued step has landed.
        Steps enqueued back to back overlap -- the next step's first chunks are
        copied in while this step's last chunks are computed and copied out --
        which removes the idle chunk at both ends of a lone step.  Until
        ``wait()`` has returned, do not touch any tensor of an enqueued step
        (inputs included) and give steps in flight separate ``out`` tensors.
        """
        if self._handle is None:
            raise RuntimeError("the pipeline is closed")
        tensors = (x, branch, weight, bias, grad_updated, grad_normalized)
        if any(t.is_cuda for t in tensors):
            raise RuntimeError("HostPipeline takes host tensors; use residual_layer_norm for device tensors")
        if x.dtype != torch.float32 or grad_updated.dtype != torch.float32:
            raise RuntimeError("x and grad_updated must use float32")
        if grad_normalized.dtype != self.normalized_dtype:
            raise RuntimeError(f"grad_normalized must use {self.normalized_dtype}")
        if branch.dtype != self.branch_dtype:
            raise RuntimeError(f"branch must use {self.branch_dtype}")
        if weight.dtype != torch.float32 or bias.dtype != torch.float32:
            raise RuntimeError("weight and bias must use float32")
        if x.ndim < 2 or x.shape[-1] != self.hidden:
            raise RuntimeError(f"x must have at least two dimensions and hidden size {self.hidden}")
        if not (branch.shape == x.shape == grad_updated.shape == grad_normalized.shape):
            raise RuntimeError("branch and the upstream gradients must match x")
        if tuple(weight.shape) != (self.hidden,) or tuple(bias.shape) != (self.hidden,):
            raise RuntimeError("weight and bias must match the hidden size")
        if not all(t.is_contiguous() for t in tensors):
            raise RuntimeError("all tensors must be contiguous")
        if x.numel() == 0:
            raise RuntimeError("empty tensors are unsupported")
        if out is None:
            out = self.allocate_outputs(x.shape)
        check_output_tensors(out, tuple(x.shape), self.hidden, self.normalized_dtype,
                             self.branch_dtype)
        updated, normalized, grad_x, grad_branch, grad_parameters = out
        rows = x.numel() // self.hidden
        active = bool(training and dropout_p > 0.0)
        entry = (_load().rln_sm100_host_forward_backward if wait
                 else _load().rln_sm100_host_forward_backward_enqueue)
        if not wait:
            # keep every tensor of the step alive until a wait has covered it
            # (the step's number is filled in once the enqueue has succeeded)
            self._in_flight.append([None, tensors, out])
        with torch.cuda.device(self.device):
            status = entry(
                self._handle,
                x.data_ptr(), branch.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                grad_updated.data_ptr(), grad_normalized.data_ptr(),
                updated.data_ptr(), normalized.data_ptr(), grad_x.data_ptr(),
                grad_branch.data_ptr(), grad_parameters.data_ptr(),
                rows, int(active), float(dropout_p), float(eps),
                int(seed), int(offset), int(row_base), int(bool(deterministic)),
            )
        if status != 0 or wait:
            # (a failed enqueue has already waited for its copies in flight)
            self._in_flight.clear()
        else:
            self._in_flight[-1][0] = self.steps_enqueued()
        _check(status, "rln_sm100_host_forward_backward")
        return out

    def steps_enqueued(self):
        """How many steps this pipeline has been given so far; right after a
        ``forward_backward(..., wait=False)`` it is that step's number for
        ``wait(step=...)``."""
        if self._handle is None:
            raise RuntimeError("the pipeline is closed")
        return int(_load().rln_sm100_host_pipeline_steps_enqueued(self._handle))

    def wait(self, step=None):
        """Blocks until every step enqueued with ``wait=False`` has landed in its
        output tensors, or, with ``step=n``, until the n-th step given to this
        pipeline has (later steps may still be in flight)."""
        if self._handle is None:
            raise RuntimeError("the pipeline is closed")
        with torch.cuda.device(self.device):
            if step is None:
                status = _load().rln_sm100_host_pipeline_wait(self._handle)
                self._in_flight.clear()
            else:
                status = _load().rln_sm100_host_pipeline_wait_step(self._handle, int(step))
                if status == 0:
                    # steps land in order: everything up to `step` may be released
                    self._in_flight = [entry for entry in self._in_flight
                                       if entry[0] is None or entry[0] > int(step)]
        _check(status, "rln_sm100_host_pipeline_wait")
