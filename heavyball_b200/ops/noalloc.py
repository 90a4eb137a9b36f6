"""ctypes access to the allocation-free cautious AdamW step (``csrc/noalloc_adamw.h``).

For callers that cannot let the optimizer allocate: the scratch the caution path needs lives in a
fixed array inside the compiled library (about 16 MiB per GPU, at most ``MAX_ELEMS`` elements per
call).  The symbol is exported with C linkage, so it is equally callable from C or any FFI; this
module is only a convenience for Python.
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import _BUILD, _NAME, load

MAX_ELEMS = 1 << 22
_lib = None


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        load()  # makes sure the shared object exists (builds it if needed) and torch's CUDA libraries are loaded
        _lib = ctypes.CDLL(os.path.join(_BUILD, _NAME + ".so"))
        fn = _lib.hb200_cautious_adamw_step_noalloc
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_longlong] + [ctypes.c_float] * 5 + [
            ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int,
        ]  # fmt: skip
    return _lib


def cautious_adamw_step(param, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay=0.0, stream=None):
    """One cautious AdamW step on fp32 CUDA tensors without any device allocation.  ``beta1`` and
    ``beta2`` are the already-debiased coefficients of this step.  Raises ``ValueError`` for sizes over
    ``MAX_ELEMS`` and ``RuntimeError`` for CUDA errors."""
    for t in (param, grad, exp_avg, exp_avg_sq):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == param.numel()):
            raise ValueError("expected contiguous fp32 CUDA tensors of equal size")
    handle = torch.cuda.current_stream(param.device).cuda_stream if stream is None else stream
    buf = ctypes.create_string_buffer(256)
    with torch.cuda.device(param.device):
        rc = library().hb200_cautious_adamw_step_noalloc(
            param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), param.numel(), lr, beta1,
            beta2, eps, weight_decay, handle, buf, len(buf),
        )  # fmt: skip
    if rc == -1:
        raise ValueError(buf.value.decode())
    if rc != 0:
        raise RuntimeError(f"CUDA error {rc}: {buf.value.decode()}")
