"""softmax / log_softmax over the last dimension, same call surface as the reference's ``kernels/softmax.py``
(``softmax`` :152-236, ``log_softmax`` :378-462): any shape, fp16 / bf16 / fp32, contiguous CUDA tensor, optional
``out`` (which may be ``x`` itself).  One launch of the hand-written kernels in ``csrc/softmax.cu`` through
``b200attn_softmax``; there is no CPU or Triton fallback."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _validate(x: torch.Tensor, out: Optional[torch.Tensor]) -> None:
    # the checks of the reference's validate_reduction / validate_input (utils/validation.py:50-63,94-97), same
    # AssertionError behaviour; the device check is "a CUDA device" rather than "Triton's active device"
    assert isinstance(x, torch.Tensor), "Input must be a tensor."
    assert x.is_cuda, "Input tensor must be a CUDA tensor."
    assert x.ndim >= 1, "Input tensor must have at least one dimension."
    assert x.is_contiguous(), "Input tensor must be contiguous."
    assert x.numel() > 0, "Input tensor must not be empty."
    assert x.shape[-1] > 0, "Last dimension must be non-empty."
    assert x.dtype in _DTYPE_CODE, "Input tensor must be float16, bfloat16 or float32."
    if out is not None:
        assert out.shape == x.shape and out.dtype == x.dtype, "Output must have the shape and dtype of the input."
        assert out.device == x.device and out.is_contiguous(), "Output must be a contiguous tensor on the input's device."


def _launch(x: torch.Tensor, out: Optional[torch.Tensor], log: bool) -> torch.Tensor:
    _validate(x, out)
    out = torch.empty_like(x) if out is None else out
    a = _native.SoftmaxArgs()
    a.x, a.out = x.data_ptr(), out.data_ptr()
    a.cols = x.shape[-1]
    a.rows = x.numel() // x.shape[-1]
    a.dtype, a.log_softmax = _DTYPE_CODE[x.dtype], int(log)
    a.device = x.device.index if x.device.index is not None else torch.cuda.current_device()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    _native.check(_native.lib().b200attn_softmax(C.byref(a), C.c_void_p(stream)), "b200attn_softmax")
    return out


def softmax(x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Softmax over the last dimension."""
    return _launch(x, out, False)


def log_softmax(x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Log-softmax over the last dimension."""
    return _launch(x, out, True)
