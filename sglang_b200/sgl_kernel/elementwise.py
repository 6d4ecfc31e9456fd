"""``sgl_kernel.elementwise`` ops used on the MoE path (``sgl-kernel/python/sgl_kernel/elementwise.py``)."""

from __future__ import annotations

from typing import Optional

import torch

from .._lib import check, dtype_code, lib


def silu_and_mul(input: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = silu(input[..., :d]) * input[..., d:]`` (kernel contract
    ``sgl-kernel/csrc/elementwise/activation.cu:82-101``); the SiLU value is rounded to the
    tensor dtype before the multiply, as ``SiluAndMul.forward_native`` does."""
    if not input.is_cuda:
        raise RuntimeError("input must be a CUDA tensor")
    if input.shape[-1] * input.element_size() % 16 != 0:
        raise ValueError("The pointers must be multiple of 16 bytes.")
    if not input.is_contiguous():
        raise RuntimeError("input must be contiguous")
    d = input.shape[-1] // 2
    if out is None:
        out = torch.empty(input.shape[:-1] + (d,), device=input.device, dtype=input.dtype)
    elif out.shape != input.shape[:-1] + (d,) or not out.is_contiguous() or out.dtype != input.dtype:
        raise RuntimeError("out must be contiguous with shape input.shape[:-1] + (d,) and input's dtype")
    rows = input.numel() // input.shape[-1] if input.shape[-1] else 0
    with torch.cuda.device(input.device):
        check(lib().sglb200_silu_and_mul(input.data_ptr(), out.data_ptr(), rows, d, dtype_code(input.dtype),
                                         torch.cuda.current_stream(input.device).cuda_stream), "silu_and_mul")
    return out
