"""Block-FP8 linear helpers (``python/sglang/srt/layers/quantization/fp8_utils.py``)."""

from __future__ import annotations

from typing import List, Optional

import torch

from .fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul, w8a8_block_fp8_matmul_ue8m0


def w8a8_block_fp8_linear(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                          weight_scale: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Quantise the activations per 1x128 group, multiply by the block-scaled weight, add bias.

    Same signature and result layout as the reference's ``*_w8a8_block_fp8_linear`` family
    (``fp8_utils.py:184-301``), which ``dispatch_w8a8_block_fp8_linear`` (``:139-149``) picks
    from; here there is one implementation.  ``weight [N, K]`` e4m3, ``weight_scale
    [ceil(N/128), ceil(K/128)]`` fp32.  Activation scales are written M-major so the GEMM's
    per-row scale loads coalesce."""
    assert input_scale is None
    input_2d = input.view(-1, input.shape[-1])
    if not input_2d.is_contiguous():
        input_2d = input_2d.contiguous()
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=True,
                                                        scale_tma_aligned=True)
    output = w8a8_block_fp8_matmul(q_input, weight, x_scale, weight_scale, block_size, output_dtype=input_2d.dtype)
    if bias is not None:
        output += bias
    return output.to(dtype=input_2d.dtype).view(*output_shape)


def dispatch_w8a8_block_fp8_linear():
    """``dispatch_w8a8_block_fp8_linear`` (``fp8_utils.py:139-149``): one back-end."""
    return w8a8_block_fp8_linear


def block_quant_dequant(x_q_block: torch.Tensor, x_s: torch.Tensor, block_size: List[int],
                        dtype: torch.dtype) -> torch.Tensor:
    """Expand block scales and dequantise (``fp8_utils.py:393-413``); offline helper."""
    block_n, block_k = block_size
    *_, n, k = x_q_block.shape
    rep = x_s.repeat_interleave(block_n, dim=-2).repeat_interleave(block_k, dim=-1)[..., :n, :k]
    return (x_q_block.to(torch.float32) * rep).to(dtype)


def w8a8_block_fp8_linear_ue8m0(input: torch.Tensor, weight: torch.Tensor, weight_scale_packed: torch.Tensor,
                                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The linear for UE8M0 checkpoints, the counterpart of ``deepgemm_w8a8_block_fp8_linear_with_fallback`` on
    Blackwell (``fp8_utils.py:217-255``): activations quantised with power-of-two group scales (packed int32,
    M-major), then the hardware block-scaled GEMM.  ``weight_scale_packed`` comes from ``pack_ue8m0_scales``."""
    input_2d = input.view(-1, input.shape[-1])
    if not input_2d.is_contiguous():
        input_2d = input_2d.contiguous()
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = sglang_per_token_group_quant_fp8(input_2d, 128, column_major_scales=True,
                                                        scale_tma_aligned=True, scale_ue8m0=True)
    output = w8a8_block_fp8_matmul_ue8m0(q_input, weight, x_scale, weight_scale_packed, output_dtype=input_2d.dtype)
    if bias is not None:
        output += bias
    return output.view(*output_shape)


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x (``fp8_utils.py:511-512``), computed on the exponent bits."""
    mant, exp = torch.frexp(x.to(torch.float32).abs())
    return torch.ldexp(torch.ones_like(mant), torch.where(mant == 0.5, exp - 1, exp))


def per_block_cast_to_fp8(x: torch.Tensor):
    """128x128 block quantisation with power-of-two (UE8M0) scales, the reference's ``per_block_cast_to_fp8``
    (``fp8_utils.py:494-507``): pad to whole blocks, block amax clamped at 1e-4, scale = the smallest power of two
    >= amax / 448, codes = e4m3(x * (1 / scale)).  Returns (codes ``[m, n]``, scales fp32 ``[ceil(m/128),
    ceil(n/128)]``).  Offline, torch ops on ``x``'s device."""
    assert x.dim() == 2
    m, n = x.shape
    m_p, n_p = -(-m // 128) * 128, -(-n // 128) * 128
    xp = torch.zeros(m_p, n_p, dtype=x.dtype, device=x.device)
    xp[:m, :n] = x
    v = xp.view(m_p // 128, 128, n_p // 128, 128)
    amax = v.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    # tensor / tensor: a true IEEE division on every device (tensor / python scalar is a multiplication by the
    # reciprocal in torch's CUDA kernels, one ulp off for some values)
    sf = ceil_to_ue8m0(amax / torch.full_like(amax, 448.0))
    q = (v * (1.0 / sf)).to(torch.float8_e4m3fn).view(m_p, n_p)[:m, :n].contiguous()
    return q, sf.view(m_p // 128, n_p // 128)


def block_quant_weight_fp8(weight: torch.Tensor, block_size: Optional[List[int]] = None):
    """Block quantisation with fp32 scales, the form block-FP8 checkpoints are made with
    (``convert_weight``, ``test/srt/cpu/utils.py:39-87``): scale = block amax / 448 (1.0 for an all-zero block),
    codes = e4m3(w / scale) with a true division; ragged edges are zero-padded for the amax and cropped.
    Returns (codes ``[N, K]`` e4m3, scales fp32 ``[ceil(N/bn), ceil(K/bk)]``).  Offline, torch ops on
    ``weight``'s device."""
    bn, bk = block_size if block_size is not None else (128, 128)
    n, k = weight.shape
    n_p, k_p = -(-n // bn) * bn, -(-k // bk) * bk
    wp = torch.zeros(n_p, k_p, dtype=torch.float32, device=weight.device)
    wp[:n, :k] = weight.to(torch.float32)
    v = wp.view(n_p // bn, bn, k_p // bk, bk)
    amax = v.abs().amax(dim=(1, 3), keepdim=True)
    s = amax / torch.full_like(amax, 448.0)  # tensor / tensor: a true IEEE division on every device
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (v / s).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(n_p, k_p)[:n, :k].contiguous()
    return q, s.view(n_p // bn, k_p // bk).contiguous()


def requant_weight_ue8m0(weight: torch.Tensor, weight_scale: torch.Tensor, block_size: List[int]):
    """Dequantise a block-FP8 weight and quantise it again with power-of-two block scales
    (``_requant_weight_ue8m0``, ``fp8_utils.py:416-491``).  Offline, torch ops."""
    assert list(block_size) == [128, 128]
    q, sf = per_block_cast_to_fp8(block_quant_dequant(weight, weight_scale, block_size, torch.float32))
    return q, sf.contiguous()
