"""Layer-level wrappers with the reference's names and signatures
(``python/sglang/srt/layers/quantization/fp8_kernel.py``): output allocation in the
reference's scale layouts, then one call into the CUDA library.  One back-end, no switches."""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ...sgl_kernel import fp8_blockwise_scaled_mm, sgl_per_token_group_quant_8bit
from ..._lib import blockwise_mm, check, dtype_code, lib

fp8_dtype = torch.float8_e4m3fn
fp8_max = torch.finfo(fp8_dtype).max
fp8_min = -fp8_max


def align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def create_per_token_group_quant_fp8_output_scale(x_shape, device, group_size, column_major_scales: bool,
                                                  scale_tma_aligned: bool, scale_ue8m0: bool):
    """Allocate the scale tensor in one of the reference's four layouts
    (``fp8_kernel.py:433-474``): row-major fp32; column-major fp32 (strides ``(1, M)``);
    column-major padded to 4 rows (strides ``(1, align(M, 4))``); UE8M0 packed int32
    ``[M, ceil(G/4)]`` with strides ``(1, align(M, 4))``."""
    if scale_ue8m0:
        assert column_major_scales and scale_tma_aligned
        *x_batch, x_q_mn, x_q_k = x_shape
        x_s_mn, x_s_k = x_q_mn, x_q_k // group_size
        aligned_mn, aligned_k = align(x_s_mn, 4), align(x_s_k, 4)
        return torch.empty((*x_batch, aligned_k // 4, aligned_mn), device=device,
                           dtype=torch.int).transpose(-1, -2)[..., :x_s_mn, :]
    if column_major_scales:
        if scale_tma_aligned:
            aligned_size = align(x_shape[-2], 4)
            return torch.empty(tuple(x_shape[:-2]) + (x_shape[-1] // group_size, aligned_size), device=device,
                               dtype=torch.float32).transpose(-1, -2)[..., : x_shape[-2], :]
        return torch.empty((x_shape[-1] // group_size,) + tuple(x_shape[:-1]), device=device,
                           dtype=torch.float32).permute(-1, -2)
    return torch.empty(tuple(x_shape[:-1]) + (x_shape[-1] // group_size,), device=device, dtype=torch.float32)


def sglang_per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
    scale_ue8m0: bool = False,
    fuse_silu_and_mul: bool = False,
    masked_m: Optional[torch.Tensor] = None,
    enable_v2: Optional[bool] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``sglang_per_token_group_quant_fp8`` (``fp8_kernel.py:477-527``): returns
    ``(x_q e4m3, x_s)`` with ``x_s`` in the requested layout.  With a 3-D ``x [E, max_m, K]`` the scales are laid out
    per expert, and ``masked_m [E]`` (int32) limits the work to the first ``masked_m[e]`` rows of every expert; the
    other rows of ``x_q`` / ``x_s`` are left unwritten (``per_token_group_quant_8bit_v2.cu:194-238``)."""
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    assert x.dim() in (2, 3), "activations must be [M, K] or, for the masked per-expert layout, [E, max_m, K]"
    assert masked_m is None or x.dim() == 3, "masked_m goes with the [E, max_m, K] layout"
    out_shape = (*x.shape[:-1], x.shape[-1] // (2 if fuse_silu_and_mul else 1))
    x_q = torch.empty(out_shape, device=x.device, dtype=fp8_dtype)
    x_s = create_per_token_group_quant_fp8_output_scale(out_shape, x.device, group_size, column_major_scales,
                                                        scale_tma_aligned, scale_ue8m0)
    if x.shape[0] > 0:
        sgl_per_token_group_quant_8bit(x, x_q, x_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0,
                                       fuse_silu_and_mul, masked_m, enable_v2=enable_v2)
    return x_q, x_s


def per_token_group_quant_fp8(x, group_size, eps: float = 1e-10, column_major_scales: bool = False,
                              scale_tma_aligned: bool = False, scale_ue8m0: bool = False):
    """The reference's Triton entry (``fp8_kernel.py:215-319``), served by the same CUDA kernel."""
    return sglang_per_token_group_quant_fp8(x, group_size, eps, column_major_scales, scale_tma_aligned, scale_ue8m0)


def w8a8_block_fp8_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                          block_size: List[int], output_dtype: torch.dtype = torch.float16,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``w8a8_block_fp8_matmul`` (``fp8_kernel.py:1149-1164``; shape rules ``:999-1044``).

    A ``[..., K]`` e4m3 contiguous, B ``[N, K]`` e4m3 contiguous, As ``[..., ceil(K/128)]`` fp32
    (row-major or M-major), Bs ``[ceil(N/128), ceil(K/128)]`` fp32; returns ``[..., N]``.  ``out`` (not in the
    reference's signature) is an optional preallocated ``[M, N]`` result with unit column stride, e.g. a row range of a
    larger tensor."""
    assert len(block_size) == 2 and block_size[0] == 128 and block_size[1] == 128, "only 128x128 blocks"
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1] and A.is_contiguous()
    assert -(-A.shape[-1] // 128) == As.shape[-1]
    assert B.ndim == 2 and B.is_contiguous() and Bs.ndim == 2
    N, K = B.shape
    assert -(-N // 128) == Bs.shape[0] and -(-K // 128) == Bs.shape[1]
    M = A.numel() // K
    A2, As2 = A.view(M, K), As.reshape(M, As.shape[-1])
    if out is not None:
        assert out.shape == (M, N) and out.dtype == output_dtype and out.stride(1) == 1 and out.device == A.device
        C = out
    else:
        C = torch.empty(A.shape[:-1] + (N,), device=A.device, dtype=output_dtype)
    if M == 0:
        return C
    ldc = C.stride(0) if out is not None and M > 1 else N
    with torch.cuda.device(A.device):
        blockwise_mm(A2.data_ptr(), B.data_ptr(), As2.data_ptr(), Bs.data_ptr(), C.data_ptr(), M, N, K, K, K, ldc,
                     As2.stride(0), As2.stride(1), Bs.stride(0), Bs.stride(1), dtype_code(output_dtype), A.device,
                     torch.cuda.current_stream(A.device).cuda_stream)
    return C


def pack_ue8m0_scales(scales: torch.Tensor) -> torch.Tensor:
    """Pack power-of-two fp32 scales ``[R, KB]`` into the UE8M0 word layout the block-scaled GEMM reads:
    int32 ``[R, ceil(KB/4)]``, byte ``j`` of word ``(r, g)`` = biased exponent of ``scales[r, 4g + j]``
    (missing k-blocks are padded with exponent 127 = 1.0).  Offline / load-time helper."""
    assert scales.dtype == torch.float32 and scales.dim() == 2
    bits = scales.contiguous().view(torch.int32)
    if bool((bits & 0x7FFFFF).ne(0).any()) or bool((bits <= 0).any()):
        raise ValueError("UE8M0 scales must be positive powers of two")
    R, KB = scales.shape
    KG = (KB + 3) // 4
    e = torch.full((R, KG * 4), 127, dtype=torch.int32, device=scales.device)
    e[:, :KB] = (bits >> 23) & 0xFF
    e = e.view(R, KG, 4)
    return (e[..., 0] | (e[..., 1] << 8) | (e[..., 2] << 16) | (e[..., 3] << 24)).to(torch.int32).contiguous()


def w8a8_block_fp8_matmul_ue8m0(A: torch.Tensor, B: torch.Tensor, As_packed: torch.Tensor, Bs_packed: torch.Tensor,
                                output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Block-FP8 GEMM with UE8M0 scales on the tensor core's block-scaling path, the counterpart of
    ``w8a8_block_fp8_matmul_deepgemm`` on Blackwell (``fp8_kernel.py:1047-1065``).

    A ``[M, K]`` e4m3; As_packed int32 ``[M, ceil(K/512)]`` with ``stride(0) == 1`` as returned by
    ``sglang_per_token_group_quant_fp8(..., column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)``;
    B ``[N, K]`` e4m3; Bs_packed int32 ``[ceil(N/128), ceil(K/512)]`` from :func:`pack_ue8m0_scales`."""
    assert A.dim() == 2 and A.is_contiguous() and B.dim() == 2 and B.is_contiguous() and A.shape[1] == B.shape[1]
    M, K = A.shape
    N = B.shape[0]
    KG = (-(-K // 128) + 3) // 4
    assert As_packed.dtype == torch.int32 and As_packed.shape == (M, KG) and (M <= 1 or As_packed.stride(0) == 1)
    assert Bs_packed.dtype == torch.int32 and Bs_packed.shape == (-(-N // 128), KG)
    C = torch.empty(M, N, device=A.device, dtype=output_dtype)
    if M == 0:
        return C
    sfa_ld = As_packed.stride(1) if KG > 1 else max(As_packed.stride(1), M)
    L = lib()
    with torch.cuda.device(A.device):
        ws_bytes = L.sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K) if M <= 64 else 0
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=A.device) if ws_bytes > 0 else None
        check(L.sglb200_fp8_ue8m0_scaled_mm_ws(
            A.data_ptr(), B.data_ptr(), As_packed.data_ptr(), Bs_packed.data_ptr(), C.data_ptr(), M, N, K, K, K, N,
            sfa_ld, Bs_packed.stride(0), Bs_packed.stride(1), dtype_code(output_dtype),
            ws.data_ptr() if ws is not None else None, ws_bytes,
            torch.cuda.current_stream(A.device).cuda_stream), "w8a8_block_fp8_matmul_ue8m0")
    return C
