"""``sgl_kernel.gemm`` ops on the block-FP8 path (``sgl-kernel/python/sgl_kernel/gemm.py:25-32,101-142``)."""

from __future__ import annotations

from typing import Optional

import torch

from .._lib import blockwise_mm, check, dtype_code, lib

FP8 = torch.float8_e4m3fn


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _cuda_check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


_EPS_CACHE = {}


def _eps_in_dtype(eps: float, dtype: torch.dtype) -> float:
    """``eps`` rounded to the input dtype (what the torch-native reference clamps with); for fp16, where 1e-10 rounds
    to zero, the fp32 value.  Cached: the rounding is a small CPU tensor op that would otherwise run on every call."""
    key = (eps, dtype)
    v = _EPS_CACHE.get(key)
    if v is None:
        v = float(eps) if dtype == torch.float32 else float(torch.tensor(eps, dtype=dtype).float())
        if v == 0.0 and eps > 0.0:
            v = float(eps)
        _EPS_CACHE[key] = v
    return v


def fp8_blockwise_scaled_mm(mat_a, mat_b, scales_a, scales_b, out_dtype):
    """Block-scaled FP8 GEMM, same contract as ``fp8_blockwise_scaled_mm``
    (``sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:368-465``).

    mat_a ``[M, K]`` e4m3 row-major; mat_b ``[K, N]`` e4m3 column-major (``weight[N, K].t()``);
    scales_a ``[M, K/128]`` fp32 (M-major as the reference requires, or row-major);
    scales_b ``[K/128, N/128]`` fp32 (``weight_scale[N/128, K/128].t()``); returns ``[M, N]``.
    Unlike the reference no padded copies of mat_a / scales_a are made for M % 4 != 0, and N
    need not be a multiple of 128 (``ceil(N/128)`` scale columns are expected then).
    """
    _cuda_check(mat_a.is_cuda, "mat_a must be a CUDA tensor")
    _cuda_check(mat_b.is_cuda, "mat_b must be a CUDA tensor")
    _cuda_check(mat_a.dim() == 2, "mat_a must be a 2D tensor")
    _cuda_check(mat_b.dim() == 2, "mat_b must be a 2D tensor")
    _cuda_check(mat_a.stride(1) == 1, "mat_a must be a row major tensor")
    _cuda_check(mat_b.stride(0) == 1, "mat_b must be a column major tensor")
    _cuda_check(mat_a.size(1) == mat_b.size(0), "mat_a and mat_b shapes cannot be multiplied")
    _cuda_check(mat_a.size(1) % 16 == 0, "mat_a must be multiple of 16 bytes for memory alignment")
    _cuda_check(mat_a.dtype == FP8, "mat_a must be Float8_e4m3fn")
    _cuda_check(mat_b.dtype == FP8, "mat_b must be Float8_e4m3fn")
    _cuda_check(out_dtype in (torch.float16, torch.bfloat16), "out_dtype must be Half or BFloat16")
    M, K = mat_a.shape
    N = mat_b.size(1)
    kt, nt = -(-K // 128), -(-N // 128)
    _cuda_check(scales_a.dim() == 2 and scales_a.size(0) == M and scales_a.size(1) == kt,
                "size of scales_a is not matched")
    _cuda_check(scales_b.dim() == 2 and scales_b.size(0) == kt and scales_b.size(1) == nt,
                "size of scales_b is not matched")
    _cuda_check(scales_a.dtype == torch.float32, "scales_a must be Float32")
    _cuda_check(scales_b.dtype == torch.float32, "scales_b must be Float32")
    _cuda_check((N * 2) % 16 == 0, "out must be multiple of 16 bytes for memory alignment")
    out = torch.empty((M, N), device=mat_a.device, dtype=out_dtype)
    if M == 0 or N == 0:
        return out
    lda = mat_a.stride(0) if M > 1 else max(mat_a.stride(0), K)
    ldb = mat_b.stride(1) if N > 1 else max(mat_b.stride(1), K)
    with torch.cuda.device(mat_a.device):
        blockwise_mm(mat_a.data_ptr(), mat_b.data_ptr(), scales_a.data_ptr(), scales_b.data_ptr(), out.data_ptr(),
                     M, N, K, lda, ldb, out.stride(0), scales_a.stride(0), scales_a.stride(1), scales_b.stride(1),
                     scales_b.stride(0), dtype_code(out_dtype), mat_a.device, _stream(mat_a))
    return out


def sgl_per_token_group_quant_8bit(
    input: torch.Tensor,
    output_q: torch.Tensor,
    output_s: torch.Tensor,
    group_size: int,
    eps: float,
    fp8_min: float,
    fp8_max: float,
    scale_ue8m0: bool = False,
    fuse_silu_and_mul: bool = False,
    masked_m: Optional[torch.Tensor] = None,
    enable_v2: Optional[bool] = None,
) -> None:
    """Per-token-group quantisation into caller-allocated ``output_q`` / ``output_s``
    (``sgl-kernel/python/sgl_kernel/gemm.py:101-137``; kernel contract
    ``sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-217``).

    ``output_s`` may be row-major ``[M, G]``, column-major (stride(0) < stride(1), optionally
    padded to a multiple of 4 rows) or, with ``scale_ue8m0``, the packed int32 layout of
    ``create_per_token_group_quant_fp8_output_scale`` (``fp8_kernel.py:433-474``).
    ``eps`` is rounded to the input dtype first, as the torch-native reference does when it
    clamps the group maximum in that dtype (``python/sglang/test/test_block_fp8.py:43``); for
    fp16, where 1e-10 rounds to zero, the fp32 value is kept.  ``enable_v2`` is accepted and
    ignored: there is one kernel.  Only the e4m3 destination is implemented.
    """
    _cuda_check(input.is_cuda and output_q.is_cuda and output_s.is_cuda, "tensors must be CUDA tensors")
    _cuda_check(input.is_contiguous(), "input must be contiguous")
    _cuda_check(output_q.is_contiguous(), "output_q must be contiguous")
    _cuda_check(output_q.dtype == FP8, "output_q must be Float8_e4m3fn (the int8 destination is not implemented)")
    hidden_in = input.size(-1)
    if input.dim() == 3:
        return _quant_batched(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0,
                              fuse_silu_and_mul, masked_m)
    _cuda_check(masked_m is None, "masked_m needs the 3-D [E, max_m, K] layout")
    _cuda_check(output_s.dim() == 2, "output_s must be 2D")
    hidden = hidden_in // 2 if fuse_silu_and_mul else hidden_in
    _cuda_check(hidden % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`")
    rows = input.numel() // hidden_in if hidden_in else 0
    _cuda_check(output_q.numel() == rows * hidden, "output_q has the wrong number of elements")
    G = hidden // group_size
    if scale_ue8m0:
        _cuda_check(output_s.dtype == torch.int32, "UE8M0 scales are packed in int32")
        _cuda_check(output_s.size(0) == rows and output_s.size(1) == -(-G // 4), "output_s shape is not matched")
    else:
        _cuda_check(output_s.dtype == torch.float32, "output_s must be Float32")
        _cuda_check(output_s.size(0) == rows and output_s.size(1) == G, "output_s shape is not matched")
    if rows == 0 or hidden == 0:
        return
    eps_eff = _eps_in_dtype(eps, input.dtype)
    L = lib()
    args = (rows, hidden, group_size, eps_eff, fp8_min, fp8_max, int(bool(scale_ue8m0)),
            output_s.stride(0), output_s.stride(1), _stream(input))
    with torch.cuda.device(input.device):
        if fuse_silu_and_mul:
            check(L.sglb200_silu_mul_group_quant_fp8(input.data_ptr(), dtype_code(input.dtype), output_q.data_ptr(),
                                                     output_s.data_ptr(), None, *args),
                  "sgl_per_token_group_quant_8bit(fuse_silu_and_mul)")
        else:
            check(L.sglb200_per_token_group_quant_fp8(input.data_ptr(), dtype_code(input.dtype),
                                                      output_q.data_ptr(), output_s.data_ptr(), *args),
                  "sgl_per_token_group_quant_8bit")


def _quant_batched(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul,
                   masked_m) -> None:
    """The ``[E, max_m, K]`` layout of the low-latency MoE path: scales addressed per expert, optional row mask
    (``sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:194-238,394-514``)."""
    E, max_m, hidden_in = input.shape
    hidden = hidden_in // 2 if fuse_silu_and_mul else hidden_in
    _cuda_check(input.dtype in (torch.bfloat16, torch.float16), "the batched layout takes bf16 / f16 input")
    _cuda_check(hidden % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`")
    _cuda_check(output_q.shape == (E, max_m, hidden), "output_q shape is not matched")
    G = hidden // group_size
    _cuda_check(output_s.dim() == 3 and output_s.size(0) == E and output_s.size(1) == max_m
                and output_s.size(2) == (-(-G // 4) if scale_ue8m0 else G), "output_s shape is not matched")
    _cuda_check(output_s.dtype == (torch.int32 if scale_ue8m0 else torch.float32), "output_s has the wrong dtype")
    mptr = None
    if masked_m is not None:
        _cuda_check(masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == E,
                    "masked_m must be a contiguous int32 tensor with one entry per expert")
        mptr = masked_m.data_ptr()
    if E == 0 or max_m == 0 or hidden == 0:
        return
    eps_eff = _eps_in_dtype(eps, input.dtype)
    with torch.cuda.device(input.device):
        check(lib().sglb200_group_quant_fp8_batched(
            input.data_ptr(), dtype_code(input.dtype), output_q.data_ptr(), output_s.data_ptr(), E, max_m, hidden,
            group_size, eps_eff, fp8_min, fp8_max, int(bool(scale_ue8m0)), int(bool(fuse_silu_and_mul)), mptr,
            output_s.stride(0), output_s.stride(1), output_s.stride(2), _stream(input)),
            "sgl_per_token_group_quant_8bit(masked)")


def sgl_per_token_group_quant_fp8(input, output_q, output_s, group_size, eps, fp8_min, fp8_max,
                                  scale_ue8m0: bool = False) -> None:
    """Legacy alias (``sgl-kernel/python/sgl_kernel/gemm.py:140-142``)."""
    sgl_per_token_group_quant_8bit(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0)
