"""``sgl_kernel.moe`` ops on the block-FP8 path (``sgl-kernel/python/sgl_kernel/moe.py:6-48,96-172``)."""

from __future__ import annotations

from typing import Optional

import torch

from .._lib import check, dtype_code, lib

FP8 = torch.float8_e4m3fn


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def prepare_moe_input(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation,
                      output_permutation, num_experts, n, k, blockscale_offsets: Optional[torch.Tensor] = None):
    """Fill the routing tables for the sorted-by-expert layout
    (``sgl-kernel/csrc/moe/prepare_moe_input.cu:13-167``).  ``expert_offsets`` has ``E + 1``
    entries.  Slots of one expert come out in ascending token order."""
    _req(topk_ids.is_cuda and topk_ids.dtype == torch.int32 and topk_ids.dim() == 2 and topk_ids.is_contiguous(),
         "topk_ids must be a contiguous 2D int32 CUDA tensor")
    _req(blockscale_offsets is None, "blockscale_offsets (the FP4 path) is not implemented")
    for name, t, numel in (("expert_offsets", expert_offsets, num_experts + 1),
                           ("problem_sizes1", problem_sizes1, num_experts * 3),
                           ("problem_sizes2", problem_sizes2, num_experts * 3),
                           ("input_permutation", input_permutation, topk_ids.numel()),
                           ("output_permutation", output_permutation, topk_ids.numel())):
        _req(t.is_cuda and t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= numel,
             f"{name} must be a contiguous int32 CUDA tensor with at least {numel} elements")
    with torch.cuda.device(topk_ids.device):
        check(lib().sglb200_prepare_moe_input(
            topk_ids.data_ptr(), expert_offsets.data_ptr(), problem_sizes1.data_ptr(), problem_sizes2.data_ptr(),
            input_permutation.data_ptr(), output_permutation.data_ptr(), topk_ids.size(0), topk_ids.size(1),
            num_experts, n, k, _stream(topk_ids)), "prepare_moe_input")


def shuffle_rows(input_tensor, dst2src_map, output_tensor_shape):
    """``output[i] = input[dst2src_map[i]]`` (``prepare_moe_input.cu:169-256``;
    Python signature ``sgl-kernel/python/sgl_kernel/moe.py``: returns a new tensor)."""
    _req(input_tensor.is_cuda and input_tensor.dim() == 2 and input_tensor.is_contiguous(),
         "input must be a contiguous 2D CUDA tensor")
    _req(dst2src_map.dtype == torch.int32 and dst2src_map.is_contiguous(), "dst2src_map must be contiguous int32")
    out = torch.empty(output_tensor_shape, device=input_tensor.device, dtype=input_tensor.dtype)
    _req(out.size(1) == input_tensor.size(1), "row length mismatch")
    _req(dst2src_map.numel() >= out.size(0), "dst2src_map is shorter than the output")
    row_bytes = input_tensor.size(1) * input_tensor.element_size()
    with torch.cuda.device(input_tensor.device):
        check(lib().sglb200_shuffle_rows(input_tensor.data_ptr(), dst2src_map.data_ptr(), out.data_ptr(),
                                         out.size(0), row_bytes, _stream(input_tensor)), "shuffle_rows")
    return out


def apply_shuffle_mul_sum(input, output, permutation, factors, round_products: bool = False):
    """``output[i] = sum_j factors[i, j] * input[permutation[i * topk + j]]`` in fp32
    (``prepare_moe_input.cu:258-392``).  ``round_products=True`` rounds every product to the
    tensor dtype before adding, the arithmetic of the torch-native expert MLP
    (``python/sglang/test/test_block_fp8.py:445-447``)."""
    _req(input.dim() == 2, "input_tensor must be 2D [m * topk, row_stride]")
    _req(output.dim() == 2, "output_tensor must be 2D [m, row_stride]")
    _req(permutation.dim() == 1 and permutation.dtype == torch.int32, "permutation must be 1D [m * topk]")
    _req(input.is_contiguous() and output.is_contiguous() and permutation.is_contiguous(), "tensors must be contiguous")
    m = output.size(0)
    topk = permutation.size(0) // m if m else 1
    _req(permutation.size(0) == m * topk, "permutation size must match m * topk")
    _req(input.dtype == output.dtype and input.size(1) == output.size(1), "input/output mismatch")
    fptr = None
    if factors is not None:
        _req(factors.dtype == output.dtype, "Factors must match output dtype")
        _req(factors.numel() == m * topk, "Factors must have shape [m * topk]")
        factors = factors.contiguous()
        fptr = factors.data_ptr()
    with torch.cuda.device(input.device):
        check(lib().sglb200_apply_shuffle_mul_sum(input.data_ptr(), output.data_ptr(), permutation.data_ptr(), fptr,
                                                  m, max(topk, 1), output.size(1), dtype_code(output.dtype),
                                                  int(bool(round_products)), _stream(input)),
              "apply_shuffle_mul_sum")


def fp8_blockwise_scaled_grouped_mm(output, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, a, b,
                                    scales_a, scales_b, stride_a, stride_b, stride_c, layout_sfa, layout_sfb,
                                    problem_sizes, expert_offsets, workspace):
    """Grouped block-scaled FP8 GEMM with the reference's 18-argument signature
    (``sgl-kernel/python/sgl_kernel/moe.py:96-135``, kernel
    ``sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:650-810``).

    ``a [rows, K]`` e4m3 sorted by expert; ``b [E, K, N]`` = ``w[E, N, K].transpose(1, 2)``
    (K contiguous); ``scales_a [rows, K/128]`` fp32; ``scales_b [E, K/128, N/128]`` =
    ``w_scale[E, N/128, K/128].transpose(1, 2)``; ``problem_sizes [E, 3]`` int32 with the row
    count of each expert in column 0; ``expert_offsets [E]`` int32.  The pointer arrays,
    stride arrays, scale-layout tables and workspace the reference needs are accepted and
    left untouched: this kernel derives everything from the offsets.
    """
    _req(a.is_cuda and a.dtype == FP8 and a.dim() == 2 and a.stride(1) == 1, "a must be a row-major 2D e4m3 CUDA tensor")
    _req(b.dtype == FP8 and b.dim() == 3 and b.stride(1) == 1, "b must be [E, K, N] e4m3 with K contiguous")
    _req(output.dim() == 2 and output.stride(1) == 1 and output.dtype in (torch.bfloat16, torch.float16),
         "output must be a row-major 2D bf16/f16 tensor")
    E, K, N = b.shape
    _req(a.size(1) == K and output.size(1) == N and output.size(0) == a.size(0), "shapes cannot be multiplied")
    _req(N % 128 == 0 and K % 128 == 0, "N and K must be multiples of 128")
    _req(scales_a.dtype == torch.float32 and scales_a.shape == (a.size(0), K // 128), "size of scales_a is not matched")
    _req(scales_b.dtype == torch.float32 and scales_b.shape == (E, K // 128, N // 128), "size of scales_b is not matched")
    _req(problem_sizes.dtype == torch.int32 and problem_sizes.is_contiguous() and problem_sizes.numel() >= 3 * E,
         "problem_sizes must be contiguous int32 [E, 3]")
    _req(expert_offsets.dtype == torch.int32 and expert_offsets.is_contiguous() and expert_offsets.numel() >= E,
         "expert_offsets must be contiguous int32 [E]")
    if a.size(0) == 0:
        return
    with torch.cuda.device(a.device):
        check(lib().sglb200_fp8_blockwise_scaled_grouped_mm(
            a.data_ptr(), b.data_ptr(), scales_a.data_ptr(), scales_b.data_ptr(), output.data_ptr(),
            expert_offsets.data_ptr(), problem_sizes.data_ptr(), a.size(0), E, N, K,
            a.stride(0), b.stride(2), b.stride(0), output.stride(0),
            scales_a.stride(0), scales_a.stride(1), scales_b.stride(0), scales_b.stride(2), scales_b.stride(1),
            dtype_code(output.dtype), _stream(a)), "fp8_blockwise_scaled_grouped_mm")


def topk_softmax(topk_weights: torch.Tensor, topk_ids: torch.Tensor, gating_output: torch.Tensor,
                 renormalize: bool = False) -> None:
    """Softmax over the experts, then the ``topk`` largest probabilities in descending order
    (``sgl-kernel/python/sgl_kernel/moe.py:28-36``; checks as
    ``sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:512-545``).  Any expert count up to 1024 runs in one
    kernel; no softmax workspace is allocated."""
    _req(gating_output.dtype in (torch.float32, torch.float16, torch.bfloat16),
         "gating_output must be float32, float16, or bfloat16")
    _req(gating_output.dim() == 2, "gating_output must be 2D tensor [num_tokens, num_experts]")
    _req(topk_weights.dim() == 2, "topk_weights must be 2D tensor [num_tokens, topk]")
    _req(topk_ids.dim() == 2, "topk_indices must be 2D tensor [num_tokens, topk]")
    _req(gating_output.size(0) == topk_weights.size(0),
         "First dimension of topk_weights must match num_tokens in gating_output")
    _req(gating_output.size(0) == topk_ids.size(0),
         "First dimension of topk_indices must match num_tokens in gating_output")
    _req(topk_weights.size(-1) == topk_ids.size(-1), "Second dimension of topk_indices must match topk in topk_weights")
    _req(topk_weights.size(-1) <= gating_output.size(-1), "topk must be less than or equal to num_experts")
    _req(topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32,
         "topk_weights must be float32 and topk_indices int32")
    _req(gating_output.is_cuda and gating_output.is_contiguous() and topk_weights.is_contiguous()
         and topk_ids.is_contiguous(), "tensors must be contiguous CUDA tensors")
    with torch.cuda.device(gating_output.device):
        check(lib().sglb200_topk_softmax(gating_output.data_ptr(), dtype_code(gating_output.dtype),
                                         topk_weights.data_ptr(), topk_ids.data_ptr(), gating_output.size(0),
                                         gating_output.size(1), topk_weights.size(1), int(bool(renormalize)),
                                         _stream(gating_output)), "topk_softmax")


def moe_align_block_size(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad,
                         cumsum_buffer, pad_sorted_token_ids=False) -> None:
    """Block-aligned sort of the routed slots (``sgl-kernel/python/sgl_kernel/moe.py:6-25``, kernel
    ``sgl-kernel/csrc/moe/moe_align_kernel.cu:302-364``).  ``num_experts`` is the number of BUCKETS, i.e. the
    caller's expert count + 1 (bucket 0 takes id -1).  Slots of one bucket come out in ascending order."""
    _req(topk_ids.is_cuda and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous(),
         "topk_ids must be a contiguous int32 CUDA tensor")
    numel = topk_ids.numel()
    cap = numel + num_experts * (block_size - 1)
    for name, t, n in (("sorted_token_ids", sorted_token_ids, cap), ("experts_ids", experts_ids, -(-cap // block_size)),
                       ("num_tokens_post_pad", num_tokens_post_pad, 1), ("cumsum_buffer", cumsum_buffer, num_experts + 1)):
        _req(t.is_cuda and t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= n,
             f"{name} must be a contiguous int32 CUDA tensor with at least {n} elements")
    with torch.cuda.device(topk_ids.device):
        check(lib().sglb200_moe_align_block_size(topk_ids.data_ptr(), numel, num_experts, block_size,
                                                 sorted_token_ids.data_ptr(), experts_ids.data_ptr(),
                                                 num_tokens_post_pad.data_ptr(), cumsum_buffer.data_ptr(),
                                                 int(bool(pad_sorted_token_ids)), _stream(topk_ids)),
              "moe_align_block_size")


def moe_sum_reduce(input_tensor, output_tensor, routed_scaling_factor=0) -> None:
    """``output[t] = routed_scaling_factor * sum_j input[t, j]`` with an fp32 sum
    (``sgl-kernel/python/sgl_kernel/moe.py:39-48``, ``sgl-kernel/csrc/moe/moe_sum_reduce.cu:227-403``).
    bf16 / f16 only; ``hidden`` must be a multiple of 8."""
    _req(input_tensor.is_cuda, "input must be CUDA tensor")
    _req(output_tensor.is_cuda, "output must be CUDA tensor")
    _req(input_tensor.dim() == 3, "input must be a 3D tensor like [token_num, topk_num, hidden_dim]")
    _req(output_tensor.dim() == 2, "output must be [token_num, hidden_dim]")
    _req(input_tensor.size(0) == output_tensor.size(0), "token dim mismatch")
    _req(input_tensor.size(2) == output_tensor.size(1), "hidden_dim mismatch")
    _req(input_tensor.is_contiguous(), "expect input to be contiguous")
    _req(output_tensor.is_contiguous(), "expect output to be contiguous")
    _req(input_tensor.dtype == output_tensor.dtype, "input/output dtype mismatch")
    with torch.cuda.device(input_tensor.device):
        check(lib().sglb200_moe_sum_reduce(input_tensor.data_ptr(), output_tensor.data_ptr(), input_tensor.size(0),
                                           input_tensor.size(1), input_tensor.size(2), dtype_code(input_tensor.dtype),
                                           float(routed_scaling_factor), _stream(input_tensor)), "moe_sum_reduce")


def moe_fused_gate(input_tensor, bias, num_expert_group, topk_group, topk, num_fused_shared_experts=0,
                   routed_scaling_factor=0, apply_routed_scaling_factor_on_output=False):
    """Sigmoid + bias + grouped top-k gate of DeepSeek-V3, renormalised; returns ``(weights fp32, ids int32)``
    (``sgl-kernel/python/sgl_kernel/moe.py:61-93``, kernel ``sgl-kernel/csrc/moe/moe_fused_gate.cu:378-525``).
    Unlike the reference the expert count need not be a power of two and a group may hold more than 32 experts."""
    _req(input_tensor.is_cuda and input_tensor.dim() == 2 and input_tensor.is_contiguous(),
         "input must be a contiguous 2D CUDA tensor [num_tokens, num_experts]")
    _req(bias.dim() == 1 and bias.size(0) == input_tensor.size(1), "input and bias should have the same num_experts")
    _req(bias.dtype == input_tensor.dtype, "input and bias should have the same dtype")
    num_rows, num_experts = input_tensor.shape
    output = torch.empty(num_rows, topk, dtype=torch.float32, device=input_tensor.device)
    indices = torch.empty(num_rows, topk, dtype=torch.int32, device=input_tensor.device)
    with torch.cuda.device(input_tensor.device):
        check(lib().sglb200_moe_fused_gate(input_tensor.data_ptr(), bias.contiguous().data_ptr(),
                                           dtype_code(input_tensor.dtype), output.data_ptr(), indices.data_ptr(),
                                           num_rows, num_experts, num_expert_group, topk_group, topk,
                                           num_fused_shared_experts, float(routed_scaling_factor),
                                           int(bool(apply_routed_scaling_factor_on_output)), _stream(input_tensor)),
              "moe_fused_gate")
    return output, indices
