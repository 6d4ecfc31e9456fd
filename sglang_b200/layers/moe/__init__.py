"""Block-FP8 fused expert MLP (``python/sglang/srt/layers/moe``): one pipeline behind the
reference's three entry signatures.

Pipeline (all CUDA, current stream): routing tables -> per-token-group quant of the
activations -> row gather into expert order -> grouped GEMM (gate_up) -> fused SiLU-and-mul +
requant -> grouped GEMM (down) -> weighted top-k combine.  Compared with the reference's
CUTLASS flow (``cutlass_moe.py:134-204``) the bf16 ``intermediate`` tensor is never written
(SiLU, multiply and requantisation are one pass) and no pointer/layout tables are filled.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, NamedTuple, Optional

import torch

from ..._lib import check, dtype_code, lib
from ...sgl_kernel import apply_shuffle_mul_sum, prepare_moe_input, shuffle_rows
from ..quantization.fp8_kernel import sglang_per_token_group_quant_fp8

FP8 = torch.float8_e4m3fn


class StandardTopKOutput(NamedTuple):
    """``StandardTopKOutput`` (``layers/moe/topk.py:149-155``)."""
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    router_logits: Optional[torch.Tensor] = None


@dataclass
class MoeRunnerConfig:
    """The fields of ``MoeRunnerConfig`` (``layers/moe/moe_runner/base.py:26-45``) this path reads."""
    num_experts: Optional[int] = None
    num_local_experts: Optional[int] = None
    hidden_size: Optional[int] = None
    intermediate_size_per_partition: Optional[int] = None
    top_k: Optional[int] = None
    activation: str = "silu"
    apply_router_weight_on_input: bool = False
    inplace: bool = False
    no_combine: bool = False
    routed_scaling_factor: Optional[float] = None


def _grouped_mm(a_q, a_s, w, w_s, out, expert_offsets):
    """out[rows of e] = block_scaled(a_q[rows of e] @ w[e].T); w ``[E, N, K]``, w_s ``[E, N/128, K/128]``."""
    E, N, K = w.shape
    with torch.cuda.device(a_q.device):
        check(lib().sglb200_fp8_blockwise_scaled_grouped_mm(
            a_q.data_ptr(), w.data_ptr(), a_s.data_ptr(), w_s.data_ptr(), out.data_ptr(),
            expert_offsets.data_ptr(), None, a_q.size(0), E, N, K,
            a_q.stride(0), w.stride(1), w.stride(0), out.stride(0),
            a_s.stride(0), a_s.stride(1), w_s.stride(0), w_s.stride(1), w_s.stride(2),
            dtype_code(out.dtype), torch.cuda.current_stream(a_q.device).cuda_stream),
            "fp8_blockwise_scaled_grouped_mm")


def fused_experts_block_fp8(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w1_scale: torch.Tensor,
                            w2_scale: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                            routed_scaling_factor: Optional[float] = None, out: Optional[torch.Tensor] = None,
                            no_combine: bool = False, apply_router_weight_on_input: bool = False) -> torch.Tensor:
    """Expert MLP with block-FP8 weights.

    hidden_states ``[M, H]`` bf16/f16; w1 ``[E, 2I, H]`` (gate rows first, then up), w2 ``[E, H, I]``
    e4m3; w1_scale ``[E, 2I/128, H/128]``, w2_scale ``[E, H/128, I/128]`` fp32; topk_weights /
    topk_ids ``[M, topk]``.  Expert ids outside ``[0, E)`` (non-local experts under expert
    parallelism, ``token_dispatcher/standard.py:74-84``) contribute zero.  Same arithmetic as
    ``torch_w8a8_block_fp8_moe`` (``python/sglang/test/test_block_fp8.py:418-447``), including its
    final combine: products with the routing weights are rounded to the activation dtype and
    then summed in fp32.

    ``out``: write the result there (it may be ``hidden_states`` itself: the activations are quantised into their own
    buffer first, so the in-place form of ``fused_moe.py:280-309`` needs no extra copy).  ``no_combine``: return the
    weighted expert outputs ``[M, topk, H]`` without the sum over top-k (``fused_moe.py:452-458,597-598``).
    ``apply_router_weight_on_input``: the routing weight multiplies the gate_up GEMM's fp32 sums instead of the expert
    output (``fused_moe_triton_kernels.py``, ``MUL_ROUTED_WEIGHT`` on the first kernel); top-1 routing only, as the
    reference's callers require.
    """
    assert hidden_states.dim() == 2 and hidden_states.is_contiguous()
    if hidden_states.size(0) == 0:
        if no_combine:
            return hidden_states.new_empty(0, topk_ids.size(1), hidden_states.size(1))
        return torch.empty_like(hidden_states) if out is None else out
    a_q, a_s = sglang_per_token_group_quant_fp8(hidden_states, 128)
    return fused_experts_block_fp8_prequant(a_q, a_s, hidden_states.dtype, w1, w2, w1_scale, w2_scale, topk_weights,
                                            topk_ids, routed_scaling_factor, out=out, no_combine=no_combine,
                                            apply_router_weight_on_input=apply_router_weight_on_input)


def fused_experts_block_fp8_prequant(a_q: torch.Tensor, a_s: torch.Tensor, out_dtype: torch.dtype, w1: torch.Tensor,
                                     w2: torch.Tensor, w1_scale: torch.Tensor, w2_scale: torch.Tensor,
                                     topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                                     routed_scaling_factor: Optional[float] = None, out: Optional[torch.Tensor] = None,
                                     no_combine: bool = False,
                                     apply_router_weight_on_input: bool = False) -> torch.Tensor:
    """The expert MLP on activations that are already quantised (``a_q [M, H]`` e4m3, ``a_s [M, H/128]`` fp32
    row-major): the form an expert-parallel rank runs on the rows it received from the dispatch, which
    travel as fp8 payload plus scales (``token_dispatcher/deepep.py:360-371``)."""
    assert a_q.dim() == 2 and a_q.is_contiguous() and a_q.dtype == FP8
    assert w1.dtype == FP8 and w2.dtype == FP8 and w1.is_contiguous() and w2.is_contiguous()
    M, H = a_q.shape
    E, two_i, H1 = w1.shape
    I = two_i // 2
    assert H1 == H and w2.shape == (E, H, I), "weight shapes do not match"
    assert H % 128 == 0 and I % 128 == 0, "hidden and intermediate sizes must be multiples of 128"
    assert a_s.shape == (M, H // 128) and a_s.dtype == torch.float32 and a_s.is_contiguous()
    assert topk_weights.shape == topk_ids.shape and topk_ids.size(0) == M
    topk = topk_ids.size(1)
    dev = a_q.device
    assert not (no_combine and out is not None), "no combine + inplace makes no sense"
    if apply_router_weight_on_input and topk != 1:
        raise NotImplementedError("apply_router_weight_on_input is implemented for top-1 routing, as the reference's "
                                  "callers require")
    if no_combine:
        out = torch.empty(M, topk, H, dtype=out_dtype, device=dev)
    elif out is None:
        out = torch.empty(M, H, dtype=out_dtype, device=dev)
    else:
        assert out.shape == (M, H) and out.dtype == out_dtype and out.is_contiguous() and out.device == dev
    if M == 0:
        return out
    ids = topk_ids.to(torch.int32).contiguous()
    rows = M * topk
    expert_offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    ps1 = torch.empty(E, 3, dtype=torch.int32, device=dev)
    ps2 = torch.empty(E, 3, dtype=torch.int32, device=dev)
    a_map = torch.empty(rows, dtype=torch.int32, device=dev)
    c_map = torch.empty(rows, dtype=torch.int32, device=dev)
    prepare_moe_input(ids, expert_offsets, ps1, ps2, a_map, c_map, E, I, H)

    rep_q = shuffle_rows(a_q, a_map, (rows, H))
    rep_s = shuffle_rows(a_s, a_map, (rows, H // 128))
    if apply_router_weight_on_input:
        # the gate_up GEMM multiplies its fp32 sums by sa[row, kb] * sb: folding the row's routing weight into its
        # group scales applies it where the reference's kernel does, before the sums are rounded to the activation type
        rep_s = rep_s * topk_weights.reshape(-1).to(torch.float32)[a_map.long()].unsqueeze(1)
    c1 = torch.empty(rows, two_i, dtype=out_dtype, device=dev)
    _grouped_mm(rep_q, rep_s, w1, w1_scale, c1, expert_offsets)
    q2, s2 = sglang_per_token_group_quant_fp8(c1, 128, fuse_silu_and_mul=True)
    c2 = torch.empty(rows, H, dtype=out_dtype, device=dev)
    _grouped_mm(q2, s2, w2, w2_scale, c2, expert_offsets)
    factors = None
    if not apply_router_weight_on_input:
        factors = topk_weights if routed_scaling_factor is None else topk_weights * routed_scaling_factor
    elif routed_scaling_factor is not None:
        factors = torch.full_like(topk_weights, routed_scaling_factor)
    if factors is not None:
        factors = factors.to(out_dtype).reshape(-1).contiguous()
    if no_combine:  # every (token, slot) is its own output row: the combine kernel with one slot per row
        apply_shuffle_mul_sum(c2, out.view(rows, H), c_map, factors, round_products=True)
    else:
        apply_shuffle_mul_sum(c2, out, c_map, factors, round_products=True)
    return out


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_output: StandardTopKOutput,
                  moe_runner_config: MoeRunnerConfig, b1=None, b2=None, use_fp8_w8a8: bool = False,
                  use_int8_w8a8: bool = False, use_int8_w8a16: bool = False, use_int4_w4a16: bool = False,
                  per_channel_quant: bool = False, w1_scale: Optional[torch.Tensor] = None,
                  w2_scale: Optional[torch.Tensor] = None, w1_zp=None, w2_zp=None, a1_scale=None, a2_scale=None,
                  block_shape: Optional[List[int]] = None):
    """``fused_experts`` (``fused_moe_triton/fused_moe.py:254-338``) for
    ``use_fp8_w8a8=True, block_shape=[128, 128]``; every other quantisation flag is refused."""
    if not use_fp8_w8a8 or block_shape is None or list(block_shape) != [128, 128]:
        raise NotImplementedError("only use_fp8_w8a8=True with block_shape=[128, 128] is implemented")
    if use_int8_w8a8 or use_int8_w8a16 or use_int4_w4a16 or per_channel_quant:
        raise NotImplementedError("integer and per-channel schemes are outside the block-FP8 path")
    if b1 is not None or b2 is not None or a1_scale is not None or a2_scale is not None:
        raise NotImplementedError("biases and static activation scales are not part of the block-FP8 path")
    if moe_runner_config.activation != "silu":
        raise NotImplementedError("only the SiLU-gated MLP is implemented")
    topk_weights, topk_ids = topk_output[0], topk_output[1]
    if moe_runner_config.inplace:
        assert not moe_runner_config.no_combine, "no combine + inplace makes no sense"
    return fused_experts_block_fp8(hidden_states, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids,
                                   moe_runner_config.routed_scaling_factor,
                                   out=hidden_states if moe_runner_config.inplace else None,
                                   no_combine=moe_runner_config.no_combine,
                                   apply_router_weight_on_input=moe_runner_config.apply_router_weight_on_input)


def cutlass_fused_experts_fp8(a, w1_q, w2_q, w1_scale, w2_scale, topk_weights, topk_ids, a1_strides=None,
                              c1_strides=None, a2_strides=None, c2_strides=None, workspace=None, a_ptrs=None,
                              b_ptrs=None, out_ptrs=None, a_scales_ptrs=None, b_scales_ptrs=None,
                              expert_offsets=None, problem_sizes1=None, problem_sizes2=None,
                              use_fp8_blockscale: bool = True):
    """``cutlass_fused_experts_fp8`` (``layers/moe/cutlass_moe.py:21-205``).  The reference passes
    transposed views: ``w1_q [E, H, 2I]`` = ``w13[E, 2I, H].transpose(1, 2)``, ``w2_q [E, I, H]``,
    and scales transposed the same way; they are viewed back here without a copy.  The stride,
    pointer, workspace and problem-size tensors are accepted for compatibility and not used."""
    assert use_fp8_blockscale, "Only support fp8 blockscale for now"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert w1_q.dtype == FP8 and w2_q.dtype == FP8
    assert a.shape[1] == w1_q.shape[1], "Hidden size mismatch w1"
    assert w1_q.shape[2] == w2_q.shape[1] * 2, "Hidden size mismatch w2"
    assert w1_q.shape[0] == w2_q.shape[0], "Expert number mismatch"
    assert a.dtype in [torch.half, torch.bfloat16], "Invalid output dtype"
    w1, w2 = w1_q.transpose(1, 2), w2_q.transpose(1, 2)
    s1, s2 = w1_scale.transpose(1, 2), w2_scale.transpose(1, 2)
    assert w1.is_contiguous() and w2.is_contiguous(), "weights must be K-contiguous ([E, N, K] storage)"
    return fused_experts_block_fp8(a, w1, w2, s1.contiguous(), s2.contiguous(), topk_weights, topk_ids)


def fused_experts_masked(hidden_states: torch.Tensor, hidden_states_scale: torch.Tensor, w13_weight: torch.Tensor,
                         w13_scale: torch.Tensor, w2_weight: torch.Tensor, w2_scale: torch.Tensor,
                         masked_m: torch.Tensor, expected_m: int, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Expert MLP in the masked per-expert layout of the low-latency dispatcher
    (``python/sglang/srt/layers/moe/moe_runner/deep_gemm.py:209-328``): ``hidden_states [E_local, max_m, H]`` e4m3
    with ``hidden_states_scale [E_local, max_m, H/128]``; expert ``e`` holds ``masked_m[e]`` valid rows.  Grouped GEMM
    (gate_up) -> fused SiLU-mul + group quant -> grouped GEMM (down); returns ``[E_local, max_m, H]``, rows past
    ``masked_m[e]`` unspecified (neither read nor written by any of the three kernels)."""
    from ..deep_gemm_wrapper import grouped_gemm_nt_f8f8bf16_masked
    E, max_m, H = hidden_states.shape
    two_i = w13_weight.shape[1]
    gate_up = torch.empty(E, max_m, two_i, dtype=out_dtype, device=hidden_states.device)
    grouped_gemm_nt_f8f8bf16_masked((hidden_states, hidden_states_scale), (w13_weight, w13_scale), gate_up, masked_m,
                                    expected_m)
    down_q, down_s = sglang_per_token_group_quant_fp8(gate_up, 128, fuse_silu_and_mul=True, masked_m=masked_m)
    out = torch.empty(E, max_m, w2_weight.shape[1], dtype=out_dtype, device=hidden_states.device)
    grouped_gemm_nt_f8f8bf16_masked((down_q, down_s), (w2_weight, w2_scale), out, masked_m, expected_m)
    return out


def _grouped_mm_ue8m0(a_q, a_sf, w, w_sf, out, expert_offsets):
    """``out[rows of e] = a_q[rows of e] @ w[e].T`` with power-of-two scales applied by the tensor core; ``a_sf
    [rows, ceil(K/512)]`` int32 in any strides, ``w_sf [E, N/128, ceil(K/512)]`` int32."""
    E, N, K = w.shape
    with torch.cuda.device(a_q.device):
        check(lib().sglb200_fp8_ue8m0_scaled_grouped_mm(
            a_q.data_ptr(), w.data_ptr(), a_sf.data_ptr(), w_sf.data_ptr(), out.data_ptr(), expert_offsets.data_ptr(),
            a_q.size(0), E, N, K, a_q.stride(0), w.stride(1), w.stride(0), out.stride(0), a_sf.stride(0),
            a_sf.stride(1) if a_sf.size(1) > 1 else max(a_sf.stride(1), 1), w_sf.stride(0), w_sf.stride(1), w_sf.stride(2),
            dtype_code(out.dtype), torch.cuda.current_stream(a_q.device).cuda_stream),
            "fp8_ue8m0_scaled_grouped_mm")


def fused_experts_block_fp8_ue8m0(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w1_sf: torch.Tensor,
                                  w2_sf: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                                  routed_scaling_factor: Optional[float] = None) -> torch.Tensor:
    """The expert MLP on a UE8M0 checkpoint (power-of-two weight block scales, packed by ``pack_ue8m0_scales`` per
    expert: ``w1_sf [E, 2I/128, ceil(H/512)]``, ``w2_sf [E, H/128, ceil(I/512)]`` int32) with power-of-two activation
    group scales: the reference's Blackwell route through DeepGEMM
    (``python/sglang/srt/layers/moe/moe_runner/deep_gemm.py:131-207``, ``DEEPGEMM_SCALE_UE8M0``).  Same pipeline as
    :func:`fused_experts_block_fp8`; both grouped GEMMs run on the tensor core's block-scaling path."""
    from ...sgl_kernel import sgl_per_token_group_quant_8bit
    assert hidden_states.dim() == 2 and hidden_states.is_contiguous()
    M, H = hidden_states.shape
    E, two_i, _ = w1.shape
    I = two_i // 2
    assert H % 128 == 0 and I % 128 == 0, "hidden and intermediate sizes must be multiples of 128"
    dev, out_dtype = hidden_states.device, hidden_states.dtype
    out = torch.empty(M, H, dtype=out_dtype, device=dev)
    if M == 0:
        return out
    topk = topk_ids.size(1)
    rows = M * topk
    kg1 = -(-(H // 128) // 4)
    a_q = torch.empty(M, H, dtype=FP8, device=dev)
    a_sf = torch.empty(M, kg1, dtype=torch.int32, device=dev)  # row-major words, so that rows can be shuffled
    sgl_per_token_group_quant_8bit(hidden_states, a_q, a_sf, 128, 1e-10, -448.0, 448.0, scale_ue8m0=True)
    ids = topk_ids.to(torch.int32).contiguous()
    expert_offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    ps1 = torch.empty(E, 3, dtype=torch.int32, device=dev)
    ps2 = torch.empty(E, 3, dtype=torch.int32, device=dev)
    a_map = torch.empty(rows, dtype=torch.int32, device=dev)
    c_map = torch.empty(rows, dtype=torch.int32, device=dev)
    prepare_moe_input(ids, expert_offsets, ps1, ps2, a_map, c_map, E, I, H)
    rep_q = shuffle_rows(a_q, a_map, (rows, H))
    rep_sf = shuffle_rows(a_sf, a_map, (rows, kg1))
    c1 = torch.empty(rows, two_i, dtype=out_dtype, device=dev)
    _grouped_mm_ue8m0(rep_q, rep_sf, w1, w1_sf, c1, expert_offsets)
    q2, sf2 = sglang_per_token_group_quant_fp8(c1, 128, column_major_scales=True, scale_tma_aligned=True,
                                               scale_ue8m0=True, fuse_silu_and_mul=True)
    c2 = torch.empty(rows, H, dtype=out_dtype, device=dev)
    _grouped_mm_ue8m0(q2, sf2, w2, w2_sf, c2, expert_offsets)
    factors = topk_weights if routed_scaling_factor is None else topk_weights * routed_scaling_factor
    apply_shuffle_mul_sum(c2, out, c_map, factors.to(out_dtype).reshape(-1).contiguous(), round_products=True)
    return out
