"""Router front end and routing tables, layer level
(``python/sglang/srt/layers/moe/topk.py:467-495`` and
``python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:17-88``)."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ...sgl_kernel import moe_align_block_size as _sgl_moe_align_block_size
from ...sgl_kernel import topk_softmax


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int, renormalize: bool,
               num_token_non_padded: Optional[torch.Tensor] = None,
               expert_location_dispatch_info=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax routing: ``(topk_weights fp32 [M, topk], topk_ids int32 [M, topk])``.  The logical-to-physical
    expert remapping and the padded-region mask of the reference are not implemented and must be ``None``."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if num_token_non_padded is not None or expert_location_dispatch_info is not None:
        raise RuntimeError("num_token_non_padded / expert_location_dispatch_info are not implemented")
    M = hidden_states.shape[0]
    topk_weights = torch.empty(M, topk, dtype=torch.float32, device=hidden_states.device)
    topk_ids = torch.empty(M, topk, dtype=torch.int32, device=hidden_states.device)
    topk_softmax(topk_weights, topk_ids, gating_output.contiguous(), renormalize)
    return topk_weights, topk_ids


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int,
                         num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(sorted_token_ids, expert_ids, num_tokens_post_padded)`` for block-wise expert GEMMs: slots sorted by
    expert, every expert padded to a multiple of ``block_size`` with the value ``topk_ids.numel()``.  Ids equal to
    -1 (experts of another rank) come first under expert id -1.  The padding is always written by the kernel, so
    no separate fill pass is made."""
    cap = topk_ids.numel() + (num_experts + 1) * (block_size - 1)
    sorted_ids = torch.empty((cap,), dtype=torch.int32, device=topk_ids.device)
    expert_ids = torch.empty((-(-cap // block_size),), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1,), dtype=torch.int32, device=topk_ids.device)
    cumsum_buffer = torch.empty((num_experts + 2,), dtype=torch.int32, device=topk_ids.device)
    _sgl_moe_align_block_size(topk_ids.contiguous(), num_experts + 1, block_size, sorted_ids, expert_ids,
                              num_tokens_post_pad, cumsum_buffer, True)
    return sorted_ids, expert_ids, num_tokens_post_pad


def biased_grouped_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, correction_bias: torch.Tensor,
                        topk: int, renormalize: bool, num_expert_group: Optional[int] = None,
                        topk_group: Optional[int] = None, num_fused_shared_experts: int = 0,
                        routed_scaling_factor: Optional[float] = None,
                        num_token_non_padded: Optional[torch.Tensor] = None, expert_location_dispatch_info=None,
                        apply_routed_scaling_factor_on_output: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """The DeepSeek-V3 gate (``python/sglang/srt/layers/moe/topk.py:691-768``): sigmoid scores, selection bias,
    group-limited top-k, renormalised weights.  One kernel for every expert count; like the reference's fused
    kernel it always renormalises, so ``renormalize=False`` is refused."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if not renormalize:
        raise RuntimeError("biased_grouped_topk: only renormalize=True is implemented (the fused gate renormalises)")
    if num_token_non_padded is not None or expert_location_dispatch_info is not None:
        raise RuntimeError("num_token_non_padded / expert_location_dispatch_info are not implemented")
    from ...sgl_kernel import moe_fused_gate
    return moe_fused_gate(gating_output.contiguous(), correction_bias.to(gating_output.dtype), num_expert_group,
                          topk_group, topk, num_fused_shared_experts,
                          routed_scaling_factor if routed_scaling_factor is not None else 0.0,
                          apply_routed_scaling_factor_on_output)
