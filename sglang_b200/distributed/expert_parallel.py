"""Expert-parallel fused MoE with all-to-all token dispatch and combine.

Experts are partitioned contiguously, ``E / ep`` per rank (``layers/moe/fused_moe_triton/layer.py:163-171``).
A token is sent ONCE to every rank that owns at least one of its top-k experts, as fp8 codes plus
per-group scales (7168 + 224 bytes per DeepSeek-V3 token instead of 14336), together with its local
expert ids and routing weights; the owner runs the grouped expert MLP on what it received and sends
one bf16 partial row back per received token; the source adds the partial rows.  This is the
dispatch / combine contract of ``token_dispatcher/deepep.py:345-504`` over NCCL
(``all_to_all_single`` with a count exchange first), one process per GPU.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def ep_owner_tables(topk_ids: torch.Tensor, num_local_experts: int, ep_size: int):
    """For every destination rank r: ``send_idx[r]`` (token indices that have an expert on r, ascending) and
    ``local_ids`` ``[M, ep, topk]`` with the expert id relative to r's first expert, or -1 for slots owned by
    another rank.  Pure index arithmetic on the routing result."""
    owner = torch.div(topk_ids, num_local_experts, rounding_mode="floor")           # [M, topk]
    ranks = torch.arange(ep_size, device=topk_ids.device).view(1, ep_size, 1)
    mine = owner.unsqueeze(1) == ranks                                               # [M, ep, topk]
    local_ids = torch.where(mine, topk_ids.unsqueeze(1) - ranks * num_local_experts,
                            torch.full_like(topk_ids.unsqueeze(1), -1)).to(torch.int32)
    has = mine.any(dim=-1)                                                           # [M, ep]
    send_idx = [torch.nonzero(has[:, r], as_tuple=False).flatten() for r in range(ep_size)]
    return send_idx, local_ids


def _all_to_all(x: torch.Tensor, in_splits, out_splits, group):
    out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
    return out


def ep_fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w1_scale: torch.Tensor,
                     w2_scale: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, ep_rank: int,
                     ep_size: int, group=None, quant_fn: Optional[Callable] = None,
                     experts_fn: Optional[Callable] = None) -> torch.Tensor:
    """Expert-parallel MoE layer for the tokens of THIS rank.

    hidden_states ``[M, H]`` (this rank's tokens); w1 / w2 / scales hold this rank's ``E / ep`` experts;
    topk_ids ``[M, topk]`` are GLOBAL expert ids.  Returns ``[M, H]``.  ``quant_fn`` / ``experts_fn`` default
    to the CUDA kernels (``sglang_per_token_group_quant_fp8``, ``fused_experts_block_fp8_prequant``)."""
    if quant_fn is None or experts_fn is None:
        from ..layers.moe import fused_experts_block_fp8_prequant
        from ..layers.quantization import sglang_per_token_group_quant_fp8
        quant_fn = quant_fn or (lambda x: sglang_per_token_group_quant_fp8(x, 128))
        experts_fn = experts_fn or fused_experts_block_fp8_prequant
    M, H = hidden_states.shape
    e_local = w1.shape[0]
    dev = hidden_states.device
    send_idx, local_ids = ep_owner_tables(topk_ids, e_local, ep_size)
    send_counts = [int(i.numel()) for i in send_idx]
    counts = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=group)
    recv_counts = [int(c) for c in recv.tolist()]

    # dispatch: fp8 codes + scales + local expert ids + weights, grouped by destination rank
    a_q, a_s = quant_fn(hidden_states)
    order = torch.cat(send_idx)
    dest = torch.cat([torch.full((n,), r, dtype=torch.long, device=dev) for r, n in enumerate(send_counts)])
    q_recv = _all_to_all(a_q.view(torch.uint8)[order], send_counts, recv_counts, group).view(a_q.dtype)
    s_recv = _all_to_all(a_s[order], send_counts, recv_counts, group)
    ids_recv = _all_to_all(local_ids[order, dest], send_counts, recv_counts, group)
    w_recv = _all_to_all(topk_weights.to(torch.float32)[order], send_counts, recv_counts, group)

    # local experts on the received rows (slots of other ranks carry id -1 and contribute nothing)
    partial = experts_fn(q_recv.contiguous(), s_recv.contiguous(), hidden_states.dtype, w1, w2, w1_scale, w2_scale,
                         w_recv, ids_recv)

    # combine: one partial row back per dispatched row, summed at the source in fp32
    back = _all_to_all(partial, recv_counts, send_counts, group)
    out = torch.zeros(M, H, dtype=torch.float32, device=dev)
    out.index_add_(0, order, back.to(torch.float32))
    return out.to(hidden_states.dtype)
