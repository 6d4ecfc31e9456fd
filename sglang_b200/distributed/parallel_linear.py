"""Column- and row-parallel block-FP8 linear layers.

Mirrors ``ColumnParallelLinear`` / ``RowParallelLinear`` (``python/sglang/srt/layers/linear.py:263-430,
1194-1386``) for block-quantised weights: one process per GPU, the weight shard of this rank,
``quant_method.apply`` for the local GEMM, and ``tensor_model_parallel_all_reduce``
(``python/sglang/srt/distributed/communication_op.py:11-13``) on the row-parallel output.
Splits must fall on 128-element block boundaries (``quantization/fp8.py:251-269``), so activation
groups and weight blocks never straddle ranks and the local quantisation is exactly the slice of
the global one.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

BLOCK = 128


def tensor_model_parallel_all_reduce(x: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over the tensor-parallel group, in place (no-op for a single rank)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, group=group)
    return x


def row_parallel_linear_overlapped(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, group=None,
                                   chunk_rows: int = 2048, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``all_reduce(x_r @ W_r^T)`` with the all-reduce of one row chunk running while the GEMM of the next one computes.

    The activations are quantised once; the GEMM then runs per chunk of ``chunk_rows`` rows into a row range of the
    result, and each range is handed to an asynchronous NCCL all-reduce as soon as its GEMM is enqueued (NCCL orders it
    after that GEMM on its own stream).  Same result as :class:`RowParallelBlockFp8Linear` without a peer exchange: the
    chunks only partition the rows.  ``bias`` (rank 0 only, as ``linear.py:1374``) is added before the reduction.
    The GEMM is a persistent kernel that fills every SM, so a concurrent NCCL kernel would have to wait for its CTAs to
    finish: callers leave SMs free for it with ``configure_deep_gemm_num_sms`` (``layers.deep_gemm_wrapper``), as the
    reference does around its overlapped GEMMs (``two_batch_overlap.py:841``)."""
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M, N = x2.shape[0], weight.shape[0]
    y = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if M == 0:
        return y.reshape(*x.shape[:-1], N)
    q, s = sglang_per_token_group_quant_fp8(x2, BLOCK, column_major_scales=True, scale_tma_aligned=True)
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    works = []
    for r0 in range(0, M, chunk_rows):
        r1 = min(M, r0 + chunk_rows)
        part = y[r0:r1]
        w8a8_block_fp8_matmul(q[r0:r1], weight, s[r0:r1], weight_scale, [BLOCK, BLOCK], x.dtype, out=part)
        if bias is not None:
            part += bias
        if multi:
            works.append(dist.all_reduce(part, group=group, async_op=True))
    for w in works:
        w.wait()
    return y.reshape(*x.shape[:-1], N)


def shard_block_fp8_weight(weight: torch.Tensor, scale: torch.Tensor, rank: int, world: int,
                           dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Slice ``weight [N, K]`` (e4m3) and ``scale [ceil(N/128), ceil(K/128)]`` for one rank along
    ``dim`` (0 = output/column-parallel, 1 = input/row-parallel).  The per-rank extent must be a
    multiple of the 128 block, as ``Fp8LinearMethod.create_weights`` requires."""
    size = weight.shape[dim]
    if size % world != 0 or (size // world) % BLOCK != 0:
        raise ValueError(f"dimension {dim} of size {size} cannot be split over {world} ranks on "
                         f"{BLOCK}-element block boundaries")
    per = size // world
    w = weight.narrow(dim, rank * per, per).contiguous()
    s = scale.narrow(dim, rank * per // BLOCK, per // BLOCK).contiguous()
    return w, s


class _ParallelBase(torch.nn.Module):
    def __init__(self, weight, scale, bias, apply_fn, group):
        super().__init__()
        self.weight = torch.nn.Parameter(weight, requires_grad=False)
        self.weight_scale_inv = torch.nn.Parameter(scale, requires_grad=False)
        self.bias = None if bias is None else torch.nn.Parameter(bias, requires_grad=False)
        self.group = group
        if apply_fn is None:
            from ..layers.quantization import Fp8Config, Fp8LinearMethod
            apply_fn = Fp8LinearMethod(Fp8Config()).apply
        self._apply = apply_fn


class ColumnParallelBlockFp8Linear(_ParallelBase):
    """``Y_r = X W_r^T``: each rank owns ``N / tp`` output features; no exchange unless
    ``gather_output`` (then an all-gather along the last dimension, ``linear.py:430``)."""

    def __init__(self, weight, scale, rank: int, world: int, bias: Optional[torch.Tensor] = None,
                 gather_output: bool = False, apply_fn: Optional[Callable] = None, group=None):
        w, s = shard_block_fp8_weight(weight, scale, rank, world, 0)
        b = None if bias is None else bias.chunk(world)[rank].contiguous()
        super().__init__(w, s, b, apply_fn, group)
        self.gather_output, self.world = gather_output, world

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._apply(self, x, self.bias)
        if self.gather_output and self.world > 1:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelBlockFp8Linear(_ParallelBase):
    """``Y = sum_r X_r W_r^T``: each rank owns ``K / tp`` input features of the weight and the
    matching slice of the activations; the partial outputs are summed with one all-reduce
    (``linear.py:1361-1386``).  The bias is added once, on rank 0, before the reduction.

    With a ``peer_exchange`` (:class:`~sglang_b200.distributed.peer_allreduce.PeerExchange`) and an output that fits
    its receive slot, the GEMM pushes its tiles into every rank's memory and the sum is taken there: no NCCL call
    (the reference switches to its custom all-reduce below a size threshold the same way,
    ``custom_all_reduce.py: should_custom_ar``); from four ranks up, outputs too large for that take the two-shot form
    (tile t reduced on rank t % world, results sent round).  Larger outputs take the multicast all-reduce of a
    ``symm_mem`` communicator (:class:`~sglang_b200.distributed.symm_mem.SymmMemCommunicator`; the GEMM writes into its
    symmetric buffer and the returned tensor is a view of it; with ``symm_mem_fused_ctas`` GEMM and all-reduce are one
    launch, with ``symm_mem_chunk_rows`` the all-reduce of a row chunk runs beside the next chunk's GEMM) when one is
    given and enabled, else the NCCL all-reduce.
    On that path the sum is taken by every rank for itself, so every rank keeps the whole bias and adds it once after
    the sum (decided here, where all ranks see the same arguments, not per rank in ``forward``)."""

    def __init__(self, weight, scale, rank: int, world: int, bias: Optional[torch.Tensor] = None,
                 input_is_parallel: bool = True, reduce_results: bool = True,
                 apply_fn: Optional[Callable] = None, group=None, peer_exchange=None, symm_mem=None,
                 symm_mem_chunk_rows: int = 0, symm_mem_blocks: int = 16, symm_mem_fused_ctas: int = 0):
        w, s = shard_block_fp8_weight(weight, scale, rank, world, 1)
        super().__init__(w, s, bias if rank == 0 else None, apply_fn, group)
        self.rank, self.world = rank, world
        self.input_is_parallel, self.reduce_results = input_is_parallel, reduce_results
        self.peer_exchange = peer_exchange
        self.symm_mem = symm_mem
        # > 0: inputs with more rows run in chunks of this many, a chunk's all-reduce beside the next chunk's GEMM
        self.symm_mem_chunk_rows, self.symm_mem_blocks = int(symm_mem_chunk_rows), int(symm_mem_blocks)
        # > 0: GEMM and all-reduce in one launch with this many communication CTAs (inputs of more than 2048 rows)
        self.symm_mem_fused_ctas = int(symm_mem_fused_ctas)
        self.bias_after_sum = None
        if (peer_exchange is not None or symm_mem is not None) and bias is not None:
            self.bias_after_sum = torch.nn.Parameter(bias, requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel:
            per = x.shape[-1] // self.world
            x = x.narrow(-1, self.rank * per, per).contiguous()
        ex = self.peer_exchange
        if (ex is not None and self.reduce_results and self.world > 1 and x.is_cuda
                and (ex.fits(x.numel() // x.shape[-1], self.weight.shape[0])
                     or ex.fits_two_shot(x.numel() // x.shape[-1], self.weight.shape[0]))):
            from .peer_allreduce import fused_row_parallel_linear
            return fused_row_parallel_linear(ex, x, self.weight, self.weight_scale_inv, self.bias_after_sum)
        sm = self.symm_mem
        if (sm is not None and not sm.disabled and self.reduce_results and self.world > 1 and x.is_cuda
                and x.dtype in (torch.bfloat16, torch.float16)
                and (x.numel() // x.shape[-1]) * self.weight.shape[0] * 2 <= sm.max_size):
            from .symm_mem import (row_parallel_linear_symm_mem, row_parallel_linear_symm_mem_fused,
                                   row_parallel_linear_symm_mem_overlapped)
            if self.symm_mem_fused_ctas > 0 and x.numel() // x.shape[-1] > 2048:
                return row_parallel_linear_symm_mem_fused(sm, x, self.weight, self.weight_scale_inv,
                                                          self.symm_mem_fused_ctas, self.bias_after_sum)
            if 0 < self.symm_mem_chunk_rows < x.numel() // x.shape[-1]:
                return row_parallel_linear_symm_mem_overlapped(sm, x, self.weight, self.weight_scale_inv,
                                                               self.symm_mem_chunk_rows, self.symm_mem_blocks,
                                                               self.bias_after_sum)
            return row_parallel_linear_symm_mem(sm, x, self.weight, self.weight_scale_inv, self.bias_after_sum)
        y = self._apply(self, x, self.bias)
        if self.reduce_results:
            y = tensor_model_parallel_all_reduce(y, self.group)
        return y
