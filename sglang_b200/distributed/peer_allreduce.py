"""GEMM + all-reduce over peer memory for the row-parallel block-FP8 linear at small M.

The reference runs the row-parallel GEMM and then a separate custom all-reduce over IPC buffers
(``python/sglang/srt/layers/linear.py:1361-1386``,
``python/sglang/srt/distributed/device_communicators/custom_all_reduce.py``,
``sgl-kernel/csrc/allreduce/custom_all_reduce.cuh:203-266``).  Here the GEMM's epilogue stores each output tile
directly into every rank's receive buffer and flags it, and a second kernel per rank waits for the flags and adds the
``world`` partial sums in rank order (``include/sglb200.h``: ``sglb200_fp8_blockwise_scaled_mm_push``,
``sglb200_peer_reduce``); for larger outputs the two-shot form sends tile ``t`` to rank ``t % world`` only, which adds
it up and sends the result round (``..._push_scatter``, ``sglb200_peer_reduce_scatter``, ``sglb200_peer_gather``).  No NCCL call is on that path; ``torch.distributed`` is used once, to exchange the IPC
handles.  Every bounded wait that runs out is reported through ``sglb200_read_device_status`` (5).
"""

from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .._lib import check, dtype_code, lib

_VP = ctypes.c_void_p


class PeerExchange:
    """Receive buffer + flag words of this rank, mapped by every rank of ``group`` (CUDA IPC), and the pointers to
    the other ranks' buffers.  ``slot_elems`` bounds ``M * N`` of one exchange.  Collective: every rank of the group
    constructs it at the same point.  Mirrors the set-up half of ``CustomAllreduce.__init__``
    (``custom_all_reduce.py``: ``create_shared_buffer`` + handle all-gather)."""

    def __init__(self, slot_elems: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise RuntimeError("PeerExchange supports at most 8 ranks (one NVLink domain)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.slot_elems = -(-int(slot_elems) // 8) * 8
        L = lib()
        self._own: List[int] = []
        self._opened: List[int] = []
        self.recv_ptrs, self.flag_ptrs = [], []
        with torch.cuda.device(self.device):
            handles = []
            for nbytes in (L.sglb200_peer_recv_bytes(self.slot_elems), L.sglb200_peer_flag_bytes()):
                ptr, h = _VP(), (ctypes.c_ubyte * 64)()
                check(L.sglb200_peer_alloc(nbytes, ctypes.byref(ptr), h), "peer_alloc")
                self._own.append(ptr.value)
                handles.append(bytes(h))
            gathered = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(gathered, handles, group=group)
            else:
                gathered[0] = handles
            for which, out in ((0, self.recv_ptrs), (1, self.flag_ptrs)):
                for r in range(self.world):
                    if r == self.rank:
                        out.append(self._own[which])
                        continue
                    ptr = _VP()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r][which])
                    check(L.sglb200_peer_open(buf, ctypes.byref(ptr)), f"peer_open(rank {r})")
                    self._opened.append(ptr.value)
                    out.append(ptr.value)
        self._recv_arr = (_VP * self.world)(*self.recv_ptrs)
        self._flag_arr = (_VP * self.world)(*self.flag_ptrs)
        if self.world > 1:
            dist.barrier(group=group)  # nobody pushes before everybody has mapped

    @property
    def completed(self) -> int:
        """Exchanges this rank has completed (the device control word; synchronises the stream-ordered work)."""
        n = ctypes.c_int64()
        with torch.cuda.device(self.device):
            check(lib().sglb200_peer_completed(self.flag_ptrs[self.rank], ctypes.byref(n)), "peer_completed")
        return n.value

    # One-shot exchange: every rank sends its whole partial sum to every other rank.  Measured against NCCL (2 and 8
    # B200s, N = 7168): ahead up to about 16 MB leaving a rank per call, behind above that.  The two-shot exchange
    # (tile t reduced on rank t % world, results sent round) moves 2 (world - 1) / world of the output per rank; measured
    # on 4 B200s it is level with one shot at 5.5 MB of one-shot traffic, ahead of it from 11 MB, and ahead of NCCL up
    # to 11 MB of its own traffic (behind at 22 MB).
    MAX_OUT_BYTES = 16 << 20
    ONE_SHOT_BYTES_FROM_FOUR_RANKS = 8 << 20

    def _fits_buffers(self, M: int, N: int) -> bool:
        return M * N <= self.slot_elems and -(-M // 128) * -(-N // 128) <= 1024

    def fits(self, M: int, N: int) -> bool:
        """The one-shot exchange is allowed and worth it for an ``[M, N]`` output."""
        limit = self.MAX_OUT_BYTES if self.world < 4 else self.ONE_SHOT_BYTES_FROM_FOUR_RANKS
        return self._fits_buffers(M, N) and (self.world - 1) * M * N * 2 <= limit

    def fits_two_shot(self, M: int, N: int) -> bool:
        """The two-shot exchange is allowed and worth it (a larger output than :meth:`fits` takes, four ranks or more,
        at least one tile per rank)."""
        return (self.world >= 4 and self._fits_buffers(M, N) and -(-M // 128) * -(-N // 128) >= self.world
                and 2 * (self.world - 1) * M * N * 2 <= self.world * self.MAX_OUT_BYTES)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (collective: all ranks first stop using them)."""
        if not self._own:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        L = lib()
        with torch.cuda.device(self.device):
            for p in self._opened:
                L.sglb200_peer_close(p)
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            for p in self._own:
                L.sglb200_peer_free(p)
        self._own, self._opened = [], []


def push_mm(ex_recv_arr, ex_flag_arr, rank: int, world: int, slot_elems: int, a_q: torch.Tensor,
            a_s: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, out_dtype: torch.dtype,
            use_workspace: bool = True) -> None:
    """One rank's half of the exchange: ``a_q [M, K_r]`` e4m3 with scales ``a_s [M, K_r/128]`` times the rank's weight
    slice ``[N, K_r]``, every output tile stored into all ranks' receive buffers.  For ``M <= 128`` a scratch buffer
    lets the library take the few-rows kernel (``use_workspace=False`` forces the 128-row kernel's push epilogue)."""
    M, K = a_q.shape
    N = weight.shape[0]
    L = lib()
    ws_bytes = L.sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes(M, N, K) if use_workspace else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a_q.device) if ws_bytes > 0 else None
    check(L.sglb200_fp8_blockwise_scaled_mm_push(
        a_q.data_ptr(), weight.data_ptr(), a_s.data_ptr(), weight_scale.data_ptr(), M, N, K, a_q.stride(0),
        weight.stride(0), a_s.stride(0), a_s.stride(1), weight_scale.stride(0), weight_scale.stride(1),
        dtype_code(out_dtype), ex_recv_arr, ex_flag_arr, rank, world, slot_elems,
        ws.data_ptr() if ws is not None else None, ws_bytes,
        torch.cuda.current_stream(a_q.device).cuda_stream), "fp8_blockwise_scaled_mm_push")


def peer_reduce(recv_ptr: int, flag_ptr: int, out: torch.Tensor, world: int, slot_elems: int,
                timeout_ns: int = 0) -> None:
    """The receiving half: wait for every rank's tiles of this epoch and add them up into ``out [M, N]``."""
    check(lib().sglb200_peer_reduce(recv_ptr, flag_ptr, out.data_ptr(), out.size(0), out.size(1), out.stride(0),
                                    dtype_code(out.dtype), world, slot_elems, timeout_ns,
                                    torch.cuda.current_stream(out.device).cuda_stream), "peer_reduce")


def push_mm_scatter(ex_recv_arr, ex_flag_arr, rank: int, world: int, slot_elems: int, a_q: torch.Tensor,
                    a_s: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, out_dtype: torch.dtype) -> None:
    """First launch of the two-shot exchange: as :func:`push_mm`, but output tile ``t`` goes to rank ``t % world``."""
    M, K = a_q.shape
    N = weight.shape[0]
    check(lib().sglb200_fp8_blockwise_scaled_mm_push_scatter(
        a_q.data_ptr(), weight.data_ptr(), a_s.data_ptr(), weight_scale.data_ptr(), M, N, K, a_q.stride(0),
        weight.stride(0), a_s.stride(0), a_s.stride(1), weight_scale.stride(0), weight_scale.stride(1),
        dtype_code(out_dtype), ex_recv_arr, ex_flag_arr, rank, world, slot_elems,
        torch.cuda.current_stream(a_q.device).cuda_stream), "fp8_blockwise_scaled_mm_push_scatter")


def peer_reduce_scatter(ex_recv_arr, ex_flag_arr, rank: int, world: int, slot_elems: int, out: torch.Tensor,
                        timeout_ns: int = 0) -> None:
    """Second launch: add up the tiles this rank owns, write them to ``out`` and send them to the other ranks."""
    check(lib().sglb200_peer_reduce_scatter(ex_recv_arr, ex_flag_arr, out.data_ptr(), out.size(0), out.size(1),
                                            out.stride(0), dtype_code(out.dtype), rank, world, slot_elems, timeout_ns,
                                            torch.cuda.current_stream(out.device).cuda_stream), "peer_reduce_scatter")


def peer_gather(recv_ptr: int, flag_ptr: int, rank: int, world: int, slot_elems: int, out: torch.Tensor,
                timeout_ns: int = 0) -> None:
    """Third launch: copy the tiles the other ranks reduced into ``out``."""
    check(lib().sglb200_peer_gather(recv_ptr, flag_ptr, out.data_ptr(), out.size(0), out.size(1), out.stride(0),
                                    dtype_code(out.dtype), rank, world, slot_elems, timeout_ns,
                                    torch.cuda.current_stream(out.device).cuda_stream), "peer_gather")


def fused_row_parallel_linear(ex: PeerExchange, x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                              bias: Optional[torch.Tensor] = None, two_shot: Optional[bool] = None) -> torch.Tensor:
    """``all_reduce(x_r @ W_r^T)`` for this rank's activation slice ``x [.., K_r]`` (bf16 / f16) and weight slice
    ``[N, K_r]`` with block scales ``[N/128, K_r/128]``: quantise, GEMM with the push epilogue, reduce.  The caller
    checks ``ex.fits(M, N)`` / ``ex.fits_two_shot(M, N)`` and takes the NCCL path otherwise
    (``RowParallelBlockFp8Linear`` does).  ``two_shot`` (default: one shot where ``ex.fits`` allows it, else two) selects
    the exchange; every rank must select the same one."""
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    x2 = x.reshape(-1, x.shape[-1])
    M, N = x2.shape[0], weight.shape[0]
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if M == 0:
        return out.reshape(*x.shape[:-1], N)
    if two_shot is None:
        two_shot = not ex.fits(M, N) and ex.fits_two_shot(M, N)
    a_q, a_s = sglang_per_token_group_quant_fp8(x2.contiguous(), 128, column_major_scales=False)
    with torch.cuda.device(x.device):
        if two_shot:
            push_mm_scatter(ex._recv_arr, ex._flag_arr, ex.rank, ex.world, ex.slot_elems, a_q, a_s, weight, weight_scale,
                            x.dtype)
            peer_reduce_scatter(ex._recv_arr, ex._flag_arr, ex.rank, ex.world, ex.slot_elems, out)
            peer_gather(ex.recv_ptrs[ex.rank], ex.flag_ptrs[ex.rank], ex.rank, ex.world, ex.slot_elems, out)
        else:
            push_mm(ex._recv_arr, ex._flag_arr, ex.rank, ex.world, ex.slot_elems, a_q, a_s, weight, weight_scale, x.dtype)
            peer_reduce(ex.recv_ptrs[ex.rank], ex.flag_ptrs[ex.rank], out, ex.world, ex.slot_elems)
    if bias is not None:
        out += bias
    return out.reshape(*x.shape[:-1], N)
