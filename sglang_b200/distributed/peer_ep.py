"""Expert-parallel MoE whose dispatch and combine run over peer memory (NVLink, CUDA-IPC mapped buffers) instead of
NCCL all-to-alls: no collective call and no host round trip for the row counts on the path, so the layer is enqueued
without ever synchronising the stream.  The contract is the one of ``token_dispatcher/deepep.py:345-504`` (dispatch fp8
rows + scales + ids + weights to the ranks that own a token's experts, run the local experts, return one partial row
per received row, add the partial rows at the source); the kernels are described in ``include/sglb200.h``
(``sglb200_ep_dispatch`` ... ``sglb200_ep_combine_reduce``).
"""

from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .._lib import check, dtype_code, lib

_VP = ctypes.c_void_p


class _Raw:
    """A range of device memory for ``torch.as_tensor`` (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def buffer_views(base_ptr: int, device, capacity: int, H: int, topk: int, world: int, m_max: int):
    """Torch views of the receive arrays inside an exchange buffer: ``(recv_q [C, H] e4m3, recv_s [C, H/128] f32,
    recv_ids [C, topk] i32, recv_w [C, topk] f32)``."""
    off = (ctypes.c_int64 * 7)()
    check(lib().sglb200_ep_buffer_offsets(capacity, H, topk, world, m_max, off), "ep_buffer_offsets")

    def view(o, nbytes, dtype, shape):
        return torch.as_tensor(_Raw(base_ptr + o, nbytes), device=device).view(dtype).view(shape)

    G = H // 128
    return (view(off[0], capacity * H, torch.float8_e4m3fn, (capacity, H)),
            view(off[1], capacity * G * 4, torch.float32, (capacity, G)),
            view(off[3], capacity * topk * 4, torch.int32, (capacity, topk)),
            view(off[4], capacity * topk * 4, torch.float32, (capacity, topk)))


class PeerEpExchange:
    """This rank's exchange buffer, mapped by every rank of ``group``, and the pointers to the other ranks' buffers.
    ``capacity`` = rows this rank can receive per call, ``m_max`` = tokens a rank may dispatch per call.  A token is
    sent to a rank at most once, so ``world * m_max`` rows always fit; a smaller ``capacity`` is refused here, because a
    full receive buffer drops rows on the device (status 23 is the only trace) and the combine would then add whatever
    an earlier exchange left in the dropped row's slot.  Collective: every rank constructs it at the same point."""

    def __init__(self, capacity: int, hidden: int, topk: int, m_max: int, group=None,
                 device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise RuntimeError("PeerEpExchange supports at most 8 ranks (one NVLink domain)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.capacity, self.hidden, self.topk, self.m_max = int(capacity), int(hidden), int(topk), int(m_max)
        if self.capacity < self.world * self.m_max:
            raise ValueError(f"capacity={self.capacity} rows cannot hold the {self.world} x {self.m_max} tokens the ranks "
                             "may dispatch to one rank: rows would be dropped")
        L = lib()
        self._opened: List[int] = []
        with torch.cuda.device(self.device):
            nbytes = L.sglb200_ep_buffer_bytes(self.capacity, self.hidden, self.topk, self.world, self.m_max)
            ptr, h = _VP(), (ctypes.c_ubyte * 64)()
            check(L.sglb200_peer_alloc(nbytes, ctypes.byref(ptr), h), "peer_alloc")
            self._own = ptr.value
            gathered = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(gathered, bytes(h), group=group)
            self.bases = []
            for r in range(self.world):
                if r == self.rank:
                    self.bases.append(self._own)
                    continue
                p = _VP()
                check(L.sglb200_peer_open((ctypes.c_ubyte * 64).from_buffer_copy(gathered[r]), ctypes.byref(p)),
                      f"peer_open(rank {r})")
                self._opened.append(p.value)
                self.bases.append(p.value)
        self._arr = (_VP * self.world)(*self.bases)
        self.recv_q, self.recv_s, self.recv_ids, self.recv_w = buffer_views(
            self._own, self.device, self.capacity, self.hidden, self.topk, self.world, self.m_max)
        self.count = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    @property
    def completed(self) -> int:
        """Exchanges this rank has completed (the device control word; synchronises the stream-ordered work)."""
        n = ctypes.c_int64()
        with torch.cuda.device(self.device):
            check(lib().sglb200_ep_completed(self._own, self.capacity, self.hidden, self.topk, self.world, self.m_max,
                                             ctypes.byref(n)), "ep_completed")
        return n.value

    def close(self) -> None:
        if self._own is None:
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
            L.sglb200_peer_free(self._own)
        self._own, self._opened = None, []


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def ep_dispatch(arr, rank, world, capacity, m_max, a_q, a_s, topk_ids, topk_weights, e_local) -> None:
    M, H = a_q.shape
    check(lib().sglb200_ep_dispatch(a_q.data_ptr(), a_s.data_ptr(), a_s.stride(0), a_s.stride(1), topk_ids.data_ptr(),
                                    topk_weights.data_ptr(), M, H, topk_ids.size(1), e_local, arr, rank, world,
                                    capacity, m_max, _stream(a_q.device)), "ep_dispatch")


def ep_dispatch_quant(arr, rank, world, capacity, m_max, x, topk_ids, topk_weights, e_local, eps=1e-10) -> None:
    """Quantise ``x [M, H]`` (bf16 / f16, unit column stride) per 128-wide group and dispatch it, in one kernel."""
    M, H = x.shape
    assert x.stride(1) == 1 or M <= 1
    check(lib().sglb200_ep_dispatch_quant(x.data_ptr(), dtype_code(x.dtype), x.stride(0) if M > 1 else H,
                                          topk_ids.data_ptr(), topk_weights.data_ptr(), M, H, topk_ids.size(1),
                                          e_local, arr, rank, world, capacity, m_max, eps, _stream(x.device)),
          "ep_dispatch_quant")


def ep_receive(arr, rank, world, H, topk, e_local, capacity, m_max, count, timeout_ns=0) -> None:
    check(lib().sglb200_ep_receive(arr, rank, world, H, topk, e_local, capacity, m_max,
                                   count.data_ptr() if count is not None else None, timeout_ns,
                                   _stream(count.device if count is not None else None)), "ep_receive")


def ep_combine_push(arr, rank, world, H, topk, e_local, capacity, m_max, partial) -> None:
    check(lib().sglb200_ep_combine_push(partial.data_ptr(), dtype_code(partial.dtype), arr, rank, world, H, topk,
                                        e_local, capacity, m_max, _stream(partial.device)), "ep_combine_push")


def ep_combine_reduce(arr, rank, world, topk_ids, out, e_local, capacity, m_max, timeout_ns=0) -> None:
    M, H = out.shape
    check(lib().sglb200_ep_combine_reduce(arr, rank, world, topk_ids.data_ptr(), out.data_ptr(),
                                          dtype_code(out.dtype), M, H, topk_ids.size(1), e_local, capacity, m_max,
                                          timeout_ns, _stream(out.device)), "ep_combine_reduce")


def ep_fused_experts_peer(ex: PeerEpExchange, hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                          w1_scale: torch.Tensor, w2_scale: torch.Tensor, topk_weights: torch.Tensor,
                          topk_ids: torch.Tensor, fuse_quant: bool = True) -> torch.Tensor:
    """The expert-parallel MoE layer for the tokens of THIS rank (same contract as
    :func:`sglang_b200.distributed.ep_fused_experts`): ``w1 / w2`` hold this rank's ``E / ep`` experts, ``topk_ids`` are
    global expert ids.  Four launches around the local expert MLP (the quantiser runs inside the dispatch kernel;
    ``fuse_quant=False`` keeps it as a launch of its own, with identical results); nothing synchronises the stream and
    the exchange counter lives on the device, so the whole layer can be captured in a CUDA graph."""
    from ..layers.moe import fused_experts_block_fp8_prequant
    from ..layers.quantization import sglang_per_token_group_quant_fp8
    M, H = hidden_states.shape
    assert H == ex.hidden and topk_ids.size(1) == ex.topk and M <= ex.m_max
    e_local = w1.shape[0]
    ids = topk_ids.to(torch.int32).contiguous()
    w = topk_weights.to(torch.float32).contiguous()
    out = torch.empty(M, H, dtype=hidden_states.dtype, device=hidden_states.device)
    args = (ex._arr, ex.rank, ex.world)
    with torch.cuda.device(hidden_states.device):
        if fuse_quant:
            ep_dispatch_quant(*args, ex.capacity, ex.m_max, hidden_states.contiguous(), ids, w, e_local)
        else:
            if M > 0:
                a_q, a_s = sglang_per_token_group_quant_fp8(hidden_states.contiguous(), 128)
            else:
                a_q = torch.empty(0, H, dtype=torch.float8_e4m3fn, device=hidden_states.device)
                a_s = torch.empty(0, H // 128, device=hidden_states.device)
            ep_dispatch(*args, ex.capacity, ex.m_max, a_q, a_s, ids, w, e_local)
        ep_receive(*args, H, ex.topk, e_local, ex.capacity, ex.m_max, ex.count)
        partial = fused_experts_block_fp8_prequant(ex.recv_q, ex.recv_s, hidden_states.dtype, w1, w2, w1_scale, w2_scale,
                                                   ex.recv_w, ex.recv_ids)
        ep_combine_push(*args, H, ex.topk, e_local, ex.capacity, ex.m_max, partial)
        ep_combine_reduce(*args, ids, out, e_local, ex.capacity, ex.m_max)
    return out
