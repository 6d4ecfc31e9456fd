"""All-reduce through NVSwitch multicast memory ("NVLS") for outputs too large for the push epilogues.

Mirrors ``SymmMemCommunicator`` (``python/sglang/srt/distributed/device_communicators/symm_mem.py:34-200``): one
symmetric buffer per rank allocated and exchanged by torch's symmetric-memory allocator (plumbing: ``cuMemCreate`` /
multicast binding / handle exchange), ``disabled`` when the node has no multicast support, ``should_symm_mem_allreduce``
and ``all_reduce(inp, out=None)`` with the reference's meaning.  The reduction itself is this library's kernel
(``sglb200_nvls_all_reduce``: ``multimem.ld_reduce`` / ``multimem.st`` on the multicast address, bounded barriers), not
``torch.ops.symm_mem.multimem_all_reduce_``.

What the reference's wrapper cannot do and this one adds: the producer writes INTO the symmetric buffer
(:meth:`view` gives the GEMM its ``out=`` tensor), so the two staging copies of ``all_reduce`` (in and out of the
buffer, ``symm_mem.py:191-199``) disappear; :func:`row_parallel_linear_symm_mem` is the row-parallel linear built that
way.  The returned tensor is a view of the buffer: it is valid until the next call that writes the same buffer.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Union

import torch
import torch.distributed as dist

from .._lib import check, dtype_code, lib

BLOCK = 128


class SymmMemCommunicator:
    """Sum over the ranks of one node through a multicast mapping.  Every rank of ``group`` must construct it, call
    it and close it in step (the kernels of all ranks pair up)."""

    def __init__(self, group, device: Union[int, str, torch.device], max_size: int = 256 << 20):
        self.disabled = True
        self.buffer = None
        self.declined_because = ""
        try:
            import torch.distributed._symmetric_memory as tsm
        except ImportError:
            return
        if isinstance(device, int):
            device = torch.device(f"cuda:{device}")
        elif isinstance(device, str):
            device = torch.device(device)
        self.device, self.group = device, group
        self.dtype = torch.bfloat16
        self.max_size = int(max_size)
        if device.type != "cuda" or not torch.cuda.is_available():
            return
        self.world_size = dist.get_world_size(group)
        if self.world_size < 2 or self.world_size > 8 or torch.cuda.get_device_capability(device)[0] != 10:
            return
        torch.cuda.set_device(device)
        # A rank that cannot set the mapping up (no multicast support, an allocator or handle-exchange error) must not
        # leave the others waiting in a later collective: every rank reports, and all decline together.
        ok, why = 1, ""
        try:
            name = group.group_name if group is not None else dist.group.WORLD.group_name
            self.buffer = tsm.empty(self.max_size // 2, device=device, dtype=self.dtype)
            handle = tsm.rendezvous(self.buffer, name)
            if handle.multicast_ptr == 0:  # no NVSwitch multicast on this node (symm_mem.py:103-110)
                ok, why = 0, "no multicast mapping"
            else:
                flag_words = lib().sglb200_nvls_flag_bytes() // 4
                self._flags = tsm.empty(flag_words, device=device, dtype=torch.int32)
                self._flags.zero_()
                fhandle = tsm.rendezvous(self._flags, name)
                self._handle, self._fhandle = handle, fhandle
                self.rank = handle.rank
                self._flag_blocks = (ctypes.c_uint64 * self.world_size)(*[int(p) for p in fhandle.buffer_ptrs])
                self._done = torch.zeros(64, device=device, dtype=torch.int32)  # row-block counters of the fused GEMM
                self.side_stream = torch.cuda.Stream(device)  # all-reduces of row chunks beside the next chunk's GEMM
        except Exception as e:  # noqa: BLE001 - declined, like the reference's wrapper; the reason is kept
            ok, why = 0, f"{type(e).__name__}: {e}"
        agreed = torch.tensor([ok], device=device, dtype=torch.int32)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)  # also: every flag block is zero before any kernel signals
        torch.cuda.synchronize(device)
        self.declined_because = why
        if int(agreed.item()) == 0:
            self.buffer = None
            return
        self.disabled = False

    # ------------------------------------------------------------------ the reference's interface
    def should_symm_mem_allreduce(self, inp: torch.Tensor) -> bool:
        """``symm_mem.py:113-135``: enabled, a 16-bit dtype this kernel adds, whole 16-byte vectors, fits the buffer."""
        if self.disabled or inp.dtype not in (torch.bfloat16, torch.float16):
            return False
        nbytes = inp.numel() * inp.element_size()
        return nbytes % 16 == 0 and nbytes <= self.max_size

    def all_reduce(self, inp: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Sum of ``inp`` over the ranks into ``out`` (a new tensor if omitted); ``None`` when disabled
        (``symm_mem.py:137-200``).  Stages through the symmetric buffer; producers that can write into the buffer
        use :meth:`view` and :meth:`all_reduce_` and skip both copies."""
        if self.disabled:
            return None
        if out is None:
            out = torch.empty_like(inp)
        staged = self.view(inp.shape, inp.dtype)
        staged.copy_(inp)
        self.all_reduce_(staged)
        out.copy_(staged)
        return out

    # ------------------------------------------------------------------ without staging
    def view(self, shape, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """A contiguous tensor of ``shape`` at the start of the symmetric buffer (the ``out=`` of the producer)."""
        if self.disabled:
            raise RuntimeError("SymmMemCommunicator is disabled (no multicast support, or not a B200 node)")
        n = 1
        for d in shape:
            n *= int(d)
        if dtype not in (torch.bfloat16, torch.float16) or n * 2 > self.max_size:
            raise ValueError(f"view of {tuple(shape)} {dtype}: 16-bit dtypes, at most {self.max_size} bytes")
        return self.buffer[:n].view(dtype).view(*shape)

    def all_reduce_(self, t: torch.Tensor, blocks: int = 0) -> torch.Tensor:
        """In-place sum of a tensor that lives in the symmetric buffer (from :meth:`view`), on the current stream.
        ``blocks`` (0 = all 128) is the kernel's grid and must be the same on every rank."""
        if self.disabled:
            raise RuntimeError("SymmMemCommunicator is disabled")
        off = t.data_ptr() - self.buffer.data_ptr()
        nbytes = t.numel() * t.element_size()
        if not t.is_contiguous() or off < 0 or off + nbytes > self.max_size or off % 16 or nbytes % 16:
            raise ValueError("all_reduce_ needs a contiguous 16-byte-aligned tensor inside the symmetric buffer")
        with torch.cuda.device(self.device):
            check(lib().sglb200_nvls_all_reduce(int(self._handle.multicast_ptr) + off, self._flag_blocks, self.rank,
                                                self.world_size, t.numel(), dtype_code(t.dtype), int(blocks),
                                                torch.cuda.current_stream(self.device).cuda_stream),
                  "nvls_all_reduce")
        return t

    def close(self) -> None:
        """Ranks leave together, with no kernel in flight, before the mappings go away."""
        if self.buffer is not None and not self.disabled:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        self.disabled = True
        self._handle = self._fhandle = None
        self._flags = None
        self.buffer = None


def row_parallel_linear_symm_mem(comm: SymmMemCommunicator, x: torch.Tensor, weight: torch.Tensor,
                                 weight_scale: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sum_r x_r @ W_r^T`` (+ bias): quantise, GEMM straight into the symmetric buffer, multicast all-reduce.
    The counterpart of ``RowParallelLinear.forward`` + ``tensor_model_parallel_all_reduce``
    (``python/sglang/srt/layers/linear.py:1361-1386``).  The result is a view of ``comm``'s buffer; ``bias`` is the
    WHOLE bias on every rank and is added once, after the sum (every rank holds the same sum)."""
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M, N = x2.shape[0], weight.shape[0]
    y = comm.view((M, N), x.dtype)
    if M:
        q, s = sglang_per_token_group_quant_fp8(x2, BLOCK, column_major_scales=True, scale_tma_aligned=True)
        w8a8_block_fp8_matmul(q, weight, s, weight_scale, [BLOCK, BLOCK], x.dtype, out=y)
        comm.all_reduce_(y)
        if bias is not None:
            y += bias
    return y.reshape(*x.shape[:-1], N)


def row_parallel_linear_symm_mem_overlapped(comm: SymmMemCommunicator, x: torch.Tensor, weight: torch.Tensor,
                                            weight_scale: torch.Tensor, chunk_rows: int = 4096, ar_blocks: int = 16,
                                            bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`row_parallel_linear_symm_mem` with the all-reduce of one row chunk running while the GEMM of the next
    chunk computes (the shape of the reference's two-batch overlap, ``two_batch_overlap.py``): the GEMM runs per chunk
    of ``chunk_rows`` rows into a row range of the symmetric buffer on ``148 - ar_blocks`` SMs
    (``configure_deep_gemm_num_sms``), and each range goes to the multicast all-reduce kernel with ``ar_blocks`` thread
    blocks on the communicator's side stream as soon as its GEMM has finished.  Same result as the unchunked form: the
    chunks only partition the rows.  Every rank must pass the same ``chunk_rows`` and ``ar_blocks``."""
    from ..layers.deep_gemm_wrapper import configure_deep_gemm_num_sms
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M, N = x2.shape[0], weight.shape[0]
    y = comm.view((M, N), x.dtype)
    if M == 0:
        return y.reshape(*x.shape[:-1], N)
    q, s = sglang_per_token_group_quant_fp8(x2, BLOCK, column_major_scales=True, scale_tma_aligned=True)
    main, side = torch.cuda.current_stream(comm.device), comm.side_stream
    sm_total = torch.cuda.get_device_properties(comm.device).multi_processor_count
    with configure_deep_gemm_num_sms(max(1, sm_total - ar_blocks)):
        for r0 in range(0, M, chunk_rows):
            r1 = min(M, r0 + chunk_rows)
            part = y[r0:r1]
            w8a8_block_fp8_matmul(q[r0:r1], weight, s[r0:r1], weight_scale, [BLOCK, BLOCK], x.dtype, out=part)
            done = torch.cuda.Event()
            done.record(main)
            side.wait_event(done)
            with torch.cuda.stream(side):
                comm.all_reduce_(part, blocks=ar_blocks)
    main.wait_stream(side)
    if bias is not None:
        y += bias
    return y.reshape(*x.shape[:-1], N)


def row_parallel_linear_symm_mem_fused(comm: SymmMemCommunicator, x: torch.Tensor, weight: torch.Tensor,
                                       weight_scale: torch.Tensor, comm_ctas: int = 16,
                                       bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`row_parallel_linear_symm_mem` with the GEMM and the all-reduce in ONE kernel launch
    (``sglb200_fp8_blockwise_scaled_mm_allreduce``): ``comm_ctas`` CTAs of the GEMM's grid sum every finished block of
    2048 output rows through the switch while the other CTAs compute the next block.  Same bits as the unfused form.
    Every rank must pass the same ``comm_ctas``; the result is a view of ``comm``'s buffer."""
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M, K = x2.shape
    N = weight.shape[0]
    y = comm.view((M, N), x.dtype)
    if M == 0:
        return y.reshape(*x.shape[:-1], N)
    q, s = sglang_per_token_group_quant_fp8(x2, BLOCK, column_major_scales=True, scale_tma_aligned=True)
    off = y.data_ptr() - comm.buffer.data_ptr()
    with torch.cuda.device(comm.device):
        check(lib().sglb200_fp8_blockwise_scaled_mm_allreduce(
            q.data_ptr(), weight.data_ptr(), s.data_ptr(), weight_scale.data_ptr(), y.data_ptr(),
            int(comm._handle.multicast_ptr) + off, comm._flag_blocks, comm._done.data_ptr(), comm.rank, comm.world_size,
            int(comm_ctas), M, N, K, q.stride(0), weight.stride(0), s.stride(0), s.stride(1), weight_scale.stride(0),
            weight_scale.stride(1), dtype_code(x.dtype), torch.cuda.current_stream(comm.device).cuda_stream),
            "fp8_blockwise_scaled_mm_allreduce")
    if bias is not None:
        y += bias
    return y.reshape(*x.shape[:-1], N)
