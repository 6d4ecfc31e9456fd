"""GEMM + all-reduce over peer memory, on ONE GPU: the ranks of a tensor-parallel group are emulated by running
every rank's push GEMM first (they never wait) and every rank's reduce afterwards (its flags are then already set),
all buffers on the same device.  The real multi-process run over NVLink is in test_multigpu_gpu.py."""

import ctypes

import pytest
import torch

import oracle
from helpers import assert_gemm_close, make_activations, row_parallel_reference

pytestmark = pytest.mark.gpu


def _buffers(world, slot_elems):
    from sglang_b200._lib import lib
    L = lib()
    recv = [torch.zeros(L.sglb200_peer_recv_bytes(slot_elems), dtype=torch.uint8, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.sglb200_peer_flag_bytes(), dtype=torch.uint8, device="cuda") for _ in range(world)]
    recv_arr = (ctypes.c_void_p * world)(*[t.data_ptr() for t in recv])
    flag_arr = (ctypes.c_void_p * world)(*[t.data_ptr() for t in flags])
    return recv, flags, recv_arr, flag_arr


def _plain_partial(a_q, a_s, w, ws):
    """The rank's partial product as the plain entry points compute it: for M <= 128 the few-rows kernel with the
    library's own K-split (scratch + reduce kernel), above that the 128-row kernel without a split - in both cases the
    kernel and the order of additions the push variant uses, stored instead of pushed."""
    from sglang_b200._lib import blockwise_mm, check, lib
    M, K = a_q.shape
    N = w.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    args = (a_q.data_ptr(), w.data_ptr(), a_s.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, a_q.stride(0), w.stride(0),
            out.stride(0), a_s.stride(0), a_s.stride(1), ws.stride(0), ws.stride(1), 0)
    if M <= 128:
        blockwise_mm(*args, a_q.device, torch.cuda.current_stream().cuda_stream)
    else:
        check(lib().sglb200_fp8_blockwise_scaled_mm(*args, torch.cuda.current_stream().cuda_stream), "mm")
    return out


@pytest.mark.parametrize("world,M,N,K", [(2, 64, 512, 1024), (4, 1, 1024, 2048), (8, 130, 640, 2048), (8, 16, 7168, 2048),
                                         (2, 128, 576, 512), (2, 16, 1024, 8192), (2, 100, 7168, 16384),
                                         (4, 130, 1152, 8192), (2, 33, 7168, 16384), (8, 64, 576, 8192)])
def test_push_and_reduce_emulated_ranks(world, M, N, K):
    from sglang_b200._lib import lib
    from sglang_b200.distributed.peer_allreduce import peer_reduce, push_mm
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    slot = -(-M * N // 8) * 8
    recv, flags, recv_arr, flag_arr = _buffers(world, slot)
    wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=torch.Generator().manual_seed(N)) * 0.05)
    kr = K // world
    shards = [(wq[:, r * kr:(r + 1) * kr].contiguous().cuda(), ws[:, r * kr // 128:(r + 1) * kr // 128].contiguous().cuda())
              for r in range(world)]
    for epoch in range(1, 6):  # both slot sets, each reused
        x = make_activations(M, K, seed=epoch, outliers=False)
        partials = []
        for r in range(world):
            a_q, a_s = sglang_per_token_group_quant_fp8(x[:, r * kr:(r + 1) * kr].contiguous().cuda(), 128)
            push_mm(recv_arr, flag_arr, r, world, slot, a_q, a_s, shards[r][0], shards[r][1], torch.bfloat16)
            partials.append(_plain_partial(a_q, a_s, *shards[r]))
        outs = []
        for r in range(world):
            out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
            peer_reduce(recv[r].data_ptr(), flags[r].data_ptr(), out, world, slot)
            outs.append(out)
        torch.cuda.synchronize()
        assert lib().sglb200_read_device_status() == 0
        want = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        for part in partials:
            want += part.float()
        want = want.bfloat16()
        for r in range(world):
            assert torch.equal(outs[r], want), f"rank {r} epoch {epoch}"
        # the tensor-parallel semantic: every rank rounds its partial sum to bf16, then the partial sums are added
        # (python/sglang/srt/layers/linear.py:1361-1386); the oracle does the same on the K-slices
        assert_gemm_close(outs[0], row_parallel_reference(x, wq, ws, world), f"epoch {epoch}")
    if M <= 128:  # the other route for few rows: the 128-row kernel's push epilogue (no scratch buffer)
        for r in range(world):
            a_q, a_s = sglang_per_token_group_quant_fp8(x[:, r * kr:(r + 1) * kr].contiguous().cuda(), 128)
            push_mm(recv_arr, flag_arr, r, world, slot, a_q, a_s, shards[r][0], shards[r][1], torch.bfloat16,
                    use_workspace=False)
        outs = []
        for r in range(world):
            out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            peer_reduce(recv[r].data_ptr(), flags[r].data_ptr(), out, world, slot)
            outs.append(out)
        torch.cuda.synchronize()
        assert lib().sglb200_read_device_status() == 0
        assert all(torch.equal(o, outs[0]) for o in outs)
        assert_gemm_close(outs[0], row_parallel_reference(x, wq, ws, world), "push epilogue route")


@pytest.mark.parametrize("world,M,N,K", [(2, 130, 640, 1024), (4, 256, 1152, 2048), (8, 300, 7168, 2048),
                                         (8, 128, 1024, 1024), (4, 100, 576, 512), (3, 515, 384, 768)])
def test_two_shot_emulated_ranks(world, M, N, K):
    """Reduce-scatter + all-gather: every rank's scatter push, then every rank's reduce-scatter (its flags are then set),
    then every rank's gather.  Same bits as the one-shot exchange; one-shot and two-shot exchanges alternate on the same
    buffers."""
    from sglang_b200._lib import lib
    from sglang_b200.distributed.peer_allreduce import (peer_gather, peer_reduce, peer_reduce_scatter, push_mm,
                                                        push_mm_scatter)
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    slot = -(-M * N // 8) * 8
    recv, flags, recv_arr, flag_arr = _buffers(world, slot)
    wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=torch.Generator().manual_seed(N)) * 0.05)
    kr = K // world
    shards = [(wq[:, r * kr:(r + 1) * kr].contiguous().cuda(), ws[:, r * kr // 128:(r + 1) * kr // 128].contiguous().cuda())
              for r in range(world)]
    for epoch, two_shot in enumerate((True, True, False, True, True, False, True), start=1):
        x = make_activations(M, K, seed=epoch, outliers=False)
        partials = []
        for r in range(world):
            a_q, a_s = sglang_per_token_group_quant_fp8(x[:, r * kr:(r + 1) * kr].contiguous().cuda(), 128)
            (push_mm_scatter if two_shot else push_mm)(recv_arr, flag_arr, r, world, slot, a_q, a_s, shards[r][0],
                                                       shards[r][1], torch.bfloat16)
            partials.append(_plain_partial(a_q, a_s, *shards[r]) if M > 64 else None)
        outs = [torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        if two_shot:
            for r in range(world):
                peer_reduce_scatter(recv_arr, flag_arr, r, world, slot, outs[r])
            for r in range(world):
                peer_gather(recv[r].data_ptr(), flags[r].data_ptr(), r, world, slot, outs[r])
        else:
            for r in range(world):
                peer_reduce(recv[r].data_ptr(), flags[r].data_ptr(), outs[r], world, slot)
        torch.cuda.synchronize()
        assert lib().sglb200_read_device_status() == 0
        done = ctypes.c_int64(-1)
        for r in range(world):
            assert lib().sglb200_peer_completed(flags[r].data_ptr(), ctypes.byref(done)) == 0 and done.value == epoch
        if M > 64:
            want = torch.zeros(M, N, dtype=torch.float32, device="cuda")
            for part in partials:
                want += part.float()
            assert torch.equal(outs[0], want.bfloat16()), f"epoch {epoch}"
        for r in range(1, world):
            assert torch.equal(outs[r], outs[0]), f"rank {r} epoch {epoch}"
        assert_gemm_close(outs[0], row_parallel_reference(x, wq, ws, world), f"epoch {epoch}")


def test_two_shot_wait_runs_out_and_rejections():
    from sglang_b200._lib import lib
    from sglang_b200.distributed.peer_allreduce import peer_gather, peer_reduce_scatter, push_mm_scatter
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    M, N, K, world = 130, 256, 256, 2
    slot = M * N
    recv, flags, recv_arr, flag_arr = _buffers(world, slot)
    wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=torch.Generator().manual_seed(1)) * 0.05)
    a_q, a_s = sglang_per_token_group_quant_fp8(make_activations(M, K, seed=1, outliers=False).cuda(), 128)
    out = [torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    push_mm_scatter(recv_arr, flag_arr, 0, world, slot, a_q, a_s, wq.cuda(), ws.cuda(), torch.bfloat16)  # rank 1 silent
    peer_reduce_scatter(recv_arr, flag_arr, 0, world, slot, out[0], timeout_ns=20_000_000)
    peer_gather(recv[0].data_ptr(), flags[0].data_ptr(), 0, world, slot, out[0], timeout_ns=20_000_000)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 5 and lib().sglb200_read_device_status() == 0
    assert (out[0] == 7.0).all()
    done = ctypes.c_int64(-1)
    assert lib().sglb200_peer_completed(flags[0].data_ptr(), ctypes.byref(done)) == 0 and done.value == 0
    # the late rank arrives: the same exchange now completes on both ranks
    push_mm_scatter(recv_arr, flag_arr, 1, world, slot, a_q, a_s, wq.cuda(), ws.cuda(), torch.bfloat16)
    for r in range(world):
        peer_reduce_scatter(recv_arr, flag_arr, r, world, slot, out[r])
    for r in range(world):
        peer_gather(recv[r].data_ptr(), flags[r].data_ptr(), r, world, slot, out[r])
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 0
    for r in range(world):
        assert lib().sglb200_peer_completed(flags[r].data_ptr(), ctypes.byref(done)) == 0 and done.value == 1
    assert torch.equal(out[0], (_plain_partial(a_q, a_s, wq.cuda(), ws.cuda()).float() * 2).bfloat16())
    assert torch.equal(out[1], out[0])
    # fewer tiles than ranks: refused before anything is launched
    recv4, flags4, recv_arr4, flag_arr4 = _buffers(4, 64 * 256)
    with pytest.raises(RuntimeError, match="fewer output tiles than ranks"):
        push_mm_scatter(recv_arr4, flag_arr4, 0, 4, 64 * 256, a_q[:64], a_s[:64], wq.cuda(), ws.cuda(), torch.bfloat16)


def test_reduce_wait_runs_out_and_reports():
    """A rank that never pushes: the bounded wait gives up, the status word says so, the output is left alone and the
    context stays usable."""
    from sglang_b200._lib import lib
    from sglang_b200.distributed.peer_allreduce import peer_reduce, push_mm
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    M, N, K, world = 32, 256, 256, 2
    slot = M * N
    recv, flags, recv_arr, flag_arr = _buffers(world, slot)
    wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=torch.Generator().manual_seed(1)) * 0.05)
    a_q, a_s = sglang_per_token_group_quant_fp8(make_activations(M, K, seed=1, outliers=False).cuda(), 128)
    push_mm(recv_arr, flag_arr, 0, world, slot, a_q, a_s, wq.cuda(), ws.cuda(), torch.bfloat16)  # rank 1 stays silent
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    peer_reduce(recv[0].data_ptr(), flags[0].data_ptr(), out, world, slot, timeout_ns=20_000_000)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 5
    assert lib().sglb200_read_device_status() == 0  # reading clears it
    assert (out == 7.0).all()
    done = ctypes.c_int64(-1)
    assert lib().sglb200_peer_completed(flags[0].data_ptr(), ctypes.byref(done)) == 0 and done.value == 0
    # the late rank arrives: the same exchange now completes and the epoch advances
    push_mm(recv_arr, flag_arr, 1, world, slot, a_q, a_s, wq.cuda(), ws.cuda(), torch.bfloat16)
    peer_reduce(recv[0].data_ptr(), flags[0].data_ptr(), out, world, slot)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 0
    assert lib().sglb200_peer_completed(flags[0].data_ptr(), ctypes.byref(done)) == 0 and done.value == 1
    assert torch.equal(out, (_plain_partial(a_q, a_s, wq.cuda(), ws.cuda()).float() * 2).bfloat16())


def test_push_rejections():
    from sglang_b200.distributed.peer_allreduce import peer_reduce, push_mm
    recv, flags, recv_arr, flag_arr = _buffers(2, 1024)
    a_q = torch.zeros(16, 128, dtype=torch.float8_e4m3fn, device="cuda")
    a_s = torch.ones(16, 1, device="cuda")
    w = torch.zeros(128, 128, dtype=torch.float8_e4m3fn, device="cuda")
    ws = torch.ones(1, 1, device="cuda")
    with pytest.raises(RuntimeError, match="does not fit a receive slot"):
        push_mm(recv_arr, flag_arr, 0, 2, 1024, a_q, a_s, w, ws, torch.bfloat16)
    with pytest.raises(RuntimeError, match="world="):
        push_mm(recv_arr, flag_arr, 2, 2, 4096, a_q, a_s, w, ws, torch.bfloat16)
    with pytest.raises(RuntimeError, match="does not fit a receive slot"):
        peer_reduce(recv[0].data_ptr(), flags[0].data_ptr(), torch.empty(16, 128, dtype=torch.bfloat16, device="cuda"),
                    2, 1024)


def test_peer_exchange_single_rank_alloc_and_linear():
    """World of one: the library allocates the buffers and exports their IPC handles; the fused linear equals the
    plain one bit for bit."""
    from sglang_b200.distributed import PeerExchange, fused_row_parallel_linear
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    ex = PeerExchange(slot_elems=64 * 512)
    try:
        assert ex.world == 1 and ex.fits(64, 512) and not ex.fits(65, 512)
        wq, ws = oracle.block_quant_weight(torch.randn(512, 384, generator=torch.Generator().manual_seed(2)) * 0.05)
        for seed in (1, 2, 3):
            x = make_activations(64, 384, seed=seed, outliers=False).cuda()
            y = fused_row_parallel_linear(ex, x, wq.cuda(), ws.cuda())
            ref = _plain_partial(*sglang_per_token_group_quant_fp8(x, 128), wq.cuda(), ws.cuda())
            torch.cuda.synchronize()
            assert torch.equal(y, ref)
        assert ex.completed == 3
        # the pair of launches replays from a CUDA graph: the epoch is read and advanced on the device
        x = make_activations(64, 384, seed=9, outliers=False).cuda()
        w_d, ws_d = wq.cuda(), ws.cuda()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fused_row_parallel_linear(ex, x, w_d, ws_d)  # warm-up on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_g = fused_row_parallel_linear(ex, x, w_d, ws_d)
        before = ex.completed
        for _ in range(3):
            y_g.zero_()
            graph.replay()
        torch.cuda.synchronize()
        assert ex.completed == before + 3
        assert torch.equal(y_g, _plain_partial(*sglang_per_token_group_quant_fp8(x, 128), w_d, ws_d))
    finally:
        ex.close()
