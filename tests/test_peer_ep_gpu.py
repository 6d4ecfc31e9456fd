"""Expert-parallel dispatch / combine over peer memory, on ONE GPU: the ranks are emulated by running every rank's
dispatch first (it never waits), then every rank's receive, expert MLP and combine-push, then every rank's combine-reduce,
all exchange buffers on the same device.  The real multi-process run over NVLink is in test_multigpu_gpu.py."""

import ctypes

import pytest
import torch

import oracle
from helpers import assert_gemm_close, expert_parallel_reference, make_activations

pytestmark = pytest.mark.gpu


def _experts(E, H, I, seed):
    g = torch.Generator().manual_seed(seed)
    w1 = [oracle.block_quant_weight(torch.randn(2 * I, H, generator=g) * 0.05) for _ in range(E)]
    w2 = [oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05) for _ in range(E)]
    return (torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1]),
            torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2]))


@pytest.mark.parametrize("world,E,topk,H,I,tokens", [(2, 8, 2, 256, 128, [40, 17]), (4, 16, 4, 512, 256, [33, 0, 64, 5]),
                                                     (8, 32, 8, 512, 128, [16] * 8)])
@pytest.mark.parametrize("fuse_quant", [False, True])
def test_ep_exchange_emulated_ranks(world, E, topk, H, I, tokens, fuse_quant):
    from sglang_b200._lib import lib
    from sglang_b200.distributed import peer_ep as pe
    from sglang_b200.layers.moe import fused_experts_block_fp8_prequant
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8
    L = lib()
    el, cap, m_max = E // world, sum(tokens), max(max(tokens), 1)
    nbytes = L.sglb200_ep_buffer_bytes(cap, H, topk, world, m_max)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    views = [pe.buffer_views(b.data_ptr(), b.device, cap, H, topk, world, m_max) for b in bufs]
    off = (ctypes.c_int64 * 7)()
    assert L.sglb200_ep_buffer_offsets(cap, H, topk, world, m_max, off) == 0
    metas = [b[off[2]:off[2] + cap * 8].view(torch.int32).view(cap, 2) for b in bufs]
    w1q, w1s, w2q, w2s = _experts(E, H, I, seed=E)
    w_dev = [(w1q[r * el:(r + 1) * el].cuda(), w2q[r * el:(r + 1) * el].cuda(), w1s[r * el:(r + 1) * el].cuda(),
              w2s[r * el:(r + 1) * el].cuda()) for r in range(world)]
    for epoch in (1, 2, 3):  # both parities of the counters and flags, and their reuse
        xs, ws_, ids_ = [], [], []
        for r in range(world):
            g = torch.Generator().manual_seed(100 * epoch + r)
            xs.append(make_activations(tokens[r], H, seed=10 * epoch + r, outliers=False) if tokens[r] else
                      torch.empty(0, H, dtype=torch.bfloat16))
            tw, ti = torch.topk(torch.softmax(torch.randn(tokens[r], E, generator=g), -1), topk)
            ws_.append(tw.float().contiguous())
            ids_.append(ti.to(torch.int32).contiguous())
        quantised = []
        for r in range(world):
            if tokens[r]:
                a_q, a_s = sglang_per_token_group_quant_fp8(xs[r].cuda(), 128)
            else:
                a_q = torch.empty(0, H, dtype=torch.float8_e4m3fn, device="cuda")
                a_s = torch.empty(0, H // 128, device="cuda")
            quantised.append((a_q, a_s))
            if fuse_quant:
                pe.ep_dispatch_quant(arr, r, world, cap, m_max, xs[r].cuda(), ids_[r].cuda(), ws_[r].cuda(), el)
            else:
                pe.ep_dispatch(arr, r, world, cap, m_max, a_q, a_s, ids_[r].cuda(), ws_[r].cuda(), el)
        counts = []
        for r in range(world):
            cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
            pe.ep_receive(arr, r, world, H, topk, el, cap, m_max, cnt)
            rq, rs, rids, rw = views[r]
            partial = fused_experts_block_fp8_prequant(rq, rs, torch.bfloat16, *w_dev[r][:2], *w_dev[r][2:], rw, rids)
            pe.ep_combine_push(arr, r, world, H, topk, el, cap, m_max, partial)
            counts.append(cnt)
        outs = []
        for r in range(world):
            out = torch.full((tokens[r], H), 7.0, dtype=torch.bfloat16, device="cuda")
            pe.ep_combine_reduce(arr, r, world, ids_[r].cuda(), out, el, cap, m_max)
            outs.append(out)
        torch.cuda.synchronize()
        assert L.sglb200_read_device_status() == 0
        # rows received = (token, destination rank) pairs addressed to that rank
        for r in range(world):
            want = sum(int(((ids_[s] // el) == r).any(dim=1).sum()) for s in range(world))
            assert int(counts[r].item()) == want, f"rank {r} received {int(counts[r].item())}, expected {want}"
            # every received row is, bit for bit, the quantised row of its (source rank, token)
            meta = metas[r][:want].cpu()
            rq, rs = views[r][0][:want].view(torch.uint8).cpu(), views[r][1][:want].cpu()
            for i in range(want):
                a_q, a_s = quantised[int(meta[i, 0])]
                tok = int(meta[i, 1])
                assert torch.equal(rq[i], a_q[tok].view(torch.uint8).cpu()) and torch.equal(rs[i], a_s[tok].cpu()), \
                    f"epoch {epoch} rank {r} row {i} (from rank {int(meta[i, 0])} token {tok})"
        for r in range(world):
            if tokens[r]:
                ref = expert_parallel_reference(xs[r], w1q, w2q, w1s, w2s, ws_[r], ids_[r], world)
                assert_gemm_close(outs[r], ref, f"epoch {epoch} rank {r}")


def test_ep_dispatch_quant_strided_f16_and_full_buffer():
    """The fused form on f16 rows with a row stride, H not a multiple of 512 (a ragged last pass over the groups), and
    its report of a full receive buffer."""
    from sglang_b200._lib import lib
    from sglang_b200.distributed import peer_ep as pe
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8
    L = lib()
    world, H, topk, el, M = 2, 768, 3, 4, 37
    cap, m_max = 2 * M, M
    nbytes = L.sglb200_ep_buffer_bytes(cap, H, topk, world, m_max)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    off = (ctypes.c_int64 * 7)()
    assert L.sglb200_ep_buffer_offsets(cap, H, topk, world, m_max, off) == 0
    wide = (make_activations(M, H + 64, seed=5, outliers=True).to(torch.float16)).cuda()
    wide[3] = 0  # an all-zero row: the scale is the floor eps / 448
    x = wide[:, :H]
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, world * el, (M, topk), generator=g, dtype=torch.int32).cuda()
    w = torch.rand(M, topk, generator=g).cuda()
    pe.ep_dispatch_quant(arr, 0, world, cap, m_max, x, ids, w, el)
    a_q, a_s = sglang_per_token_group_quant_fp8(x.contiguous(), 128)
    torch.cuda.synchronize()
    assert L.sglb200_read_device_status() == 0
    for r in range(world):
        rq, rs, rids, rw = pe.buffer_views(bufs[r].data_ptr(), bufs[r].device, cap, H, topk, world, m_max)
        meta = bufs[r][off[2]:off[2] + cap * 8].view(torch.int32).view(cap, 2)
        toks = ((ids // el) == r).any(dim=1).nonzero().flatten()
        n = toks.numel()
        order = meta[:n, 1].long()
        assert sorted(order.tolist()) == toks.tolist() and bool((meta[:n, 0] == 0).all())
        assert torch.equal(rq[:n].view(torch.uint8), a_q[order].view(torch.uint8)) and torch.equal(rs[:n], a_s[order])
        want_ids = torch.where((ids[order] // el) == r, ids[order] - r * el, torch.full_like(ids[order], -1))
        assert torch.equal(rids[:n], want_ids) and torch.equal(rw[:n], w[order])
    # 37 more rows for rank 0 into a buffer that has room for 4: reported, nothing written past the buffer
    small = L.sglb200_ep_buffer_bytes(4, H, topk, world, m_max)
    bufs2 = [torch.zeros(small + 4096, dtype=torch.uint8, device="cuda") for _ in range(world)]
    arr2 = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs2])
    pe.ep_dispatch_quant(arr2, 0, world, 4, m_max, x, torch.zeros_like(ids), w, el)
    torch.cuda.synchronize()
    assert L.sglb200_read_device_status() == 23
    assert all(int(b[small:].sum()) == 0 for b in bufs2)


def test_ep_receive_wait_runs_out_and_full_buffer_reports():
    from sglang_b200._lib import lib
    from sglang_b200.distributed import peer_ep as pe
    L = lib()
    world, H, topk, el, cap, m_max = 2, 256, 2, 4, 4, 16
    nbytes = L.sglb200_ep_buffer_bytes(cap, H, topk, world, m_max)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    a_q = torch.zeros(16, H, dtype=torch.float8_e4m3fn, device="cuda")
    a_s = torch.ones(16, 2, device="cuda")
    ids = torch.zeros(16, topk, dtype=torch.int32, device="cuda")  # every token goes to rank 0: 16 rows into 4 slots
    w = torch.ones(16, topk, device="cuda")
    pe.ep_dispatch(arr, 0, world, cap, m_max, a_q, a_s, ids, w, el)
    torch.cuda.synchronize()
    assert L.sglb200_read_device_status() == 23  # receive buffer full: rows dropped, reported
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    pe.ep_receive(arr, 0, world, H, topk, el, cap, m_max, cnt, timeout_ns=20_000_000)  # rank 1 never dispatched
    torch.cuda.synchronize()
    assert L.sglb200_read_device_status() == 21 and int(cnt.item()) == 0
    assert L.sglb200_read_device_status() == 0


def test_peer_ep_exchange_single_rank():
    """World of one through the allocating class (CUDA-IPC export included): equals the plain fused MoE bit for bit."""
    from sglang_b200.distributed import PeerEpExchange, ep_fused_experts_peer
    from sglang_b200.layers.moe import fused_experts_block_fp8
    E, topk, H, I, M = 8, 2, 256, 128, 50
    w1q, w1s, w2q, w2s = _experts(E, H, I, seed=3)
    ex = PeerEpExchange(capacity=M, hidden=H, topk=topk, m_max=M)
    try:
        for seed in (1, 2, 3):
            x = make_activations(M, H, seed=seed, outliers=False).cuda()
            g = torch.Generator().manual_seed(seed)
            tw, ti = torch.topk(torch.softmax(torch.randn(M, E, generator=g), -1), topk)
            out = ep_fused_experts_peer(ex, x, w1q.cuda(), w2q.cuda(), w1s.cuda(), w2s.cuda(), tw.cuda(), ti.cuda(),
                                        fuse_quant=seed != 2)
            ref = fused_experts_block_fp8(x, w1q.cuda(), w2q.cuda(), w1s.cuda(), w2s.cuda(), tw.cuda(),
                                          ti.to(torch.int32).cuda())
            torch.cuda.synchronize()
            assert torch.equal(out, ref)
        assert ex.completed == 3
        # the whole layer replays from a CUDA graph: nothing on the path synchronises, the exchange counter is on the device
        x = make_activations(M, H, seed=9, outliers=False).cuda()
        g = torch.Generator().manual_seed(9)
        tw, ti = torch.topk(torch.softmax(torch.randn(M, E, generator=g), -1), topk)
        args = (x, w1q.cuda(), w2q.cuda(), w1s.cuda(), w2s.cuda(), tw.cuda(), ti.cuda())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ep_fused_experts_peer(ex, *args)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_g = ep_fused_experts_peer(ex, *args)
        before = ex.completed
        for _ in range(3):
            y_g.zero_()
            graph.replay()
        torch.cuda.synchronize()
        assert ex.completed == before + 3
        assert torch.equal(y_g, fused_experts_block_fp8(x, *args[1:5], tw.cuda(), ti.to(torch.int32).cuda()))
    finally:
        ex.close()
