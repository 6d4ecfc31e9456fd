"""Two-GPU runs of the sharded paths (skipped on a single-GPU box): tensor-parallel column/row linear with the
NCCL all-reduce, and expert-parallel MoE with all-to-all dispatch/combine, against the CPU oracle."""

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        from helpers import assert_gemm_close, expert_parallel_reference, row_parallel_reference
        from sglang_b200.distributed import (ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear,
                                             ep_fused_experts)
        g = torch.Generator().manual_seed(0)
        # ---- tensor parallel MLP: column-parallel up, row-parallel down + all-reduce
        M, H, I = 200, 1024, 1536
        x = torch.randn(M, H, generator=g).bfloat16()
        w_up, s_up = oracle.block_quant_weight(torch.randn(I, H, generator=g) * 0.05)
        w_dn, s_dn = oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05)
        up = ColumnParallelBlockFp8Linear(w_up.cuda(), s_up.cuda(), rank, world)
        down = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world)
        y = down(up(x.cuda()))
        torch.cuda.synchronize()
        q1, a1 = oracle.per_token_group_quant_fp8(x, 128)
        h = oracle.w8a8_block_fp8_matmul(q1, w_up, a1, s_up)
        q2, a2 = oracle.per_token_group_quant_fp8(h.contiguous(), 128)
        ref = oracle.w8a8_block_fp8_matmul(q2, w_dn, a2, s_dn)
        assert_gemm_close(y, ref, "tp mlp")

        # ---- expert parallel MoE
        E, topk, Hm, Im = 16, 4, 512, 256
        w1 = [oracle.block_quant_weight(torch.randn(2 * Im, Hm, generator=g) * 0.05) for _ in range(E)]
        w2 = [oracle.block_quant_weight(torch.randn(Hm, Im, generator=g) * 0.05) for _ in range(E)]
        w1q, w1s = torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1])
        w2q, w2s = torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2])
        Mr = [150, 90][rank]
        gr = torch.Generator().manual_seed(50 + rank)
        xm = torch.randn(Mr, Hm, generator=gr).bfloat16()
        tw, ti = torch.topk(torch.softmax(torch.randn(Mr, E, generator=gr), -1), topk)
        el = E // world
        lo, hi = rank * el, (rank + 1) * el
        out = ep_fused_experts(xm.cuda(), w1q[lo:hi].cuda(), w2q[lo:hi].cuda(), w1s[lo:hi].cuda(), w2s[lo:hi].cuda(),
                               tw.cuda(), ti.cuda(), rank, world)
        torch.cuda.synchronize()
        refm = oracle.fused_experts_block_fp8(xm, w1q, w2q, w1s, w2s, tw, ti)
        rel = float((out.cpu().float() - refm.float()).norm() / refm.float().norm())
        assert rel <= 1e-2, f"ep moe rel-L2 {rel}"
        # ---- row-parallel linear with the GEMM pushing its tiles into every rank's memory (no NCCL on the path)
        from sglang_b200.distributed import PeerExchange
        ex = PeerExchange(slot_elems=128 * H)
        try:
            fused = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world, peer_exchange=ex)
            for it, Ms in enumerate([64, 1, 128, 33, 64, 64, 100]):
                xs = torch.randn(Ms, I, generator=g).bfloat16()
                xr = xs[:, rank * (I // world):(rank + 1) * (I // world)].contiguous().cuda()
                y_f = fused(xr)
                y_n = down(xr)  # the same shard through NCCL
                torch.cuda.synchronize()
                assert ex.completed == it + 1
                assert_gemm_close(y_f, row_parallel_reference(xs, w_dn, s_dn, world), f"fused row-parallel {it}")
                assert_gemm_close(y_f, y_n.cpu(), f"fused vs nccl {it}", allow_one_ulp=True)
                both = [torch.empty_like(y_f) for _ in range(world)]
                dist.all_gather(both, y_f)
                assert torch.equal(both[0], both[1]), "ranks must hold identical bits"
            big = fused(torch.randn(512, I // world, generator=g).bfloat16().cuda())  # does not fit: NCCL path
            assert big.shape == (512, H) and ex.completed == 7
            # a bias with the exchange: every rank adds the whole bias once, after the sum, and the ranks stay in step
            bias = torch.randn(H, generator=g).bfloat16()
            fused_b = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world, bias=bias.cuda(), peer_exchange=ex)
            for it in range(2):
                xs = torch.randn(64, I, generator=g).bfloat16()
                xr = xs[:, rank * (I // world):(rank + 1) * (I // world)].contiguous().cuda()
                y_b = fused_b(xr)
                torch.cuda.synchronize()
                ref_b = (row_parallel_reference(xs, w_dn, s_dn, world).float() + bias.float()).bfloat16()
                assert_gemm_close(y_b, ref_b, f"fused row-parallel with bias {it}", allow_one_ulp=True)
            assert ex.completed == 9
        finally:
            ex.close()
        # ---- the two-shot form (tile t reduced on rank t % world, results sent round), alternating with the one-shot form
        from sglang_b200.distributed import fused_row_parallel_linear
        ex2 = PeerExchange(slot_elems=300 * H)
        try:
            shard = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world)
            for it, Ms in enumerate([300, 130, 256, 300]):
                xs = torch.randn(Ms, I, generator=g).bfloat16()
                xr = xs[:, rank * (I // world):(rank + 1) * (I // world)].contiguous().cuda()
                y_2 = fused_row_parallel_linear(ex2, xr, shard.weight, shard.weight_scale_inv, two_shot=True)
                y_1 = fused_row_parallel_linear(ex2, xr, shard.weight, shard.weight_scale_inv, two_shot=False)
                torch.cuda.synchronize()
                assert ex2.completed == 2 * (it + 1)
                assert torch.equal(y_2, y_1), f"two-shot and one-shot bits differ ({it})"
                both = [torch.empty_like(y_2) for _ in range(world)]
                dist.all_gather(both, y_2)
                assert torch.equal(both[0], both[1]), "ranks must hold identical bits"
            assert_gemm_close(y_2, row_parallel_reference(xs, w_dn, s_dn, world), "two-shot row-parallel")
        finally:
            ex2.close()
        # ---- the same expert-parallel layer with dispatch / combine over peer memory (no NCCL, no host sync)
        from sglang_b200.distributed import PeerEpExchange, ep_fused_experts_peer
        epx = PeerEpExchange(capacity=2 * 150, hidden=Hm, topk=topk, m_max=150)
        try:
            done = []
            for it in range(6):
                gi = torch.Generator().manual_seed(70 + 10 * it + rank)
                Mi = [150, 90, 1, 77][(it + rank) % 4]
                xi = torch.randn(Mi, Hm, generator=gi).bfloat16()
                twi, tii = torch.topk(torch.softmax(torch.randn(Mi, E, generator=gi), -1), topk)
                out_p = ep_fused_experts_peer(epx, xi.cuda(), w1q[lo:hi].cuda(), w2q[lo:hi].cuda(), w1s[lo:hi].cuda(),
                                              w2s[lo:hi].cuda(), twi.cuda(), tii.cuda())
                done.append((it, out_p, xi, twi, tii))
            torch.cuda.synchronize()
            # the references are computed after the loop: the waits inside the exchange are bounded (2 s), and seconds of
            # CPU work on one rank between two layers would let the other rank's wait run out
            for it, out_p, xi, twi, tii in done:
                refi = expert_parallel_reference(xi, w1q, w2q, w1s, w2s, twi, tii, world)
                assert_gemm_close(out_p, refi, f"peer ep moe {it}")
        finally:
            epx.close()
        from sglang_b200._lib import lib
        assert lib().sglb200_read_device_status() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_and_ep_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
