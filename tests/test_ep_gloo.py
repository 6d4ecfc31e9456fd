"""Expert-parallel dispatch / combine on two CPU ranks (gloo): routing tables, the count exchange, the fp8
payload all-to-all and the partial-row combine.  The quantiser and the expert MLP are the CPU oracle here
(test stand-ins); on GPUs the same function runs the CUDA kernels."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from sglang_b200.distributed import ep_fused_experts, ep_owner_tables
        E, topk, H, I = 8, 3, 256, 128
        g = torch.Generator().manual_seed(0)
        w1 = [oracle.block_quant_weight(torch.randn(2 * I, H, generator=g) * 0.05) for _ in range(E)]
        w2 = [oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05) for _ in range(E)]
        w1q, w1s = torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1])
        w2q, w2s = torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2])
        M = [13, 7][rank]                       # ragged token counts per rank
        gr = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(M, H, generator=gr).bfloat16()
        p = torch.softmax(torch.randn(M, E, generator=gr), -1)
        tw, ti = torch.topk(p, topk)

        el = E // world
        send_idx, local_ids = ep_owner_tables(ti, el, world)
        for r in range(world):
            has = ((ti // el) == r).any(-1)
            assert torch.equal(send_idx[r], torch.nonzero(has).flatten())
            lid = local_ids[:, r]
            assert bool(((lid >= 0) == ((ti // el) == r)).all())
            assert bool((lid[lid >= 0] == (ti - r * el)[lid >= 0]).all())

        def quant_fn(t):
            return oracle.per_token_group_quant_fp8(t, 128)

        def experts_fn(a_q, a_s, dtype, w1_, w2_, s1_, s2_, w_, ids_):
            # oracle expert MLP on pre-quantised rows: dequantise-free restatement through the oracle pieces
            rows, tk = ids_.shape
            out = torch.zeros(rows, w2_.shape[1], dtype=torch.float32)
            for e in range(w1_.shape[0]):
                for j in range(tk):
                    m = ids_[:, j] == e
                    if m.any():
                        h = oracle.w8a8_block_fp8_matmul(a_q[m], w1_[e], a_s[m], s1_[e], output_dtype=dtype)
                        act = oracle.silu_and_mul(h).contiguous()
                        q2, s2 = oracle.per_token_group_quant_fp8(act, 128)
                        y = oracle.w8a8_block_fp8_matmul(q2, w2_[e], s2, s2_[e], output_dtype=dtype)
                        out[m] += (y * w_[m, j:j + 1].to(dtype)).float()
            return out.to(dtype)

        lo, hi = rank * el, (rank + 1) * el
        y = ep_fused_experts(x, w1q[lo:hi], w2q[lo:hi], w1s[lo:hi], w2s[lo:hi], tw, ti, rank, world,
                             quant_fn=quant_fn, experts_fn=experts_fn)
        ref = oracle.fused_experts_block_fp8(x, w1q, w2q, w1s, w2s, tw, ti)
        rel = float((y.float() - ref.float()).norm() / ref.float().norm())
        assert y.shape == (M, H) and rel < 1e-2, rel
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
