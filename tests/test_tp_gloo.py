"""Tensor-parallel host logic on two CPU ranks (gloo): weight/scale sharding on block boundaries,
local quantisation equal to the slice of the global one, and the row-parallel all-reduce.  The
local GEMM is the CPU oracle here (test stand-in); on GPUs the layers call Fp8LinearMethod.apply."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_apply(layer, x, bias=None):
    import oracle
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    q, s = oracle.per_token_group_quant_fp8(x2, 128)
    y = oracle.w8a8_block_fp8_matmul(q, layer.weight.data, s, layer.weight_scale_inv.data)
    if bias is not None:
        y = y + bias
    return y.reshape(*x.shape[:-1], layer.weight.shape[0])


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from sglang_b200.distributed import (ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear,
                                             shard_block_fp8_weight)
        g = torch.Generator().manual_seed(0)
        M, H, I = 24, 512, 768
        x = torch.randn(M, H, generator=g).bfloat16()
        w_up, s_up = oracle.block_quant_weight(torch.randn(I, H, generator=g) * 0.05)
        w_dn, s_dn = oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05)
        bias = torch.randn(H, generator=g).bfloat16()

        up = ColumnParallelBlockFp8Linear(w_up, s_up, rank, world, apply_fn=_oracle_apply)
        down = RowParallelBlockFp8Linear(w_dn, s_dn, rank, world, bias=bias, apply_fn=_oracle_apply)
        assert up.weight.shape == (I // world, H) and up.weight_scale_inv.shape == (I // 128 // world, H // 128)
        assert down.weight.shape == (H, I // world) and down.weight_scale_inv.shape == (H // 128, I // 128 // world)

        h_local = up(x)                      # [M, I / world]
        y = down(h_local)                    # all-reduced [M, H]

        # single-rank reference of the same two layers
        class L:  # noqa: D401
            pass
        ref_up, ref_dn = L(), L()
        ref_up.weight, ref_up.weight_scale_inv = torch.nn.Parameter(w_up, False), torch.nn.Parameter(s_up, False)
        ref_dn.weight, ref_dn.weight_scale_inv = torch.nn.Parameter(w_dn, False), torch.nn.Parameter(s_dn, False)
        h_ref = _oracle_apply(ref_up, x)
        per = I // world
        assert torch.equal(h_local, h_ref[:, rank * per:(rank + 1) * per]), "column shard differs from the slice"
        # local activation quantisation == slice of the global one (groups do not straddle ranks)
        q_g, s_g = oracle.per_token_group_quant_fp8(h_ref.contiguous(), 128)
        q_l, s_l = oracle.per_token_group_quant_fp8(h_local.contiguous(), 128)
        assert torch.equal(q_l.view(torch.uint8), q_g[:, rank * per:(rank + 1) * per].view(torch.uint8))
        assert torch.equal(s_l, s_g[:, rank * per // 128:(rank + 1) * per // 128])
        y_ref = _oracle_apply(ref_dn, h_ref, bias)
        rel = float((y.float() - y_ref.float()).norm() / y_ref.float().norm())
        assert rel < 1e-2, rel   # partial sums are rounded to bf16 per rank before the reduction

        gathered = ColumnParallelBlockFp8Linear(w_up, s_up, rank, world, gather_output=True, apply_fn=_oracle_apply)(x)
        assert torch.equal(gathered, h_ref)
        # a symmetric-memory communicator that declined (no GPU here) leaves the layer on the collective library's
        # all-reduce, with the bias on rank 0 before the sum, whatever the one-launch / chunk options say
        from sglang_b200.distributed import SymmMemCommunicator
        comm = SymmMemCommunicator(dist.group.WORLD, "cpu")
        assert comm.disabled
        down_sm = RowParallelBlockFp8Linear(w_dn, s_dn, rank, world, bias=bias, apply_fn=_oracle_apply, symm_mem=comm,
                                            symm_mem_fused_ctas=16, symm_mem_chunk_rows=8)
        assert torch.equal(down_sm(h_local), y)
        comm.close()
        try:
            shard_block_fp8_weight(w_up[:640], s_up[:5], rank, world, 0)   # 320 rows per rank: not a block multiple
            raise AssertionError("bad split accepted")
        except ValueError:
            pass
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_row_parallel_bias_with_peer_exchange_is_decided_in_the_constructor(monkeypatch):
    """With a peer exchange every rank takes the sum for itself, so every rank must hold the whole bias and add it after
    the sum; no rank may raise or skip it on its own (the ranks would leave the exchange out of step)."""
    import oracle
    import sglang_b200.distributed.peer_allreduce as pa
    from sglang_b200.distributed import RowParallelBlockFp8Linear

    class FakeExchange:
        def fits(self, m, n):
            return True

        def fits_two_shot(self, m, n):
            return False

    calls = []

    def fake_fused(ex, x, w, ws, bias=None, two_shot=None):
        calls.append(bias)
        return torch.zeros(x.shape[0], w.shape[0]) + (0 if bias is None else bias)

    monkeypatch.setattr(pa, "fused_row_parallel_linear", fake_fused)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    g = torch.Generator().manual_seed(0)
    w, s = oracle.block_quant_weight(torch.randn(256, 512, generator=g) * 0.05)
    bias = torch.randn(256, generator=g)
    outs = []
    for rank in range(2):
        layer = RowParallelBlockFp8Linear(w, s, rank, 2, bias=bias, apply_fn=_oracle_apply, peer_exchange=FakeExchange())
        assert layer.bias_after_sum is not None and torch.equal(layer.bias_after_sum, bias)
        outs.append(layer(torch.zeros(3, 256)))
    assert len(calls) == 2 and all(c is not None and torch.equal(c, bias) for c in calls)
    assert torch.equal(outs[0], outs[1])


def _overlap_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        import sglang_b200.layers.quantization.fp8_kernel as fk
        from sglang_b200.distributed import row_parallel_linear_overlapped

        # CPU stand-ins for the two CUDA calls, so that the chunking, the row-range outputs and the asynchronous
        # reductions run for real on two gloo ranks
        def fake_quant(x, g, column_major_scales=False, scale_tma_aligned=False, **kw):
            return oracle.per_token_group_quant_fp8(x, g)

        def fake_mm(a, b, a_s, b_s, block, dtype, out=None):
            y = oracle.w8a8_block_fp8_matmul(a, b, a_s.contiguous(), b_s, output_dtype=dtype)
            out.copy_(y)
            return out

        fk.sglang_per_token_group_quant_fp8, fk.w8a8_block_fp8_matmul = fake_quant, fake_mm
        g = torch.Generator().manual_seed(0)
        M, N, K = 300, 256, 512
        x = torch.randn(M, K, generator=g).bfloat16()
        wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05)
        kr = K // world
        y = row_parallel_linear_overlapped(x[:, rank * kr:(rank + 1) * kr].contiguous(),
                                           wq[:, rank * kr:(rank + 1) * kr].contiguous(),
                                           ws[:, rank * kr // 128:(rank + 1) * kr // 128].contiguous(), chunk_rows=128)
        ref = oracle.row_parallel_reference(x, wq, ws, world)
        # gloo adds the bf16 partial products in bf16; two ranks: one addition, the same bits as the fp32 sum rounded
        assert torch.equal(y, ref), float((y.float() - ref.float()).abs().max())
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


def test_overlapped_row_parallel_linear_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_overlap_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_bf16_sum_bound_covers_any_order_of_a_library_all_reduce():
    """The bound used for the NCCL paths: a sum of the ranks' bf16 partial results taken in bf16, in ring order from any
    starting rank or as a pairwise tree, lies within `sum_in_storage_type_bound` of the fp32 sum rounded once."""
    import oracle
    g = torch.Generator().manual_seed(0)
    world = 8
    x = torch.randn(48, 2048, generator=g).bfloat16()
    wq, ws = oracle.block_quant_weight(torch.randn(256, 2048, generator=g) * 0.05)
    parts = oracle.row_parallel_partials(x, wq, ws, world)
    ref = oracle.row_parallel_reference(x, wq, ws, world).double()
    slack = oracle.sum_in_storage_type_bound(parts)
    worst = 0.0
    for start in range(world):  # ring orders
        acc = parts[start].clone()
        for i in range(1, world):
            acc = (acc.float() + parts[(start + i) % world].float()).bfloat16()
        assert bool(((acc.double() - ref).abs() <= slack).all())
        worst = max(worst, float((acc.double() - ref).abs().max() / ref.pow(2).mean().sqrt()))
    level = list(parts)  # pairwise tree
    while len(level) > 1:
        level = [(level[i].float() + level[i + 1].float()).bfloat16() for i in range(0, len(level), 2)]
    assert bool(((level[0].double() - ref).abs() <= slack).all())
    assert worst > 2e-2, "with eight bf16 additions the plain 2e-2 x RMS bar is expected to be missed by some element"
