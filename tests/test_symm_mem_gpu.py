"""Two-GPU run of the multicast (NVSwitch) all-reduce and the row-parallel linear built on it; skipped on a single-GPU
box and reported as skipped when the node offers no multicast mapping.  The reference checks its custom all-reduce
against ``dist.all_reduce`` in child processes the same way (``test/srt/test_custom_allreduce.py:16-60``)."""

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
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    comm = None
    try:
        import oracle
        from helpers import assert_gemm_close, row_parallel_reference
        from sglang_b200._lib import lib
        from sglang_b200.distributed import (RowParallelBlockFp8Linear, SymmMemCommunicator,
                                             row_parallel_linear_symm_mem, row_parallel_linear_symm_mem_fused,
                                             row_parallel_linear_symm_mem_overlapped)
        dev = torch.device("cuda", rank)
        comm = SymmMemCommunicator(dist.group.WORLD, dev, max_size=64 << 20)
        if comm.disabled:
            q.put((rank, "skip: no multicast support on this node"))
            return
        g = torch.Generator().manual_seed(7)  # the same stream of numbers on both ranks; rank r takes part r

        def parts_of(shape, dtype):
            return [(torch.randn(*shape, generator=g) * 3).to(dtype) for _ in range(world)]

        # ---- plain sums: sizes that do and do not split evenly over the ranks, both dtypes, repeated (epochs advance)
        for it, (shape, dtype) in enumerate([((1000, 1024), torch.bfloat16), ((8,), torch.bfloat16),
                                             ((3, 8), torch.float16), ((777, 72), torch.bfloat16),
                                             ((4096, 7168), torch.bfloat16), ((1000, 1024), torch.float16)]):
            parts = parts_of(shape, dtype)
            t = comm.view(shape, dtype)
            t.copy_(parts[rank])
            comm.all_reduce_(t)
            torch.cuda.synchronize()
            want = sum(p.double() for p in parts)
            got = t.cpu().double()
            # The switch's adder does not round to nearest: on this pool its sums lie within ONE unit in the last place
            # of the exact sum, on either side (a sum rounded to nearest would lie within half a unit).
            ulp = torch.ldexp(torch.ones_like(want), torch.frexp(want.abs().clamp(min=1e-30))[1] - 1 - (7 if dtype == torch.bfloat16 else 10))
            err = (got - want) / ulp
            print(f"[rank {rank}] sum {it} {tuple(shape)} {dtype}: error in ulps min {float(err.min()):.4f} max "
                  f"{float(err.max()):.4f}", flush=True)
            assert bool((err.abs() <= 1.0001).all()), f"sum {it}: more than one ulp off"
            both = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(both, t.clone())
            assert torch.equal(both[0], both[1]), "ranks must hold identical bits"
        assert lib().sglb200_read_device_status() == 0

        # ---- the reference's interface: staged in, new tensor out
        parts = parts_of((130, 256), torch.bfloat16)
        inp = parts[rank].cuda()
        assert comm.should_symm_mem_allreduce(inp)
        assert not comm.should_symm_mem_allreduce(torch.zeros(4, device=dev))              # fp32
        assert not comm.should_symm_mem_allreduce(torch.zeros(3, device=dev).bfloat16())   # not whole vectors
        out = comm.all_reduce(inp)
        torch.cuda.synchronize()
        assert out.data_ptr() != inp.data_ptr() and torch.equal(inp.cpu(), parts[rank])
        want = sum(p.float() for p in parts).bfloat16()
        assert float((out.cpu().float() - want.float()).abs().max()) <= float(want.float().abs().max()) * 2.0 ** -7

        # ---- replayed CUDA graph: the epochs live on the device
        parts = parts_of((512, 512), torch.bfloat16)
        src = parts[rank].cuda()
        t = comm.view((512, 512))
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                t.copy_(src)
                comm.all_reduce_(t)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            t.copy_(src)
            comm.all_reduce_(t)
        want = sum(p.float() for p in parts)
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert float((t.cpu().float() - want).abs().max()) <= float(want.abs().max()) * 2.0 ** -7
        assert lib().sglb200_read_device_status() == 0

        # ---- row-parallel linear: GEMM into the symmetric buffer, multicast all-reduce, against the oracle and NCCL
        H, I = 1024, 1536
        w_dn, s_dn = oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05)
        plain = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world)
        bias = torch.randn(H, generator=g).bfloat16()
        layer = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world, symm_mem=comm)
        layer_f = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world, symm_mem=comm, symm_mem_fused_ctas=12)
        layer_b = RowParallelBlockFp8Linear(w_dn.cuda(), s_dn.cuda(), rank, world, bias=bias.cuda(), symm_mem=comm,
                                            symm_mem_chunk_rows=256, symm_mem_blocks=8)  # chunked from 257 rows up
        for it, Ms in enumerate([200, 1, 2048 + 2048 + 130, 333]):  # the third: three row blocks, the last one ragged
            xs = torch.randn(Ms, I, generator=g).bfloat16()
            xr = xs[:, rank * (I // world):(rank + 1) * (I // world)].contiguous().cuda()
            y = layer(xr).clone()
            y_direct = row_parallel_linear_symm_mem(comm, xr, plain.weight, plain.weight_scale_inv).clone()
            y_b = layer_b(xr).clone()
            # chunks of rows, each chunk's all-reduce (16 blocks, side stream) beside the next chunk's GEMM: same bits
            y_ovl = row_parallel_linear_symm_mem_overlapped(comm, xr, plain.weight, plain.weight_scale_inv,
                                                            chunk_rows=512, ar_blocks=16).clone()
            # GEMM and all-reduce in one launch (communication CTAs inside the GEMM's grid): same bits again
            y_fused = row_parallel_linear_symm_mem_fused(comm, xr, plain.weight, plain.weight_scale_inv,
                                                         comm_ctas=[8, 16, 1, 32][it]).clone()
            y_lf = layer_f(xr).clone()  # one launch from 2049 rows up, the plain multicast form below
            y_n = plain(xr)
            torch.cuda.synchronize()
            assert lib().sglb200_read_device_status() == 0
            assert torch.equal(y_fused, y_lf)
            ref = row_parallel_reference(xs, w_dn, s_dn, world)
            assert_gemm_close(y, ref, f"symm-mem row-parallel {it}", allow_one_ulp=True)
            assert torch.equal(y, y_direct)
            assert torch.equal(y, y_ovl), f"chunk-overlapped form differs ({it})"
            assert torch.equal(y, y_fused), f"fused GEMM + all-reduce differs ({it})"
            # NCCL rounds the same sum to nearest: the two results differ by less than two units in the last place
            d = (y.float() - y_n.float()).abs().cpu().double()
            ulp = torch.ldexp(torch.ones_like(d), torch.frexp(ref.double().abs().clamp(min=1e-30))[1] - 8)
            assert bool((d <= 2.0001 * ulp).all()), f"symm-mem vs nccl {it}"
            # the bias is added to the finished sum, once, on every rank
            assert torch.equal(y_b, (y.float() + bias.cuda().float()).bfloat16()), f"bias after the sum {it}"
            both = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(both, y)
            assert torch.equal(both[0], both[1]), "ranks must hold identical bits"
        # an output larger than the buffer takes the NCCL path
        big = layer(torch.randn(40000, I // world, generator=g).bfloat16().cuda())
        torch.cuda.synchronize()
        assert big.shape == (40000, H)
        assert lib().sglb200_read_device_status() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        # ranks leave together with nothing in flight, then the mappings go away
        try:
            torch.cuda.synchronize()
            if comm is not None:
                comm.close()
        finally:
            dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_symm_mem_all_reduce_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=500) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    if all(str(r[1]).startswith("skip") for r in results):
        pytest.skip(results[0][1])
    for r in results:
        assert r[1] == "ok", r[1]
