"""The allocation-free split-K GEMM entry (sglb200_fp8_blockwise_scaled_mm_noalloc), called through the C ABI.

Some callers of this library are not allowed to allocate device memory at the point where they run the GEMM (an
engine that owns all device memory through its own pool, a no-allocation region, a bare C host).  For them the
split-K scratch is a fixed array inside the library.  This file checks that entry against the existing split-K
entry (caller-provided scratch) on two consecutive calls with different inputs, so stale scratch contents from the
first call would show up in the second, and that shapes beyond the built-in buffer are refused.  It is collected
last on purpose: a run that stops at the first failure has already run everything else.
"""

import pytest
import torch

import oracle
from helpers import assert_gemm_close, make_activations, make_weight

pytestmark = pytest.mark.gpu


def _args(aq, a_s, wq, ws, out):
    M, K = aq.shape
    N = wq.shape[0]
    return (aq.data_ptr(), wq.data_ptr(), a_s.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, K, K, N,
            a_s.stride(0), a_s.stride(1), ws.stride(0), ws.stride(1), 0)


def test_noalloc_entry_matches_workspace_entry_twice():
    from sglang_b200._lib import check, lib
    L = lib()
    assert L.sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes() == 16 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    for call, (M, N, K, seed) in enumerate([(16, 7168, 8192, 1), (64, 1536, 4096, 2)]):
        a = make_activations(M, K, seed=seed)
        aq_c, as_c = oracle.per_token_group_quant_fp8(a, 128)
        wq_c, ws_c = make_weight(N, K, seed=seed + 10)
        aq, a_s, wq, ws = aq_c.cuda(), as_c.cuda(), wq_c.cuda(), ws_c.cuda()
        need = L.sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K)
        assert 0 < need <= L.sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes(), "shape must use split-K and fit"
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        want = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        check(L.sglb200_fp8_blockwise_scaled_mm_ws(*_args(aq, a_s, wq, ws, want), scratch.data_ptr(), need, stream),
              "workspace entry")
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        check(L.sglb200_fp8_blockwise_scaled_mm_noalloc(*_args(aq, a_s, wq, ws, got), stream), "no-alloc entry")
        torch.cuda.synchronize()
        assert L.sglb200_read_device_status() == 0
        # same kernels, same split, same order of additions: the two entries agree bit for bit
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"
        assert_gemm_close(got, oracle.w8a8_block_fp8_matmul(aq_c, wq_c, as_c, ws_c), f"call {call} vs oracle")


def test_noalloc_entry_rejects_oversized_scratch_and_runs_large_m():
    from sglang_b200._lib import lib
    L = lib()
    stream = torch.cuda.current_stream().cuda_stream
    # M=128, N=7168, K=16384 splits six ways: 22 MB of partial sums, more than the built-in 16 MiB: refused before any launch
    M, N, K = 128, 7168, 16384
    assert L.sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K) > L.sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes()
    rc = L.sglb200_fp8_blockwise_scaled_mm_noalloc(None, None, None, None, None, M, N, K, K, K, N, 1, M, K // 128, 1, 0,
                                                   stream)
    assert rc == -7 and b"built-in buffer" in L.sglb200_last_error_detail()
    # a shape that does not use split-K at all runs through the same entry
    M, N, K = 300, 512, 1024
    a = make_activations(M, K, seed=5)
    aq_c, as_c = oracle.per_token_group_quant_fp8(a, 128)
    wq_c, ws_c = make_weight(N, K, seed=6)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    aq, a_s, wq, ws = aq_c.cuda(), as_c.cuda(), wq_c.cuda(), ws_c.cuda()
    assert L.sglb200_fp8_blockwise_scaled_mm_noalloc(*_args(aq, a_s, wq, ws, out), stream) == 0
    torch.cuda.synchronize()
    assert_gemm_close(out, oracle.w8a8_block_fp8_matmul(aq_c, wq_c, as_c, ws_c), "large M through no-alloc entry")
