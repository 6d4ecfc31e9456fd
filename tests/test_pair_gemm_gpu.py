"""The CTA-pair GEMM (tcgen05 cta_group::2, 256 x 128 and 256 x 256 tiles) through its C-ABI entry against the CPU
oracle, and bit for bit against the single-CTA kernel (both add the k-blocks of a row in the same order)."""

import pytest
import torch

import oracle
from helpers import assert_gemm_close, bits, make_activations, make_weight

pytestmark = pytest.mark.gpu


def _pair(aq, a_s, wq, ws, tile_n, out_dtype=torch.bfloat16):
    from sglang_b200._lib import check, dtype_code, lib
    M, K = aq.shape
    N = wq.shape[0]
    out = torch.empty(M, N, dtype=out_dtype, device="cuda")
    check(lib().sglb200_fp8_blockwise_scaled_mm_pair(
        aq.data_ptr(), wq.data_ptr(), a_s.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, aq.stride(0), wq.stride(0),
        out.stride(0), a_s.stride(0), a_s.stride(1), ws.stride(0), ws.stride(1), dtype_code(out_dtype), tile_n,
        torch.cuda.current_stream().cuda_stream), "fp8_blockwise_scaled_mm_pair")
    return out


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (129, 576, 1024), (300, 1536, 384), (2100, 2368, 512),
                                   (512, 4096, 4096)])
def test_pair_gemm_matches_oracle_and_single_cta_kernel(M, N, K, tile_n):
    from sglang_b200._lib import check, lib
    a = make_activations(M, K, seed=M + N)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=K + N)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    aq_d, as_d, wq_d, ws_d = aq.cuda(), a_s.cuda(), wq.cuda(), ws.cuda()
    if M % 2:
        as_d = as_d.t().contiguous().t()  # M-major scales
    out = _pair(aq_d, as_d, wq_d, ws_d, tile_n)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 0
    assert_gemm_close(out, ref, f"pair tile_n={tile_n} M={M} N={N} K={K}")
    if M > 64:  # the plain entry runs the 128 x 128 kernel without a K-split here
        plain = torch.empty_like(out)
        check(lib().sglb200_fp8_blockwise_scaled_mm(
            aq_d.data_ptr(), wq_d.data_ptr(), as_d.data_ptr(), ws_d.data_ptr(), plain.data_ptr(), M, N, K, K, K, N,
            as_d.stride(0), as_d.stride(1), ws_d.stride(0), ws_d.stride(1), 0, torch.cuda.current_stream().cuda_stream),
            "mm")
        torch.cuda.synchronize()
        assert torch.equal(bits(out), bits(plain))


def test_pair_gemm_full_size_rows_sample_and_f16():
    M, N, K = 4096, 7168, 16384
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(M, K, generator=g, device="cuda").bfloat16()
    from sglang_b200.layers.quantization import block_quant_weight_fp8, sglang_per_token_group_quant_fp8
    wq, ws = block_quant_weight_fp8(torch.randn(N, K, generator=g, device="cuda") * 0.02)
    q, s = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:48].sort().values.cuda()
    ref = oracle.w8a8_block_fp8_matmul(q[rows].cpu(), wq.cpu(), s[rows].cpu().contiguous(), ws.cpu(),
                                       output_dtype=torch.float16)
    for tile_n in (128, 256):
        out = _pair(q, s, wq, ws, tile_n, out_dtype=torch.float16)
        torch.cuda.synchronize()
        assert_gemm_close(out[rows], ref, f"pair tile_n={tile_n} full size")


def test_pair_gemm_refuses_bad_arguments():
    from sglang_b200._lib import lib
    L = lib()
    assert L.sglb200_fp8_blockwise_scaled_mm_pair(None, None, None, None, None, 128, 128, 128, 128, 128, 128, 1, 1, 1, 1, 0,
                                                  192, None) == -1
    assert L.sglb200_fp8_blockwise_scaled_mm_pair(None, None, None, None, None, 128, 128, 128, 128, 128, 128, 1, 1, 1, 1, 0,
                                                  128, None) == -6
