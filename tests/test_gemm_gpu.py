"""Parity of the tcgen05 block-scaled FP8 GEMM (through the C ABI) with the CPU oracle.
Tolerance for bf16/f16 outputs: rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS of the reference."""

import numpy as np
import pytest
import torch

import oracle
from helpers import FP8, as_bf16, as_fp8, as_t, assert_gemm_close, load_golden, make_activations, make_weight

pytestmark = pytest.mark.gpu


def _status():
    from sglang_b200._lib import lib
    return lib().sglb200_read_device_status()


def _run(aq, a_s, wq, ws, out_dtype=torch.bfloat16, m_major=False):
    from sglang_b200.layers.quantization import w8a8_block_fp8_matmul
    a_s_d = a_s.cuda()
    if m_major:
        a_s_d = a_s_d.t().contiguous().t()
    out = w8a8_block_fp8_matmul(aq.cuda(), wq.cuda(), a_s_d, ws.cuda(), [128, 128], out_dtype)
    torch.cuda.synchronize()
    assert _status() == 0, "a bounded wait in the GEMM kernel timed out"
    return out


@pytest.mark.parametrize("name", ["m37_n320_k384", "m1_n128_k128", "m130_n576_k256"])
def test_golden_vectors(name):
    z = load_golden("gemm.npz")
    out = _run(as_fp8(z[f"{name}_aq"]), as_t(z[f"{name}_as"]), as_fp8(z[f"{name}_wq"]), as_t(z[f"{name}_ws"]))
    assert_gemm_close(out, as_bf16(z[f"{name}_c"]), name)


@pytest.mark.parametrize("M", [1, 5, 127, 128, 129, 300])
@pytest.mark.parametrize("N,K", [(128, 128), (256, 512), (576, 1024), (1536, 384), (4096, 4096)])
def test_shapes_match_oracle(M, N, K):
    a = make_activations(M, K, seed=M + N + K)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=N * 3 + K)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    out = _run(aq, a_s, wq, ws, m_major=(M % 2 == 1))
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    assert_gemm_close(out, ref, f"M={M} N={N} K={K}")


def test_f16_output_and_ragged_k():
    M, N, K = 70, 384, 320  # K = 2.5 blocks: the tail block is zero-filled by the loader
    a = make_activations(M, 384, seed=2)[:, :K].contiguous()
    aq, a_s = oracle.per_token_group_quant_fp8(torch.nn.functional.pad(a, (0, 64)), 128)
    aq = aq[:, :K].contiguous()
    wq, ws = make_weight(N, K, seed=9)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws, output_dtype=torch.float16)
    out = _run(aq, a_s, wq, ws, out_dtype=torch.float16)
    assert out.dtype == torch.float16
    assert_gemm_close(out, ref, "f16 ragged K")


def test_many_tiles_persistent_schedule():
    """More tiles than SMs, ragged M and N, so every CTA loops over several tiles."""
    M, N, K = 2100, 2304 + 64, 512
    a = make_activations(M, K, seed=11)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=12)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    assert_gemm_close(_run(aq, a_s, wq, ws), ref, "persistent")


def test_sweep_shape_rows_sample():
    """A full-size point of the DeepSeek-V3 sweep (M=2048, N=7168, K=16384): a sample of rows is
    checked against the oracle, the rest through linearity in the activation scales."""
    M, N, K = 2048, 7168, 16384
    a = make_activations(M, K, seed=21)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=22)
    out = _run(aq, a_s, wq, ws, m_major=True)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(3))[:96]
    ref = oracle.w8a8_block_fp8_matmul(aq[rows], wq, a_s[rows], ws)
    assert_gemm_close(out[rows.cuda()], ref, "sweep rows")
    out2 = _run(aq, a_s * 2.0, wq, ws, m_major=True)
    assert torch.equal(out2.float(), (out.float() * 2.0).bfloat16().float())  # power-of-two scaling is exact


def test_sgl_kernel_signature():
    """fp8_blockwise_scaled_mm with the reference's operand layout: mat_b = weight.t(),
    scales_a M-major, scales_b = weight_scale.t()."""
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm
    M, N, K = 77, 512, 1024
    a = make_activations(M, K, seed=31)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=32)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    sa = a_s.cuda().t().contiguous().t()
    out = fp8_blockwise_scaled_mm(aq.cuda(), wq.cuda().t(), sa, ws.cuda().t(), torch.bfloat16)
    torch.cuda.synchronize()
    assert_gemm_close(out, ref, "sgl_kernel signature")
    with pytest.raises(RuntimeError, match="column major"):
        fp8_blockwise_scaled_mm(aq.cuda(), wq.cuda().t().contiguous(), sa, ws.cuda().t(), torch.bfloat16)
    with pytest.raises(RuntimeError, match="scales_a"):
        fp8_blockwise_scaled_mm(aq.cuda(), wq.cuda().t(), sa[:, :-1], ws.cuda().t(), torch.bfloat16)
    with pytest.raises(RuntimeError, match="out_dtype"):
        fp8_blockwise_scaled_mm(aq.cuda(), wq.cuda().t(), sa, ws.cuda().t(), torch.float32)
    assert fp8_blockwise_scaled_mm(aq.cuda()[:0], wq.cuda().t(), sa[:0], ws.cuda().t(), torch.bfloat16).shape == (0, N)


def test_linear_method_apply():
    """Fp8LinearMethod.apply = quant + GEMM + bias, against the oracle's two steps."""
    from sglang_b200.layers.quantization import Fp8Config, Fp8LinearMethod
    M, N, K = 45, 768, 1024
    x = make_activations(3 * 15, K, seed=41).view(3, 15, K)
    wq, ws = make_weight(N, K, seed=42)
    bias = torch.randn(N).bfloat16()
    layer = torch.nn.Module()
    method = Fp8LinearMethod(Fp8Config.from_config({"quant_method": "fp8", "weight_block_size": [128, 128]}))
    method.create_weights(layer, K, [N], K, N, torch.bfloat16, device="cuda")
    layer.weight.data.copy_(wq.cuda().view(torch.uint8).view(FP8))
    layer.weight_scale_inv.data.copy_(ws)
    y = method.apply(layer, x.cuda(), bias.cuda())
    torch.cuda.synchronize()
    aq, a_s = oracle.per_token_group_quant_fp8(x.view(M, K), 128)
    ref = (oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws) + bias).view(3, 15, N)
    assert y.shape == (3, 15, N) and y.dtype == torch.bfloat16
    assert_gemm_close(y, ref, "linear apply")


@pytest.mark.parametrize("M", [1, 16, 64, 128])
@pytest.mark.parametrize("N,K", [(576, 7168), (7168, 8192), (1536, 4096)])
def test_small_m_split_k(M, N, K):
    """Small M: the split-K path (fp32 partial sums in a scratch buffer + reduce) against the oracle.  M <= 64 runs
    the weight-streaming kernel with swapped operands, M = 128 the 128 x 128 kernel."""
    from sglang_b200._lib import lib
    a = make_activations(M, K, seed=M * 3 + N)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=N + K)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    assert lib().sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K) > 0, "expected split-K for this shape"
    out = _run(aq, a_s, wq, ws, m_major=True)
    assert_gemm_close(out, ref, f"split-K M={M} N={N} K={K}")
    assert lib().sglb200_fp8_blockwise_scaled_mm_workspace_bytes(4096, N, K) == 0


@pytest.mark.parametrize("M", [2, 16, 17, 32, 33, 48, 64, 65, 96, 127, 128, 129])
@pytest.mark.parametrize("N,K", [(128, 128), (576, 1024), (1536, 384), (4096, 4096), (7168, 2048)])
def test_few_rows_kernel_boundaries(M, N, K):
    """The weight-streaming kernel (M <= 64, token columns padded to 16 / 32 / 64) on both sides of every padding
    boundary, with ragged N, with and without split-K, both scale layouts; M = 65 is the first size of the 128-row
    kernel."""
    a = make_activations(M, K, seed=M * 7 + N + K)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, ws = make_weight(N, K, seed=N * 5 + K)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)
    out = _run(aq, a_s, wq, ws, m_major=(M % 2 == 0))
    assert_gemm_close(out, ref, f"few rows M={M} N={N} K={K}")
    from sglang_b200._lib import check, lib  # the plain entry point: same kernel, never split
    a_d, w_d, s_d, ws_d = aq.cuda(), wq.cuda(), a_s.cuda(), ws.cuda()
    out2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    check(lib().sglb200_fp8_blockwise_scaled_mm(a_d.data_ptr(), w_d.data_ptr(), s_d.data_ptr(), ws_d.data_ptr(),
                                                out2.data_ptr(), M, N, K, K, K, N, s_d.stride(0), s_d.stride(1),
                                                ws_d.stride(0), ws_d.stride(1), 0, torch.cuda.current_stream().cuda_stream),
          "mm")
    torch.cuda.synchronize()
    assert _status() == 0
    assert_gemm_close(out2, ref, f"few rows, plain entry M={M} N={N} K={K}")


@pytest.mark.parametrize("M", [24, 100])  # one sub-tile of 32 rows; two sub-tiles of 64 rows
def test_few_rows_f16_ragged_k_and_strided_output(M):
    N, K = 384, 320  # K = 2.5 blocks
    a = make_activations(M, 384, seed=5)[:, :K].contiguous()
    aq, a_s = oracle.per_token_group_quant_fp8(torch.nn.functional.pad(a, (0, 64)), 128)
    aq = aq[:, :K].contiguous()
    wq, ws = make_weight(N, K, seed=6)
    ref = oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws, output_dtype=torch.float16)
    out = _run(aq, a_s, wq, ws, out_dtype=torch.float16)
    assert_gemm_close(out, ref, "few rows f16 ragged K")
    from sglang_b200._lib import check, lib  # output rows 512 elements apart
    a_d, w_d, s_d, ws_d = aq.cuda(), wq.cuda(), a_s.cuda(), ws.cuda()
    wide = torch.full((M, 512), 3.0, dtype=torch.float16, device="cuda")
    check(lib().sglb200_fp8_blockwise_scaled_mm(a_d.data_ptr(), w_d.data_ptr(), s_d.data_ptr(), ws_d.data_ptr(),
                                                wide.data_ptr(), M, N, K, K, K, 512, s_d.stride(0), s_d.stride(1),
                                                ws_d.stride(0), ws_d.stride(1), 1, torch.cuda.current_stream().cuda_stream),
          "mm")
    torch.cuda.synchronize()
    assert torch.equal(wide[:, :N], out) and (wide[:, N:] == 3.0).all()
