"""The UE8M0 path: activations with power-of-two group scales and the hardware block-scaled GEMM
(tcgen05.mma kind::mxf8f6f4.block_scale) against the oracle.  With power-of-two scales the scaled products are the
oracle's exactly; the fp32 sum over K is taken inside the tensor core in another order, so about 0.2 % of the bf16
outputs land one ulp away from the oracle's.  Tolerance: rel-L2 <= 1e-2 (measured 1e-4 .. 1e-8) and max-abs <=
2e-2 x RMS or one bf16 ulp of the element (see helpers.assert_gemm_close)."""

import pytest
import torch

import oracle
from helpers import FP8, assert_gemm_close, make_activations, rel_l2

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 10 ** (torch.rand(M, 1, generator=g) * 4 - 2)).bfloat16()
    w = torch.randn(N, K, generator=g) * 0.02 * (10 ** (torch.rand(N, 1, generator=g) * 2 - 1))
    wq, ws = oracle.block_quant_weight(w, scale_ue8m0=True)
    aq, a_s = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
    return x, wq, ws, aq, a_s, oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)


@pytest.mark.parametrize("M,N,K", [(128, 224, 128), (1, 576, 512), (5, 128, 384), (200, 576, 2048), (1000, 1536, 4096),
                                   (2048, 1920, 4096), (333, 7168, 1536),
                                   # up to 64 rows: the weight-streaming kernel, with and without split-K
                                   (16, 7168, 8192), (17, 1536, 4096), (33, 576, 7168), (64, 4096, 7168), (48, 384, 640),
                                   (65, 7168, 2048)])
def test_ue8m0_gemm_matches_oracle(M, N, K):
    from sglang_b200._lib import lib
    from sglang_b200.layers.quantization import (pack_ue8m0_scales, sglang_per_token_group_quant_fp8,
                                                 w8a8_block_fp8_matmul_ue8m0)
    x, wq, ws, aq_ref, as_ref, ref = _case(M, N, K, M + N + K)
    aq, asp = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                               scale_ue8m0=True)
    out = w8a8_block_fp8_matmul_ue8m0(aq, wq.cuda(), asp, pack_ue8m0_scales(ws.cuda()), torch.bfloat16)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 0
    assert torch.equal(aq.cpu().view(torch.uint8), aq_ref.view(torch.uint8))
    assert_gemm_close(out, ref, f"ue8m0 M={M} N={N} K={K}", allow_one_ulp=True)
    assert rel_l2(out.float().cpu(), ref.float()) < 2e-3


def test_ue8m0_sustained_launches_full_size():
    """Thirteen back-to-back launches of a DeepSeek-V3 gate_up-sized problem, then the rows of a sample against
    the oracle (the sequence that an earlier two-issuer version of the kernel did not survive)."""
    from sglang_b200._lib import lib
    from sglang_b200.layers.quantization import pack_ue8m0_scales, w8a8_block_fp8_matmul_ue8m0
    M, N, K = 8192, 36864, 7168
    g = torch.Generator(device="cuda").manual_seed(0)
    a = (torch.randn(M, K, device="cuda", generator=g) * 30).to(FP8)
    b = (torch.randn(N, K, device="cuda", generator=g) * 30).to(FP8)
    e_a = torch.randint(120, 134, (M, K // 128), device="cuda", generator=g)
    e_b = torch.randint(115, 125, (N // 128, K // 128), device="cuda", generator=g)
    sa = torch.ldexp(torch.ones_like(e_a, dtype=torch.float32), e_a - 127)
    sb = torch.ldexp(torch.ones_like(e_b, dtype=torch.float32), e_b - 127)
    sfa = pack_ue8m0_scales(sa).t().contiguous().t()  # M-major, as the quantiser writes it
    sfb = pack_ue8m0_scales(sb)
    for _ in range(13):
        out = w8a8_block_fp8_matmul_ue8m0(a, b, sfa, sfb, torch.bfloat16)
    torch.cuda.synchronize()
    assert lib().sglb200_read_device_status() == 0
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:64]
    ref = oracle.w8a8_block_fp8_matmul(a[rows.cuda()].cpu(), b.cpu(), sa[rows.cuda()].cpu(), sb.cpu())
    assert_gemm_close(out[rows.cuda()], ref, "sustained ue8m0", allow_one_ulp=True)


def test_linear_method_picks_ue8m0_for_power_of_two_scales():
    from sglang_b200.layers.quantization import Fp8Config, Fp8LinearMethod
    M, N, K = 77, 768, 1024
    x, wq, ws, aq, a_s, ref = _case(M, N, K, 5)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(9)).bfloat16()
    method = Fp8LinearMethod(Fp8Config())
    layer = torch.nn.Module()
    method.create_weights(layer, K, [N], K, N, torch.bfloat16, device="cuda")
    layer.weight.data.copy_(wq.cuda().view(torch.uint8).view(FP8))
    layer.weight_scale_inv.data.copy_(ws)
    method.process_weights_after_loading(layer)
    assert layer.weight_scale_ue8m0 is not None and layer.weight_scale_ue8m0.dtype == torch.int32
    y = method.apply(layer, x.cuda().view(7, 11, K), bias.cuda())
    torch.cuda.synchronize()
    assert_gemm_close(y.view(M, N), ref + bias, "ue8m0 linear", allow_one_ulp=True)
    # scales that are not powers of two keep the fp32-scale GEMM ...
    wq2, ws2 = oracle.block_quant_weight(torch.randn(N, K, generator=torch.Generator().manual_seed(3)) * 0.02)
    layer2 = torch.nn.Module()
    method.create_weights(layer2, K, [N], K, N, torch.bfloat16, device="cuda")
    layer2.weight.data.copy_(wq2.cuda().view(torch.uint8).view(FP8))
    layer2.weight_scale_inv.data.copy_(ws2)
    method.process_weights_after_loading(layer2)
    assert layer2.weight_scale_ue8m0 is None
    # ... unless the config asks for requantisation (the reference's Blackwell behaviour): then parity is looser
    method_r = Fp8LinearMethod(Fp8Config(requant_weight_ue8m0=True))
    method_r.process_weights_after_loading(layer2)
    assert layer2.weight_scale_ue8m0 is not None
    y2 = method_r.apply(layer2, x.cuda())
    torch.cuda.synchronize()
    q2, s2 = oracle.per_token_group_quant_fp8(x, 128)
    ref2 = oracle.w8a8_block_fp8_matmul(q2, wq2, s2, ws2)
    assert rel_l2(y2.float().cpu(), ref2.float()) < 6e-2  # requantisation error of weights and power-of-two activation scales


def _ue8m0_experts(E, H, I, seed):
    from sglang_b200.layers.quantization import pack_ue8m0_scales
    g = torch.Generator().manual_seed(seed)
    w1 = [oracle.block_quant_weight(torch.randn(2 * I, H, generator=g) * 0.05, scale_ue8m0=True) for _ in range(E)]
    w2 = [oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05, scale_ue8m0=True) for _ in range(E)]
    w1q, w1s = torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1])
    w2q, w2s = torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2])
    w1p = torch.stack([pack_ue8m0_scales(s) for s in w1s])
    w2p = torch.stack([pack_ue8m0_scales(s) for s in w2s])
    return w1q, w1s, w2q, w2s, w1p, w2p


@pytest.mark.parametrize("rows_per_expert,N,K", [([5, 0, 300, 128, 1], 448, 512), ([130, 129, 2], 2048, 1024),
                                                 ([0, 0, 7], 224, 128), ([64] * 16, 4096, 7168)])
def test_grouped_ue8m0_gemm_matches_oracle(rows_per_expert, N, K):
    """Grouped form: ragged expert segments (empty ones included), row-major scale words as after a row shuffle."""
    from sglang_b200.layers.moe import _grouped_mm_ue8m0
    from sglang_b200.layers.quantization import pack_ue8m0_scales
    E, total = len(rows_per_expert), sum(rows_per_expert)
    x = make_activations(total, K, seed=total + N, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
    g = torch.Generator().manual_seed(N)
    ws = [oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05, scale_ue8m0=True) for _ in range(E)]
    wq, wsc = torch.stack([w[0] for w in ws]), torch.stack([w[1] for w in ws])
    wp = torch.stack([pack_ue8m0_scales(t) for t in wsc])
    offs = torch.tensor([0] + list(torch.tensor(rows_per_expert).cumsum(0)), dtype=torch.int32)
    out = torch.full((total, N), 7.0, dtype=torch.bfloat16, device="cuda")
    _grouped_mm_ue8m0(q.cuda(), pack_ue8m0_scales(s).cuda(), wq.cuda(), wp.cuda(), out, offs.cuda())
    torch.cuda.synchronize()
    from sglang_b200._lib import lib
    assert lib().sglb200_read_device_status() == 0
    for e in range(E):
        r0, r1 = int(offs[e]), int(offs[e + 1])
        if r1 > r0:
            ref = oracle.w8a8_block_fp8_matmul(q[r0:r1], wq[e], s[r0:r1], wsc[e])
            assert_gemm_close(out[r0:r1], ref, f"expert {e}", allow_one_ulp=True)


@pytest.mark.parametrize("M,E,topk,H,I", [(1, 8, 2, 512, 256), (100, 16, 4, 512, 256), (700, 32, 8, 1024, 384)])
def test_fused_experts_ue8m0_matches_oracle(M, E, topk, H, I):
    from sglang_b200.layers.moe import fused_experts_block_fp8_ue8m0
    a = make_activations(M, H, seed=M, outliers=False)
    w1q, w1s, w2q, w2s, w1p, w2p = _ue8m0_experts(E, H, I, seed=E)
    g = torch.Generator().manual_seed(M + 1)
    w, ids = torch.topk(torch.softmax(torch.randn(M, E, generator=g), dim=-1), topk)
    ids = ids.to(torch.int32)
    if M >= 100:
        ids[5, 1] = -1
    ref = oracle.fused_experts_block_fp8(a, w1q, w2q, w1s, w2s, w, ids, scale_ue8m0=True)
    out = fused_experts_block_fp8_ue8m0(a.cuda(), w1q.cuda(), w2q.cuda(), w1p.cuda(), w2p.cuda(), w.cuda(), ids.cuda())
    torch.cuda.synchronize()
    from sglang_b200._lib import lib
    assert lib().sglb200_read_device_status() == 0
    assert_gemm_close(out, ref, "fused experts, UE8M0", allow_one_ulp=True)
