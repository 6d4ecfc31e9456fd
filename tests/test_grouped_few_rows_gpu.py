"""The grouped GEMM on few rows per expert (the decode case of a mixture-of-experts layer): the weight-streaming kernel
with swapped operands against the oracle run expert by expert, and bit for bit against the 128 x 128 grouped kernel on
the same inputs.  The reference checks its grouped kernel against a per-expert loop of the torch-native block matmul the
same way (sgl-kernel/tests/test_fp8_blockwise_moe.py:122-221)."""

import contextlib

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, make_activations

pytestmark = pytest.mark.gpu


@contextlib.contextmanager
def few_rows_limit(limit):
    from sglang_b200._lib import lib
    L = lib()
    before = L.sglb200_get_grouped_few_rows()
    assert L.sglb200_set_grouped_few_rows(limit) == 0
    try:
        yield
    finally:
        assert L.sglb200_set_grouped_few_rows(before) == 0


def _weights(E, N, K, seed, ue8m0=False):
    g = torch.Generator().manual_seed(seed)
    ws = [oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05, scale_ue8m0=ue8m0) for _ in range(E)]
    return torch.stack([w[0] for w in ws]), torch.stack([w[1] for w in ws])


def _run_sorted(aq, a_s, wq, wsc, counts, out_dtype=torch.bfloat16, pad_rows=3):
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_grouped_mm
    E, N, K = wq.shape
    rows = sum(counts)
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    ps = torch.tensor([[c, N, K] for c in counts], dtype=torch.int32)
    out = torch.full((rows + pad_rows, N), 7.0, dtype=out_dtype, device="cuda")
    d = torch.empty(0, device="cuda")
    fp8_blockwise_scaled_grouped_mm(out[:rows], d, d, d, d, d, aq.cuda(), wq.cuda().transpose(1, 2), a_s.cuda(),
                                    wsc.cuda().transpose(1, 2), d, d, d, d, d, ps.cuda(),
                                    torch.from_numpy(offs[:-1].copy()).cuda(), d)
    torch.cuda.synchronize()
    from sglang_b200._lib import lib
    assert lib().sglb200_read_device_status() == 0
    return out.cpu(), offs


@pytest.mark.parametrize("counts,N,K", [
    ([3, 0, 17, 1, 9, 0, 40, 2], 384, 512),      # 16-row chunks; experts with 2 and 3 chunks; empty experts
    ([0, 0, 7], 256, 128),                       # one k-block, leading empty experts
    ([20] * 12, 256, 1024),                      # 32-row chunks
    ([33, 40, 1, 64, 50], 512, 640),             # 64-row chunks, one exactly full
    ([1] * 64, 128, 7168),                       # one row each, a long K
    ([16, 16, 16, 16], 2048, 256),               # full 16-row chunks
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_few_rows_grouped_matches_oracle_and_tile_kernel(counts, N, K, out_dtype):
    E, rows = len(counts), sum(counts)
    a = make_activations(rows, K, seed=rows + N)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, wsc = _weights(E, N, K, seed=K)
    with few_rows_limit(64):
        got, offs = _run_sorted(aq, a_s, wq, wsc, counts, out_dtype)
    with few_rows_limit(0):
        tiled, _ = _run_sorted(aq, a_s, wq, wsc, counts, out_dtype)
    assert (got[rows:] == 7.0).all(), "rows past the last expert were written"
    assert torch.equal(got.view(torch.int16), tiled.view(torch.int16)), "few-rows kernel and 128 x 128 kernel differ"
    ref = torch.cat([oracle.w8a8_block_fp8_matmul(aq[offs[e]:offs[e + 1]], wq[e], a_s[offs[e]:offs[e + 1]], wsc[e],
                                                  output_dtype=out_dtype) for e in range(E) if counts[e]])
    assert_gemm_close(got[:rows], ref, f"few rows {counts}")


def test_few_rows_grouped_offsets_without_problem_sizes():
    """The C entry point with expert_offsets [E + 1] alone (no problem-size table), as the fused MoE calls it."""
    from sglang_b200.layers.moe import _grouped_mm
    counts, N, K = [2, 0, 11, 5, 0, 0, 30, 1], 200, 384  # a ragged last weight tile
    E, rows = len(counts), sum(counts)
    a = make_activations(rows, K, seed=5)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, wsc = _weights(E, N, K, seed=6)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    outs = []
    for limit in (64, 0):
        out = torch.full((rows, N), 7.0, dtype=torch.bfloat16, device="cuda")
        with few_rows_limit(limit):
            _grouped_mm(aq.cuda(), a_s.cuda(), wq.cuda(), wsc.cuda(), out, offs.cuda())
        torch.cuda.synchronize()
        outs.append(out.cpu())
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    ref = torch.cat([oracle.w8a8_block_fp8_matmul(aq[offs[e]:offs[e + 1]], wq[e], a_s[offs[e]:offs[e + 1]], wsc[e])
                     for e in range(E) if counts[e]])
    assert_gemm_close(outs[0], ref, "offsets only")


@pytest.mark.parametrize("G,max_m", [(6, 16), (5, 24), (4, 64)])
def test_few_rows_masked_layout(G, max_m):
    from sglang_b200.layers.deep_gemm_wrapper import grouped_gemm_nt_f8f8bf16_masked
    N, K = 384, 512
    masked = torch.randint(0, max_m + 1, (G,), generator=torch.Generator().manual_seed(G), dtype=torch.int32)
    masked[0], masked[1] = max_m, 0
    x = make_activations(G * max_m, K, seed=max_m, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128)
    wq, ws = _weights(G, N, K, seed=3)
    outs = []
    for limit in (64, 0):
        out = torch.full((G, max_m, N), 7.0, dtype=torch.bfloat16, device="cuda")
        with few_rows_limit(limit):
            grouped_gemm_nt_f8f8bf16_masked((q.view(G, max_m, K).cuda(), s.view(G, max_m, -1).cuda()),
                                            (wq.cuda(), ws.cuda()), out, masked.cuda(), max_m)
        torch.cuda.synchronize()
        outs.append(out.cpu())
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    for g in range(G):
        m = int(masked[g])
        assert (outs[0][g, m:] == 7.0).all(), f"group {g}: rows past masked_m were written"
        if m:
            ref = oracle.w8a8_block_fp8_matmul(q.view(G, max_m, K)[g, :m], wq[g], s.view(G, max_m, -1)[g, :m], ws[g])
            assert_gemm_close(outs[0][g, :m], ref, f"group {g}")


@pytest.mark.parametrize("counts,N,K", [([3, 0, 17, 1, 9, 0, 40, 2], 448, 512), ([20] * 6, 256, 1152), ([1] * 32, 128, 7168)])
def test_few_rows_grouped_ue8m0(counts, N, K):
    """Power-of-two scales: the few-rows kernel decodes the packed exponent words and applies the scales after each
    k-block, exactly; within the output rounding of the oracle, and within one unit in the last place of the block-scaled
    tensor-core kernel (which applies the scales inside the MMA, before its fp32 accumulation)."""
    from sglang_b200.layers.moe import _grouped_mm_ue8m0
    from sglang_b200.layers.quantization import pack_ue8m0_scales
    E, rows = len(counts), sum(counts)
    x = make_activations(rows, K, seed=rows + N, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
    wq, wsc = _weights(E, N, K, seed=N, ue8m0=True)
    wp = torch.stack([pack_ue8m0_scales(t) for t in wsc])
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    outs = []
    for limit in (64, 0):
        out = torch.full((rows, N), 7.0, dtype=torch.bfloat16, device="cuda")
        with few_rows_limit(limit):
            _grouped_mm_ue8m0(q.cuda(), pack_ue8m0_scales(s).cuda(), wq.cuda(), wp.cuda(), out, offs.cuda())
        torch.cuda.synchronize()
        from sglang_b200._lib import lib
        assert lib().sglb200_read_device_status() == 0
        outs.append(out.cpu())
    for e in range(E):
        r0, r1 = int(offs[e]), int(offs[e + 1])
        if r1 > r0:
            ref = oracle.w8a8_block_fp8_matmul(q[r0:r1], wq[e], s[r0:r1], wsc[e])
            assert_gemm_close(outs[0][r0:r1], ref, f"expert {e}, few-rows kernel")
            assert_gemm_close(outs[1][r0:r1], ref, f"expert {e}, tile kernel", allow_one_ulp=True)
            assert_gemm_close(outs[0][r0:r1], outs[1][r0:r1], f"expert {e}, kernels against each other", allow_one_ulp=True)


def test_few_rows_limit_setter_rejects_bad_values():
    from sglang_b200._lib import lib
    L = lib()
    before = L.sglb200_get_grouped_few_rows()
    assert L.sglb200_set_grouped_few_rows(-1) != 0
    assert L.sglb200_set_grouped_few_rows(65) != 0
    assert L.sglb200_get_grouped_few_rows() == before


@pytest.mark.parametrize("tokens", [4, 48])
def test_fused_experts_decode_sizes_same_bits_on_both_kernels(tokens):
    """A whole fused-expert layer at decode sizes (few tokens, many experts) takes the few-rows grouped kernel for both
    GEMMs; its output equals the 128 x 128 path's bit for bit and the oracle's within the output-rounding bar."""
    from sglang_b200.layers.moe import fused_experts_block_fp8
    E, topk, H, I = 32, 4, 512, 256
    g = torch.Generator().manual_seed(tokens)
    x = make_activations(tokens, H, seed=tokens, outliers=False)
    w13, w13s = _weights(E, 2 * I, H, seed=11)
    w2, w2s = _weights(E, H, I, seed=12)
    scores = torch.randn(tokens, E, generator=g)
    tw, ti = torch.topk(torch.softmax(scores, -1), topk)
    tw = (tw / tw.sum(-1, keepdim=True)).float()
    outs = []
    for limit in (64, 0):
        with few_rows_limit(limit):
            y = fused_experts_block_fp8(x.cuda(), w13.cuda(), w2.cuda(), w13s.cuda(), w2s.cuda(), tw.cuda(),
                                        ti.int().cuda())
        torch.cuda.synchronize()
        outs.append(y.cpu())
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    ref = oracle.fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti)
    assert_gemm_close(outs[0], ref, f"fused experts, {tokens} tokens")
