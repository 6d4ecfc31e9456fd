"""The masked per-expert layout ([E, max_m, K] with masked_m valid rows per expert) against the oracle run expert by
expert (the reference checks DeepGEMM's masked kernel against a per-batch loop of its torch-native matmul the same
way, python/sglang/test/test_block_fp8.py:549-563,586-635)."""

import pytest
import torch

import oracle
from helpers import assert_gemm_close, make_activations

pytestmark = pytest.mark.gpu


def _weights(G, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    ws = [oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05) for _ in range(G)]
    return torch.stack([w[0] for w in ws]), torch.stack([w[1] for w in ws])


@pytest.mark.parametrize("G,max_m,N,K", [(4, 256, 512, 512), (8, 64, 128, 128), (3, 300, 1024, 384), (32, 128, 256, 7168)])
@pytest.mark.parametrize("mn_major", [False, True])
def test_masked_grouped_gemm(G, max_m, N, K, mn_major):
    from sglang_b200.layers.deep_gemm_wrapper import grouped_gemm_nt_f8f8bf16_masked
    gen = torch.Generator().manual_seed(G + N)
    masked = torch.randint(0, max_m + 1, (G,), generator=gen, dtype=torch.int32)
    masked[0] = max_m
    if G > 2:
        masked[1] = 0
        masked[2] = 1
    x = make_activations(G * max_m, K, seed=K, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128)
    wq, ws = _weights(G, N, K, seed=N)
    a_s = s.view(G, max_m, K // 128).cuda()
    if mn_major:  # scales of a group stored K-block by K-block (the layout DeepGEMM asks for)
        a_s = a_s.transpose(1, 2).contiguous().transpose(1, 2)
    out = torch.full((G, max_m, N), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm_nt_f8f8bf16_masked((q.view(G, max_m, K).cuda(), a_s), (wq.cuda(), ws.cuda()), out, masked.cuda(), max_m)
    torch.cuda.synchronize()
    out = out.cpu()
    for g in range(G):
        m = int(masked[g])
        assert (out[g, m:] == 7.0).all(), f"group {g}: rows past masked_m were written"
        if m:
            ref = oracle.w8a8_block_fp8_matmul(q.view(G, max_m, K)[g, :m], wq[g], s.view(G, max_m, -1)[g, :m], ws[g])
            assert_gemm_close(out[g, :m], ref, f"group {g}")


def test_masked_grouped_gemm_clamps_and_rejects():
    from sglang_b200.layers.deep_gemm_wrapper import grouped_gemm_nt_f8f8bf16_masked
    G, max_m, N, K = 2, 64, 128, 128
    x = make_activations(G * max_m, K, seed=1, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128)
    wq, ws = _weights(G, N, K, seed=2)
    out = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device="cuda")
    masked = torch.tensor([1000, -5], dtype=torch.int32, device="cuda")  # clamped to [0, max_m]
    grouped_gemm_nt_f8f8bf16_masked((q.view(G, max_m, K).cuda(), s.view(G, max_m, 1).cuda()), (wq.cuda(), ws.cuda()), out,
                                    masked, max_m)
    torch.cuda.synchronize()
    assert_gemm_close(out[0].cpu(), oracle.w8a8_block_fp8_matmul(q[:max_m], wq[0], s[:max_m], ws[0]), "clamped")
    assert (out[1] == 0).all()
    with pytest.raises(RuntimeError, match="masked_m"):
        grouped_gemm_nt_f8f8bf16_masked((q.view(G, max_m, K).cuda(), s.view(G, max_m, 1).cuda()), (wq.cuda(), ws.cuda()),
                                        out, masked[:1], max_m)


def test_fused_experts_masked_matches_oracle():
    from sglang_b200.layers.moe import fused_experts_masked
    E, max_m, H, I = 6, 96, 512, 256
    gen = torch.Generator().manual_seed(4)
    masked = torch.tensor([96, 0, 5, 33, 64, 1], dtype=torch.int32)
    x = make_activations(E * max_m, H, seed=3, outliers=False)
    q, s = oracle.per_token_group_quant_fp8(x, 128)
    w13, w13s = _weights(E, 2 * I, H, seed=5)
    w2, w2s = _weights(E, H, I, seed=6)
    out = fused_experts_masked(q.view(E, max_m, H).cuda(), s.view(E, max_m, -1).cuda(), w13.cuda(), w13s.cuda(), w2.cuda(),
                               w2s.cuda(), masked.cuda(), 48)
    torch.cuda.synchronize()
    for e in range(E):
        m = int(masked[e])
        if not m:
            continue
        h = oracle.w8a8_block_fp8_matmul(q.view(E, max_m, H)[e, :m], w13[e], s.view(E, max_m, -1)[e, :m], w13s[e])
        act = oracle.silu_and_mul(h)
        aq, a_s = oracle.per_token_group_quant_fp8(act.contiguous(), 128)
        ref = oracle.w8a8_block_fp8_matmul(aq, w2[e], a_s, w2s[e])
        assert_gemm_close(out[e, :m], ref, f"expert {e}")
