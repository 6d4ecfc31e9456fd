"""Parity of the MoE side of the path (routing tables, row movers, grouped GEMM, fused expert
MLP) with the CPU oracle.  Integer tables and pure data movement are bit-exact; bf16 outputs
use rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS."""

import numpy as np
import pytest
import torch

import oracle
from helpers import FP8, as_bf16, as_fp8, as_t, assert_gemm_close, load_golden, make_activations

pytestmark = pytest.mark.gpu


def _routing(M, E, topk, seed):
    g = torch.Generator().manual_seed(seed)
    p = torch.softmax(torch.randn(M, E, generator=g), dim=-1, dtype=torch.float32)
    w, ids = torch.topk(p, topk)
    return w, ids.to(torch.int32)


def _experts(E, H, I, seed, std=0.05):
    g = torch.Generator().manual_seed(seed)
    w1 = [oracle.block_quant_weight(torch.randn(2 * I, H, generator=g) * std) for _ in range(E)]
    w2 = [oracle.block_quant_weight(torch.randn(H, I, generator=g) * std) for _ in range(E)]
    return (torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1]),
            torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2]))


def _prepare(ids, E, n, k):
    from sglang_b200.sgl_kernel import prepare_moe_input
    L = ids.numel()
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    ps1 = torch.empty(E, 3, dtype=torch.int32, device="cuda")
    ps2 = torch.empty(E, 3, dtype=torch.int32, device="cuda")
    a_map = torch.empty(L, dtype=torch.int32, device="cuda")
    c_map = torch.empty(L, dtype=torch.int32, device="cuda")
    prepare_moe_input(ids.cuda(), offs, ps1, ps2, a_map, c_map, E, n, k)
    torch.cuda.synchronize()
    return offs, ps1, ps2, a_map, c_map


@pytest.mark.parametrize("M,E,topk", [(1, 4, 2), (9, 4, 2), (50, 7, 4), (333, 64, 6), (4096, 256, 8), (16384, 256, 8)])
def test_prepare_moe_input_exact(M, E, topk):
    _, ids = _routing(M, E, topk, seed=M + E)
    if M >= 50:
        ids[3, 1] = -1  # a non-local expert
        ids[7, 0] = E + 5
    got = _prepare(ids, E, 128, 256)
    want = oracle.prepare_moe_input(ids.numpy(), E, 128, 256)
    for g, w, name in zip(got, want, ["offsets", "ps1", "ps2", "a_map", "c_map"]):
        assert np.array_equal(g.cpu().numpy().reshape(w.shape), w), name


def test_shuffle_rows_and_combine_exact():
    from sglang_b200.sgl_kernel import apply_shuffle_mul_sum, shuffle_rows
    M, E, topk, H = 77, 8, 3, 512
    w, ids = _routing(M, E, topk, seed=5)
    ids[2, 2] = -1
    _, _, _, a_map, c_map = oracle.prepare_moe_input(ids.numpy(), E, 64, H)
    x = make_activations(M, H, seed=6)
    for t in (x, x.to(FP8), torch.randn(M, 4)):  # bf16 rows, fp8 rows, 16-byte scale rows
        got = shuffle_rows(t.cuda(), torch.from_numpy(a_map).cuda(), (M * topk, t.shape[1]))
        want = oracle.shuffle_rows(t, a_map)
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))
    c2 = make_activations(M * topk, H, seed=7, outliers=False)
    out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    apply_shuffle_mul_sum(c2.cuda(), out, torch.from_numpy(c_map).cuda(), w.bfloat16().cuda().reshape(-1))
    want = oracle.apply_shuffle_mul_sum(c2, c_map, w.bfloat16(), M)
    assert torch.equal(out.cpu(), want)
    apply_shuffle_mul_sum(c2.cuda(), out, torch.from_numpy(c_map).cuda(), None)
    assert torch.equal(out.cpu(), oracle.apply_shuffle_mul_sum(c2, c_map, None, M))


def test_silu_and_mul():
    from sglang_b200.sgl_kernel import silu_and_mul
    x = make_activations(65, 2 * 384, seed=8, outliers=False)
    got = silu_and_mul(x.cuda()).cpu()
    want = oracle.silu_and_mul(x)
    assert float((got != want).float().mean()) < 1e-3  # expf differs from the CPU's in the last place, rarely
    assert bool(((got.float() - want.float()).abs() <= want.float().abs() * 2.0 ** -7 + 1e-30).all())
    with pytest.raises(ValueError):
        silu_and_mul(torch.zeros(4, 6, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("counts", [[5, 0, 130, 1], [0, 0, 7], [128, 128], [300, 1, 0, 0, 77, 129, 0, 2]])
def test_grouped_gemm_matches_oracle(counts):
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_grouped_mm
    E, N, K = len(counts), 384, 512
    rows = sum(counts)
    a = make_activations(rows, K, seed=rows)
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    g = torch.Generator().manual_seed(3)
    ws = [oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05) for _ in range(E)]
    wq, wsc = torch.stack([w[0] for w in ws]), torch.stack([w[1] for w in ws])
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    ps = torch.tensor([[c, N, K] for c in counts], dtype=torch.int32)
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    dummy = torch.empty(0, device="cuda")
    fp8_blockwise_scaled_grouped_mm(out, dummy, dummy, dummy, dummy, dummy, aq.cuda(), wq.cuda().transpose(1, 2),
                                    a_s.cuda(), wsc.cuda().transpose(1, 2), dummy, dummy, dummy, dummy, dummy,
                                    ps.cuda(), torch.from_numpy(offs[:-1].copy()).cuda(), dummy)
    torch.cuda.synchronize()
    from sglang_b200._lib import lib
    assert lib().sglb200_read_device_status() == 0
    ref = torch.cat([oracle.w8a8_block_fp8_matmul(aq[offs[e]:offs[e + 1]], wq[e], a_s[offs[e]:offs[e + 1]], wsc[e])
                     for e in range(E)])
    assert not bool(torch.isnan(out.float()).any()), "a row was not written"
    assert_gemm_close(out, ref, f"grouped {counts}")


@pytest.mark.parametrize("name,topk", [("m9_e4_k2", 2), ("m33_e6_k3", 3)])
def test_fused_moe_golden(name, topk):
    from sglang_b200.layers.moe import fused_experts_block_fp8
    z = load_golden("moe.npz")
    a = as_bf16(z[f"{name}_a"])
    p = torch.softmax(as_t(z[f"{name}_score"]), dim=-1, dtype=torch.float32)
    w, ids = torch.topk(p, topk)
    out = fused_experts_block_fp8(a.cuda(), as_fp8(z[f"{name}_w1q"]).cuda(), as_fp8(z[f"{name}_w2q"]).cuda(),
                                  as_t(z[f"{name}_w1s"]).cuda(), as_t(z[f"{name}_w2s"]).cuda(), w.cuda(),
                                  ids.to(torch.int32).cuda())
    torch.cuda.synchronize()
    assert_gemm_close(out, as_bf16(z[f"{name}_y"]), name)


@pytest.mark.parametrize("M,E,topk,H,I", [(1, 8, 2, 256, 128), (100, 16, 4, 512, 256), (700, 32, 8, 1024, 384)])
def test_fused_moe_matches_oracle(M, E, topk, H, I):
    from sglang_b200.layers.moe import MoeRunnerConfig, StandardTopKOutput, cutlass_fused_experts_fp8, fused_experts
    a = make_activations(M, H, seed=M, outliers=False)
    w1q, w1s, w2q, w2s = _experts(E, H, I, seed=E)
    w, ids = _routing(M, E, topk, seed=M + 1)
    if M >= 100:
        ids[5, 1] = -1  # dropped by an expert-parallel dispatcher
    ref = oracle.fused_experts_block_fp8(a, w1q, w2q, w1s, w2s, w, ids)
    cfg = MoeRunnerConfig(num_experts=E, num_local_experts=E, top_k=topk, inplace=False)
    out = fused_experts(a.cuda(), w1q.cuda(), w2q.cuda(), StandardTopKOutput(w.cuda(), ids.cuda(), None), cfg,
                        use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])
    torch.cuda.synchronize()
    assert_gemm_close(out, ref, "fused_experts")
    out2 = cutlass_fused_experts_fp8(a.cuda(), w1q.cuda().transpose(1, 2), w2q.cuda().transpose(1, 2),
                                     w1s.cuda().transpose(1, 2), w2s.cuda().transpose(1, 2), w.cuda(), ids.cuda())
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    with pytest.raises(NotImplementedError):
        fused_experts(a.cuda(), w1q.cuda(), w2q.cuda(), StandardTopKOutput(w.cuda(), ids.cuda(), None), cfg,
                      use_int8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])


def test_fused_experts_options_no_combine_inplace_and_router_weight_on_input():
    """The options of ``fused_experts`` (``fused_moe_triton/fused_moe.py:254-338``): ``no_combine`` returns the
    weighted rows per (token, slot); ``inplace`` writes into ``hidden_states`` (no second buffer); with
    ``apply_router_weight_on_input`` (top-1 routing) the weight scales the gate_up result instead of the expert output."""
    from sglang_b200.layers.moe import MoeRunnerConfig, StandardTopKOutput, fused_experts
    M, E, topk, H, I = 150, 8, 2, 512, 256
    a = make_activations(M, H, seed=3, outliers=False)
    w1q, w1s, w2q, w2s = _experts(E, H, I, seed=5)
    w, ids = _routing(M, E, topk, seed=6)
    dev = [t.cuda() for t in (w1q, w2q, w1s, w2s)]

    def run(cfg, x, tw, ti):
        return fused_experts(x, dev[0], dev[1], StandardTopKOutput(tw.cuda(), ti.cuda(), None), cfg, use_fp8_w8a8=True,
                             w1_scale=dev[2], w2_scale=dev[3], block_shape=[128, 128])

    plain = run(MoeRunnerConfig(top_k=topk), a.cuda(), w, ids)
    # no_combine: [M, topk, H]; summing it in fp32 gives the combined result
    nc = run(MoeRunnerConfig(top_k=topk, no_combine=True), a.cuda(), w, ids)
    assert nc.shape == (M, topk, H)
    ref_nc = oracle.fused_experts_block_fp8(a, w1q, w2q, w1s, w2s, w, ids, no_combine=True)
    assert_gemm_close(nc.reshape(M * topk, H), ref_nc.reshape(M * topk, H), "no_combine")
    assert torch.equal(nc.float().sum(dim=1).bfloat16(), plain)
    # inplace: the result lands in the input tensor, same bits as the out-of-place call
    x = a.cuda().clone()
    got = run(MoeRunnerConfig(top_k=topk, inplace=True), x, w, ids)
    assert got.data_ptr() == x.data_ptr() and torch.equal(x, plain)
    with pytest.raises(AssertionError):
        run(MoeRunnerConfig(top_k=topk, inplace=True, no_combine=True), a.cuda().clone(), w, ids)
    # router weight on the input side, top-1
    w1_, ids1 = w[:, :1].contiguous(), ids[:, :1].contiguous()
    rw = run(MoeRunnerConfig(top_k=1, apply_router_weight_on_input=True), a.cuda(), w1_, ids1)
    ref_rw = oracle.fused_experts_block_fp8(a, w1q, w2q, w1s, w2s, w1_, ids1, apply_router_weight_on_input=True)
    assert_gemm_close(rw, ref_rw, "apply_router_weight_on_input")
    with pytest.raises(NotImplementedError):
        run(MoeRunnerConfig(top_k=topk, apply_router_weight_on_input=True), a.cuda(), w, ids)
    torch.cuda.synchronize()
