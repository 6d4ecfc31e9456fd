"""The compiled torch registration (``torch.ops.sgl_kernel.*``, schemas of the reference's common_extension.cc) against
the oracle, and CUDA-graph capture of the layer-level calls (a replay must reproduce the eager result bit for bit)."""

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, bits, make_activations, make_weight

SCHEMAS = {
    "fp8_blockwise_scaled_mm": "sgl_kernel::fp8_blockwise_scaled_mm(Tensor mat_a, Tensor mat_b, Tensor scales_a, "
                               "Tensor scales_b, ScalarType out_dtype) -> Tensor",
    "sgl_per_token_group_quant_8bit": "sgl_kernel::sgl_per_token_group_quant_8bit(Tensor input, Tensor output_q, "
                                      "Tensor output_s, int group_size, float eps, float fp8_min, float fp8_max, "
                                      "bool scale_ue8m0) -> ()",
    "prepare_moe_input": "sgl_kernel::prepare_moe_input(Tensor topk_ids, Tensor expert_offsets, Tensor? "
                         "blockscale_offsets, Tensor problem_sizes1, Tensor problem_sizes2, Tensor input_permutation, "
                         "Tensor output_permutation, int num_experts, int n, int k) -> ()",
    "shuffle_rows": "sgl_kernel::shuffle_rows(Tensor input, Tensor dst2src_map, Tensor output) -> ()",
    "apply_shuffle_mul_sum": "sgl_kernel::apply_shuffle_mul_sum(Tensor input, Tensor output, Tensor permutation, "
                             "Tensor? factors) -> ()",
}


def _ops():
    from sglang_b200.sgl_kernel import load_torch_ops
    load_torch_ops()
    return torch.ops.sgl_kernel


def test_ops_are_registered_with_the_reference_schemas():
    ops = _ops()
    for name, schema in SCHEMAS.items():
        assert str(getattr(ops, name).default._schema) == schema
    for name in ("sgl_per_token_group_quant_8bit_v2", "fp8_blockwise_scaled_grouped_mm", "silu_and_mul", "moe_sum_reduce"):
        assert getattr(ops, name).default is not None


@pytest.mark.gpu
def test_quant_and_gemm_ops_match_oracle():
    ops = _ops()
    M, N, K = 77, 512, 1024
    x = make_activations(M, K, seed=5)
    wq, ws = make_weight(N, K, seed=6)
    xq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    xs = torch.empty(K // 128, M, dtype=torch.float32, device="cuda").t()  # M-major, as the reference GEMM requires
    ops.sgl_per_token_group_quant_8bit.default(x.cuda(), xq, xs, 128, 1e-10, -448.0, 448.0, False)
    q_ref, s_ref = oracle.per_token_group_quant_fp8(x, 128)
    assert torch.equal(bits(xq.cpu()), bits(q_ref)) and torch.equal(bits(xs.cpu().contiguous()), bits(s_ref))
    out = ops.fp8_blockwise_scaled_mm.default(xq, wq.cuda().t(), xs, ws.cuda().t(), torch.bfloat16)
    torch.cuda.synchronize()
    assert_gemm_close(out, oracle.w8a8_block_fp8_matmul(q_ref, wq, s_ref, ws), "torch op GEMM")
    small = ops.fp8_blockwise_scaled_mm.default(xq[:8], wq.cuda().t(), xs[:8], ws.cuda().t(), torch.bfloat16)
    assert_gemm_close(small, oracle.w8a8_block_fp8_matmul(q_ref[:8], wq, s_ref[:8], ws), "torch op GEMM, few rows")
    with pytest.raises(RuntimeError, match="column major"):
        ops.fp8_blockwise_scaled_mm.default(xq, wq.cuda().t().contiguous(), xs, ws.cuda().t(), torch.bfloat16)
    # fused SiLU-mul + quant through the v2 schema
    g = make_activations(M, 2 * K, seed=7, outliers=False)
    q2 = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    s2 = torch.empty(M, K // 128, dtype=torch.float32, device="cuda")
    ops.sgl_per_token_group_quant_8bit_v2.default(g.cuda(), q2, s2, 128, 1e-10, -448.0, 448.0, False, True, None)
    qa, sa = oracle.per_token_group_quant_fp8(oracle.silu_and_mul(g).contiguous(), 128)
    assert torch.equal(bits(q2.cpu()), bits(qa)) and torch.equal(bits(s2.cpu()), bits(sa))


@pytest.mark.gpu
def test_moe_ops_match_oracle():
    ops = _ops()
    E, topk, H, I, M = 8, 2, 256, 128, 90
    gen = torch.Generator().manual_seed(11)
    ids = torch.stack([torch.randperm(E, generator=gen)[:topk] for _ in range(M)]).to(torch.int32)
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    ps1 = torch.empty(E, 3, dtype=torch.int32, device="cuda")
    ps2 = torch.empty(E, 3, dtype=torch.int32, device="cuda")
    a_map = torch.empty(M * topk, dtype=torch.int32, device="cuda")
    c_map = torch.empty(M * topk, dtype=torch.int32, device="cuda")
    ops.prepare_moe_input.default(ids.cuda(), offs, None, ps1, ps2, a_map, c_map, E, I, H)
    o_ref, p1_ref, p2_ref, a_ref, c_ref = oracle.prepare_moe_input(ids.numpy(), E, I, H)
    assert np.array_equal(offs.cpu().numpy(), o_ref) and np.array_equal(ps1.cpu().numpy(), p1_ref)
    assert np.array_equal(a_map.cpu().numpy(), a_ref) and np.array_equal(c_map.cpu().numpy(), c_ref)
    # grouped GEMM over the sorted rows
    x = make_activations(M, H, seed=12, outliers=False)
    xq, xs = oracle.per_token_group_quant_fp8(x, 128)
    rep_q = torch.empty(M * topk, H, dtype=torch.float8_e4m3fn, device="cuda")
    ops.shuffle_rows.default(xq.cuda(), a_map, rep_q)
    rep_s = torch.empty(M * topk, H // 128, dtype=torch.float32, device="cuda")
    ops.shuffle_rows.default(xs.cuda(), a_map, rep_s)
    w = [make_weight(2 * I, H, seed=20 + e, std=0.05) for e in range(E)]
    wq, wsc = torch.stack([t[0] for t in w]), torch.stack([t[1] for t in w])
    out = torch.full((M * topk, 2 * I), float("nan"), dtype=torch.bfloat16, device="cuda")
    d = torch.empty(0, device="cuda")
    ops.fp8_blockwise_scaled_grouped_mm.default(out, d, d, d, d, d, rep_q, wq.cuda().transpose(1, 2), rep_s,
                                                wsc.cuda().transpose(1, 2), d, d, d, d, d, ps1, offs, d)
    torch.cuda.synchronize()
    rq, rs = xq[torch.from_numpy(a_ref).long()], xs[torch.from_numpy(a_ref).long()]
    ref = torch.cat([oracle.w8a8_block_fp8_matmul(rq[o_ref[e]:o_ref[e + 1]], wq[e], rs[o_ref[e]:o_ref[e + 1]], wsc[e])
                     for e in range(E)])
    assert_gemm_close(out, ref, "torch op grouped GEMM")
    # combine with fp32 products (the reference kernel's arithmetic)
    fac = torch.rand(M, topk, generator=gen).bfloat16()
    y = torch.empty(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    ops.apply_shuffle_mul_sum.default(out, y, c_map, fac.cuda().reshape(-1))
    want = oracle.apply_shuffle_mul_sum(out.cpu(), c_ref, fac, M)
    assert torch.equal(bits(y.cpu()), bits(want))


@pytest.mark.gpu
def test_linear_and_fused_experts_replay_in_a_cuda_graph():
    """Neither call synchronises, allocates outside torch's allocator or reads the host: both can be captured, and a
    replay on new input contents gives the eager result bit for bit."""
    from sglang_b200.layers.moe import fused_experts_block_fp8
    from sglang_b200.layers.quantization import Fp8Config, Fp8LinearMethod
    M, N, K = 200, 640, 1024
    wq, ws = make_weight(N, K, seed=31)
    layer = torch.nn.Module()
    method = Fp8LinearMethod(Fp8Config())
    method.create_weights(layer, K, [N], K, N, torch.bfloat16, device="cuda")
    layer.weight.data, layer.weight_scale_inv.data = wq.cuda(), ws.cuda()
    E, topk, H, I = 8, 2, 256, 128
    w1 = [make_weight(2 * I, H, seed=40 + e, std=0.05) for e in range(E)]
    w2 = [make_weight(H, I, seed=60 + e, std=0.05) for e in range(E)]
    w1q, w1s = torch.stack([t[0] for t in w1]).cuda(), torch.stack([t[1] for t in w1]).cuda()
    w2q, w2s = torch.stack([t[0] for t in w2]).cuda(), torch.stack([t[1] for t in w2]).cuda()
    gen = torch.Generator().manual_seed(3)
    tw, ti = torch.topk(torch.softmax(torch.randn(M, E, generator=gen), -1), topk)
    tw, ti = tw.cuda(), ti.to(torch.int32).cuda()
    x_lin = make_activations(M, K, seed=1).cuda()
    x_moe = make_activations(M, H, seed=2, outliers=False).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (per-device set-up calls)
        method.apply(layer, x_lin)
        fused_experts_block_fp8(x_moe, w1q, w2q, w1s, w2s, tw, ti)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_lin = method.apply(layer, x_lin)
        y_moe = fused_experts_block_fp8(x_moe, w1q, w2q, w1s, w2s, tw, ti)
    for seed in (7, 8):
        x_lin.copy_(make_activations(M, K, seed=seed).cuda())
        x_moe.copy_(make_activations(M, H, seed=seed + 10, outliers=False).cuda())
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(bits(y_lin), bits(method.apply(layer, x_lin)))
        assert torch.equal(bits(y_moe), bits(fused_experts_block_fp8(x_moe, w1q, w2q, w1s, w2s, tw, ti)))
