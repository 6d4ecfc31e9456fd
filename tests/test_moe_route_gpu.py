"""Parity of the router-side helpers (softmax + top-k, block-aligned sort, top-k sum) with the CPU oracle and
the fixtures made from the reference's own functions.  Integer tables and the sum are bit-exact; softmax
weights are compared within 1e-5 relative (expf differs by units in the last place between CPU and GPU), and
expert ids are compared exactly wherever the selection is not decided by a gap of under 1e-6 relative."""

import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

ROUTING = np.load(os.path.join(os.path.dirname(__file__), "golden", "routing.npz"))


def _topk(g, k, renorm):
    from sglang_b200.sgl_kernel import topk_softmax
    w = torch.empty(g.size(0), k, dtype=torch.float32, device="cuda")
    ids = torch.empty(g.size(0), k, dtype=torch.int32, device="cuda")
    topk_softmax(w, ids, g.cuda(), renorm)
    torch.cuda.synchronize()
    return w.cpu(), ids.cpu()


def _check_topk(g, k, renorm):
    w, ids = _topk(g, k, renorm)
    w_ref, ids_ref = oracle.topk_softmax(g, k, renorm)
    torch.testing.assert_close(w, w_ref, rtol=1e-5, atol=1e-9)
    p = torch.softmax(g.float(), -1)
    top = torch.sort(p, dim=-1, descending=True).values[:, :min(k + 1, p.size(1))]
    gap = (top[:, :-1] - top[:, 1:]) / top[:, :-1]
    tied = gap == 0  # exact ties follow the index rule on both sides
    clear = ((gap > 1e-6) | tied).all(dim=1)
    assert clear.float().mean() > 0.9
    assert torch.equal(ids[clear], ids_ref[clear])
    # everywhere: the selected experts carry the weights the oracle reports (a near-tie may swap two ids)
    sel = p.gather(1, ids.long())
    if renorm:
        sel = sel / sel.sum(-1, keepdim=True)
    torch.testing.assert_close(sel, w_ref, rtol=1e-5, atol=1e-9)
    assert (ids >= 0).all() and (ids < g.size(1)).all()
    assert all(len(set(r.tolist())) == k for r in ids[:64])  # no expert twice


@pytest.mark.parametrize("name,dtype,renorm", [("t33_e8_k2", torch.float32, False), ("t17_e64_k6_rn", torch.float32, True),
                                               ("t29_e256_k8_rn", torch.bfloat16, True),
                                               ("t5_e160_k4", torch.float16, False)])
def test_topk_softmax_golden(name, dtype, renorm):
    g = torch.from_numpy(ROUTING[f"topk_{name}_g"]).to(dtype)
    w_ref, ids_ref = ROUTING[f"topk_{name}_w"], ROUTING[f"topk_{name}_ids"]
    w, ids = _topk(g, ids_ref.shape[1], renorm)
    np.testing.assert_allclose(w.numpy(), w_ref, rtol=1e-5, atol=1e-9)
    _check_topk(g, ids_ref.shape[1], renorm)


@pytest.mark.parametrize("T,E,k", [(1, 4, 1), (16, 8, 2), (128, 64, 4), (512, 256, 8), (2048, 128, 4), (1000, 160, 6),
                                   (300, 257, 8), (64, 1024, 32), (7, 33, 33), (4096, 384, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("renorm", [False, True])
def test_topk_softmax_parity(T, E, k, dtype, renorm):
    gen = torch.Generator().manual_seed(T * 7 + E + k)
    g = (torch.randn(T, E, generator=gen) * 3.0).to(dtype)
    _check_topk(g, k, renorm)


def test_topk_softmax_edge_cases():
    # identical logits everywhere: the first k experts, in order, each 1 / E
    g = torch.zeros(5, 48)
    w, ids = _topk(g, 6, False)
    assert torch.equal(ids, torch.arange(6, dtype=torch.int32).repeat(5, 1))
    torch.testing.assert_close(w, torch.full((5, 6), 1.0 / 48), rtol=1e-6, atol=0)
    # huge spread: no overflow, the rest underflow to zero
    g = torch.full((3, 16), -1e4)
    g[:, 11] = 1e4
    w, ids = _topk(g, 2, True)
    assert (ids[:, 0] == 11).all() and (ids[:, 1] == 0).all()
    assert torch.equal(w, torch.tensor([[1.0, 0.0]] * 3))
    # empty batch
    w, ids = _topk(torch.zeros(0, 8), 2, False)
    assert w.shape == (0, 2)
    from sglang_b200.sgl_kernel import topk_softmax
    with pytest.raises(RuntimeError, match="topk must be less than or equal"):
        topk_softmax(torch.empty(2, 9, device="cuda"), torch.empty(2, 9, dtype=torch.int32, device="cuda"),
                     torch.zeros(2, 8, device="cuda"))
    with pytest.raises(RuntimeError, match="num_experts"):
        topk_softmax(torch.empty(2, 2, device="cuda"), torch.empty(2, 2, dtype=torch.int32, device="cuda"),
                     torch.zeros(2, 2048, device="cuda"))


def _align(ids, E, bs, pad):
    from sglang_b200.sgl_kernel import moe_align_block_size
    numel = ids.numel()
    cap = numel + (E + 1) * (bs - 1)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device="cuda")
    if not pad:
        sorted_ids.fill_(numel)
    expert_ids = torch.full((-(-cap // bs),), -7, dtype=torch.int32, device="cuda")
    post = torch.empty(1, dtype=torch.int32, device="cuda")
    cumsum = torch.empty(E + 2, dtype=torch.int32, device="cuda")
    moe_align_block_size(ids.cuda(), E + 1, bs, sorted_ids, expert_ids, post, cumsum, pad)
    torch.cuda.synchronize()
    return sorted_ids.cpu().numpy(), expert_ids.cpu().numpy(), int(post.item()), cumsum.cpu().numpy()


def _check_align(ids, E, bs, pad):
    s, e, post, cs = _align(ids, E, bs, pad)
    s_ref, e_ref, post_ref, cs_ref = oracle.moe_align_block_size(ids.numpy(), bs, E)
    assert post == post_ref
    assert np.array_equal(e[:post // bs], e_ref)
    assert (e[post // bs:] == -7).all()  # blocks past the padded length are left alone
    assert np.array_equal(s[:post], s_ref[:post])
    if not pad:
        assert np.array_equal(s, s_ref)
    assert np.array_equal(cs[:E + 2], cs_ref)


@pytest.mark.parametrize("name,E,bs", [("t1_k1_e8_b4", 8, 4), ("t13_k2_e8_b4", 8, 4), ("t40_k4_e16_b16", 16, 16),
                                       ("t64_k8_e64_b32", 64, 32), ("t7_k3_e33_b64", 33, 64)])
@pytest.mark.parametrize("pad", [False, True])
def test_moe_align_golden(name, E, bs, pad):
    ids = torch.from_numpy(ROUTING[f"align_{name}_ids"])
    s, e, post, _ = _align(ids, E, bs, pad)
    assert post == int(ROUTING[f"align_{name}_post"][0])
    assert np.array_equal(e[:post // bs], ROUTING[f"align_{name}_experts"])
    assert np.array_equal(s[:post], ROUTING[f"align_{name}_sorted"][:post])


@pytest.mark.parametrize("bs", [32, 64, 128, 256])
@pytest.mark.parametrize("T,topk", [(1, 1), (2, 8), (16, 2), (64, 64), (256, 8), (1024, 4), (4096, 8), (4096, 64)])
@pytest.mark.parametrize("E", [64, 160, 256, 257, 264])
def test_moe_align_parity(bs, T, topk, E):
    gen = torch.Generator().manual_seed(bs + T + topk + E)
    ids = torch.argsort(torch.rand(T, E, generator=gen), dim=1)[:, :topk].to(torch.int32).contiguous()
    _check_align(ids, E, bs, pad=bool((T + E) & 1))


def test_moe_align_filtered_and_empty():
    # expert-parallel case: ids of experts another rank owns arrive as -1 and land in bucket 0 (expert id -1)
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 32, (333, 6), generator=gen, dtype=torch.int32)
    ids[torch.rand(333, 6, generator=gen) < 0.4] = -1
    _check_align(ids, 32, 64, pad=True)
    s, e, post, cs = _align(ids, 32, 64, True)
    n_filtered = int((ids == -1).sum())
    assert (e[:-(-n_filtered // 64)] == -1).all() and cs[1] == -(-n_filtered // 64) * 64
    # all slots on one expert; and no slots at all
    _check_align(torch.full((100, 2), 5, dtype=torch.int32), 8, 16, pad=True)
    _check_align(torch.zeros(0, 4, dtype=torch.int32), 8, 16, pad=True)
    # the largest expert count the kernel takes (1024 buckets)
    ids = torch.randint(0, 1023, (2000, 8), generator=gen, dtype=torch.int32)
    _check_align(ids, 1023, 16, pad=False)
    from sglang_b200.sgl_kernel import moe_align_block_size
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="at least"):
        moe_align_block_size(z, 9, 16, z, z, z, z)


def _sum(x, scale):
    from sglang_b200.sgl_kernel import moe_sum_reduce
    y = torch.empty(x.size(0), x.size(2), dtype=x.dtype, device="cuda")
    moe_sum_reduce(x.cuda(), y, scale)
    torch.cuda.synchronize()
    return y.cpu()


@pytest.mark.parametrize("name,dtype", [("t33_k6_h128", torch.bfloat16), ("t7_k8_h256_s", torch.bfloat16),
                                        ("t5_k2_h64_f16", torch.float16)])
def test_moe_sum_reduce_golden(name, dtype):
    x = torch.from_numpy(ROUTING[f"sum_{name}_x"]).view(dtype)
    y = _sum(x, float(ROUTING[f"sum_{name}_scale"]))
    assert np.array_equal(y.view(torch.int16).numpy(), ROUTING[f"sum_{name}_y"])


@pytest.mark.parametrize("T", [1, 33, 64, 222, 4096])
@pytest.mark.parametrize("topk", [1, 2, 6, 8, 9])
@pytest.mark.parametrize("H", [128, 1024, 7168])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_sum_reduce_exact(T, topk, H, dtype):
    if T * topk * H > 4096 * 8 * 7168:
        pytest.skip("larger than the serving shape")
    gen = torch.Generator().manual_seed(T + topk + H)
    x = torch.randn(T, topk, H, generator=gen).to(dtype)
    scale = 2.5 if topk % 2 else 1.0
    y = _sum(x, scale)
    assert torch.equal(y.view(torch.int16), oracle.moe_sum_reduce(x, scale).view(torch.int16))


def test_moe_sum_reduce_rejects():
    from sglang_b200.sgl_kernel import moe_sum_reduce
    x = torch.zeros(4, 2, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 8"):
        moe_sum_reduce(x, torch.empty(4, 100, dtype=torch.bfloat16, device="cuda"), 1.0)
    with pytest.raises(RuntimeError, match="hidden_dim mismatch"):
        moe_sum_reduce(x, torch.empty(4, 96, dtype=torch.bfloat16, device="cuda"), 1.0)
    _sum(torch.zeros(0, 2, 128, dtype=torch.bfloat16), 1.0)  # empty batch: nothing launched


@pytest.mark.parametrize("name,topk", [("m9_e4_k2", 2), ("m33_e6_k3", 3)])
def test_routed_moe_from_logits_golden(name, topk):
    """Router logits -> fused_topk -> fused expert MLP, all on the GPU, against the reference's torch-native
    MoE (which takes the logits) on the stored inputs."""
    from helpers import as_bf16, as_fp8, as_t, assert_gemm_close, load_golden
    from sglang_b200.layers.moe import fused_experts_block_fp8
    from sglang_b200.layers.moe.topk import fused_topk, moe_align_block_size
    z = load_golden("moe.npz")
    a = as_bf16(z[f"{name}_a"]).cuda()
    w, ids = fused_topk(a, as_t(z[f"{name}_score"]).cuda(), topk, renormalize=False)
    out = fused_experts_block_fp8(a, as_fp8(z[f"{name}_w1q"]).cuda(), as_fp8(z[f"{name}_w2q"]).cuda(),
                                  as_t(z[f"{name}_w1s"]).cuda(), as_t(z[f"{name}_w2s"]).cuda(), w, ids)
    torch.cuda.synchronize()
    assert_gemm_close(out, as_bf16(z[f"{name}_y"]), name)
    E = z[f"{name}_w1q"].shape[0]
    s, e, post = moe_align_block_size(ids, 16, E)
    s_ref, e_ref, post_ref, _ = oracle.moe_align_block_size(ids.cpu().numpy(), 16, E)
    assert int(post) == post_ref and np.array_equal(s.cpu().numpy()[:post_ref], s_ref[:post_ref])
    assert np.array_equal(e.cpu().numpy()[:post_ref // 16], e_ref)


def _gate(x, bias, G, tg, k, n_shared=0, rsf=2.5, apply=False):
    from sglang_b200.sgl_kernel import moe_fused_gate
    w, ids = moe_fused_gate(x.cuda(), bias.cuda(), G, tg, k, n_shared, rsf, apply)
    torch.cuda.synchronize()
    return w.cpu(), ids.cpu()


def _check_gate(x, bias, G, tg, k, n_shared, rsf, apply):
    w, ids = _gate(x, bias, G, tg, k, n_shared, rsf, apply)
    w_ref, ids_ref = oracle.moe_fused_gate(x, bias, G, tg, k, n_shared, rsf, apply)
    E = x.size(1)
    k_real = k - n_shared
    assert torch.equal(ids[:, k_real:], ids_ref[:, k_real:])  # shared slots: E, E + 1, ...
    # rows whose group choice and expert choice are decided by gaps above 1e-6 must agree id for id
    s = torch.sigmoid(x.float()).to(x.dtype)
    b = (s + bias).to(x.dtype).float()
    gs = torch.sort(b.view(x.size(0), G, E // G), dim=-1, descending=True).values[..., :2].sum(-1)
    gsorted = torch.sort(gs, dim=-1, descending=True).values
    clear = torch.ones(x.size(0), dtype=torch.bool)
    if tg < G:
        d = gsorted[:, tg - 1] - gsorted[:, tg]
        clear &= (d > 1e-6 * gsorted[:, tg - 1].abs()) | (d == 0)
    rows = torch.arange(x.size(0))
    picked = b[rows[:, None], ids_ref[:, :k_real].long()]
    kept = torch.zeros(x.size(0), G, dtype=torch.bool)
    kept.scatter_(1, torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :tg], True)
    rest = b.masked_fill(~kept.repeat_interleave(E // G, dim=1), -float("inf"))
    rest[rows[:, None], ids_ref[:, :k_real].long()] = -float("inf")
    seq = torch.cat([picked, rest.max(-1, keepdim=True).values], dim=1)
    d = seq[:, :-1] - seq[:, 1:]
    if x.dtype == torch.float32:
        clear &= ((d > 1e-6 * seq[:, :-1].abs()) | (d == 0)).all(dim=1)
    assert clear.float().mean() > 0.8 or x.size(0) < 16
    if x.dtype == torch.float32:
        assert torch.equal(ids[clear], ids_ref[clear])
        torch.testing.assert_close(w[clear], w_ref[clear], rtol=1e-5, atol=1e-7)
    else:
        # a sigmoid within an fp32 ulp of a 16-bit rounding boundary may round the other way on the GPU and move
        # one selection: nearly all rows must agree id for id, and those rows within one 16-bit ulp in weight
        same = (ids == ids_ref).all(dim=1) & clear
        assert same.float().mean() > 0.97
        torch.testing.assert_close(w[same], w_ref[same], rtol=1e-2, atol=1e-7)
    total = w[:, :k_real].sum(-1) / (rsf if apply else 1.0)
    torch.testing.assert_close(total, torch.ones_like(total), rtol=1e-5, atol=0)
    assert (ids[:, :k_real] >= 0).all() and (ids[:, :k_real] < E).all()


@pytest.mark.parametrize("name,G,tg,n_shared,rsf,apply", [
    ("t37_e256_g8_tg4_k8", 8, 4, 0, 2.5, False), ("t21_e256_g8_tg4_k9_s1", 8, 4, 1, 2.5, True),
    ("t9_e128_g4_tg2_k4", 4, 2, 0, 2.5, True), ("t13_e512_g16_tg8_k16", 16, 8, 0, 1.0, False),
    ("t11_e96_g6_tg3_k5", 6, 3, 0, 2.5, False)])
def test_moe_fused_gate_golden(name, G, tg, n_shared, rsf, apply):
    x, bias = torch.from_numpy(ROUTING[f"gate_{name}_x"]), torch.from_numpy(ROUTING[f"gate_{name}_bias"])
    w_ref, ids_ref = ROUTING[f"gate_{name}_w"], ROUTING[f"gate_{name}_ids"]
    w, ids = _gate(x, bias, G, tg, ids_ref.shape[1], n_shared, rsf, apply)
    o = np.argsort(ids.numpy(), axis=1, kind="stable")
    o_ref = np.argsort(ids_ref, axis=1, kind="stable")
    assert np.array_equal(np.take_along_axis(ids.numpy(), o, 1), np.take_along_axis(ids_ref, o_ref, 1))
    np.testing.assert_allclose(np.take_along_axis(w.numpy(), o, 1), np.take_along_axis(w_ref, o_ref, 1), rtol=1e-5)


@pytest.mark.parametrize("T", [1, 7, 64, 1024, 8192])
@pytest.mark.parametrize("E,G,tg,k", [(128, 4, 2, 4), (256, 8, 4, 8), (512, 16, 8, 16), (96, 6, 3, 5), (1024, 32, 4, 32),
                                      (64, 1, 1, 6)])
@pytest.mark.parametrize("n_shared", [0, 1, 2])
@pytest.mark.parametrize("apply", [False, True])
def test_moe_fused_gate_parity(T, E, G, tg, k, n_shared, apply):
    gen = torch.Generator().manual_seed(T + E + n_shared)
    x = torch.rand(T, E, generator=gen) if (T & 1) else torch.randn(T, E, generator=gen)
    bias = torch.rand(E, generator=gen)
    if k + n_shared > 32:
        k -= n_shared
    _check_gate(x, bias, G, tg, k + n_shared, n_shared, 2.5, apply)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_fused_gate_16bit(dtype):
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(512, 256, generator=gen).to(dtype)
    bias = (torch.rand(256, generator=gen) * 0.1).to(dtype)
    _check_gate(x, bias, 8, 4, 8, 0, 2.5, False)


def test_moe_fused_gate_rejects_and_layer_entry():
    from sglang_b200.layers.moe.topk import biased_grouped_topk
    from sglang_b200.sgl_kernel import moe_fused_gate
    x = torch.zeros(4, 256, device="cuda")
    bias = torch.zeros(256, device="cuda")
    with pytest.raises(RuntimeError, match="num_expert_group"):
        moe_fused_gate(x, bias, 7, 4, 8)
    with pytest.raises(RuntimeError, match="fit into the selected groups"):
        moe_fused_gate(x, bias, 32, 1, 9)
    with pytest.raises(RuntimeError, match="same num_experts"):
        moe_fused_gate(x, bias[:128], 8, 4, 8)
    # identical scores everywhere: groups 0..3, experts 0..7, equal weights
    w, ids = biased_grouped_topk(x, x, bias, 8, True, 8, 4, routed_scaling_factor=2.5)
    assert torch.equal(ids.cpu(), torch.arange(8, dtype=torch.int32).repeat(4, 1))
    torch.testing.assert_close(w.cpu(), torch.full((4, 8), 0.125))
    with pytest.raises(RuntimeError, match="renormalize"):
        biased_grouped_topk(x, x, bias, 8, False, 8, 4)
