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
