"""The CPU oracle against the golden vectors produced by the reference's own functions
(tests/golden/make_golden.py), plus the oracle's own layout and integer helpers."""

import hashlib
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import FP8, as_bf16, as_f16, as_fp8, as_t, bits, load_golden


@pytest.mark.parametrize("name,dec,g", [("bf16_g128", as_bf16, 128), ("bf16_g64", as_bf16, 64),
                                        ("f16_g128", as_f16, 128), ("f32_g128", as_t, 128)])
def test_quant_matches_reference_bits(name, dec, g):
    z = load_golden("quant.npz")
    x = dec(z[f"{name}_x"])
    q, s = oracle.per_token_group_quant_fp8(x, g)
    assert np.array_equal(bits(q).numpy(), z[f"{name}_q"])
    assert np.array_equal(bits(s).numpy(), z[f"{name}_s"].view(np.int32))


@pytest.mark.parametrize("name", ["m37_n320_k384", "m1_n128_k128", "m130_n576_k256"])
def test_gemm_matches_reference_bits(name):
    z = load_golden("gemm.npz")
    c = oracle.w8a8_block_fp8_matmul(as_fp8(z[f"{name}_aq"]), as_fp8(z[f"{name}_wq"]),
                                     as_t(z[f"{name}_as"]), as_t(z[f"{name}_ws"]))
    assert np.array_equal(bits(c).numpy(), z[f"{name}_c"])


@pytest.mark.parametrize("name,topk", [("m9_e4_k2", 2), ("m33_e6_k3", 3)])
def test_moe_matches_reference_bits(name, topk):
    z = load_golden("moe.npz")
    y = oracle.moe_block_fp8_from_scores(as_bf16(z[f"{name}_a"]), as_fp8(z[f"{name}_w1q"]),
                                         as_fp8(z[f"{name}_w2q"]), as_t(z[f"{name}_w1s"]),
                                         as_t(z[f"{name}_w2s"]), as_t(z[f"{name}_score"]), topk)
    assert np.array_equal(bits(y).numpy(), z[f"{name}_y"])


def test_config1_digests():
    """The reference-runnable benchmark case (M=128, K=N=4096, seed 0)."""
    z = load_golden("config1.npz")
    torch.manual_seed(0)
    A = torch.randn(128, 4096).bfloat16()
    W = torch.randn(4096, 4096) * 0.02
    aq, asc = oracle.per_token_group_quant_fp8(A, 128)
    wq, ws = oracle.block_quant_weight(W)
    sha = lambda t: hashlib.sha256(bits(t).numpy().tobytes()).hexdigest()
    if sha(aq) != str(z["aq_sha"]):
        pytest.skip("torch RNG stream differs from the one that made the fixture")
    assert sha(asc) == str(z["as_sha"]) and sha(wq) == str(z["wq_sha"]) and sha(ws) == str(z["ws_sha"])
    c = oracle.w8a8_block_fp8_matmul(aq, wq, asc, ws)
    assert np.array_equal(bits(c[:8, :64]).numpy(), z["c_corner"])
    assert sha(c) == str(z["c_sha"])


def test_ue8m0_is_exact_ceiling():
    s = torch.tensor([1.0, 1.0000001, 0.99999994, 2.2331343e-13, 3.0, 2.0 ** -20, 2.0 ** -20 * 1.5])
    r = oracle.ceil_to_ue8m0(s)
    assert torch.equal(r, torch.tensor([1.0, 2.0, 1.0, 2.0 ** -42, 4.0, 2.0 ** -20, 2.0 ** -19]))
    # agrees with the reference's formula (fp8_utils.py:511-512) on scales that real bf16 data make
    x = (torch.randn(64, 1024) * 3).bfloat16()
    amax = x.view(-1, 128).abs().amax(-1).float() / 448.0
    assert torch.equal(oracle.ceil_to_ue8m0(amax), torch.pow(2.0, torch.ceil(torch.log2(amax))))


def test_ue8m0_quant_divides_by_power_of_two():
    x = (torch.randn(8, 256) * 5).bfloat16()
    q, s = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
    q0, s0 = oracle.per_token_group_quant_fp8(x, 128)
    assert bool(((s.view(torch.int32) & 0x7FFFFF) == 0).all())
    assert bool((s >= s0).all()) and bool((s < 2 * s0).all())


def test_scale_layouts():
    M, G = 6, 5
    s = torch.arange(M * G, dtype=torch.float32).view(M, G) + 1
    assert oracle.pack_scales(s, "row").stride() == (G, 1)
    c = oracle.pack_scales(s, "col")
    assert c.stride() == (1, M) and torch.equal(c, s)
    t = oracle.pack_scales(s, "col_tma")
    assert t.stride() == (1, 8) and t.shape == (M, G) and torch.equal(t, s)
    p2 = torch.ldexp(torch.ones(M, G), torch.arange(M * G).view(M, G) - 10)
    u = oracle.pack_scales(p2, "ue8m0")
    assert u.dtype == torch.int32 and u.shape == (M, 2) and u.stride() == (1, 8)
    by = u.contiguous().view(torch.uint8).view(M, 2, 4)
    for m in range(M):
        for g in range(8):
            want = (m * G + g - 10 + 127) if g < G else 0
            assert int(by[m, g // 4, g % 4]) == want


def test_prepare_moe_input_tables():
    rng = np.random.default_rng(0)
    M, topk, E = 50, 4, 7
    ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    ids[3, 1] = -1  # a non-local expert
    offs, ps1, ps2, a_map, c_map = oracle.prepare_moe_input(ids, E, n=128, k=256)
    flat = ids.reshape(-1)
    total = int((flat >= 0).sum())
    assert offs[0] == 0 and offs[-1] == total
    assert (ps1[:, 1] == 256).all() and (ps1[:, 2] == 256).all() and (ps2[:, 1] == 256).all() and (ps2[:, 2] == 128).all()
    for e in range(E):
        seg = a_map[offs[e]:offs[e + 1]]
        assert (ps1[e, 0] == len(seg)) and (np.diff(seg) >= 0).all()  # stable order
        assert all(e in ids[t] for t in seg)
    for i, r in enumerate(c_map):
        if flat[i] < 0:
            assert r == -1
        else:
            assert offs[flat[i]] <= r < offs[flat[i] + 1] and a_map[r] == i // topk
    assert sorted(c_map[c_map >= 0]) == list(range(total))


def test_shuffle_and_combine_roundtrip():
    M, topk, E, H = 10, 2, 4, 16
    rng = np.random.default_rng(1)
    ids = np.stack([rng.permutation(E)[:topk] for _ in range(M)]).astype(np.int32)
    _, _, _, a_map, c_map = oracle.prepare_moe_input(ids, E, 8, 16)
    x = torch.randn(M, H).bfloat16()
    rep = oracle.shuffle_rows(x, a_map)
    w = torch.rand(M, topk).bfloat16()
    y = oracle.apply_shuffle_mul_sum(rep, c_map, w, M)
    want = (x.float() * w[:, 0:1].float() + x.float() * w[:, 1:2].float()).bfloat16()
    assert torch.equal(y, want)
    q = oracle.shuffle_rows(x.to(FP8), a_map)
    assert q.dtype == FP8 and torch.equal(q.view(torch.uint8)[0], x.to(FP8).view(torch.uint8)[a_map[0]])


# ---- routing helpers: tests/golden/routing.npz (made by tests/golden/make_golden_routing.py) ----------
ROUTING = np.load(os.path.join(os.path.dirname(__file__), "golden", "routing.npz"))
TOPK_CASES = {"t33_e8_k2": (torch.float32, False), "t17_e64_k6_rn": (torch.float32, True),
              "t29_e256_k8_rn": (torch.bfloat16, True), "t5_e160_k4": (torch.float16, False)}
ALIGN_CASES = {"t1_k1_e8_b4": (8, 4), "t13_k2_e8_b4": (8, 4), "t40_k4_e16_b16": (16, 16),
               "t64_k8_e64_b32": (64, 32), "t7_k3_e33_b64": (33, 64)}
SUM_CASES = {"t33_k6_h128": torch.bfloat16, "t7_k8_h256_s": torch.bfloat16, "t5_k2_h64_f16": torch.float16}


@pytest.mark.parametrize("name", sorted(TOPK_CASES))
def test_oracle_topk_softmax_matches_reference(name):
    dtype, renorm = TOPK_CASES[name]
    g = torch.from_numpy(ROUTING[f"topk_{name}_g"]).to(dtype)
    w_ref, ids_ref = ROUTING[f"topk_{name}_w"], ROUTING[f"topk_{name}_ids"]
    k = ids_ref.shape[1]
    w, ids = oracle.topk_softmax(g, k, renorm)
    assert np.array_equal(w.numpy(), w_ref)
    # torch.topk leaves the order of equal probabilities open (they occur with 16-bit logits); the kernel
    # takes the lower index first (moe_topk_softmax_kernels.cu:372).  Rows without a tie must agree exactly.
    top = torch.sort(torch.softmax(g.float(), -1), dim=-1, descending=True).values[:, :k + 1].numpy()
    untied = (np.diff(top, axis=1) != 0).all(axis=1)
    assert untied.sum() >= len(untied) // 2
    assert np.array_equal(ids.numpy()[untied], ids_ref[untied])
    p = torch.softmax(g.float(), -1).numpy()
    assert np.array_equal(np.take_along_axis(p, ids.numpy().astype(np.int64), 1),
                          np.take_along_axis(p, ids_ref.astype(np.int64), 1))


@pytest.mark.parametrize("name", sorted(ALIGN_CASES))
def test_oracle_moe_align_matches_reference(name):
    E, bs = ALIGN_CASES[name]
    ids = ROUTING[f"align_{name}_ids"]
    sorted_ids, expert_ids, post, cumsum = oracle.moe_align_block_size(ids, bs, E)
    assert post == int(ROUTING[f"align_{name}_post"][0])
    assert np.array_equal(expert_ids, ROUTING[f"align_{name}_experts"])
    assert np.array_equal(sorted_ids, ROUTING[f"align_{name}_sorted"])
    assert cumsum[0] == 0 and cumsum[1] == 0  # bucket 0 (id -1) is empty without expert parallelism


@pytest.mark.parametrize("name", sorted(SUM_CASES))
def test_oracle_moe_sum_reduce_matches_fixture(name):
    dtype = SUM_CASES[name]
    x = torch.from_numpy(ROUTING[f"sum_{name}_x"]).view(dtype)
    y = oracle.moe_sum_reduce(x, float(ROUTING[f"sum_{name}_scale"]))
    assert np.array_equal(y.view(torch.int16).numpy(), ROUTING[f"sum_{name}_y"])
    # the reference test's bar (sgl-kernel/tests/test_moe_align.py:261-268) against torch's own sum
    if float(ROUTING[f"sum_{name}_scale"]) == 1.0:
        torch.testing.assert_close(y, x.sum(dim=1), atol=2e-2, rtol=0)


GATE_CASES = {"t37_e256_g8_tg4_k8": (8, 4, 0, 2.5, False), "t21_e256_g8_tg4_k9_s1": (8, 4, 1, 2.5, True),
              "t9_e128_g4_tg2_k4": (4, 2, 0, 2.5, True), "t13_e512_g16_tg8_k16": (16, 8, 0, 1.0, False),
              "t11_e96_g6_tg3_k5": (6, 3, 0, 2.5, False)}


def by_id(w, ids):
    """Rows sorted by expert id: the torch-native gate returns its selection in no particular order."""
    order = np.argsort(ids, axis=1, kind="stable")
    return np.take_along_axis(w, order, 1), np.take_along_axis(ids, order, 1)


@pytest.mark.parametrize("name", sorted(GATE_CASES))
def test_oracle_moe_fused_gate_matches_reference(name):
    G, tg, n_shared, rsf, apply = GATE_CASES[name]
    x, bias = torch.from_numpy(ROUTING[f"gate_{name}_x"]), torch.from_numpy(ROUTING[f"gate_{name}_bias"])
    w_ref, ids_ref = ROUTING[f"gate_{name}_w"], ROUTING[f"gate_{name}_ids"]
    w, ids = oracle.moe_fused_gate(x, bias, G, tg, ids_ref.shape[1], n_shared, rsf, apply)
    w, ids = w.numpy(), ids.numpy()
    assert (ids_ref[:, ids_ref.shape[1] - n_shared:] >= x.shape[1]).all()
    w_s, ids_s = by_id(w, ids)
    w_rs, ids_rs = by_id(w_ref, ids_ref)
    assert np.array_equal(ids_s, ids_rs)
    np.testing.assert_allclose(w_s, w_rs, rtol=2e-6, atol=0)  # the sum is taken in a different order
    # the kernel's order: descending biased score among the routed slots
    k_real = ids.shape[1] - n_shared
    b = (torch.sigmoid(x) + bias).numpy()
    picked = np.take_along_axis(b, ids[:, :k_real].astype(np.int64), 1)
    assert (np.diff(picked, axis=1) <= 0).all()
