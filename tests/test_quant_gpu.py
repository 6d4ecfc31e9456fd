"""Parity of the CUDA per-token-group quantiser (through the C ABI) with the CPU oracle:
e4m3 codes and scales must be bit-exact in every scale layout."""

import numpy as np
import pytest
import torch

import oracle
from helpers import FP8, as_bf16, as_f16, as_t, bits, load_golden, make_activations

pytestmark = pytest.mark.gpu


def _quant(x, g=128, **kw):
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8
    q, s = sglang_per_token_group_quant_fp8(x.cuda(), g, **kw)
    torch.cuda.synchronize()
    return q, s


def _same_bits(a, b):
    return torch.equal(bits(a.cpu()), bits(b.cpu()))


@pytest.mark.parametrize("name,dec,g", [("bf16_g128", as_bf16, 128), ("bf16_g64", as_bf16, 64),
                                        ("f16_g128", as_f16, 128), ("f32_g128", as_t, 128)])
def test_golden_vectors(name, dec, g):
    z = load_golden("quant.npz")
    x = dec(z[f"{name}_x"])
    q, s = _quant(x, g)
    assert np.array_equal(bits(q.cpu()).numpy(), z[f"{name}_q"])
    assert np.array_equal(bits(s.cpu()).numpy(), z[f"{name}_s"].view(np.int32))


@pytest.mark.parametrize("M,K", [(1, 128), (3, 256), (5, 1536), (130, 7168), (1001, 2048), (64, 18432)])
@pytest.mark.parametrize("layout", ["row", "col", "col_tma", "ue8m0"])
def test_random_matches_oracle(M, K, layout):
    x = make_activations(M, K, seed=M * 7 + K, row_scale=True)
    x[0, :128] = 0
    kw = dict(row={}, col=dict(column_major_scales=True),
              col_tma=dict(column_major_scales=True, scale_tma_aligned=True),
              ue8m0=dict(column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True))[layout]
    q, s = _quant(x, 128, **kw)
    q_ref, s_ref = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=(layout == "ue8m0"))
    assert _same_bits(q, q_ref), f"{int((bits(q.cpu()) != bits(q_ref)).sum())} code mismatches"
    want = oracle.pack_scales(s_ref, layout)
    assert s.shape == want.shape and s.stride() == want.stride() and s.dtype == want.dtype
    assert _same_bits(s, want)
    if layout == "ue8m0" and (K // 128) % 4:
        # bytes of the last word past the last group are zero
        by = torch.empty(s.shape, dtype=s.dtype).copy_(s.cpu()).view(torch.uint8).view(M, -1, 4)
        assert int(by[:, -1, (K // 128) % 4:].max()) == 0


@pytest.mark.parametrize("g", [16, 32, 64])
def test_small_groups(g):
    x = make_activations(33, 512, seed=g)
    q, s = _quant(x, g)
    q_ref, s_ref = oracle.per_token_group_quant_fp8(x, g)
    assert _same_bits(q, q_ref) and _same_bits(s, s_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_other_input_dtypes(dtype):
    x = make_activations(40, 1024, seed=3, dtype=dtype)
    q, s = _quant(x, 128)
    q_ref, s_ref = oracle.per_token_group_quant_fp8(x, 128)
    assert _same_bits(q, q_ref) and _same_bits(s, s_ref)


def test_bandwidth_case_full_size():
    """M=16384 x 7168 (the quant bandwidth configuration): layouts agree with each other and a
    sample of rows agrees with the oracle bit for bit."""
    M, K = 16384, 7168
    x = make_activations(M, K, seed=0, outliers=False, row_scale=True)
    q_row, s_row = _quant(x, 128)
    q_col, s_col = _quant(x, 128, column_major_scales=True, scale_tma_aligned=True)
    q_ue, s_ue = _quant(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    assert s_col.stride() == (1, M) and s_ue.shape == (M, 14) and s_ue.stride() == (1, M)
    assert torch.equal(q_row.view(torch.uint8), q_col.view(torch.uint8))
    assert torch.equal(s_row, s_col)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:512]
    xs = x[rows].contiguous()
    q_ref, s_ref = oracle.per_token_group_quant_fp8(xs, 128)
    assert _same_bits(q_row[rows.cuda()], q_ref) and _same_bits(s_row[rows.cuda()], s_ref)
    q_ref, s_ref = oracle.per_token_group_quant_fp8(xs, 128, scale_ue8m0=True)
    assert _same_bits(q_ue[rows.cuda()], q_ref)
    assert _same_bits(s_ue[rows.cuda()].contiguous(), oracle.pack_scales(s_ref, "ue8m0").contiguous())
    # dequantised codes reproduce the input to within half an e4m3 step of the group maximum
    deq = q_row[:256].float().view(256, -1, 128) * s_row[:256].unsqueeze(-1)
    err = (deq.view(256, K) - x[:256].cuda().float()).abs().view(256, -1, 128).amax(-1)
    assert bool((err <= s_row[:256] * 16.01 + 1e-30).all())


def test_empty_and_errors():
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8
    from sglang_b200.sgl_kernel import sgl_per_token_group_quant_8bit
    q, s = sglang_per_token_group_quant_fp8(torch.empty(0, 256, dtype=torch.bfloat16, device="cuda"), 128)
    assert q.shape == (0, 256) and s.shape == (0, 2)
    with pytest.raises(AssertionError):
        sglang_per_token_group_quant_fp8(torch.zeros(4, 200, dtype=torch.bfloat16, device="cuda"), 128)
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        sgl_per_token_group_quant_8bit(x, torch.empty(4, 256, dtype=torch.int8, device="cuda"),
                                       torch.empty(4, 2, device="cuda"), 128, 1e-10, -448.0, 448.0)
    with pytest.raises(RuntimeError):
        sgl_per_token_group_quant_8bit(x, torch.empty(4, 256, dtype=FP8, device="cuda"),
                                       torch.empty(4, 3, device="cuda"), 128, 1e-10, -448.0, 448.0)
    with pytest.raises(RuntimeError):  # the C ABI itself rejects an unsupported group size
        sgl_per_token_group_quant_8bit(x, torch.empty(4, 256, dtype=FP8, device="cuda"),
                                       torch.empty(4, 32, device="cuda"), 8, 1e-10, -448.0, 448.0)


def test_fused_silu_mul_quant():
    """Fused SiLU-and-mul + quant: codes and scales equal the unfused CUDA pipeline's bit for
    bit, and the activation is within one bf16 step of the oracle's."""
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8
    from sglang_b200.sgl_kernel import silu_and_mul
    x = make_activations(77, 2 * 1024, seed=5, outliers=False).cuda()
    act = silu_and_mul(x)
    q0, s0 = sglang_per_token_group_quant_fp8(act, 128)
    q1, s1 = sglang_per_token_group_quant_fp8(x, 128, fuse_silu_and_mul=True)
    assert torch.equal(q0.view(torch.uint8), q1.view(torch.uint8)) and torch.equal(s0, s1)
    ref = oracle.silu_and_mul(x.cpu())
    d = (act.cpu().float() - ref.float()).abs()
    assert bool((d <= ref.float().abs() * 2.0 ** -7 + 1e-30).all())
    assert float((act.cpu() != ref).float().mean()) < 1e-3


@pytest.mark.parametrize("layout", ["row", "col_tma", "ue8m0"])
@pytest.mark.parametrize("fuse", [False, True])
def test_masked_per_expert_layout(layout, fuse):
    """[E, max_m, K] with masked_m valid rows per expert: valid rows equal the flat kernel's output bit for bit (and
    with that the oracle's), the other rows of codes and scales are not touched."""
    from sglang_b200.layers.quantization import (create_per_token_group_quant_fp8_output_scale,
                                                 sglang_per_token_group_quant_fp8)
    from sglang_b200.sgl_kernel import sgl_per_token_group_quant_8bit
    E, max_m, K = 5, 37, 512
    masked = torch.tensor([37, 0, 1, 20, 36], dtype=torch.int32)
    x = make_activations(E * max_m, K * (2 if fuse else 1), seed=9, outliers=False).view(E, max_m, -1).cuda()
    ue = layout == "ue8m0"
    kw = dict(column_major_scales=layout != "row", scale_tma_aligned=layout != "row", scale_ue8m0=ue)
    q = torch.full((E, max_m, K), 0.5, device="cuda").to(FP8)
    s = create_per_token_group_quant_fp8_output_scale((E, max_m, K), "cuda", 128, **kw)
    s.fill_(77 if ue else 77.0)
    sgl_per_token_group_quant_8bit(x, q, s, 128, 1e-10, -448.0, 448.0, ue, fuse, masked.cuda())
    torch.cuda.synchronize()
    sentinel_q = torch.full((1,), 0.5).to(FP8).view(torch.uint8).item()
    for e in range(E):
        m = int(masked[e])
        q_ref, s_ref = sglang_per_token_group_quant_fp8(x[e].contiguous(), 128, fuse_silu_and_mul=fuse, **kw)
        assert torch.equal(q[e, :m].view(torch.uint8), q_ref[:m].view(torch.uint8)), f"expert {e} codes"
        assert torch.equal(s[e, :m], s_ref[:m]), f"expert {e} scales"
        assert (q[e, m:].view(torch.uint8) == sentinel_q).all(), f"expert {e}: codes past masked_m were written"
        if not ue:  # UE8M0 words hold four k-blocks: rows past masked_m keep the whole word
            assert (s[e, m:] == 77.0).all(), f"expert {e}: scales past masked_m were written"
        else:
            assert (s[e, m:] == 77).all()
    # the allocating wrapper, unmasked 3-D input: every expert as the flat call
    q3, s3 = sglang_per_token_group_quant_fp8(x, 128, fuse_silu_and_mul=fuse, **kw)
    q2, s2 = sglang_per_token_group_quant_fp8(x.view(E * max_m, -1), 128, fuse_silu_and_mul=fuse, **kw)
    assert torch.equal(q3.view(torch.uint8).view(E * max_m, K), q2.view(torch.uint8))
    if layout == "row":
        assert torch.equal(s3.reshape(E * max_m, -1), s2)
    with pytest.raises(RuntimeError, match="masked_m"):
        sgl_per_token_group_quant_8bit(x, q, s, 128, 1e-10, -448.0, 448.0, ue, fuse, masked[:2].cuda())
    with pytest.raises(RuntimeError, match="3-D"):
        sgl_per_token_group_quant_8bit(x.view(E * max_m, -1), q.view(E * max_m, K),
                                       torch.empty(E * max_m, K // 128, device="cuda"), 128, 1e-10, -448.0, 448.0,
                                       False, fuse, masked.cuda())
