"""The product-side weight block quantisers against the reference's own outputs (``tests/golden/weights.npz``, made by
``make_golden_weights.py`` from ``per_block_cast_to_fp8`` and ``convert_weight``) and against the oracle: bit for bit."""

import pytest
import torch

import oracle
from helpers import as_fp8, as_t, bits, load_golden
from sglang_b200.layers.quantization.fp8_utils import (block_quant_dequant, block_quant_weight_fp8,
                                                       per_block_cast_to_fp8, requant_weight_ue8m0)

NAMES = ["n256_k384", "n200_k320", "n128_k128"]


@pytest.mark.parametrize("name", NAMES)
def test_fp32_scale_quantiser_matches_reference(name):
    z = load_golden("weights.npz")
    w = as_t(z[f"{name}_w"])
    q, s = block_quant_weight_fp8(w, [128, 128])
    assert torch.equal(bits(q), bits(as_fp8(z[f"{name}_f32_q"])))
    assert torch.equal(bits(s), bits(as_t(z[f"{name}_f32_s"])))
    qo, so = oracle.block_quant_weight(w)
    assert torch.equal(bits(q), bits(qo)) and torch.equal(bits(s), bits(so))


@pytest.mark.parametrize("name", NAMES)
def test_ue8m0_quantiser_matches_reference(name):
    z = load_golden("weights.npz")
    w = as_t(z[f"{name}_w"])
    q, s = per_block_cast_to_fp8(w)
    assert torch.equal(bits(q), bits(as_fp8(z[f"{name}_ue8m0_q"])))
    assert torch.equal(bits(s.contiguous()), bits(as_t(z[f"{name}_ue8m0_s"])))
    assert bool(((bits(s.contiguous()) & 0x7FFFFF) == 0).all()), "scales must be powers of two"


def test_requant_roundtrip_is_power_of_two_and_close():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(384, 256, generator=g) * 0.02
    q, s = block_quant_weight_fp8(w)
    q2, s2 = requant_weight_ue8m0(q, s, [128, 128])
    assert bool(((bits(s2) & 0x7FFFFF) == 0).all())
    back = block_quant_dequant(q2, s2, [128, 128], torch.float32)
    first = block_quant_dequant(q, s, [128, 128], torch.float32)
    assert float((back - first).norm() / first.norm()) < 0.05


@pytest.mark.gpu
def test_quantisers_on_the_gpu_give_the_same_bits():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(640, 896, generator=g) * 0.02
    q, s = block_quant_weight_fp8(w)
    qd, sd = block_quant_weight_fp8(w.cuda())
    assert torch.equal(bits(qd.cpu()), bits(q)) and torch.equal(bits(sd.cpu()), bits(s))
    q, s = per_block_cast_to_fp8(w)
    qd, sd = per_block_cast_to_fp8(w.cuda())
    assert torch.equal(bits(qd.cpu()), bits(q)) and torch.equal(bits(sd.cpu().contiguous()), bits(s.contiguous()))
