"""Shared helpers for the tests: fixture decoding and seeded workload builders."""

import os

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def as_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def as_f16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float16)


def as_fp8(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(FP8)


def as_t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def bits(t):
    """Bit pattern of a tensor as an integer tensor, for exact comparisons."""
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)
    if t.dtype == FP8:
        return t.view(torch.uint8)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


def rel_l2(x, ref):
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm().clamp(min=1e-30))


def max_abs_over_rms(x, ref):
    x, ref = x.double(), ref.double()
    rms = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return float((x - ref).abs().max() / rms)


# ----------------------------------------------------------------------------- workloads
def make_activations(M, K, seed=0, outliers=True, dtype=torch.bfloat16, row_scale=False):
    """Seeded activations ~N(0,1) on the CPU; 1% of entries x50 (the sweep's outliers) and
    optionally a per-row scale drawn log-uniform in [1e-2, 1e2] (the quant bandwidth case)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if outliers:
        x = torch.where(torch.rand(M, K, generator=g) < 0.01, x * 50.0, x)
    if row_scale:
        x = x * 10 ** (torch.rand(M, 1, generator=g) * 4 - 2)
    return x.to(dtype).contiguous()


def make_weight(N, K, seed=1, std=0.02):
    """Seeded weight ~N(0, std) block-quantised 128x128 by the oracle: (codes e4m3, scales fp32)."""
    import oracle
    g = torch.Generator().manual_seed(seed)
    return oracle.block_quant_weight(torch.randn(N, K, generator=g) * std)


def assert_gemm_close(out, ref, what="", allow_one_ulp=False):
    """The tolerance of the GEMM / MoE outputs: rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS(ref).

    ``allow_one_ulp``: an element may also differ from the reference by one unit in the last place of its 16-bit
    format.  One bf16 ulp of an element five times the RMS is already 2-4 % of the RMS, so an implementation whose
    fp32 sums differ from the oracle's in the last bits (another accumulation order inside the tensor core) cannot
    meet the max-abs bar on millions of outputs; the rel-L2 bar is unaffected."""
    o, r_ = out.float().cpu(), ref.float().cpu()
    r = rel_l2(o, r_)
    diff = (o.double() - r_.double()).abs()
    rms = r_.double().pow(2).mean().sqrt().clamp(min=1e-30)
    bound = torch.full_like(diff, 2e-2 * float(rms))
    if allow_one_ulp:
        mant_bits = 7 if ref.dtype == torch.bfloat16 else 10
        ulp = torch.ldexp(torch.ones_like(diff), torch.frexp(r_.double().abs().clamp(min=1e-30))[1] - 1 - mant_bits)
        bound = torch.maximum(bound, ulp * 1.001)
    m = float((diff / rms).max())
    bad = int((diff > bound).sum())
    assert r <= 1e-2 and bad == 0, (f"{what}: rel-L2 {r:.3e} (<=1e-2), max-abs/RMS {m:.3e} (<=2e-2"
                                    f"{' or one ulp' if allow_one_ulp else ''}), {bad} elements over")
    return r, m


def row_parallel_reference(x, wq, ws, world):
    """Oracle of the row-parallel linear (``oracle.row_parallel_reference``)."""
    import oracle
    return oracle.row_parallel_reference(x, wq, ws, world)


def expert_parallel_reference(x, w1q, w2q, w1s, w2s, topk_w, topk_ids, world):
    """Oracle of the expert-parallel MoE (``oracle.expert_parallel_reference``)."""
    import oracle
    return oracle.expert_parallel_reference(x, w1q, w2q, w1s, w2s, topk_w, topk_ids, world)
