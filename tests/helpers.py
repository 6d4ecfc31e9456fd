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


def assert_gemm_close(out, ref, what=""):
    """The tolerance of the GEMM / MoE outputs: rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS(ref)."""
    r, m = rel_l2(out.float().cpu(), ref.float().cpu()), max_abs_over_rms(out.float().cpu(), ref.float().cpu())
    assert r <= 1e-2 and m <= 2e-2, f"{what}: rel-L2 {r:.3e} (<=1e-2), max-abs/RMS {m:.3e} (<=2e-2)"
    return r, m
