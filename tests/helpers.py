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
