"""Grouped block-FP8 GEMM entry points with the signatures of
``python/sglang/srt/layers/deep_gemm_wrapper/entrypoint.py`` (there they forward to the third-party DeepGEMM
package; here they call the library's grouped kernel).  No JIT, no warm-up hook: ``expected_m`` is accepted and
unused."""

from __future__ import annotations

from contextlib import contextmanager
from typing import Optional, Tuple

import torch

from ..._lib import check, dtype_code, lib

FP8 = torch.float8_e4m3fn


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def grouped_gemm_nt_f8f8bf16_masked(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor],
                                    out: torch.Tensor, masked_m: torch.Tensor, expected_m: int) -> None:
    """``out[g, :masked_m[g]] = lhs[g, :masked_m[g]] @ rhs[g].T`` with 1x128 activation scales and 128x128 weight
    scales (``entrypoint.py:26-49``).  ``lhs = (a [G, max_m, K] e4m3, a_s [G, max_m, K/128] fp32)``,
    ``a_s`` in any strides, e.g. MN-major per group; ``rhs = (w [G, N, K] e4m3, w_s [G, N/128, K/128] fp32)``, ``out [G, max_m, N]`` bf16 / f16, ``masked_m [G]``
    int32.  Rows at and past ``masked_m[g]`` are left untouched."""
    a, a_s = lhs
    w, w_s = rhs
    _req(a.is_cuda and a.dtype == FP8 and a.dim() == 3 and a.is_contiguous(), "lhs must be a contiguous [G, max_m, K] e4m3 tensor")
    _req(w.dtype == FP8 and w.dim() == 3 and w.stride(2) == 1, "rhs must be [G, N, K] e4m3 with K contiguous")
    G, max_m, K = a.shape
    N = w.shape[1]
    _req(w.shape[0] == G and w.shape[2] == K, "lhs and rhs shapes cannot be multiplied")
    _req(out.shape == (G, max_m, N) and out.is_contiguous() and out.dtype in (torch.bfloat16, torch.float16),
         "out must be a contiguous [G, max_m, N] bf16/f16 tensor")
    kt, nt = -(-K // 128), -(-N // 128)
    _req(a_s.dtype == torch.float32 and a_s.shape == (G, max_m, kt), "lhs scales must be fp32 [G, max_m, ceil(K/128)]")
    _req(w_s.dtype == torch.float32 and w_s.shape == (G, nt, kt), "rhs scales must be fp32 [G, ceil(N/128), ceil(K/128)]")
    _req(masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == G,
         "masked_m must be a contiguous int32 tensor with one entry per group")
    if G == 0 or max_m == 0 or N == 0:
        return
    with torch.cuda.device(a.device):
        check(lib().sglb200_fp8_blockwise_scaled_masked_grouped_mm(
            a.data_ptr(), w.data_ptr(), a_s.data_ptr(), w_s.data_ptr(), out.data_ptr(), masked_m.data_ptr(), G, max_m, N, K,
            a.stride(1), w.stride(1), w.stride(0), out.stride(1), a_s.stride(0), a_s.stride(1), a_s.stride(2), w_s.stride(0),
            w_s.stride(1), w_s.stride(2), dtype_code(out.dtype), torch.cuda.current_stream(a.device).cuda_stream),
            "grouped_gemm_nt_f8f8bf16_masked")


@contextmanager
def configure_deep_gemm_num_sms(num_sms: Optional[int]):
    """Run the GEMMs inside the block on at most ``num_sms`` SMs (``entrypoint.py:94-104``): the way the reference keeps
    SMs free for a communication kernel that overlaps a GEMM.  ``None`` changes nothing."""
    if num_sms is None:
        yield
        return
    L = lib()
    original = L.sglb200_get_num_sms()
    check(L.sglb200_set_num_sms(int(num_sms)), "set_num_sms")
    try:
        yield
    finally:
        L.sglb200_set_num_sms(original)
