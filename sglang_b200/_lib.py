"""ctypes binding of the C-ABI library ``libsglb200.so`` (declared in ``include/sglb200.h``).

There is no CPU fallback: if the library is missing, :func:`lib` raises and tells the user to
build it (``python -m sglang_b200.build``); if a call returns a negative status, :func:`check`
raises ``RuntimeError`` with the library's own description, before anything ran on the GPU
(the reference raises ``RuntimeError`` from ``TORCH_CHECK`` the same way,
``sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:374-406``).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libsglb200.so")

_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float

# name -> argument types; every function returns int (status) unless listed in _RESTYPES
SIGNATURES = {
    "sglb200_per_token_group_quant_fp8": [_P, _I, _P, _P, _L, _L, _I, _F, _F, _F, _I, _L, _L, _P],
    "sglb200_silu_mul_group_quant_fp8": [_P, _I, _P, _P, _P, _L, _L, _I, _F, _F, _F, _I, _L, _L, _P],
    "sglb200_group_quant_fp8_batched": [_P, _I, _P, _P, _L, _L, _L, _I, _F, _F, _F, _I, _I, _P, _L, _L, _L, _P],
    "sglb200_fp8_blockwise_scaled_mm": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P],
    "sglb200_fp8_blockwise_scaled_mm_ws": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P, _L, _P],
    "sglb200_fp8_blockwise_scaled_mm_workspace_bytes": [_L, _L, _L],
    "sglb200_fp8_blockwise_scaled_mm_noalloc": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P],
    "sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes": [],
    "sglb200_fp8_blockwise_scaled_mm_pair": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _I, _P],
    "sglb200_fp8_ue8m0_scaled_mm": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P],
    "sglb200_fp8_ue8m0_scaled_mm_ws": [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P, _L, _P],
    "sglb200_fp8_ue8m0_scaled_grouped_mm": [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L,
                                            _I, _P],
    "sglb200_fp8_blockwise_scaled_grouped_mm": [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L,
                                                _L, _L, _L, _I, _P],
    "sglb200_fp8_blockwise_scaled_masked_grouped_mm": [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L,
                                                       _L, _L, _L, _L, _I, _P],
    "sglb200_prepare_moe_input": [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P],
    "sglb200_shuffle_rows": [_P, _P, _P, _L, _L, _P],
    "sglb200_apply_shuffle_mul_sum": [_P, _P, _P, _P, _L, _L, _L, _I, _I, _P],
    "sglb200_silu_and_mul": [_P, _P, _L, _L, _I, _P],
    "sglb200_topk_softmax": [_P, _I, _P, _P, _L, _L, _L, _I, _P],
    "sglb200_moe_fused_gate": [_P, _P, _I, _P, _P, _L, _L, _L, _L, _L, _L, _F, _I, _P],
    "sglb200_moe_align_block_size": [_P, _L, _L, _L, _P, _P, _P, _P, _I, _P],
    "sglb200_moe_sum_reduce": [_P, _P, _L, _L, _L, _I, _F, _P],
    "sglb200_fp8_blockwise_scaled_mm_push": [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P, _P, _I, _I,
                                             _L, _P, _L, _P],
    "sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes": [_L, _L, _L],
    "sglb200_fp8_blockwise_scaled_mm_push_scatter": [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P, _P, _I,
                                                     _I, _L, _P],
    "sglb200_peer_reduce_scatter": [_P, _P, _P, _L, _L, _L, _I, _I, _I, _L, _L, _P],
    "sglb200_peer_gather": [_P, _P, _P, _L, _L, _L, _I, _I, _I, _L, _L, _P],
    "sglb200_peer_reduce": [_P, _P, _P, _L, _L, _L, _I, _I, _L, _L, _P],
    "sglb200_ep_buffer_bytes": [_L, _L, _L, _L, _L],
    "sglb200_ep_buffer_offsets": [_L, _L, _L, _L, _L, _P],
    "sglb200_ep_dispatch": [_P, _P, _L, _L, _P, _P, _L, _L, _L, _L, _P, _I, _I, _L, _L, _P],
    "sglb200_ep_dispatch_quant": [_P, _I, _L, _P, _P, _L, _L, _L, _L, _P, _I, _I, _L, _L, _F, _P],
    "sglb200_ep_receive": [_P, _I, _I, _L, _L, _L, _L, _L, _P, _L, _P],
    "sglb200_ep_combine_push": [_P, _I, _P, _I, _I, _L, _L, _L, _L, _L, _P],
    "sglb200_ep_combine_reduce": [_P, _I, _I, _P, _P, _I, _L, _L, _L, _L, _L, _L, _L, _P],
    "sglb200_ep_completed": [_P, _L, _L, _L, _L, _L, _P],
    "sglb200_peer_completed": [_P, _P],
    "sglb200_peer_flag_bytes": [],
    "sglb200_peer_recv_bytes": [_L],
    "sglb200_peer_alloc": [_L, _P, _P],
    "sglb200_peer_open": [_P, _P],
    "sglb200_peer_close": [_P],
    "sglb200_peer_free": [_P],
    "sglb200_read_device_status": [],
    "sglb200_status_string": [_I],
    "sglb200_last_error_detail": [],
    "sglb200_version": [],
    "sglb200_set_num_sms": [_I],
    "sglb200_get_num_sms": [],
    "sglb200_set_grouped_few_rows": [_I],
    "sglb200_get_grouped_few_rows": [],
    "sglb200_nvls_all_reduce": [ctypes.c_uint64, _P, _I, _I, _L, _I, _I, _P],
    "sglb200_nvls_flag_bytes": [],
    "sglb200_fp8_blockwise_scaled_mm_allreduce": [_P, _P, _P, _P, _P, ctypes.c_uint64, _P, _P, _I, _I, _I, _L, _L, _L, _L,
                                                  _L, _L, _L, _L, _L, _I, _P],
}
_RESTYPES = {"sglb200_fp8_blockwise_scaled_mm_workspace_bytes": c_int64,
             "sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes": c_int64,
             "sglb200_ep_buffer_bytes": c_int64, "sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes": c_int64, "sglb200_peer_flag_bytes": c_int64, "sglb200_nvls_flag_bytes": c_int64, "sglb200_peer_recv_bytes": c_int64, "sglb200_status_string": c_char_p, "sglb200_last_error_detail": c_char_p, "sglb200_version": c_char_p}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library (loaded on first use).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m sglang_b200.build` "
                "(needs nvcc with sm_100a support). sglang_b200 has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = header and library out of step
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, c_int)
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        raise RuntimeError(f"{what}: {L.sglb200_status_string(status).decode()} "
                           f"({L.sglb200_last_error_detail().decode()})")


def blockwise_mm(a_ptr, b_ptr, sa_ptr, sb_ptr, out_ptr, M, N, K, lda, ldb, ldc, sa_m, sa_k, sb_n, sb_k, out_code, device,
                 stream) -> None:
    """One dense block-scaled GEMM launch; picks the split-K entry with a torch-allocated scratch buffer when the
    library asks for one (small M), else the plain entry."""
    import torch
    L = lib()
    ws_bytes = L.sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K)
    if ws_bytes > 0:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        check(L.sglb200_fp8_blockwise_scaled_mm_ws(a_ptr, b_ptr, sa_ptr, sb_ptr, out_ptr, M, N, K, lda, ldb, ldc, sa_m,
                                                   sa_k, sb_n, sb_k, out_code, ws.data_ptr(), ws_bytes, stream),
              "fp8_blockwise_scaled_mm (split-K)")
    else:
        check(L.sglb200_fp8_blockwise_scaled_mm(a_ptr, b_ptr, sa_ptr, sb_ptr, out_ptr, M, N, K, lda, ldb, ldc, sa_m,
                                                sa_k, sb_n, sb_k, out_code, stream), "fp8_blockwise_scaled_mm")


DTYPE_CODES = {"torch.bfloat16": 0, "torch.float16": 1, "torch.float32": 2}


def dtype_code(dtype) -> int:
    try:
        return DTYPE_CODES[str(dtype)]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype}: expected bfloat16, float16 or float32") from None
