"""Drop-in replacements for the ``sgl_kernel`` ops on the block-FP8 W8A8 path.

Same names, argument order and error behaviour as ``sgl-kernel/python/sgl_kernel/{gemm,moe,
elementwise}.py``; every op validates on the host and then calls the C-ABI library
(``include/sglb200.h``) on the current CUDA stream.  Nothing here computes in PyTorch.
"""

from .elementwise import silu_and_mul  # noqa: F401
from .gemm import (  # noqa: F401
    fp8_blockwise_scaled_mm,
    sgl_per_token_group_quant_8bit,
    sgl_per_token_group_quant_fp8,
)
from .moe import (  # noqa: F401
    apply_shuffle_mul_sum,
    fp8_blockwise_scaled_grouped_mm,
    moe_align_block_size,
    moe_fused_gate,
    moe_sum_reduce,
    prepare_moe_input,
    shuffle_rows,
    topk_softmax,
)


_TORCH_OPS_LOADED = False


def load_torch_ops() -> None:
    """Register the ops with torch's dispatcher under the reference's namespace, so that they can be called the way
    ``sgl-kernel/python/sgl_kernel/{gemm,moe}.py`` call them: ``torch.ops.sgl_kernel.fp8_blockwise_scaled_mm.default(...)``,
    ``torch.ops.sgl_kernel.prepare_moe_input.default(...)`` and so on (schemas of ``sgl-kernel/csrc/common_extension.cc:
    82-83,168-181,262-263,274-290``).  Loads ``lib/libsgl_kernel_ops.so`` (built by ``python -m
    sglang_b200.build_torch_ops``), a thin compiled layer over the C ABI; raises if it has not been built."""
    global _TORCH_OPS_LOADED
    if _TORCH_OPS_LOADED:
        return
    import os

    import torch
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libsgl_kernel_ops.so")
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m sglang_b200.build_torch_ops`")
    torch.ops.load_library(path)
    _TORCH_OPS_LOADED = True
