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
