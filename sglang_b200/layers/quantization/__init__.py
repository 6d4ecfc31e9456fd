from .fp8 import Fp8Config, Fp8LinearMethod  # noqa: F401
from .fp8_kernel import (  # noqa: F401
    create_per_token_group_quant_fp8_output_scale,
    pack_ue8m0_scales,
    per_token_group_quant_fp8,
    sglang_per_token_group_quant_fp8,
    w8a8_block_fp8_matmul,
    w8a8_block_fp8_matmul_ue8m0,
)
from .fp8_utils import (  # noqa: F401
    block_quant_dequant,
    block_quant_weight_fp8,
    per_block_cast_to_fp8,
    requant_weight_ue8m0,
    w8a8_block_fp8_linear,
)
