"""CPU oracle for the block-FP8 W8A8 hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory: it is the checker used by
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``.

Parity status: PINNED.  ``tests/golden/make_golden.py`` executes the reference's own
torch-native functions (``native_per_token_group_quant_fp8``,
``native_w8a8_block_fp8_matmul``, ``torch_w8a8_block_fp8_moe`` from
``python/sglang/test/test_block_fp8.py``) on seeded inputs and stores their outputs under
``tests/golden/``; ``tests/test_oracle_golden.py`` checks this restatement against those
files bit for bit.  The UE8M0 scale variant is defined by composition
(``ceil_to_ue8m0(amax / 448)`` from ``fp8_utils.py:511-512`` applied inside the native
quant function); no reference test pins it on random data.  The routing helpers (``topk_softmax``,
``moe_fused_gate``, ``moe_align_block_size``, ``moe_sum_reduce``) are pinned by ``tests/golden/make_golden_routing.py``, which runs
``fused_topk_torch_native`` and ``biased_grouped_topk_impl`` (``python/sglang/srt/layers/moe/topk.py:402-431,594-665``) and the reference test's staged
block-aligned sort (``sgl-kernel/tests/test_moe_align.py:17-148``) into ``tests/golden/routing.npz``.
"""

from .block_fp8 import (  # noqa: F401
    FP8_MAX,
    apply_shuffle_mul_sum,
    block_quant_weight,
    ceil_to_ue8m0,
    expert_parallel_reference,
    fused_experts_block_fp8,
    moe_align_block_size,
    moe_block_fp8_from_scores,
    moe_fused_gate,
    moe_sum_reduce,
    pack_scales,
    per_token_group_quant_fp8,
    prepare_moe_input,
    row_parallel_partials,
    row_parallel_reference,
    shuffle_rows,
    silu_and_mul,
    sum_in_storage_type_bound,
    topk_softmax,
    w8a8_block_fp8_matmul,
)
