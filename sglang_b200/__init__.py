"""sglang_b200 — B200 (sm_100a) implementation of SGLang's block-FP8 W8A8 linear / fused-MoE path.

Python here is host glue over ``libsglb200.so`` (C ABI in ``include/sglb200.h``); there is no
CPU fallback.  ``sglang_b200.sgl_kernel`` mirrors the ``sgl_kernel`` op names,
``sglang_b200.layers`` the layer-level functions of ``sglang.srt.layers``.
"""

__version__ = "0.1"
