"""Golden vectors for the weight block quantisers, made by the REFERENCE's own functions.

    python tests/golden/make_golden_weights.py /path/to/reference

``per_block_cast_to_fp8`` / ``ceil_to_ue8m0`` (``python/sglang/srt/layers/quantization/fp8_utils.py:494-512``) and
``convert_weight`` (``test/srt/cpu/utils.py:39-87``) are taken out of their files' syntax trees and executed unchanged on
seeded weights; inputs and outputs go to ``tests/golden/weights.npz``.  No reference source is written here.
"""

import ast
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _functions(path, names, ns):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    missing = set(names) - set(ns)
    assert not missing, f"{missing} not found in {path}"
    return ns


def raw(t):
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def main(ref_root):
    from typing import List, Tuple
    ns = {"torch": torch, "Tuple": Tuple, "List": List, "math": math,
          "align": lambda x, a: (x + a - 1) // a * a}  # fp8_utils.py imports align from sglang.srt.utils (ceil to a multiple)
    _functions(os.path.join(ref_root, "python/sglang/srt/layers/quantization/fp8_utils.py"),
               {"per_block_cast_to_fp8", "ceil_to_ue8m0"}, ns)
    _functions(os.path.join(ref_root, "test/srt/cpu/utils.py"), {"convert_weight"}, ns)
    gen = torch.Generator().manual_seed(7)
    out = {}
    for name, n, k in [("n256_k384", 256, 384), ("n200_k320", 200, 320), ("n128_k128", 128, 128)]:
        w = torch.randn(n, k, generator=gen) * 0.02
        w[:64, :64] *= 37.0      # blocks of very different magnitude
        if n > 128:
            w[128:, :128] = 0.0  # an all-zero block
        q, s = ns["per_block_cast_to_fp8"](w)
        q2, s2, _ = ns["convert_weight"](w, [128, 128], torch.bfloat16)
        out.update({f"{name}_w": raw(w), f"{name}_ue8m0_q": raw(q), f"{name}_ue8m0_s": raw(s.contiguous()),
                    f"{name}_f32_q": raw(q2), f"{name}_f32_s": raw(s2)})
    np.savez_compressed(os.path.join(HERE, "weights.npz"), **out)
    print("wrote weights.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_weights.py <reference checkout>")
    main(sys.argv[1])
