"""Generate tests/golden/routing.npz from the REFERENCE's own routing functions.

    python tests/golden/make_golden_routing.py /path/to/reference

* ``fused_topk_torch_native`` (``python/sglang/srt/layers/moe/topk.py:402-431``) is taken out of the
  module's syntax tree and executed unchanged: softmax -> top-k -> optional renormalisation.
* ``moe_align_block_size_triton`` and its four stage functions (``sgl-kernel/tests/test_moe_align.py:17-148``)
  are the reference test's second implementation of the block-aligned sort.  They only use scalar
  ``tl.load`` / ``tl.store`` / ``tl.program_id`` / ``tl.cdiv`` / ``tl.minimum``, so they are executed
  unchanged with a few-line stand-in for those five names (one Python call per program id).
* ``biased_grouped_topk_impl`` (``python/sglang/srt/layers/moe/topk.py:594-665``), the torch-native twin the
  reference tests ``moe_fused_gate`` against (``sgl-kernel/tests/test_moe_fused_gate.py:44-56``), is executed
  unchanged without its ``torch.compile`` decorator; the two id post-processing hooks it calls are identity here.
* ``moe_sum_reduce``: the reference test's expectation is ``input.sum(dim=1)`` (``test_moe_align.py:261-268``);
  the kernel's own order (fp32, ascending j, then the factor, ``moe_sum_reduce.cu:146-170``) is stored.

No reference source is written to this repository; only outputs on seeded inputs are stored.
"""

import ast
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


# ---- a scalar stand-in for the five triton.language names the stage functions use ----------------
class Ptr:
    def __init__(self, arr, off=0):
        self.arr, self.off = arr, int(off)

    def __add__(self, k):
        return Ptr(self.arr, self.off + int(k))

    def __sub__(self, k):
        return Ptr(self.arr, self.off - int(k))


class _Launcher:
    def __init__(self, fn, tl):
        self.fn, self.tl = fn, tl

    def __getitem__(self, grid):
        def run(*args):
            args = [Ptr(a.view(-1).numpy()) if isinstance(a, torch.Tensor) else a for a in args]
            for pid in range(grid[0]):
                self.tl._pid = pid
                self.fn(*args)
        return run


def fake_triton():
    tl = types.SimpleNamespace(_pid=0, constexpr=int)
    tl.program_id = lambda axis: tl._pid
    tl.load = lambda p: int(p.arr[p.off])
    tl.cdiv = lambda a, b: (a + b - 1) // b
    tl.minimum = min

    def store(p, v):
        p.arr[p.off] = v
    tl.store = store
    triton = types.SimpleNamespace(jit=lambda fn: _Launcher(fn, tl))
    return triton, tl


def load_align(ref_root):
    path = os.path.join(ref_root, "sgl-kernel/tests/test_moe_align.py")
    tree = ast.parse(open(path).read())
    triton, tl = fake_triton()
    ns = {"torch": torch, "triton": triton, "tl": tl}
    want = {"ceil_div", "moe_align_block_size_triton"} | {f"moe_align_block_size_stage{i}" for i in (1, 2, 3, 4)}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in want:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    assert want <= set(ns)
    return ns["moe_align_block_size_triton"]


def load_topk(ref_root):
    path = os.path.join(ref_root, "python/sglang/srt/layers/moe/topk.py")
    tree = ast.parse(open(path).read())
    ns = {"torch": torch, "F": torch.nn.functional}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == "fused_topk_torch_native":
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    return ns["fused_topk_torch_native"]


def load_gate(ref_root):
    from typing import Optional
    path = os.path.join(ref_root, "python/sglang/srt/layers/moe/topk.py")
    tree = ast.parse(open(path).read())
    ns = {"torch": torch, "Optional": Optional, "ExpertLocationDispatchInfo": object,
          "topk_ids_logical_to_physical": lambda ids, info: ids,
          "_mask_topk_ids_padded_region": lambda ids, n: None}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == "biased_grouped_topk_impl":
            node.decorator_list = []
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    return ns["biased_grouped_topk_impl"]


def main(ref_root):
    gen = torch.Generator().manual_seed(1)
    out = {}

    # ---- topk_softmax
    topk_ref = load_topk(ref_root)
    for name, M, E, k, renorm, dtype in [("t33_e8_k2", 33, 8, 2, False, torch.float32),
                                         ("t17_e64_k6_rn", 17, 64, 6, True, torch.float32),
                                         ("t29_e256_k8_rn", 29, 256, 8, True, torch.bfloat16),
                                         ("t5_e160_k4", 5, 160, 4, False, torch.float16)]:
        g = (torch.randn(M, E, generator=gen) * 2.0).to(dtype)
        w, ids = topk_ref(torch.empty(M, 1), g, k, renorm)
        out[f"topk_{name}_g"] = g.float().numpy()
        out[f"topk_{name}_w"] = w.float().numpy()
        out[f"topk_{name}_ids"] = ids.to(torch.int32).numpy()

    # ---- moe_align_block_size (ids in [0, E); the caller passes E + 1 buckets)
    align_ref = load_align(ref_root)
    for name, T, k, E, bs in [("t1_k1_e8_b4", 1, 1, 8, 4), ("t13_k2_e8_b4", 13, 2, 8, 4),
                              ("t40_k4_e16_b16", 40, 4, 16, 16), ("t64_k8_e64_b32", 64, 8, 64, 32),
                              ("t7_k3_e33_b64", 7, 3, 33, 64)]:
        ids = torch.argsort(torch.rand(T, E, generator=gen), dim=1)[:, :k].to(torch.int32).contiguous()
        cap = ids.numel() + (E + 1) * (bs - 1)
        sorted_ids = torch.full((cap,), ids.numel(), dtype=torch.int32)
        expert_ids = torch.zeros(cap // bs + 1, dtype=torch.int32)
        post = torch.zeros(1, dtype=torch.int32)
        align_ref(ids, E + 1, bs, sorted_ids, expert_ids, post)
        out[f"align_{name}_ids"] = ids.numpy()
        out[f"align_{name}_sorted"] = sorted_ids.numpy()
        out[f"align_{name}_experts"] = expert_ids.numpy()[: int(post) // bs]
        out[f"align_{name}_post"] = post.numpy()

    # ---- moe_fused_gate (always renormalised, as the kernel)
    gate_ref = load_gate(ref_root)
    for name, T, E, G, tg, k, ns_, rsf, apply, dtype, kind in [
            ("t37_e256_g8_tg4_k8", 37, 256, 8, 4, 8, 0, 2.5, False, torch.float32, "rand"),
            ("t21_e256_g8_tg4_k9_s1", 21, 256, 8, 4, 9, 1, 2.5, True, torch.float32, "randn"),
            ("t9_e128_g4_tg2_k4", 9, 128, 4, 2, 4, 0, 2.5, True, torch.float32, "randn"),
            ("t13_e512_g16_tg8_k16", 13, 512, 16, 8, 16, 0, 1.0, False, torch.float32, "rand"),
            ("t11_e96_g6_tg3_k5", 11, 96, 6, 3, 5, 0, 2.5, False, torch.float32, "randn")]:
        x = (torch.rand(T, E, generator=gen) if kind == "rand" else torch.randn(T, E, generator=gen)).to(dtype)
        bias = (torch.rand(E, generator=gen) * (1.0 if kind == "rand" else 0.1)).to(dtype)
        torch.manual_seed(0)  # the shared-expert id of the torch-native function is random
        w, ids = gate_ref(x, x, bias, k, True, G, tg, ns_, rsf, None, None, apply)
        out[f"gate_{name}_x"] = x.float().numpy()
        out[f"gate_{name}_bias"] = bias.float().numpy()
        out[f"gate_{name}_w"] = w.float().numpy()
        out[f"gate_{name}_ids"] = ids.to(torch.int32).numpy()

    # ---- moe_sum_reduce
    for name, T, k, H, scale, dtype in [("t33_k6_h128", 33, 6, 128, 1.0, torch.bfloat16),
                                        ("t7_k8_h256_s", 7, 8, 256, 2.5, torch.bfloat16),
                                        ("t5_k2_h64_f16", 5, 2, 64, 0.5, torch.float16)]:
        x = torch.randn(T, k, H, generator=gen).to(dtype)
        acc = torch.zeros(T, H)
        for j in range(k):
            acc = acc + x[:, j].float()
        y = (acc * scale).to(dtype)
        out[f"sum_{name}_x"] = x.view(torch.int16).numpy()
        out[f"sum_{name}_y"] = y.view(torch.int16).numpy()
        out[f"sum_{name}_scale"] = np.float32(scale)
    np.savez_compressed(os.path.join(HERE, "routing.npz"), **out)
    print("wrote routing.npz with", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: {os.path.basename(__file__)} <reference checkout>")
    main(sys.argv[1])
