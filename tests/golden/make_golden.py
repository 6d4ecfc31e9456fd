"""Generate the golden vectors under tests/golden/ from the REFERENCE's own functions.

Run once in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference module ``python/sglang/test/test_block_fp8.py`` cannot be imported without
the ``sglang`` / ``sgl_kernel`` packages, so the three torch-native functions are taken out
of its syntax tree and executed unchanged (no reference source is written to this
repository; only their outputs on seeded inputs are stored).  The fixtures hold inputs
AND outputs, so the tests that read them need neither the reference nor a matching RNG.
"""

import ast
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
WANT = {"native_per_token_group_quant_fp8", "native_w8a8_block_fp8_matmul", "torch_w8a8_block_fp8_moe"}


def load_reference(ref_root):
    path = os.path.join(ref_root, "python/sglang/test/test_block_fp8.py")
    tree = ast.parse(open(path).read())

    class _SiluAndMul:  # layers/activation.py:68-70, forward_native
        def forward_native(self, x):
            d = x.shape[-1] // 2
            return torch.nn.functional.silu(x[..., :d]) * x[..., d:]

    ns = {"torch": torch, "SiluAndMul": _SiluAndMul}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANT:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    assert WANT <= set(ns), "reference functions not found"
    return ns


def raw(t):
    """Bit pattern of a tensor as a numpy array (bf16 -> int16, e4m3 -> uint8)."""
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    if t.dtype == torch.float16:
        return t.contiguous().view(torch.int16).numpy()
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def block_quant(w):
    """Builder-side 128x128 weight quantiser (inputs only; mirrors oracle.block_quant_weight)."""
    N, K = w.shape
    Np, Kp = -(-N // 128) * 128, -(-K // 128) * 128
    wp = torch.zeros(Np, Kp)
    wp[:N, :K] = w
    v = wp.view(Np // 128, 128, Kp // 128, 128)
    s = v.abs().amax(dim=(1, 3), keepdim=True) / 448.0
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (v / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(Np, Kp)[:N, :K].contiguous()
    return q, s.view(Np // 128, Kp // 128).contiguous()


def quant_inputs(gen, M, K, dtype):
    x = torch.randn(M, K, generator=gen)
    r = 10 ** (torch.rand(M, 1, generator=gen) * 4 - 2)  # per-row scale, log-uniform 1e-2..1e2
    x = x * r
    x[torch.rand(M, K, generator=gen) < 0.01] *= 50.0
    x[0, :128] = 0.0                      # an all-zero group (eps path)
    x[1, :128] = 1e-12                    # below eps
    x[2, 128:256] = 0.0
    x[2, 130] = -3e-39                    # sub-normal magnitudes only
    x[3, :128] = torch.linspace(-448, 448, 128)  # amax = 448 -> scale exactly 1
    x[4, :128] = torch.linspace(-7, 7, 128) * 2.0 ** 20  # amax = 7 * 2^k -> power-of-two scale
    x[5, 0] = 3.0e38
    x[5, 1] = -1.0e-30
    return x.to(dtype).contiguous()


def main(ref_root):
    ref = load_reference(ref_root)
    q_ref, mm_ref, moe_ref = (ref[n] for n in sorted(WANT))
    q_ref = ref["native_per_token_group_quant_fp8"]
    mm_ref = ref["native_w8a8_block_fp8_matmul"]
    moe_ref = ref["torch_w8a8_block_fp8_moe"]
    gen = torch.Generator().manual_seed(0)

    # ---- Q: quant, three input dtypes, two group sizes
    out = {}
    for name, dtype, M, K, g in [("bf16_g128", torch.bfloat16, 37, 512, 128),
                                 ("bf16_g64", torch.bfloat16, 16, 256, 64),
                                 ("f16_g128", torch.float16, 19, 384, 128),
                                 ("f32_g128", torch.float32, 11, 256, 128)]:
        x = quant_inputs(gen, M, K, dtype)
        if dtype == torch.float16:
            x = x.float().clamp(-6e4, 6e4).to(dtype)
            # fp16(1e-10) == 0, so the reference turns an all-zero fp16 group into 0/0 = NaN codes;
            # keep such groups out of the fixture (the CUDA kernel keeps eps in fp32 there)
            zero = x.view(M, K // g, g).abs().amax(-1) == 0
            x.view(M, K // g, g)[..., 0][zero] = 1e-3
        q, s = q_ref(x, g)
        out[f"{name}_x"] = raw(x)
        out[f"{name}_q"] = raw(q)
        out[f"{name}_s"] = raw(s)
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)

    # ---- G: GEMM, ragged N (2.5 blocks) and odd M
    out = {}
    for name, M, N, K in [("m37_n320_k384", 37, 320, 384), ("m1_n128_k128", 1, 128, 128),
                          ("m130_n576_k256", 130, 576, 256)]:
        a = torch.randn(M, K, generator=gen).bfloat16()
        aq, asc = q_ref(a, 128)
        wq, ws = block_quant(torch.randn(N, K, generator=gen) * 0.02)
        c = mm_ref(aq, wq, asc, ws, [128, 128], torch.bfloat16)
        out.update({f"{name}_aq": raw(aq), f"{name}_as": raw(asc), f"{name}_wq": raw(wq),
                    f"{name}_ws": raw(ws), f"{name}_c": raw(c)})
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **out)

    # ---- ME: fused MoE (routing included)
    out = {}
    for name, M, E, topk, H, I in [("m9_e4_k2", 9, 4, 2, 256, 128), ("m33_e6_k3", 33, 6, 3, 256, 128)]:
        a = torch.randn(M, H, generator=gen).bfloat16()
        score = torch.randn(M, E, generator=gen)
        w1 = [block_quant(torch.randn(2 * I, H, generator=gen) * 0.05) for _ in range(E)]
        w2 = [block_quant(torch.randn(H, I, generator=gen) * 0.05) for _ in range(E)]
        w1q, w1s = torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1])
        w2q, w2s = torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2])
        y = moe_ref(a, w1q, w2q, w1s, w2s, score, topk, [128, 128])
        out.update({f"{name}_a": raw(a), f"{name}_score": raw(score), f"{name}_w1q": raw(w1q),
                    f"{name}_w1s": raw(w1s), f"{name}_w2q": raw(w2q), f"{name}_w2s": raw(w2s),
                    f"{name}_y": raw(y)})
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)

    # ---- the reference-runnable benchmark case: M=128, K=4096, N=4096, seed 0.  Only digests
    # and a corner of the output are stored (the full output is 1 MiB).
    torch.manual_seed(0)
    A = torch.randn(128, 4096).bfloat16()
    W = torch.randn(4096, 4096) * 0.02
    aq, asc = q_ref(A, 128)
    wq, ws = block_quant(W)
    c = mm_ref(aq, wq, asc, ws, [128, 128], torch.bfloat16)
    sha = lambda t: hashlib.sha256(raw(t).tobytes()).hexdigest()
    np.savez_compressed(os.path.join(HERE, "config1.npz"),
                        aq_sha=sha(aq), as_sha=sha(asc), wq_sha=sha(wq), ws_sha=sha(ws), c_sha=sha(c),
                        c_corner=raw(c[:8, :64]), as_corner=raw(asc[:8, :8]))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: {os.path.basename(__file__)} <reference checkout>")
    main(sys.argv[1])
