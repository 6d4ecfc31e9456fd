"""Parity at the sizes the benchmark reports: the DeepSeek-V3 projection sweep (fp32-scale kernel), the Llama-3-70B
tensor-parallel shard shapes and the DeepSeek-V3 expert layer, each at its full size on the GPU and checked against the
CPU oracle on a seeded sample of rows / tokens (the oracle is row-independent, so a sample pins every sampled output
exactly as a full run would).  Bars as everywhere: quant codes and scales bit-exact, bf16 outputs rel-L2 <= 1e-2 and
max-abs <= 2e-2 x RMS of the reference.

Inputs are generated on the GPU from a seeded generator (the weights alone are up to 11 GB) and the sampled rows are
copied to the host for the oracle; both sides therefore see the same bits.
"""

import pytest
import torch

import oracle
from helpers import assert_gemm_close, bits

pytestmark = pytest.mark.gpu

DSV3 = [(24576, 1536), (576, 7168), (7168, 16384), (36864, 7168), (7168, 18432)]


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _activations(M, K, seed, outliers=True):
    g = _gen(seed)
    x = torch.randn(M, K, generator=g, device="cuda")
    if outliers:  # 1 % of the entries x50, as the sweep's inputs
        x = torch.where(torch.rand(M, K, generator=g, device="cuda") < 0.01, x * 50.0, x)
    return x.bfloat16()


def _weight(N, K, seed):
    from sglang_b200.layers.quantization import block_quant_weight_fp8
    w = torch.randn(N, K, generator=_gen(seed), device="cuda") * 0.02
    return block_quant_weight_fp8(w)


def _status():
    from sglang_b200._lib import lib
    return lib().sglb200_read_device_status()


def _check_linear(M, N, K, seed, n_rows=64, via_apply=False):
    """quant + GEMM at full size on the GPU; `n_rows` sampled rows against the oracle."""
    from sglang_b200.layers.quantization import (Fp8Config, Fp8LinearMethod, sglang_per_token_group_quant_fp8,
                                                 w8a8_block_fp8_matmul)
    x = _activations(M, K, seed)
    wq, ws = _weight(N, K, seed + 1)
    q, s = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
    y = w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)
    if via_apply:
        layer = torch.nn.Module()
        method = Fp8LinearMethod(Fp8Config(weight_block_size=[128, 128]))
        method.create_weights(layer, K, [N], K, N, torch.bfloat16, device="cuda")
        layer.weight.data, layer.weight_scale_inv.data = wq, ws
        method.process_weights_after_loading(layer)
        y2 = method.apply(layer, x)
        assert torch.equal(bits(y2), bits(y)), "Fp8LinearMethod.apply differs from quant + GEMM"
    torch.cuda.synchronize()
    assert _status() == 0, "a bounded wait in the GEMM kernel timed out"
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(seed))[:min(n_rows, M)].sort().values
    rows_d = rows.cuda()
    q_ref, s_ref = oracle.per_token_group_quant_fp8(x[rows_d].cpu(), 128)
    assert torch.equal(bits(q[rows_d].cpu()), bits(q_ref)), "quant codes differ from the oracle"
    assert torch.equal(bits(s[rows_d].cpu().contiguous()), bits(s_ref)), "quant scales differ from the oracle"
    ref = oracle.w8a8_block_fp8_matmul(q_ref, wq.cpu(), s_ref, ws.cpu())
    assert_gemm_close(y[rows_d], ref, f"M={M} N={N} K={K}")


@pytest.mark.parametrize("M", [8192, 512])
@pytest.mark.parametrize("N,K", DSV3)
def test_dsv3_sweep_shapes_fp32_scale_kernel(M, N, K):
    _check_linear(M, N, K, seed=N + K + M, n_rows=64)


@pytest.mark.parametrize("M", [128, 2048])
@pytest.mark.parametrize("N,K", [(576, 7168), (7168, 16384)])
def test_dsv3_sweep_mid_sizes(M, N, K):
    _check_linear(M, N, K, seed=N + K + M + 5, n_rows=64)


# Llama-3-70B projections, M = 8192: (name, N, K, split) with split "col" (N / tp) or "row" (K / tp)
LLAMA = [("qkv", 10240, 8192, "col"), ("o", 8192, 8192, "row"), ("gate_up", 57344, 8192, "col"),
         ("down", 8192, 28672, "row")]


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
@pytest.mark.parametrize("name,N,K,split", LLAMA)
def test_llama70b_tp_shard_shapes(name, N, K, split, tp):
    """One rank's shard of every projection through Fp8LinearMethod.apply: column-parallel shards cut N, row-parallel
    shards cut K (the rank's partial product, before the all-reduce)."""
    n, k = (N // tp, K) if split == "col" else (N, K // tp)
    assert n % 128 == 0 and k % 128 == 0
    _check_linear(8192, n, k, seed=1000 + tp * 17 + N % 97, n_rows=48, via_apply=True)


# ------------------------------------------------------------------------------------------------ DeepSeek-V3 expert layer
E, TOPK, H, I = 256, 8, 7168, 2048


@pytest.fixture(scope="module")
def dsv3_experts():
    from sglang_b200.layers.quantization import block_quant_weight_fp8
    g = _gen(77)
    w1q = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device="cuda")
    w1s = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float32, device="cuda")
    w2q = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device="cuda")
    w2s = torch.empty(E, H // 128, I // 128, dtype=torch.float32, device="cuda")
    for e in range(E):
        w1q[e], w1s[e] = block_quant_weight_fp8(torch.randn(2 * I, H, generator=g, device="cuda") * 0.02)
        w2q[e], w2s[e] = block_quant_weight_fp8(torch.randn(H, I, generator=g, device="cuda") * 0.02)
    yield w1q, w1s, w2q, w2s
    del w1q, w1s, w2q, w2s
    torch.cuda.empty_cache()


@pytest.mark.parametrize("M", [256, 4096, 16384])
def test_dsv3_moe_layer_shape(dsv3_experts, M):
    """256 experts, top-8 of a softmax over random logits, hidden 7168, intermediate 2048: the whole layer on the GPU,
    a sample of tokens against the oracle.  The oracle is given only the experts those tokens hit (ids remapped)."""
    from sglang_b200.layers.moe import fused_experts_block_fp8
    w1q, w1s, w2q, w2s = dsv3_experts
    a = _activations(M, H, seed=M, outliers=False)
    logits = torch.randn(M, E, generator=_gen(M + 1), device="cuda")
    tw, ti = torch.topk(torch.softmax(logits, dim=-1, dtype=torch.float32), TOPK)
    out = fused_experts_block_fp8(a, w1q, w2q, w1s, w2s, tw, ti.to(torch.int32))
    torch.cuda.synchronize()
    assert _status() == 0
    tok = torch.randperm(M, generator=torch.Generator().manual_seed(M))[:16].sort().values.cuda()
    ids = ti[tok]
    need, inv = torch.unique(ids, return_inverse=True)
    ref = oracle.fused_experts_block_fp8(a[tok].cpu(), w1q[need].cpu(), w2q[need].cpu(), w1s[need].cpu(),
                                         w2s[need].cpu(), tw[tok].cpu(), inv.cpu())
    assert_gemm_close(out[tok], ref, f"DeepSeek-V3 expert layer M={M}")
