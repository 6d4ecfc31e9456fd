"""Torch/numpy CPU restatement of the reference's block-FP8 W8A8 arithmetic.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Every function names the reference
lines it follows.  All tensors live on the CPU; the arithmetic is the reference's own
torch-native arithmetic, so results are compared bit for bit with the golden files that
were produced by executing the reference's functions.
"""

from __future__ import annotations

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


# --------------------------------------------------------------------------------------
# Q: per-token-group quantisation
# --------------------------------------------------------------------------------------
def ceil_to_ue8m0(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s, for positive finite fp32 ``s``.

    Follows ``python/sglang/srt/layers/quantization/fp8_utils.py:511-512``
    (``2 ** ceil(log2(|x|))``) but with exact integer arithmetic on the fp32 exponent, so
    the answer does not depend on libm's ``log2f`` rounding.
    """
    s = s.to(torch.float32).abs()
    mant, exp = torch.frexp(s)  # s = mant * 2**exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp)
    return torch.ldexp(torch.ones_like(s), e)


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128, eps: float = 1e-10,
                              scale_ue8m0: bool = False):
    """``native_per_token_group_quant_fp8`` (``python/sglang/test/test_block_fp8.py:23-48``).

    amax is taken and clamped in the INPUT dtype (so eps becomes bf16(eps) for bf16 input),
    then widened to fp32; scale = amax / 448 is an IEEE fp32 division; codes are
    RNE_e4m3(clamp(x / scale)) with a true fp32 division per element.  With
    ``scale_ue8m0`` the scale is rounded up to a power of two first (the reference's
    Blackwell path, ``fp8_kernel.py:441-452`` + ``fp8_utils.py:511-512``).

    Returns (codes e4m3 with x's shape, scales fp32 ``x.shape[:-1] + (K // group_size,)``).
    """
    assert x.shape[-1] % group_size == 0 and x.is_contiguous()
    x_ = x.reshape(x.numel() // group_size, group_size)
    amax = x_.abs().max(dim=-1, keepdim=True)[0].clamp(min=eps).to(torch.float32)
    s = amax / FP8_MAX
    if scale_ue8m0:
        s = ceil_to_ue8m0(s)
    q = (x_ / s).clamp(min=-FP8_MAX, max=FP8_MAX).to(FP8)
    return q.reshape(x.shape), s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


def pack_scales(s: torch.Tensor, layout: str) -> torch.Tensor:
    """Lay a logical ``[M, G]`` fp32 scale matrix out the way the reference allocates it
    (``create_per_token_group_quant_fp8_output_scale``, ``fp8_kernel.py:433-474``).

    layout:
      "row"     -> contiguous ``[M, G]``
      "col"     -> shape ``[M, G]``, strides ``(1, M)``
      "col_tma" -> shape ``[M, G]``, strides ``(1, align(M, 4))``
      "ue8m0"   -> int32 ``[M, ceil(G/4)]``, strides ``(1, align(M, 4))``; byte ``g % 4`` of
                   int ``g // 4`` holds the biased exponent of scale g (scales must be
                   powers of two); unused bytes are zero
                   (``per_token_group_quant_8bit.cu:54-61,94-97``).
    Padding rows (M..align(M,4)) are zero-filled here; the kernels leave them untouched.
    """
    M, G = s.shape
    if layout == "row":
        return s.contiguous()
    if layout == "col":
        return s.t().contiguous().t()
    Ma = _align(M, 4)
    if layout == "col_tma":
        buf = torch.zeros(G, Ma, dtype=torch.float32)
        buf[:, :M] = s.t()
        return buf.t()[:M, :]
    if layout == "ue8m0":
        bits = s.contiguous().view(torch.int32)
        assert bool(((bits & 0x7FFFFF) == 0).all()), "UE8M0 scales must be powers of two"
        expo = ((bits >> 23) & 0xFF).to(torch.uint8)  # [M, G]
        Gp = _align(G, 4)
        buf = torch.zeros(Gp // 4, Ma, 4, dtype=torch.uint8)
        e = torch.zeros(M, Gp, dtype=torch.uint8)
        e[:, :G] = expo
        buf[:, :M, :] = e.view(M, Gp // 4, 4).permute(1, 0, 2)
        return buf.view(torch.int32).view(Gp // 4, Ma).t()[:M, :]
    raise ValueError(layout)


# --------------------------------------------------------------------------------------
# W: 128x128 block quantisation of weights (offline)
# --------------------------------------------------------------------------------------
def block_quant_weight(w: torch.Tensor, block=(128, 128), scale_ue8m0: bool = False):
    """Block-quantise ``w [N, K]`` to e4m3 with fp32 scales ``[ceil(N/bn), ceil(K/bk)]``.

    scale = block amax / 448 (1.0 for an all-zero block), code = RNE_e4m3(w / scale), as
    ``convert_weight`` in ``test/srt/cpu/utils.py:39-87``; ragged edges are zero-padded
    for the amax and cropped afterwards.
    """
    bn, bk = block
    N, K = w.shape
    Np, Kp = _align(N, bn), _align(K, bk)
    wp = torch.zeros(Np, Kp, dtype=torch.float32)
    wp[:N, :K] = w.to(torch.float32)
    v = wp.view(Np // bn, bn, Kp // bk, bk)
    s = v.abs().amax(dim=(1, 3), keepdim=True) / FP8_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    if scale_ue8m0:  # power-of-two block scales, as the reference requantises weights for Blackwell (fp8_utils.py:494-512)
        s = ceil_to_ue8m0(s)
    q = (v / s).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(Np, Kp)[:N, :K].contiguous()
    return q, s.view(Np // bn, Kp // bk).contiguous()


# --------------------------------------------------------------------------------------
# G: block-scaled GEMM
# --------------------------------------------------------------------------------------
def w8a8_block_fp8_matmul(A, B, As, Bs, block_size=(128, 128), output_dtype=torch.bfloat16):
    """``native_w8a8_block_fp8_matmul`` (``python/sglang/test/test_block_fp8.py:273-325``).

    ``C[:, nb] += (A[:, kb] @ B[nb, kb].T) * (As[:, kb] * Bs[nb, kb])`` in fp32, k-block
    outer loop, n-block inner loop, then one cast to ``output_dtype``.  A ``[..., K]`` codes
    (or fp32 values of codes), B ``[N, K]``, As ``[..., ceil(K/bk)]``, Bs ``[ceil(N/bn),
    ceil(K/bk)]``.
    """
    bn, bk = block_size
    A = A.to(torch.float32)
    B = B.to(torch.float32)
    K = A.shape[-1]
    N = B.shape[0]
    lead = A.shape[:-1]
    A = A.reshape(-1, K)
    nt, kt = -(-N // bn), -(-K // bk)
    As = As.reshape(A.shape[0], kt).to(torch.float32)
    assert Bs.shape == (nt, kt) and As.shape[1] == kt
    C = torch.zeros(A.shape[0], N, dtype=torch.float32)
    for i in range(kt):
        a = A[:, i * bk:min((i + 1) * bk, K)]
        for j in range(nt):
            b = B[j * bn:min((j + 1) * bn, N), i * bk:min((i + 1) * bk, K)]
            s = As[:, i:i + 1] * Bs[j][i]
            C[:, j * bn:min((j + 1) * bn, N)] += torch.matmul(a, b.t()) * s
    return C.reshape(lead + (N,)).to(output_dtype)


# --------------------------------------------------------------------------------------
# SA / ME: activation and the fused expert MLP
# --------------------------------------------------------------------------------------
def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """``SiluAndMul.forward_native`` (``python/sglang/srt/layers/activation.py:68-70``):
    ``silu(x[..., :d]) * x[..., d:]`` evaluated in x's dtype (for bf16 that is: silu in
    fp32 rounded to bf16, then a bf16 multiply)."""
    d = x.shape[-1] // 2
    return torch.nn.functional.silu(x[..., :d]) * x[..., d:]


def fused_experts_block_fp8(a, w1, w2, w1_s, w2_s, topk_weight, topk_ids, block_shape=(128, 128), scale_ue8m0=False,
                            no_combine=False, apply_router_weight_on_input=False):
    """Expert MLP of ``torch_w8a8_block_fp8_moe`` (``test_block_fp8.py:418-447``) with the
    routing result passed in.  a ``[M, H]`` bf16; w1 ``[E, 2I, H]``, w2 ``[E, H, I]`` e4m3;
    w1_s ``[E, 2I/128, H/128]``, w2_s ``[E, H/128, I/128]``; topk_* ``[M, topk]``.
    Experts with id < 0 or >= E contribute zero (non-local experts under expert
    parallelism, ``fused_moe_triton_kernels.py:421-437``).  ``scale_ue8m0`` rounds both activation quantisations'
    scales up to powers of two (the Blackwell DeepGEMM route, ``fp8_utils.py:511-512``).
    ``no_combine`` returns the weighted expert outputs ``[M, topk, H]`` without the sum over top-k
    (``fused_moe_triton/fused_moe.py:452-458,597-598``).  ``apply_router_weight_on_input`` multiplies the gate_up
    GEMM's fp32 result by the routing weight before it is rounded (the first kernel's ``MUL_ROUTED_WEIGHT``,
    ``fused_moe.py:523``) and leaves the expert output unweighted."""
    Bt, D = a.shape
    topk = topk_ids.shape[1]
    bk = block_shape[1]
    rep = a.view(Bt, -1, D).repeat(1, topk, 1).reshape(-1, D)
    out = torch.zeros(Bt * topk, w2.shape[1], dtype=a.dtype)
    ids = topk_ids.reshape(-1)
    a_q, a_s = per_token_group_quant_fp8(rep, bk, scale_ue8m0=scale_ue8m0)
    a_q = a_q.to(torch.float32)
    wflat = topk_weight.reshape(-1).to(torch.float32)
    for e in range(w1.shape[0]):
        mask = ids == e
        if mask.sum():
            if apply_router_weight_on_input:
                h = (w8a8_block_fp8_matmul(a_q[mask], w1[e], a_s[mask], w1_s[e], block_shape, torch.float32)
                     * wflat[mask].unsqueeze(1)).to(a.dtype)
            else:
                h = w8a8_block_fp8_matmul(a_q[mask], w1[e], a_s[mask], w1_s[e], block_shape, a.dtype)
            act = silu_and_mul(h)
            act_q, act_s = per_token_group_quant_fp8(act.contiguous(), bk, scale_ue8m0=scale_ue8m0)
            out[mask] = w8a8_block_fp8_matmul(act_q, w2[e], act_s, w2_s[e], block_shape, a.dtype)
    weighted = out.view(Bt, -1, w2.shape[1])
    if not apply_router_weight_on_input:
        weighted = weighted * topk_weight.view(Bt, -1, 1).to(out.dtype)
    return weighted if no_combine else weighted.sum(dim=1)


def moe_block_fp8_from_scores(a, w1, w2, w1_s, w2_s, score, topk, block_shape=(128, 128)):
    """``torch_w8a8_block_fp8_moe`` including its routing: fp32 softmax then ``torch.topk``
    with no renormalisation (``test_block_fp8.py:424-425``)."""
    p = torch.softmax(score, dim=-1, dtype=torch.float32)
    w, ids = torch.topk(p, topk)
    return fused_experts_block_fp8(a, w1, w2, w1_s, w2_s, w, ids, block_shape)


# --------------------------------------------------------------------------------------
# MP / MS: integer routing tables and the row shuffles
# --------------------------------------------------------------------------------------
def prepare_moe_input(topk_ids: np.ndarray, num_experts: int, n: int, k: int):
    """Routing tables of ``prepare_moe_input`` (``sgl-kernel/csrc/moe/prepare_moe_input.cu:13-167``).

    Returns int32 arrays ``expert_offsets [E+1]``, ``problem_sizes1 [E,3] = (cnt, 2n, k)``,
    ``problem_sizes2 [E,3] = (cnt, k, n)``, ``a_map [M*topk]`` (sorted row -> source token)
    and ``c_map [M*topk]`` (token-major slot -> sorted row).  The reference hands out slots
    inside one expert's segment in atomic order; here the order is the stable one
    (ascending flat index), which is one of the orders the reference can produce.  Ids
    outside ``[0, E)`` get no row: their ``c_map`` entry is -1.
    """
    ids = np.asarray(topk_ids, dtype=np.int64)
    topk = ids.shape[1]
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < num_experts)
    cnt = np.bincount(flat[valid], minlength=num_experts).astype(np.int32)
    offs = np.zeros(num_experts + 1, dtype=np.int32)
    offs[1:] = np.cumsum(cnt)
    ps1 = np.stack([cnt, np.full_like(cnt, 2 * n), np.full_like(cnt, k)], axis=1).astype(np.int32)
    ps2 = np.stack([cnt, np.full_like(cnt, k), np.full_like(cnt, n)], axis=1).astype(np.int32)
    total = int(offs[-1])
    order = np.argsort(np.where(valid, flat, num_experts), kind="stable")[:total]
    a_map = np.full(flat.shape[0], 0, dtype=np.int32)
    a_map[:total] = (order // topk).astype(np.int32)
    c_map = np.full(flat.shape[0], -1, dtype=np.int32)
    c_map[order] = np.arange(total, dtype=np.int32)
    return offs, ps1, ps2, a_map, c_map


def shuffle_rows(x: torch.Tensor, dst2src: np.ndarray, n_dst: int | None = None) -> torch.Tensor:
    """``shuffle_rows`` (``prepare_moe_input.cu:169-256``): ``out[i] = x[dst2src[i]]``."""
    idx = torch.as_tensor(np.asarray(dst2src[: n_dst if n_dst is not None else len(dst2src)]),
                          dtype=torch.long)
    if x.dtype == FP8:
        return x.view(torch.uint8)[idx].view(FP8)
    return x[idx]


def apply_shuffle_mul_sum(c2: torch.Tensor, c_map: np.ndarray, factors: torch.Tensor | None,
                          m: int) -> torch.Tensor:
    """``apply_shuffle_mul_sum`` (``prepare_moe_input.cu:258-392``):
    ``out[i] = cast(sum_j fp32(factors[i,j]) * fp32(c2[c_map[i*topk+j]]))`` with the sum taken
    in fp32 in ascending j.  Slots with ``c_map < 0`` (non-local experts) are skipped."""
    cm = torch.as_tensor(np.asarray(c_map), dtype=torch.long).view(m, -1)
    topk = cm.shape[1]
    acc = torch.zeros(m, c2.shape[1], dtype=torch.float32)
    f = None if factors is None else factors.reshape(m, topk).to(torch.float32)
    for j in range(topk):
        ok = cm[:, j] >= 0
        rows = c2[cm[:, j].clamp(min=0)].to(torch.float32)
        term = rows if f is None else rows * f[:, j:j + 1]
        acc = acc + torch.where(ok[:, None], term, torch.zeros_like(term))
    return acc.to(c2.dtype)


def topk_softmax(gating_output: torch.Tensor, topk: int, renormalize: bool = False):
    """``topk_softmax`` as the torch-native router states it (``python/sglang/srt/layers/moe/topk.py:426-431``;
    the kernel ``sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:512-590`` is tested against the same two torch
    calls, ``sgl-kernel/tests/test_moe_topk_softmax.py:33-44``).  Returns ``(weights fp32 [T, topk],
    ids int32 [T, topk])``; equal probabilities go to the lower expert index, the kernel's rule
    (``moe_topk_softmax_kernels.cu:372``; ``torch.topk`` leaves that order open)."""
    p = torch.softmax(gating_output.float(), dim=-1)
    # stable descending sort = torch.topk's order, with the tie rule made explicit
    order = torch.sort(p, dim=-1, descending=True, stable=True).indices[:, :topk]
    w = p.gather(1, order)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, order.to(torch.int32)


def moe_align_block_size(topk_ids: np.ndarray, block_size: int, num_experts: int):
    """``moe_align_block_size`` (``sgl-kernel/csrc/moe/moe_align_kernel.cu:56-229,302-364`` with the caller's
    ``num_experts + 1`` buckets, ``moe_align_block_size.py:57-85``): bucket ``id + 1`` per slot, every bucket
    padded to a multiple of ``block_size``; ``expert_ids[block] = bucket - 1``; padding entries hold ``numel``.
    Inside a bucket the slots are in ascending order (the order of the reference test's second implementation,
    ``sgl-kernel/tests/test_moe_align.py:71-97``; the CUDA kernel's order there is unspecified).
    Returns ``(sorted_token_ids [capacity], expert_ids [post_pad / block_size], post_pad, cumsum [B + 1])``."""
    flat = np.asarray(topk_ids, dtype=np.int64).reshape(-1)
    numel, B = flat.shape[0], num_experts + 1
    counts = np.bincount(flat + 1, minlength=B)[:B]
    padded = (counts + block_size - 1) // block_size * block_size
    cumsum = np.concatenate([[0], np.cumsum(padded)]).astype(np.int32)
    post_pad = int(cumsum[-1])
    cap = numel + B * (block_size - 1)
    sorted_ids = np.full(cap, numel, dtype=np.int32)
    expert_ids = np.zeros(post_pad // block_size, dtype=np.int32)
    order = np.argsort(flat, kind="stable")
    pos = 0
    for b in range(B):
        c = int(counts[b])
        sorted_ids[cumsum[b]:cumsum[b] + c] = order[pos:pos + c]
        pos += c
        expert_ids[cumsum[b] // block_size:cumsum[b + 1] // block_size] = b - 1
    return sorted_ids, expert_ids, post_pad, cumsum


def moe_sum_reduce(x: torch.Tensor, routed_scaling_factor: float = 1.0) -> torch.Tensor:
    """``moe_sum_reduce`` (``sgl-kernel/csrc/moe/moe_sum_reduce.cu:146-170``): fp32 sum over the top-k axis in
    ascending order, one multiplication by the factor, one cast."""
    acc = torch.zeros(x.shape[0], x.shape[2], dtype=torch.float32)
    for j in range(x.shape[1]):
        acc = acc + x[:, j].float()
    return (acc * torch.tensor(routed_scaling_factor, dtype=torch.float32)).to(x.dtype)


def moe_fused_gate(x: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
                   num_fused_shared_experts: int = 0, routed_scaling_factor: float = 0.0,
                   apply_routed_scaling_factor_on_output: bool = False):
    """``moe_fused_gate`` (``sgl-kernel/csrc/moe/moe_fused_gate.cu:104-258``; torch-native twin
    ``biased_grouped_topk_impl``, ``python/sglang/srt/layers/moe/topk.py:611-661``): sigmoid, plus bias, group score =
    sum of the two largest biased scores of a group, the ``topk_group`` best groups stay, the best biased scores
    inside them are taken and weighted by the unbiased sigmoid, shared-expert slots get ``sum / factor``, everything
    is divided by the routed sum.  Ties follow the kernel: lower group (``:147-150``), lower expert (``:192-196``);
    the shared slots get the ids ``E, E + 1, ...`` (``:226-243``)."""
    T, E = x.shape
    s = torch.sigmoid(x.float()).to(x.dtype)
    b = (s + bias.unsqueeze(0)).to(x.dtype)
    gsz = E // num_expert_group
    top2 = torch.sort(b.view(T, num_expert_group, gsz).float(), dim=-1, descending=True).values[..., :2]
    gscore = (top2[..., 0].to(x.dtype) + top2[..., 1].to(x.dtype)).float()
    gorder = torch.sort(gscore, dim=-1, descending=True, stable=True).indices[:, :topk_group]
    gmask = torch.zeros(T, num_expert_group, dtype=torch.bool)
    gmask.scatter_(1, gorder, True)
    masked = b.float().masked_fill(~gmask.repeat_interleave(gsz, dim=1), float("-inf"))
    k_real = topk - num_fused_shared_experts
    ids = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :k_real]
    w = s.float().gather(1, ids)
    total = torch.zeros(T, dtype=torch.float32)
    for j in range(k_real):  # the kernel adds the weights in selection order
        total = total + w[:, j]
    if num_fused_shared_experts:
        shared_w = (total / torch.tensor(routed_scaling_factor, dtype=torch.float32))[:, None]
        w = torch.cat([w, shared_w.expand(T, num_fused_shared_experts)], dim=1)
        ids = torch.cat([ids, (E + torch.arange(num_fused_shared_experts)).expand(T, -1)], dim=1)
    w = w / total[:, None]
    if apply_routed_scaling_factor_on_output:
        w = w * torch.tensor(routed_scaling_factor, dtype=torch.float32)
    return w, ids.to(torch.int32)


# --------------------------------------------------------------------------------------
# AR / A2A: the sharded forms, evaluated the way the sharding defines the arithmetic
# --------------------------------------------------------------------------------------
def row_parallel_partials(x, wq, ws, world):
    """The partial products of the row-parallel linear, one per rank, each rounded to the output type as the rank's GEMM
    leaves it (``python/sglang/srt/layers/linear.py:1361-1378``)."""
    K = x.shape[1]
    kr = K // world
    parts = []
    for r in range(world):
        q, s = per_token_group_quant_fp8(x[:, r * kr:(r + 1) * kr].contiguous(), 128)
        parts.append(w8a8_block_fp8_matmul(q, wq[:, r * kr:(r + 1) * kr].contiguous(), s,
                                           ws[:, r * kr // 128:(r + 1) * kr // 128].contiguous(), output_dtype=x.dtype))
    return parts


def row_parallel_reference(x, wq, ws, world):
    """Row-parallel linear: every rank quantises its K-slice, rounds its partial product to the output type, and the
    partial products are added (``python/sglang/srt/layers/linear.py:1361-1386``); fp32 sum here, one cast."""
    ref = torch.zeros(x.shape[0], wq.shape[0], dtype=torch.float32)
    for part in row_parallel_partials(x, wq, ws, world):
        ref += part.float()
    return ref.to(x.dtype)


def sum_in_storage_type_bound(parts):
    """How far a sum of ``parts`` taken IN their 16-bit type, in any order (what an all-reduce library does with bf16
    buffers, ``python/sglang/srt/distributed/device_communicators/pynccl.py:143-160``), can lie from the fp32 sum rounded
    once: every one of the ``len(parts) - 1`` additions rounds a running sum no larger than ``sum |part|``, half a unit
    in the last place each, plus half a unit for the final rounding of the reference itself.  Element-wise, fp64."""
    mant = 8 if parts[0].dtype == torch.bfloat16 else 11
    mag = torch.zeros(parts[0].shape, dtype=torch.float64)
    for part in parts:
        mag += part.double().abs()
    ulp = torch.ldexp(torch.ones_like(mag), torch.frexp(mag.clamp(min=1e-300))[1] - mant)
    return 0.5 * ulp * len(parts)


def expert_parallel_reference(x, w1q, w2q, w1s, w2s, topk_w, topk_ids, world):
    """Expert-parallel MoE: every rank adds up the contributions of ITS experts to a token and returns that partial row
    in the activation type; the partial rows are added at the source in fp32
    (``python/sglang/srt/layers/moe/token_dispatcher/deepep.py:466-492``)."""
    E = w1q.shape[0]
    el = E // world
    total = torch.zeros(x.shape[0], w2q.shape[1], dtype=torch.float32)
    for r in range(world):
        local = torch.where((topk_ids // el) == r, topk_ids, torch.full_like(topk_ids, -1))
        if bool((local >= 0).any()):
            total += fused_experts_block_fp8(x, w1q, w2q, w1s, w2s, topk_w, local).float()
    return total.to(x.dtype)
