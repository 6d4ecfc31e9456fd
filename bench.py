#!/usr/bin/env python
"""Benchmark of the block-FP8 W8A8 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M]

Workload ("dsv3_linear_sweep"): one step = one forward of the block-FP8 linear (per-token-group
quant of the bf16 activations + block-scaled FP8 GEMM, bf16 out) for each of the five
DeepSeek-V3 projection shapes (N, K) at M tokens.  With N GPUs the same layers are
tensor-parallel, the way the model shards them: column-parallel for q_b_proj (24576, 1536) and
gate_up (36864, 7168); row-parallel with an NCCL all-reduce for o_proj (7168, 16384) and
down_proj (7168, 18432); kv_a_proj (576, 7168) replicated.  Total work is fixed ("strong").
Synthetic data: activations ~N(0,1) with 1% of entries x50, weights ~N(0, 0.02) block-quantised.

Prints ONE JSON line.  `value` = TFLOP/s of the whole step (2*M*N*K summed over the shapes, inputs
resident in HBM); `e2e` = the same through Fp8LinearMethod.apply from pinned host buffers with the
result copied back; `roofline` = the GEMM kernel alone (CUDA events around each launch) against
2 x the measured dense bf16 rate, with the other kernels the path is judged on under `roofline.others`
(the per-token-group quant kernel on M=16384 x 7168 against measured HBM bandwidth, before and after
the GEMM sweep; the UE8M0 GEMM; the fused MoE); `breakdown` = device time per kind of kernel and the
host gap of one step; `cpu_baseline` = the reference's CPU kernel (or the oracle port) on the same five
shapes.  With N > 1: `parity` = one small tensor-parallel and one small expert-parallel layer checked
against the CPU oracle on rank 0 before anything is timed, for the NCCL path and for the peer-memory
paths.  `--impl reference` times only the CPU path.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [  # (name, N, K, tensor-parallel mode)
    ("q_b_proj", 24576, 1536, "column"),
    ("kv_a_proj", 576, 7168, "replicated"),
    ("o_proj", 7168, 16384, "row"),
    ("gate_up_proj", 36864, 7168, "column"),
    ("down_proj", 7168, 18432, "row"),
]
METRIC = "block_fp8_linear_tflops"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- clock sampling
_SAMPLER_CHILD = r"""
import sys, time
uuid, path = sys.argv[1], sys.argv[2]
with open(path, "w", buffering=1) as f:
    try:
        import pynvml as n
        n.nvmlInit()
        h = n.nvmlDeviceGetHandleByUUID(uuid)
        f.write("max %d\n" % n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))
        while True:
            f.write("%.6f %d %d\n" % (time.time(), n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM),
                                      n.nvmlDeviceGetCurrentClocksEventReasons(h)))
            time.sleep(0.004)
    except Exception as e:
        f.write("error %r\n" % (e,))
"""


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while timed regions run.  The NVML polling (read-only queries,
    every 4 ms) runs in ONE CHILD PROCESS for the whole run, writing to a scratch file: a polling thread inside the
    benchmark process takes the interpreter lock away from the thread that launches the kernels, which showed as idle GPU
    time in steps of one or two milliseconds.  start() / stop() mark the wall-clock window whose samples count."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))
    _child = None
    _path = None

    def __init__(self, gpu_uuid: str):
        self.t0 = self.t1 = None
        if gpu_uuid is None:  # ranks whose line is not printed do not sample
            return
        if ClockSampler._child is None:
            import tempfile
            fd, ClockSampler._path = tempfile.mkstemp(prefix="sglb200_clocks_", suffix=".txt")
            os.close(fd)
            try:
                ClockSampler._child = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, gpu_uuid, ClockSampler._path],
                                                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
                import atexit
                atexit.register(ClockSampler.shutdown)
            except OSError:
                ClockSampler._child = None

    @staticmethod
    def shutdown():
        if ClockSampler._child is not None:
            ClockSampler._child.terminate()
            ClockSampler._child = None
        if ClockSampler._path and os.path.exists(ClockSampler._path):
            os.remove(ClockSampler._path)

    def start(self):
        self.t0 = time.time()

    def stop(self):
        self.t1 = time.time()
        if ClockSampler._child is None or not ClockSampler._path:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampler unavailable"]}
        time.sleep(0.01)
        clk, near, mx, reasons, err = [], [], None, set(), None
        with open(ClockSampler._path) as f:
            for line in f:
                fld = line.split()
                if len(fld) == 2 and fld[0] == "max":
                    mx = int(fld[1])
                elif fld and fld[0] == "error":
                    err = line.strip()
                elif len(fld) == 3:
                    t, c, r = float(fld[0]), int(fld[1]), int(fld[2])
                    if self.t0 <= t <= self.t1:
                        clk.append(c)
                        for name, bit in self.REASONS:
                            if r & bit:
                                reasons.add(name)
                    elif self.t0 - 0.05 <= t <= self.t1 + 0.05:
                        near.append(c)
        if err is not None and not clk:
            return {"sm_mhz": None, "sm_max_mhz": mx, "reasons": [err]}
        use = clk or near  # a region shorter than the polling period: the samples right beside it
        return {"sm_mhz": statistics.median(use) if use else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clk), "source": "nvml (child process)"}


# --------------------------------------------------------------------------- CPU arm
def host_cores() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_arm(steps: int, warmup: int, m_sample: int):
    """The reference's CPU implementation of the path on this host: sgl-kernel's AMX
    fp8_scaled_mm_cpu (W8A16) built from the reference sources when it loads here, else the
    torch-native oracle port.  One pass = the five shapes at `m_sample` rows, on every core this
    process may use (torch.distributed.run exports OMP_NUM_THREADS=1; the thread count is raised
    here, after import, so the arm is not measured on one core)."""
    import torch
    torch.set_num_threads(host_cores())
    import oracle
    from oracle.build_ref import load_ref
    ops = load_ref()
    kind = "reference" if ops is not None else "port"
    if ops is None:
        m_sample = min(m_sample, 64)
    g = torch.Generator().manual_seed(0)
    layers = []
    for name, N, K, _ in SHAPES:
        if ops is None and N * K > 24576 * 1536:
            continue  # the torch-native port is ~100x slower: keep the two small shapes
        w = (torch.randn(N, K, generator=g) * 0.02)
        wq, ws = oracle.block_quant_weight(w)
        x = torch.randn(m_sample, K, generator=g).bfloat16()
        layers.append((x, ops.convert_weight_packed(wq) if ops is not None else wq, ws, N, K))
    flops = sum(2.0 * m_sample * N * K for _, _, _, N, K in layers)

    def one_pass():
        for x, wq, ws, N, K in layers:
            if ops is not None:
                ops.fp8_scaled_mm_cpu(x, wq, ws, [128, 128], None, torch.bfloat16, True)
            else:
                aq, a_s = oracle.per_token_group_quant_fp8(x, 128)
                oracle.w8a8_block_fp8_matmul(aq, wq, a_s, ws)

    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / steps
    names = "+".join(s[0] for s in SHAPES if any(l[3] == s[1] and l[4] == s[2] for l in layers))
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "M_sample": m_sample,
            "sample": f"{names} at M={m_sample} rows, {steps} passes after {warmup} warm-up; "
                      + ("sgl-kernel fp8_scaled_mm_cpu (AMX bf16, W8A16)" if ops is not None
                         else "torch-native oracle (W8A8)"),
            "ms_per_pass": dt * 1e3}


def moe_section(torch, dev, gen, Ms=(16, 64, 256, 4096, 16384), E=256, topk=8, H=7168, I=2048, gpu_uuid=None):
    """Block-FP8 fused MoE, DeepSeek-V3 layer shape: 256 experts, top-8 of softmax(random logits), hidden 7168,
    moe_intermediate 2048, M tokens; random e4m3 expert weights (11.3 GB).  Two checkpoints: fp32 block scales
    (software promotion) and power-of-two (UE8M0) scales (grouped GEMMs on the hardware block-scaling path)."""
    from sglang_b200._lib import lib
    from sglang_b200.layers.moe import fused_experts_block_fp8, fused_experts_block_fp8_ue8m0
    from sglang_b200.layers.quantization import pack_ue8m0_scales

    def rand_fp8(*shape):
        t = torch.empty(shape, device=dev, dtype=torch.float8_e4m3fn)
        flat = t.view(-1)
        for i in range(0, flat.numel(), 1 << 28):
            n = min(1 << 28, flat.numel() - i)
            flat[i:i + n] = (torch.randn(n, device=dev, generator=gen) * 20).to(torch.float8_e4m3fn)
        return t

    def pow2_packed(e, nb, kb):
        ex = torch.randint(-12, -8, (e * nb, kb), device=dev, generator=gen).float()
        return pack_ue8m0_scales(torch.exp2(ex)).view(e, nb, -1)

    w1, w2 = rand_fp8(E, 2 * I, H), rand_fp8(E, H, I)
    w1s = torch.rand(E, 2 * I // 128, H // 128, device=dev, generator=gen) * 1e-3
    w2s = torch.rand(E, H // 128, I // 128, device=dev, generator=gen) * 1e-3
    w1p, w2p = pow2_packed(E, 2 * I // 128, H // 128), pow2_packed(E, H // 128, I // 128)
    out = {"workload": f"fused_experts block-FP8 E={E} top{topk} H={H} I={I}", "weight_bytes": w1.numel() + w2.numel(),
           "kernels_per_call": 9, "cases": []}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def board_state():
        """SM clock and board power right after a timed loop (NVML, read-only)."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = (pynvml.nvmlDeviceGetHandleByUUID(gpu_uuid) if gpu_uuid
                 else pynvml.nvmlDeviceGetHandleByIndex(dev.index or 0))
            return {"sm_mhz_after": pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                    "watts_after": pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0}
        except Exception:  # noqa: BLE001 - the clock note is optional
            return {}

    for M in Ms:
        a = torch.randn(M, H, device=dev, generator=gen).bfloat16()
        tw, ti = torch.topk(torch.softmax(torch.randn(M, E, device=dev, generator=gen), -1), topk)
        ti = ti.to(torch.int32)
        flops = M * topk * (2.0 * H * 2 * I + 2.0 * I * H)
        # weights of the experts that received a row: what a call has to stream from HBM
        routed = int(torch.unique(ti).numel())
        w_bytes = routed * (w1.numel() + w2.numel()) // E
        case = {"M": M, "experts_with_rows": routed, "routed_weight_bytes": w_bytes}
        few_rows = M * topk <= lib().sglb200_get_grouped_few_rows() * E  # the grouped GEMMs take the few-rows kernel
        variants = [("fp32_scales", lambda: fused_experts_block_fp8(a, w1, w2, w1s, w2s, tw, ti), None),
                    ("ue8m0", lambda: fused_experts_block_fp8_ue8m0(a, w1, w2, w1p, w2p, tw, ti), None)]
        if few_rows:  # the same calls with the few-rows kernel switched off: the 128 x 128 grouped kernels
            variants += [("fp32_scales_tile_kernel", variants[0][1], 0), ("ue8m0_tile_kernel", variants[1][1], 0)]
        for name, fn, limit in variants:
            before = lib().sglb200_get_grouped_few_rows()
            if limit is not None:
                lib().sglb200_set_grouped_few_rows(limit)
            # Sustained figures: a call is milliseconds long and the board needs about a second of load to settle under
            # its power cap, so a handful of calls would read the clock the PREVIOUS variant left behind (the 128 x 128
            # kernel on few rows per expert pulls the SM clock to ~1.1 GHz at 1000 W, the few-rows kernel stays at
            # ~1.75 GHz).  About 0.3 s of untimed calls, then about 0.3 s timed.
            try:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                n = max(5, min(150, int(300.0 / max(e0.elapsed_time(e1), 0.05))))
                for _ in range(n):
                    fn()
                torch.cuda.synchronize()
                e0.record()
                for _ in range(n):
                    fn()
                e1.record()
                torch.cuda.synchronize()
            finally:
                lib().sglb200_set_grouped_few_rows(before)
            ms = e0.elapsed_time(e1) / n
            case[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                          "weight_tbs": w_bytes / (ms * 1e-3) / 1e12, "calls_timed": n, **board_state()}
        out["cases"].append(case)
    return out


def tp_llama_section(torch, dist, dev, gen, world, rank, M=8192, iters=5, mc=None, mc_chunk=4096, mc_blocks=16):
    """Tensor-parallel decoder projections at the Llama-3-70B shape (hidden 8192, intermediate 28672, 64 q / 8 kv
    heads of 128): column-parallel QKV and gate_up, row-parallel o and down, each followed by an NCCL all-reduce of the
    [M, 8192] bf16 output (none at tp1).  One step = the four linears of a layer on M tokens; device time, max over
    ranks."""
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    layers_ = [("qkv", 10240, 8192, "column"), ("o", 8192, 8192, "row"), ("gate_up", 57344, 8192, "column"),
               ("down", 8192, 28672, "row")]
    built, flops = [], 0.0
    for name, N, K, mode in layers_:
        n_loc, k_loc = (N // world, K) if mode == "column" else (N, K // world)
        w = (torch.randn(n_loc, k_loc, device=dev, generator=gen) * 20).to(torch.float8_e4m3fn)
        ws = torch.rand(n_loc // 128, k_loc // 128, device=dev, generator=gen) * 1e-3
        x = torch.randn(M, k_loc, device=dev, generator=gen).bfloat16()
        built.append((mode, w, ws, x))
        flops += 2.0 * M * N * K

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(use_mc):
        for mode, w, ws, x in built:
            q, sc = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
            row = mode == "row" and world > 1
            y = w8a8_block_fp8_matmul(q, w, sc, ws, [128, 128], torch.bfloat16,
                                      out=mc.view((M, w.shape[0])) if row and use_mc else None)
            if row and use_mc:
                mc.all_reduce_(y)
            elif row:
                dist.all_reduce(y)

    def timed(fn):
        for _ in range(3):
            fn()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    ms = timed(lambda: step(False))
    out = {"workload": f"Llama-3-70B layer projections, M={M}, tp{world}: qkv/gate_up column-parallel, o/down "
                       "row-parallel + NCCL all-reduce", "ms_per_layer": ms, "tflops": flops / (ms * 1e-3) / 1e12,
           "allreduce_bytes_per_layer": 2 * M * 8192 * 2 if world > 1 else 0}
    if mc is not None and world > 1 and 2 * M * 8192 <= mc.max_size:
        ms_mc = timed(lambda: step(True))
        out["multicast_allreduce"] = {"ms_per_layer": ms_mc, "tflops": flops / (ms_mc * 1e-3) / 1e12,
                                      "how": "row-parallel GEMMs write into NVSwitch multicast memory, one multimem "
                                             "kernel (ld_reduce + st) per all-reduce"}
        from sglang_b200.distributed import row_parallel_linear_symm_mem_fused, row_parallel_linear_symm_mem_overlapped

        def step_fused():
            for mode, w, ws, x in built:
                if mode == "row":
                    row_parallel_linear_symm_mem_fused(mc, x, w, ws, comm_ctas=16)
                else:
                    q, sc = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
                    w8a8_block_fp8_matmul(q, w, sc, ws, [128, 128], torch.bfloat16)

        ms_fu = timed(step_fused)
        out["gemm_allreduce_one_launch"] = {
            "ms_per_layer": ms_fu, "tflops": flops / (ms_fu * 1e-3) / 1e12,
            "how": "row-parallel GEMM and multicast all-reduce in one cooperative launch, 16 communication CTAs"}

        def step_ovl():
            for mode, w, ws, x in built:
                if mode == "row":
                    row_parallel_linear_symm_mem_overlapped(mc, x, w, ws, chunk_rows=mc_chunk, ar_blocks=mc_blocks)
                else:
                    q, sc = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
                    w8a8_block_fp8_matmul(q, w, sc, ws, [128, 128], torch.bfloat16)

        ms_ov = timed(step_ovl)
        out["multicast_allreduce_overlapped"] = {
            "ms_per_layer": ms_ov, "tflops": flops / (ms_ov * 1e-3) / 1e12,
            "how": f"the same in chunks of {mc_chunk} rows: the all-reduce of a chunk ({mc_blocks} blocks, side stream) "
                   "runs beside the next chunk's GEMM"}
    return out


def ep_moe_section(torch, dist, dev, gen, world, rank, M_total=4096, E=256, topk=8, H=7168, I=2048, iters=5,
                   decode_graph=True):
    """Expert-parallel fused MoE at the DeepSeek-V3 layer shape: E / ep experts and M_total / ep tokens per rank,
    all-to-all dispatch of e4m3 rows + scales, local grouped GEMMs, all-to-all combine.  Device time, max over ranks."""
    from sglang_b200.distributed import PeerEpExchange, ep_fused_experts, ep_fused_experts_peer
    el, m_loc = E // world, M_total // world
    w1 = (torch.randn(el, 2 * I, H, device=dev, generator=gen) * 20).to(torch.float8_e4m3fn)
    w2 = (torch.randn(el, H, I, device=dev, generator=gen) * 20).to(torch.float8_e4m3fn)
    w1s = torch.rand(el, 2 * I // 128, H // 128, device=dev, generator=gen) * 1e-3
    w2s = torch.rand(el, H // 128, I // 128, device=dev, generator=gen) * 1e-3
    a = torch.randn(m_loc, H, device=dev, generator=gen).bfloat16()
    tw, ti = torch.topk(torch.softmax(torch.randn(m_loc, E, device=dev, generator=gen), -1), topk)
    ti = ti.to(torch.int32)
    for _ in range(2):
        ep_fused_experts(a, w1, w2, w1s, w2s, tw, ti, rank, world)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        ep_fused_experts(a, w1, w2, w1s, w2s, tw, ti, rank, world)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    flops = M_total * topk * (2.0 * H * 2 * I + 2.0 * I * H)
    res = {"workload": f"fused MoE E={E} top{topk} H={H} I={I}, {M_total} tokens over ep{world} ({m_loc} per rank)",
           "nccl": {"ms": float(ms), "tflops": flops / (float(ms) * 1e-3) / 1e12,
                    "how": "NCCL all-to-all dispatch/combine with a host-side count exchange"}}
    # the same layer with dispatch / combine over peer memory: no NCCL call, no host round trip
    ex = PeerEpExchange(capacity=M_total, hidden=H, topk=topk, m_max=m_loc)
    try:
        def timed_peer(fuse):
            for _ in range(2):
                y = ep_fused_experts_peer(ex, a, w1, w2, w1s, w2s, tw, ti, fuse_quant=fuse)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(iters):
                y = ep_fused_experts_peer(ex, a, w1, w2, w1s, w2s, tw, ti, fuse_quant=fuse)
            e1.record()
            dist.barrier()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t, y

        ms_u, _ = timed_peer(False)
        ms_p, out_p = timed_peer(True)
        out_n = ep_fused_experts(a, w1, w2, w1s, w2s, tw, ti, rank, world)
        err = float((out_p.float() - out_n.float()).norm() / out_n.float().norm())
        res["peer"] = {"ms": float(ms_p), "tflops": flops / (float(ms_p) * 1e-3) / 1e12, "rel_l2_vs_nccl": err,
                       "ms_with_separate_quant_launch": float(ms_u),
                       "how": "quantise-and-dispatch / combine kernels over CUDA-IPC peer memory, device-side row counts"}
        if not decode_graph or m_loc < 64:
            return res
        # decode size: 64 tokens per rank.  The peer version is one CUDA graph (nothing on its path synchronises); the
        # NCCL version needs the received-row counts on the host and cannot be captured.
        md = 64
        ad, twd, tid = a[:md].contiguous(), tw[:md].contiguous(), ti[:md].contiguous()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                ep_fused_experts_peer(ex, ad, w1, w2, w1s, w2s, twd, tid)
        torch.cuda.current_stream().wait_stream(side)
        dist.barrier()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ep_fused_experts_peer(ex, ad, w1, w2, w1s, w2s, twd, tid)
        times = {}
        for name, fn in (("peer_graph", graph.replay),
                         ("nccl_eager", lambda: ep_fused_experts(ad, w1, w2, w1s, w2s, twd, tid, rank, world))):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(20):
                fn()
            e1.record()
            dist.barrier()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 20], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times[name] = float(t) * 1e3
        res["decode_64_tokens_per_rank_us"] = times
        del graph
    finally:
        ex.close()
    return res


def parity_section(torch, dist, dev, world, rank):
    """N > 1: one small row-parallel linear and one small expert-parallel layer on all ranks, checked on rank 0 against
    the CPU oracle evaluated the way the sharding defines the arithmetic (every rank rounds its partial result to bf16,
    the partial results are added).  Bars: rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS(reference).  The oracle is used here
    as the checker only, outside every timed region."""
    from sglang_b200._lib import lib
    from sglang_b200.distributed import (PeerEpExchange, PeerExchange, RowParallelBlockFp8Linear, ep_fused_experts,
                                         ep_fused_experts_peer, fused_row_parallel_linear)
    import oracle

    def verdict(out, ref, slack=None):
        """rel-L2 <= 1e-2 and max-abs <= 2e-2 x RMS(ref); with `slack` (element-wise) an element may instead lie within
        that distance of the reference: the bound on a sum that the collective library takes in bf16."""
        o, r = out.float().cpu().double(), ref.float().double()
        rel = float((o - r).norm() / r.norm().clamp(min=1e-30))
        rms = r.pow(2).mean().sqrt().clamp(min=1e-30)
        diff = (o - r).abs()
        mx = float(diff.max() / rms)
        bound = torch.full_like(diff, 2e-2 * float(rms))
        res = {"rel_l2": rel, "max_abs_over_rms": mx}
        if slack is not None:
            bound = torch.maximum(bound, slack)
            res["bar"] = ("rel-L2 <= 1e-2; max-abs <= 2e-2 x RMS or the rounding of a sum of the ranks' bf16 partial results "
                          "taken in bf16 (NCCL adds bf16 buffers in bf16 and the NVSwitch adder does not round to nearest; "
                          "the oracle adds them in fp32 and rounds once)")
        res["elements_over"] = int((diff > bound).sum())
        res["pass"] = bool(rel <= 1e-2 and res["elements_over"] == 0)
        return res

    res = {}
    g = torch.Generator().manual_seed(4321)  # the same inputs on every rank
    M, N, K = 192, 1024, 2048
    x = torch.randn(M, K, generator=g).bfloat16()
    wq, ws = oracle.block_quant_weight(torch.randn(N, K, generator=g) * 0.05)
    kr = K // world
    xr = x[:, rank * kr:(rank + 1) * kr].contiguous().to(dev)
    layer = RowParallelBlockFp8Linear(wq.to(dev), ws.to(dev), rank, world)
    outs = {"tp_nccl_allreduce": layer(xr)}
    from sglang_b200.distributed import row_parallel_linear_overlapped
    outs["tp_nccl_overlapped_chunks"] = row_parallel_linear_overlapped(xr, layer.weight, layer.weight_scale_inv, chunk_rows=128)
    from sglang_b200.distributed import SymmMemCommunicator, row_parallel_linear_symm_mem
    mc = SymmMemCommunicator(dist.group.WORLD, dev, max_size=8 << 20)
    try:
        if not mc.disabled:
            outs["tp_multicast_allreduce"] = row_parallel_linear_symm_mem(mc, xr, layer.weight,
                                                                          layer.weight_scale_inv).clone()
            from sglang_b200.distributed import row_parallel_linear_symm_mem_fused
            outs["tp_multicast_gemm_allreduce_one_launch"] = row_parallel_linear_symm_mem_fused(
                mc, xr, layer.weight, layer.weight_scale_inv, comm_ctas=8).clone()
            torch.cuda.synchronize()
    finally:
        mc.close()
    ex = PeerExchange(slot_elems=M * N)
    try:
        outs["tp_peer_one_shot"] = fused_row_parallel_linear(ex, xr, layer.weight, layer.weight_scale_inv, two_shot=False)
        if -(-M // 128) * -(-N // 128) >= world:
            outs["tp_peer_two_shot"] = fused_row_parallel_linear(ex, xr, layer.weight, layer.weight_scale_inv, two_shot=True)
        torch.cuda.synchronize()
    finally:
        ex.close()
    # expert parallel: E experts over the ranks, 48 tokens per rank
    E, topk, H, I, m_loc = 16, 4, 512, 256, 48
    w1 = [oracle.block_quant_weight(torch.randn(2 * I, H, generator=g) * 0.05) for _ in range(E)]
    w2 = [oracle.block_quant_weight(torch.randn(H, I, generator=g) * 0.05) for _ in range(E)]
    w1q, w1s = torch.stack([w[0] for w in w1]), torch.stack([w[1] for w in w1])
    w2q, w2s = torch.stack([w[0] for w in w2]), torch.stack([w[1] for w in w2])
    gr = torch.Generator().manual_seed(100 + rank)
    xm = torch.randn(m_loc, H, generator=gr).bfloat16()
    tw, ti = torch.topk(torch.softmax(torch.randn(m_loc, E, generator=gr), -1), topk)
    el = E // world
    lo, hi = rank * el, (rank + 1) * el
    loc = [t[lo:hi].to(dev) for t in (w1q, w2q, w1s, w2s)]
    ep_outs = {"ep_nccl_all_to_all": ep_fused_experts(xm.to(dev), loc[0], loc[1], loc[2], loc[3], tw.to(dev),
                                                      ti.to(torch.int32).to(dev), rank, world)}
    epx = PeerEpExchange(capacity=world * m_loc, hidden=H, topk=topk, m_max=m_loc)
    try:
        ep_outs["ep_peer_dispatch_combine"] = ep_fused_experts_peer(epx, xm.to(dev), loc[0], loc[1], loc[2], loc[3],
                                                                    tw.to(dev), ti.to(torch.int32).to(dev))
        torch.cuda.synchronize()
    finally:
        epx.close()
    status = lib().sglb200_read_device_status()
    dist.barrier()
    if rank == 0:  # the oracle runs after all device work: the peer exchanges assume ranks in step
        parts = oracle.row_parallel_partials(x, wq, ws, world)
        ref = oracle.row_parallel_reference(x, wq, ws, world)
        slack = oracle.sum_in_storage_type_bound(parts)
        for k, v in outs.items():
            res[k] = verdict(v, ref, slack if ("nccl" in k or "multicast" in k) else None)
        ref_ep = oracle.expert_parallel_reference(xm, w1q, w2q, w1s, w2s, tw, ti, world)
        for k, v in ep_outs.items():
            res[k] = verdict(v, ref_ep)
        res["device_status"] = status
        res["shapes"] = {"tp": [M, N, K], "ep": {"experts": E, "topk": topk, "hidden": H, "intermediate": I,
                                                "tokens_per_rank": m_loc}}
        res["pass"] = bool(all(v["pass"] for k, v in res.items() if isinstance(v, dict) and "pass" in v) and status == 0)
    dist.barrier()
    return res if rank == 0 else None


def decode_section(torch, dev, peaks, shapes=None, ms=(1, 16, 64, 128)):
    """The five layers at decode batch sizes (M = 1, 16, 64, 128): weight streaming, HBM-bound.  Each measurement is one
    CUDA graph holding one GEMM call per weight copy (enough copies that the working set exceeds L2), replayed ten
    times back to back; reported per call."""
    from sglang_b200.layers.quantization import w8a8_block_fp8_matmul
    out = {"workload": "block-FP8 linear at M = 1 / 16 / 64 / 128, per-call device time inside a replayed CUDA graph over "
                       "rotating weight copies (working set > L2)", "unit": "us", "peak_gbs": peaks["hbm_gbs"],
           "cases": []}
    for name, N, K, _ in (shapes or SHAPES):
        copies = max(4, min(32, int(400e6 // (N * K)) + 1))
        ws_ = [torch.randint(-60, 60, (N, K), device=dev, dtype=torch.int8).view(torch.float8_e4m3fn) for _ in range(copies)]
        sc = torch.rand(-(-N // 128), K // 128, device=dev) * 0.01
        for M in ms:
            a = torch.randint(-60, 60, (M, K), device=dev, dtype=torch.int8).view(torch.float8_e4m3fn)
            sa = torch.rand(M, K // 128, device=dev)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for w in ws_[:2]:
                    w8a8_block_fp8_matmul(a, w, sa, sc, [128, 128], torch.bfloat16)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for w in ws_:
                    w8a8_block_fp8_matmul(a, w, sa, sc, [128, 128], torch.bfloat16)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 10 / copies
            nbytes = N * K + N * K / 16384 * 4 + M * K + M * K / 128 * 4 + 2 * M * N
            out["cases"].append({"layer": name, "N": N, "K": K, "M": M, "us": us, "gbs": nbytes / us / 1e3,
                                 "frac": nbytes / us / 1e3 / peaks["hbm_gbs"]})
            del graph
        del ws_
        torch.cuda.empty_cache()
    return out


def fused_allreduce_section(torch, dist, dev, world, rank, layers, iters=30):
    """Row-parallel layers at decode batch sizes: quant + GEMM + NCCL all-reduce against quant + GEMM with the push
    epilogue + peer reduce (no NCCL).  Device time per layer call, max over ranks, median over `iters` calls."""
    from sglang_b200.distributed import PeerExchange, fused_row_parallel_linear
    from sglang_b200.layers.quantization import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul
    rows = [L for L in layers if L["mode"] == "row"]
    ex = PeerExchange(slot_elems=1024 * max(L["N"] for L in rows))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {"workload": "row-parallel o_proj / down_proj at decode batch sizes: quant + GEMM + all-reduce as one CUDA "
                       "graph, device us per replay (max over ranks, median), L2 flushed before every replay",
           "cases": []}
    try:
        for L in rows:
            for m in (16, 64, 128, 256, 512, 1024):
                x = L["x"][:m].contiguous()
                w, ws = L["layer"].weight, L["layer"].weight_scale_inv

                def nccl_call():
                    q, s = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
                    y = w8a8_block_fp8_matmul(q, w, s, ws, [128, 128], torch.bfloat16)
                    dist.all_reduce(y)
                    return y

                def fused_call():  # measured at every size, also where PeerExchange.fits would choose NCCL
                    return fused_row_parallel_linear(ex, x, w, ws, two_shot=False)

                def two_shot_call():
                    return fused_row_parallel_linear(ex, x, w, ws, two_shot=True)

                variants = [("nccl", nccl_call), ("fused", fused_call)]
                if m > 64 and -(-m // 128) * -(-L["N"] // 128) >= world:
                    variants.append(("two_shot", two_shot_call))
                res = {}
                for name, fn in variants:
                    # one call captured in a CUDA graph (how a decode step is launched), replayed with the L2 flushed
                    # before every replay; device time of the replay alone
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        for _ in range(3):
                            fn()
                    torch.cuda.current_stream().wait_stream(side)
                    dist.barrier()
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        fn()
                    evs = []
                    for _ in range(iters + 3):
                        flush.zero_()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        graph.replay()
                        e1.record()
                        evs.append((e0, e1))
                    torch.cuda.synchronize()
                    t = torch.tensor([a.elapsed_time(b) for a, b in evs[3:]], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    res[name] = float(t.median()) * 1e3
                    del graph
                y_f, y_n = fused_call(), nccl_call()
                torch.cuda.synchronize()
                err = float((y_f.float() - y_n.float()).norm() / y_n.float().norm())
                case = {"layer": L["name"], "M": m, "N": L["N"], "K_local": L["k_loc"],
                        "nccl_us": res["nccl"], "fused_us": res["fused"],
                        "speedup": res["nccl"] / res["fused"], "rel_l2_vs_nccl": err,
                        "library_choice": "one_shot" if ex.fits(m, L["N"]) else
                                          "two_shot" if ex.fits_two_shot(m, L["N"]) else "nccl"}
                if "two_shot" in res:
                    y_2 = two_shot_call()
                    torch.cuda.synchronize()
                    case.update(two_shot_us=res["two_shot"], two_shot_speedup=res["nccl"] / res["two_shot"],
                                two_shot_equals_one_shot=bool(torch.equal(y_2, y_f)))
                out["cases"].append(case)
    finally:
        ex.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=8192, help="tokens per step")
    ap.add_argument("--cpu-m", type=int, default=0, help="rows of the CPU arm (0: the same M as the GPU arm)")
    ap.add_argument("--overlap", type=int, default=-1,
                    help="N > 1: 1 = the all-reduce of a row chunk overlaps the next chunk's GEMM; 0 = all-reduce after "
                         "each row-parallel GEMM on the same stream; -1 (default) = time both during set-up and keep the faster")
    ap.add_argument("--multicast", type=int, default=-1,
                    help="N > 1: 1 = row-parallel GEMMs write into NVSwitch multicast memory and this library's "
                         "multimem kernel adds them; 0 = never; -1 = tried with the other orders, the fastest is kept")
    ap.add_argument("--ar-blocks", type=int, default=0,
                    help="thread blocks of the multicast all-reduce kernel when it overlaps the next row chunk's GEMM; "
                         "0 = 4, 8, 16 and 32 are tried")
    ap.add_argument("--chunk-rows", type=int, default=0,
                    help="rows per chunk of the overlapped row-parallel linear; 0 = M / 4 and M / 2 are both tried")
    ap.add_argument("--comm-sms", type=int, default=0, help="SMs the GEMMs leave free for NCCL while overlapping")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="upper bound on NCCL's CTAs per collective (0: NCCL's own)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-moe", action="store_true", help="skip the fused-MoE section (11.3 GB of expert weights)")
    ap.add_argument("--only", default="all", choices=["all", "gemm", "quant", "ue8m0", "decode", "moe"],
                    help="profiling aid: run only the linear sweep ('gemm'), the quant bandwidth case, the UE8M0 sweep, "
                         "the decode-size section (with --shape and --m for one case) or the fused MoE at --m tokens")
    ap.add_argument("--moe-experts", type=int, default=256, help="profiling aid for --only moe: number of experts")
    ap.add_argument("--shape", default=None, help="profiling aid: restrict the sweep to one layer name")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "dsv3_linear_sweep", "M": args.m, "shapes_NK": [[s[1], s[2]] for s in SHAPES],
              "parallelism": f"tp{world}", "block": [128, 128], "group": 128,
              "l2": "working set per step (weights 555 MB + activations) exceeds the 126 MB L2; no explicit flush"}

    cpu_m = args.cpu_m if args.cpu_m > 0 else args.m
    if args.impl == "reference":
        if rank != 0:
            return
        cb = cpu_arm(args.steps, args.warmup, cpu_m)
        if cb["M_sample"] != args.m:  # the torch-native port is too slow for the full M: say so in the config
            config["M_sample"] = cb["M_sample"]
        line = {"metric": METRIC, "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": cb["ms_per_pass"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic", "config": config,
                "impl": "reference", "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from sglang_b200.layers.quantization import (Fp8Config, Fp8LinearMethod, block_quant_weight_fp8, pack_ue8m0_scales,
                                                 per_block_cast_to_fp8, sglang_per_token_group_quant_fp8,
                                                 w8a8_block_fp8_matmul, w8a8_block_fp8_matmul_ue8m0)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        opts = None
        if args.nccl_max_ctas > 0:
            try:  # fewer, not more, CTAs per collective: the GEMMs running beside it keep the other SMs
                opts = dist.ProcessGroupNCCL.Options()
                opts.config.max_ctas = args.nccl_max_ctas
            except Exception:  # noqa: BLE001 - an older torch without the config field: NCCL's default
                opts = None
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    peaks = load_peaks()
    M = args.m
    gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid).replace("GPU-", "") if rank == 0 else None
    ClockSampler(gpu_uuid)  # starts the polling child now: it needs a moment to come up
    parity = None
    if world > 1 and args.only == "all":
        try:
            parity = parity_section(torch, dist, dev, world, rank)
        except Exception as e:  # noqa: BLE001 - reported, never hidden: a failed check shows up as pass = false
            parity = {"pass": False, "error": f"{type(e).__name__}: {e}"}
    if args.only == "moe":
        gen_m = torch.Generator(device=dev).manual_seed(0)
        print(json.dumps({"metric": METRIC, "only": "moe",
                          "moe": moe_section(torch, dev, gen_m, Ms=(args.m,), E=args.moe_experts, gpu_uuid=gpu_uuid)}))
        return
    if args.only == "decode":
        sel = [sh for sh in SHAPES if args.shape in (None, sh[0])]
        ms_sel = (args.m,) if args.m <= 64 else (1, 16, 64)
        print(json.dumps({"metric": METRIC, "only": "decode", "decode": decode_section(torch, dev, peaks, sel, ms_sel)}))
        return

    # ---- quant kernel on the bandwidth configuration (M=16384 x 7168), L2 flushed before every launch.  Measured twice:
    # before the GEMM sweep (GPU not yet at its power cap) and after it (SM clock pulled down under sw_power_cap).
    def quant_case(when):
        from sglang_b200.layers.quantization import create_per_token_group_quant_fp8_output_scale
        from sglang_b200.sgl_kernel import sgl_per_token_group_quant_8bit
        sampler_q = ClockSampler(gpu_uuid)
        gen_q = torch.Generator(device=dev).manual_seed(1)
        Mq, Kq, sets = 16384, 7168, 3
        xs, qs, ss = [], [], []
        for _ in range(sets):  # three input / output sets used in turn: 1.07 GB in flight, nothing is re-used from L2
            xq = torch.randn(Mq, Kq, device=dev, generator=gen_q)
            xs.append((xq * 10 ** (torch.rand(Mq, 1, device=dev, generator=gen_q) * 4 - 2)).bfloat16())
            qs.append(torch.empty(Mq, Kq, dtype=torch.float8_e4m3fn, device=dev))
            ss.append(create_per_token_group_quant_fp8_output_scale((Mq, Kq), dev, 128, True, True, False))
        del xq

        def launch(i):
            sgl_per_token_group_quant_8bit(xs[i % sets], qs[i % sets], ss[i % sets], 128, 1e-10, -448.0, 448.0, False)

        n = 21
        for i in range(4):
            launch(i)
        torch.cuda.synchronize()
        sampler_q.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
        clocks_q = sampler_q.stop()
        qms = e0.elapsed_time(e1) / n
        # the same kernel as a single launch after a 256 MB write flush (the dirty lines of the flush are written back
        # during the launch, and a launch after an idle gap starts slower): a lower figure, kept for comparison
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
        iso = []
        for i in range(12):
            flush.zero_()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            launch(i)
            f1.record()
            torch.cuda.synchronize()
            if i >= 3:
                iso.append(f0.elapsed_time(f1))
        del flush
        qbytes = Mq * Kq * 3 + Mq * (Kq // 128) * 4
        mhz = clocks_q.get("sm_mhz")
        return {"workload": "per_token_group_quant_fp8 M=16384 K=7168 bf16 -> e4m3 + f32 column-major scales",
                "when": when, "bytes": qbytes, "ms": qms, "gbs": qbytes / (qms * 1e-3) / 1e9,
                "peak_gbs": peaks["hbm_gbs"], "frac": qbytes / (qms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "peak_source": peaks["source"],
                "l2": f"inputs larger than L2: {sets} input / output sets of 356 MB used in turn, {n} launches back to back "
                      "between one pair of CUDA events, no flush",
                "single_launch_after_write_flush_us": statistics.median(iso) * 1e3,
                "clocks": clocks_q, "us_x_sm_mhz": qms * 1e3 * mhz if mhz else None, "launches": n}

    quant = None
    if rank == 0 and args.only not in ("gemm", "ue8m0"):
        quant = quant_case("before the GEMM sweep")

    # ---- synthetic layers, sharded for this rank
    method = Fp8LinearMethod(Fp8Config(), tp_size=world)
    layers = []
    gen = torch.Generator(device=dev).manual_seed(0)

    total_flops = 0.0
    shapes = [s for s in SHAPES if args.shape in (None, s[0])]
    if args.shape is not None:
        config["shapes_NK"] = [[s[1], s[2]] for s in shapes]
    for name, N, K, mode in shapes:
        total_flops += 2.0 * M * N * K
        n_loc, k_loc = N, K
        if world > 1 and mode == "column":
            n_loc = N // world
        if world > 1 and mode == "row":
            k_loc = K // world
        w = torch.randn(n_loc, k_loc, device=dev, generator=gen) * 0.02
        wq, ws = block_quant_weight_fp8(w)
        wq_u, ws_u = per_block_cast_to_fp8(w)  # power-of-two block scales (a UE8M0 checkpoint)
        ws_u = ws_u.contiguous()
        del w
        layer = torch.nn.Module()
        method.create_weights(layer, k_loc, [n_loc], K, N, torch.bfloat16, device=dev)
        layer.weight.data = wq
        layer.weight_scale_inv.data = ws
        x = torch.randn(M, k_loc, device=dev, generator=gen)
        x = torch.where(torch.rand(M, k_loc, device=dev, generator=gen) < 0.01, x * 50.0, x).bfloat16()
        layers.append({"name": name, "N": N, "K": K, "mode": mode, "n_loc": n_loc, "k_loc": k_loc, "layer": layer,
                       "x": x, "gemm_ms": [], "wq_u": wq_u, "ws_u": pack_ue8m0_scales(ws_u), "ev_u": []})

    overlap = world > 1 and args.overlap == 1
    mc, multicast = None, False
    if world > 1:
        from sglang_b200.distributed import (SymmMemCommunicator, row_parallel_linear_overlapped,
                                             row_parallel_linear_symm_mem_fused,
                                             row_parallel_linear_symm_mem_overlapped)
        from sglang_b200.layers.deep_gemm_wrapper import configure_deep_gemm_num_sms
        sm_total = torch.cuda.get_device_properties(dev).multi_processor_count
        if args.multicast != 0:
            mc = SymmMemCommunicator(dist.group.WORLD, dev,
                                     max_size=2 * M * max([L["N"] for L in layers if L["mode"] == "row"] + [8192]))
            if mc.disabled:
                mc = None
        multicast = mc is not None and args.multicast == 1
        overlap = overlap and not multicast

    chunk_rows = [args.chunk_rows if args.chunk_rows > 0 else max(128, M // 4)]
    own_launches = [0]  # kernels of this library launched by step(): one quantiser + one GEMM per layer (per chunk)

    mc_chunk = [0]  # > 0: the multicast all-reduce runs per chunk of this many rows beside the next chunk's GEMM
    ar_blocks = [args.ar_blocks if args.ar_blocks > 0 else 16]
    fused_ctas = [0]  # > 0: GEMM and multicast all-reduce in one launch, this many communication CTAs

    def step(record=False):
        for L in layers:
            if multicast and fused_ctas[0] > 0 and L["mode"] == "row":
                own_launches[0] += 2
                y = row_parallel_linear_symm_mem_fused(mc, L["x"], L["layer"].weight, L["layer"].weight_scale_inv,
                                                       comm_ctas=fused_ctas[0])
                continue
            if multicast and mc_chunk[0] > 0 and L["mode"] == "row":
                own_launches[0] += 1 + 2 * -(-M // mc_chunk[0])
                y = row_parallel_linear_symm_mem_overlapped(mc, L["x"], L["layer"].weight, L["layer"].weight_scale_inv,
                                                            chunk_rows=mc_chunk[0], ar_blocks=ar_blocks[0])
                continue
            if overlap and L["mode"] == "row":
                own_launches[0] += 1 + -(-M // chunk_rows[0])
                with configure_deep_gemm_num_sms(sm_total - args.comm_sms if args.comm_sms > 0 else None):
                    y = row_parallel_linear_overlapped(L["x"], L["layer"].weight, L["layer"].weight_scale_inv,
                                                       chunk_rows=chunk_rows[0])
                continue
            own_launches[0] += 2
            use_mc = multicast and L["mode"] == "row"
            q, s = sglang_per_token_group_quant_fp8(L["x"], 128, column_major_scales=True, scale_tma_aligned=True)
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            y = w8a8_block_fp8_matmul(q, L["layer"].weight, s, L["layer"].weight_scale_inv, [128, 128], torch.bfloat16,
                                      out=mc.view((M, L["n_loc"])) if use_mc else None)
            if record:
                e1.record()
                L["ev"].append((e0, e1))
            if use_mc:
                own_launches[0] += 1
                mc.all_reduce_(y)
            elif world > 1 and L["mode"] == "row":
                dist.all_reduce(y)
        return y

    def breakdown_pass(n_steps=3):
        """Device time per kind of kernel for one step in the plain order (quant, GEMM, then the all-reduce on the same
        stream), CUDA events around every launch; and the host time to enqueue a step."""
        evs = {"quant": [], "gemm": [], "allreduce": []}

        def mark(kind, fn):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            evs[kind].append((e0, e1))
            return out

        def plain_step():
            for L in layers:
                q, s = mark("quant", lambda: sglang_per_token_group_quant_fp8(L["x"], 128, column_major_scales=True,
                                                                              scale_tma_aligned=True))
                use_mc = multicast and L["mode"] == "row"
                y = mark("gemm", lambda: w8a8_block_fp8_matmul(q, L["layer"].weight, s, L["layer"].weight_scale_inv,
                                                               [128, 128], torch.bfloat16,
                                                               out=mc.view((M, L["n_loc"])) if use_mc else None))
                if use_mc:
                    mark("allreduce", lambda: mc.all_reduce_(y))
                elif world > 1 and L["mode"] == "row":
                    mark("allreduce", lambda: dist.all_reduce(y))

        plain_step()
        fence()
        for k in evs:
            evs[k].clear()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        h0 = time.perf_counter()
        for _ in range(n_steps):
            plain_step()
        host_ms = (time.perf_counter() - h0) * 1e3 / n_steps
        b1.record()
        fence()
        out = {k + "_ms": sum(a.elapsed_time(b) for a, b in v) / n_steps for k, v in evs.items()}
        t = torch.tensor([b0.elapsed_time(b1) / n_steps, out["quant_ms"], out["gemm_ms"], out["allreduce_ms"], host_ms],
                         device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, qm, gm, am, hm = (float(v) for v in t)
        return {"order": ("multicast all-reduce kernel after each row-parallel GEMM" if multicast
                          else "plain (no overlap)") + ", max over ranks", "step_ms": step_ms, "quant_ms": qm, "gemm_ms": gm,
                "allreduce_ms": am, "host_gap_ms": step_ms - (qm + gm + am), "host_enqueue_ms": hm,
                "launches_per_step": sum(len(v) for v in evs.values()) // n_steps}

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(gpu_uuid)  # its child process needs a moment to come up: created before the warm-up
    if world > 1:  # set-up, not a step: NCCL builds its channels and buffers for this message size on first use
        warm = torch.zeros(M, max(L["N"] for L in layers if L["mode"] == "row"), dtype=torch.bfloat16, device=dev)
        for _ in range(5):
            dist.all_reduce(warm)
        del warm
        fence()
    if world > 1 and args.overlap < 0 and args.multicast != 1:
        # set-up, not a step: time the orders of a step (three steps each after one warm-up step, device time, max over
        # ranks) and keep the fastest for the warm-up and the timed region
        tried = {}
        chunk_choices = [args.chunk_rows] if args.chunk_rows > 0 else [max(128, M // 4), max(128, M // 2)]
        blocks_choices = [args.ar_blocks] if args.ar_blocks > 0 else [4, 8, 16, 32]
        for mode in (["plain"] + [f"overlapped_{c}" for c in chunk_choices]
                     + (["multicast"] + [f"multicast_overlapped_{c}_{b}" for c in chunk_choices for b in blocks_choices]
                        + [f"multicast_fused_{c}" for c in (8, 16, 24)] if mc is not None else [])):
            overlap, multicast = mode.startswith("overlapped"), mode.startswith("multicast")
            mc_chunk[0] = int(mode.split("_")[2]) if mode.startswith("multicast_overlapped") else 0
            fused_ctas[0] = int(mode.split("_")[2]) if mode.startswith("multicast_fused") else 0
            if mc_chunk[0]:
                ar_blocks[0] = int(mode.split("_")[3])
            if overlap:
                chunk_rows[0] = int(mode.split("_")[1])
            # an order that the library refuses on this box (a host-side status, nothing launched) is left out on every
            # rank alike: the ranks agree on the outcome before the next one is tried
            failed = 0
            try:
                step()
                fence()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(3):
                    step()
                a1.record()
            except RuntimeError as e:
                failed = 1
                config.setdefault("step_refused", {})[mode] = str(e)[:200]
            fence()
            tt = torch.tensor([a0.elapsed_time(a1) / 3 if not failed else float("inf"), float(failed)], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            if float(tt[1]) > 0:
                continue
            tried[mode] = float(tt[0])
        best = min(tried, key=tried.get)
        overlap, multicast = best.startswith("overlapped"), best.startswith("multicast")
        mc_chunk[0] = int(best.split("_")[2]) if best.startswith("multicast_overlapped") else 0
        fused_ctas[0] = int(best.split("_")[2]) if best.startswith("multicast_fused") else 0
        if mc_chunk[0]:
            ar_blocks[0] = int(best.split("_")[3])
        if overlap:
            chunk_rows[0] = int(best.split("_")[1])
        config["step_tried_ms"] = tried
        # The trials loaded the board for a few hundred milliseconds; at N = 1 the warm-up starts from an idle board.  Give
        # the power controller the same starting point here (set-up, outside every timed region).
        fence()
        time.sleep(1.0)
        fence()
        config["after_trials"] = "1 s idle before the warm-up steps"
    if world > 1:
        config["step"] = ((f"row-parallel layers in chunks of {chunk_rows[0]} rows, the NCCL all-reduce of a chunk overlaps "
                           f"the next chunk's GEMM" + (f"; GEMMs on {sm_total - args.comm_sms} of {sm_total} SMs"
                                                       if args.comm_sms > 0 else "")) if overlap
                          else (f"row-parallel GEMM and multicast all-reduce in ONE launch: {fused_ctas[0]} CTAs of the GEMM's "
                                "grid sum every finished block of 2048 output rows through the switch (multimem ld_reduce + "
                                "st) while the other CTAs compute the next block") if multicast and fused_ctas[0]
                          else (f"row-parallel GEMMs in chunks of {mc_chunk[0]} rows on {sm_total - ar_blocks[0]} SMs write "
                                f"into NVSwitch multicast memory; this library's multimem kernel ({ar_blocks[0]} blocks, side "
                                "stream) adds a chunk in place while the next chunk's GEMM runs") if multicast and mc_chunk[0]
                          else ("row-parallel GEMMs write into NVSwitch multicast memory; this library's multimem kernel "
                                "(ld_reduce + st, one launch) adds them in place, same stream") if multicast
                          else "NCCL all-reduce after each row-parallel GEMM, same stream")
    for _ in range(args.warmup if args.only not in ("quant", "ue8m0") else 0):
        step()
    for L in layers:
        L["ev"] = []
    main_steps = args.steps if args.only not in ("quant", "ue8m0") else 1
    fence()
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    own_launches[0] = 0
    t0.record()
    for _ in range(main_steps):
        step(record=True)
    t1.record()
    timed_launches = own_launches[0]
    fence()
    clocks = sampler.stop()
    ms = torch.tensor([t0.elapsed_time(t1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / main_steps
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    breakdown = None
    if args.only in ("all", "gemm"):
        breakdown = breakdown_pass()
        if overlap or (multicast and (mc_chunk[0] > 0 or fused_ctas[0] > 0)):
            breakdown["overlap_saves_ms"] = breakdown["step_ms"] - ms_per_step
        if world == 1:
            # the same step as one replayed CUDA graph: what is left of the host gap when nothing is launched from Python
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            torch.cuda.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(main_steps):
                graph.replay()
            g1.record()
            torch.cuda.synchronize()
            breakdown["graph_replay_ms_per_step"] = g0.elapsed_time(g1) / main_steps
            del graph
            # host microseconds of one Fp8LinearMethod.apply call (allocation, checks, tensor maps, two launches)
            torch.cuda.synchronize()
            h0 = time.perf_counter()
            for _ in range(20):
                method.apply(layers[1]["layer"], layers[1]["x"][:256])
            breakdown["host_us_per_apply_call"] = (time.perf_counter() - h0) * 1e6 / 20
            torch.cuda.synchronize()

    # GEMM kernel alone: CUDA events around every launch in the timed region
    gemm_ms, gemm_flops, per_shape = 0.0, 0.0, {}
    for L in layers:
        if not L["ev"]:
            continue
        t = [a.elapsed_time(b) for a, b in L["ev"]]
        f = 2.0 * M * L["n_loc"] * L["k_loc"]
        gemm_ms += sum(t)
        gemm_flops += f * len(t)
        per_shape[L["name"]] = {"N": L["n_loc"], "K": L["k_loc"], "gemm_ms": statistics.median(t),
                                "gemm_tflops": f / (statistics.median(t) * 1e-3) / 1e12}
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    # DRAM traffic per launch: algorithmic operand + output bytes x 1.05, the read + write / algorithmic ratio of one ncu
    # capture of this kernel at M = 2048, N = 7168, K = 16384 (189.0 MB measured, 180.4 MB algorithmic), scaled up
    alg_bytes = sum(L["n_loc"] * L["k_loc"] + M * L["k_loc"] + 2.0 * M * L["n_loc"] for L in layers) / len(layers)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                "frac": achieved / fp8_peak, "traffic": 1.05 * alg_bytes,
                "traffic_note": "bytes per launch averaged over the layers; ncu ratio 1.05 on a smaller M scaled up",
                "kernel": "fp8_block_gemm_kernel",
                "peak_source": f"2 x bf16_tflops_sustained ({peaks['source']}); nominal dense FP8 is 4500",
                "frac_of_nominal_fp8": achieved / 4500.0, "launches": sum(len(L["ev"]) for L in layers),
                "avg_launch_ms": gemm_ms / max(1, sum(len(L["ev"]) for L in layers)), "others": []}
    if overlap or (multicast and (mc_chunk[0] > 0 or fused_ctas[0] > 0)):
        roofline["note"] = ("column-parallel and replicated layers only: the row-parallel GEMMs run in chunks beside "
                            "the all-reduce")

    # ---- the same sweep on a UE8M0 checkpoint (power-of-two weight block scales, power-of-two activation group
    # scales): the tensor core applies the scales itself (tcgen05.mma kind::mxf8f6f4.block_scale)
    def step_u(record=False):
        for L in layers:
            q, s = sglang_per_token_group_quant_fp8(L["x"], 128, column_major_scales=True, scale_tma_aligned=True,
                                                    scale_ue8m0=True)
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            y = w8a8_block_fp8_matmul_ue8m0(q, L["wq_u"], s, L["ws_u"], torch.bfloat16)
            if record:
                e1.record()
                L["ev_u"].append((e0, e1))
            if world > 1 and L["mode"] == "row":
                dist.all_reduce(y)
        return y

    ue8m0 = None
    if args.only in ("all", "ue8m0"):
        sampler_u = ClockSampler(gpu_uuid)
        for _ in range(args.warmup):
            step_u()
        fence()
        sampler_u.start()
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        u0.record()
        for _ in range(args.steps):
            step_u(record=True)
        u1.record()
        fence()
        clocks_u = sampler_u.stop()
        ms_u = torch.tensor([u0.elapsed_time(u1)], device=dev)
        if world > 1:
            dist.all_reduce(ms_u, op=dist.ReduceOp.MAX)
        ms_u_step = float(ms_u) / args.steps
        g_ms, g_fl, shp = 0.0, 0.0, {}
        for L in layers:
            tt = [a.elapsed_time(b) for a, b in L["ev_u"]]
            f = 2.0 * M * L["n_loc"] * L["k_loc"]
            g_ms += sum(tt)
            g_fl += f * len(tt)
            shp[L["name"]] = {"gemm_ms": statistics.median(tt), "gemm_tflops": f / (statistics.median(tt) * 1e-3) / 1e12}
        ach_u = g_fl / (g_ms * 1e-3) / 1e12
        ue8m0 = {"workload": "same five layers, UE8M0 checkpoint: power-of-two weight block scales and activation "
                             "group scales, hardware block-scaled MMA",
                 "value": total_flops / (ms_u_step * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_u_step,
                 "roofline": {"bound": "tensor", "achieved": ach_u, "peak": 2.0 * peaks["bf16_tflops_sustained"],
                              "unit": "TFLOP/s", "frac": ach_u / (2.0 * peaks["bf16_tflops_sustained"]),
                              "frac_of_nominal_fp8": ach_u / 4500.0, "kernel": "fp8_ue8m0_gemm_kernel"},
                 "per_shape": shp, "clocks": clocks_u, "gpu_launches": args.steps * len(layers) * 2}

    quant_after = None
    if rank == 0 and args.only in ("all", "quant"):
        quant_after = quant_case("after the GEMM sweeps")
    for qc in (quant, quant_after):
        if qc is not None:
            roofline["others"].append({"kernel": "group_quant16_kernel", "bound": "hbm", "achieved": qc["gbs"],
                                       "peak": qc["peak_gbs"], "unit": "GB/s", "frac": qc["frac"], "when": qc["when"],
                                       "us": qc["ms"] * 1e3, "us_x_sm_mhz": qc["us_x_sm_mhz"], "clocks": qc["clocks"],
                                       "workload": "M=16384 K=7168 bf16 -> e4m3 + f32 scales (355.99 MB)"})
    if ue8m0 is not None:
        roofline["others"].append(dict(ue8m0["roofline"], workload="the same sweep on a UE8M0 checkpoint",
                                       note="outputs may differ from the oracle by one bf16 ulp (the K loop is summed "
                                            "inside the tensor core); rel-L2 bar unchanged"))

    if args.only != "all":
        if rank == 0:
            print(json.dumps({"metric": METRIC, "only": args.only, "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "config": config,
                              "clocks": clocks, "roofline": roofline, "quant": quant, "per_shape": per_shape,
                              "ue8m0": ue8m0, "breakdown": breakdown}))
        if mc is not None:
            mc.close()
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- fused MoE at the DeepSeek-V3 layer shape (BASELINE config 5), reported beside the headline
    moe = None
    if rank == 0 and world == 1 and not args.no_moe:
        try:
            moe = moe_section(torch, dev, gen, gpu_uuid=gpu_uuid)
        except Exception as e:  # noqa: BLE001 - the headline must not depend on this section
            moe = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()
        for case in (moe.get("cases") or []):
            for ck in ("fp32_scales", "ue8m0"):
                wl = f"E=256 top-8 H=7168 I=2048 M={case['M']}"
                if case["M"] <= 256:
                    # few rows per expert: bound by streaming the weights of the experts that have rows
                    gbs = case[ck]["weight_tbs"] * 1e3
                    entry = {"kernel": f"fused_experts ({ck}), nine launches", "bound": "hbm", "achieved": gbs,
                             "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                             "ms": case[ck]["ms"],
                             "workload": wl + f", {case['experts_with_rows']} experts with rows"}
                    if ck + "_tile_kernel" in case:
                        entry["ms_with_128x128_grouped_kernel"] = case[ck + "_tile_kernel"]["ms"]
                    roofline["others"].append(entry)
                else:
                    roofline["others"].append({"kernel": f"fused_experts ({ck}), nine launches", "bound": "tensor",
                                               "achieved": case[ck]["tflops"], "peak": fp8_peak, "unit": "TFLOP/s",
                                               "frac": case[ck]["tflops"] / fp8_peak, "ms": case[ck]["ms"],
                                               "workload": wl})

    # ---- the mid sizes of the sweep (M = 128 / 512 / 2048): GEMM kernel alone per shape
    per_shape_mid = None
    if rank == 0 and world == 1:
        per_shape_mid = []
        for L in layers:
            for m_mid in (128, 512, 2048):
                if m_mid >= M:
                    continue
                xm = L["x"][:m_mid].contiguous()
                qm_, sm_ = sglang_per_token_group_quant_fp8(xm, 128, column_major_scales=True, scale_tma_aligned=True)
                ev = []
                for i in range(8):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    w8a8_block_fp8_matmul(qm_, L["layer"].weight, sm_, L["layer"].weight_scale_inv, [128, 128], torch.bfloat16)
                    e1.record()
                    ev.append((e0, e1))
                torch.cuda.synchronize()
                tms = statistics.median(a.elapsed_time(b) for a, b in ev[3:])
                per_shape_mid.append({"layer": L["name"], "M": m_mid, "N": L["n_loc"], "K": L["k_loc"], "gemm_us": tms * 1e3,
                                      "gemm_tflops": 2.0 * m_mid * L["n_loc"] * L["k_loc"] / (tms * 1e-3) / 1e12})

    # ---- end to end through the public API from pinned host memory
    host_x = [L["x"].cpu().pin_memory() for L in layers]
    # results that are identical on every rank (all-reduced row-parallel outputs, the replicated layer) go back to the
    # host once, from rank 0; every rank returns its own column-parallel shard
    returns = [world == 1 or L["mode"] == "column" or rank == 0 for L in layers]
    host_y = [torch.empty(M, L["n_loc"], dtype=torch.bfloat16).pin_memory() if r else None for L, r in zip(layers, returns)]
    h2d = sum(t.numel() * 2 for t in host_x)
    d2h = sum(t.numel() * 2 for t in host_y if t is not None)

    # Three streams: the upload of layer i + 1 and the download of layer i - 1 run under the compute of layer i (PCIe is
    # full duplex), as a serving loop that owns its copy engines would do it.  Every byte still crosses inside the timed
    # region; the device input buffers are allocated once.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    dev_x = [torch.empty_like(L["x"]) for L in layers]

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)  # the previous step's GEMMs have read the input buffers
        for L, hx, hy, xd in zip(layers, host_x, host_y, dev_x):
            with torch.cuda.stream(s_in):
                xd.copy_(hx, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            cur.wait_event(ev_in)
            y = method.apply(L["layer"], xd)
            if world > 1 and L["mode"] == "row":
                dist.all_reduce(y)
            if hy is None:
                continue
            ev_out = torch.cuda.Event()
            ev_out.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_out)
                hy.copy_(y, non_blocking=True)
                y.record_stream(s_out)
        cur.wait_stream(s_out)  # the step ends when its last result has reached the host buffer

    e2e_steps = max(3, min(args.steps, 5))
    for _ in range(2):
        e2e_step()
    fence()
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    fence()
    ms = torch.tensor([t0.elapsed_time(t1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(ms) / e2e_steps
    e2e = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "api": "Fp8LinearMethod.apply on pinned-host activations, result copied back to pinned host; uploads, "
                  "compute and downloads on three streams"}

    decode = None
    if rank == 0 and world == 1:
        try:
            decode = decode_section(torch, dev, peaks)
        except Exception as e:  # noqa: BLE001 - the headline must not depend on this section
            decode = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()

    fused_ar = None
    if world > 1:
        try:
            fused_ar = fused_allreduce_section(torch, dist, dev, world, rank, layers)
        except Exception as e:  # noqa: BLE001 - the headline must not depend on this section
            fused_ar = {"error": f"{type(e).__name__}: {e}"}

    tp_llama, ep_moe = None, None
    if world > 1:
        for L in layers:  # free the sweep's weights first
            L.clear()
        layers_n = len(layers)
        torch.cuda.empty_cache()
        try:
            tp_llama = tp_llama_section(torch, dist, dev, gen, world, rank, mc=mc, mc_chunk=mc_chunk[0] or M // 2,
                                        mc_blocks=ar_blocks[0])
        except Exception as e:  # noqa: BLE001
            tp_llama = {"error": f"{type(e).__name__}: {e}"}
        if mc is not None:
            mc.close()
            mc = None
        torch.cuda.empty_cache()
        if not args.no_moe:
            ep_moe = []
            for m_total in (256, 4096, 16384):
                try:
                    ep_moe.append(ep_moe_section(torch, dist, dev, gen, world, rank, M_total=m_total,
                                                 decode_graph=(m_total == 4096)))
                except Exception as e:  # noqa: BLE001
                    ep_moe.append({"M_total": m_total, "error": f"{type(e).__name__}: {e}"})
                torch.cuda.empty_cache()
    else:
        layers_n = len(layers)
        if rank == 0:
            for L in layers:
                L.clear()
            torch.cuda.empty_cache()
            try:  # the tp1 point: the base of the tensor-parallel scaling of this layer
                tp_llama = tp_llama_section(torch, dist, dev, gen, 1, 0)
            except Exception as e:  # noqa: BLE001
                tp_llama = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_arm(3, 1, cpu_m)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic", "config": config, "clocks": clocks,
                "e2e": e2e, "gpu_launches": timed_launches, "roofline": roofline,
                "cpu_baseline": cpu_baseline, "breakdown": breakdown, "parity": parity, "quant": quant,
                "quant_after": quant_after, "moe": moe, "per_shape": per_shape, "per_shape_mid": per_shape_mid,
                "ue8m0": ue8m0, "decode": decode, "fused_allreduce": fused_ar, "tp_llama70b": tp_llama, "ep_moe": ep_moe,
                "impl": "ours"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
