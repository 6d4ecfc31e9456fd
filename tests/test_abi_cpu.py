"""CPU-side checks: the C-ABI library loads without a GPU and exports every symbol the header
declares; host-side validation raises before anything could launch; the quantiser's FMA division
is checked against the IEEE division on a sample of the exhaustive host test."""

import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sglb200.h")


@pytest.fixture(scope="module")
def built_lib():
    from sglang_b200 import build
    path = build.build()
    assert os.path.exists(path)
    return path


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sglb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    from sglang_b200._lib import SIGNATURES, lib
    handle = lib()
    declared = _declared_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared in include/sglb200.h but not exported"
    assert sorted(SIGNATURES) == declared, "ctypes signatures and header are out of step"
    assert handle.sglb200_version().decode() == "0.2"
    assert handle.sglb200_status_string(0).decode() == "ok"
    assert "alignment" in handle.sglb200_status_string(-2).decode()


def test_header_cites_the_reference_for_each_kernel_entry():
    text = open(HEADER).read()
    for name in ["per_token_group_quant_8bit.cu", "fp8_blockwise_gemm_kernel.cu", "fp8_blockwise_moe_kernel.cu",
                 "prepare_moe_input.cu", "activation.cu", "common_extension.cc"]:
        assert name in text


def test_host_validation_without_gpu(built_lib):
    """Shape / dtype / null checks come first, so they are reachable on a machine with no GPU."""
    from sglang_b200._lib import check, lib
    L = lib()
    assert L.sglb200_per_token_group_quant_fp8(None, 0, None, None, 4, 200, 128, 1e-10, -448.0, 448.0, 0, 2, 1, None) == -1
    assert "multiple of group_size" in L.sglb200_last_error_detail().decode()
    assert L.sglb200_per_token_group_quant_fp8(None, 0, None, None, 4, 256, 8, 1e-10, -448.0, 448.0, 0, 2, 1, None) == -1
    assert L.sglb200_per_token_group_quant_fp8(None, 7, None, None, 4, 256, 128, 1e-10, -448.0, 448.0, 0, 2, 1, None) == -5
    assert L.sglb200_per_token_group_quant_fp8(None, 0, None, None, 4, 256, 128, 1e-10, -448.0, 448.0, 0, 2, 1, None) == -6
    assert L.sglb200_per_token_group_quant_fp8(None, 0, None, None, 0, 256, 128, 1e-10, -448.0, 448.0, 0, 2, 1, None) == 0
    assert L.sglb200_fp8_blockwise_scaled_mm(None, None, None, None, None, 4, 128, 100, 100, 100, 128, 1, 4, 1, 1, 0, None) == -1
    assert L.sglb200_fp8_blockwise_scaled_mm(None, None, None, None, None, 4, 128, 128, 128, 128, 128, 1, 4, 1, 1, 2, None) == -5
    assert L.sglb200_fp8_blockwise_scaled_mm(None, None, None, None, None, 0, 128, 128, 128, 128, 128, 1, 4, 1, 1, 0, None) == 0
    assert L.sglb200_shuffle_rows(None, None, None, 4, 6, None) == -1
    assert L.sglb200_prepare_moe_input(None, None, None, None, None, None, 4, 2, 5000, 1, 1, None) == -1
    with pytest.raises(RuntimeError, match="bad shape"):
        check(-1, "op")


def test_ops_refuse_cpu_tensors(built_lib):
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm, silu_and_mul
    a = torch.zeros(4, 128, dtype=torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fp8_blockwise_scaled_mm(a, a.t(), torch.ones(4, 1), torch.ones(1, 1), torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        silu_and_mul(torch.zeros(4, 16, dtype=torch.bfloat16))


def test_missing_library_fails_loudly(monkeypatch):
    import sglang_b200._lib as L
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", "/nonexistent/libsglb200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        L.lib()


@pytest.mark.parametrize("fmt", ["bf16", "f16"])
def test_fma_division_matches_ieee_on_a_sample(tmp_path, fmt):
    """tests/csrc/check_quant_math.cpp with stride 97 (the full run, stride 1, takes ~15 s per format)."""
    exe = str(tmp_path / "check_quant_math")
    subprocess.check_call(["g++", "-O2", "-fopenmp", "-x", "c++", "-o", exe,
                           os.path.join(ROOT, "tests", "csrc", "check_quant_math.cpp"),
                           "-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lgomp"])
    out = subprocess.run([exe, fmt, "97"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert "code_mismatch=0" in out.stdout and "scale_mismatch=0" in out.stdout


def test_linear_method_create_weights_checks():
    from sglang_b200.layers.quantization import Fp8Config, Fp8LinearMethod
    cfg = Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    layer = torch.nn.Module()
    Fp8LinearMethod(cfg, tp_size=1).create_weights(layer, 7168, [576], 7168, 576, torch.bfloat16)
    assert layer.weight.shape == (576, 7168) and layer.weight.dtype == torch.float8_e4m3fn
    assert layer.weight_scale_inv.shape == (5, 56) and layer.input_scale is None
    with pytest.raises(ValueError, match="block_k"):
        Fp8LinearMethod(cfg, tp_size=8).create_weights(torch.nn.Module(), 200, [512], 1600, 512, torch.bfloat16)
    with pytest.raises(ValueError, match="block_n"):
        Fp8LinearMethod(cfg, tp_size=1).create_weights(torch.nn.Module(), 1024, [192, 192], 1024, 384, torch.bfloat16)
    with pytest.raises(ValueError):
        Fp8Config(weight_block_size=[64, 64])
    with pytest.raises(ValueError):
        Fp8Config(activation_scheme="static")


def test_scale_allocator_layouts():
    from sglang_b200.layers.quantization import create_per_token_group_quant_fp8_output_scale as alloc
    assert alloc((6, 640), "cpu", 128, False, False, False).stride() == (5, 1)
    assert alloc((6, 640), "cpu", 128, True, False, False).stride() == (1, 6)
    t = alloc((6, 640), "cpu", 128, True, True, False)
    assert t.shape == (6, 5) and t.stride() == (1, 8)
    u = alloc((6, 640), "cpu", 128, True, True, True)
    assert u.dtype == torch.int32 and u.shape == (6, 2) and u.stride() == (1, 8)


def test_host_validation_of_routing_and_exchange_entries(built_lib):
    """The routing, masked-layout and peer-exchange entry points check their arguments before touching a device too."""
    import ctypes
    from sglang_b200._lib import lib
    L = lib()
    detail = lambda: L.sglb200_last_error_detail().decode()
    assert L.sglb200_topk_softmax(None, 2, None, None, 4, 2048, 2, 0, None) == -1 and "num_experts" in detail()
    assert L.sglb200_topk_softmax(None, 2, None, None, 4, 8, 9, 0, None) == -1 and "topk" in detail()
    assert L.sglb200_topk_softmax(None, 2, None, None, 0, 8, 2, 0, None) == 0
    assert L.sglb200_moe_fused_gate(None, None, 2, None, None, 4, 256, 7, 4, 8, 0, 2.5, 0, None) == -1
    assert "num_expert_group" in detail()
    assert L.sglb200_moe_fused_gate(None, None, 2, None, None, 4, 256, 8, 4, 8, 2, 0.0, 0, None) == -1
    assert "routed_scaling_factor" in detail()
    assert L.sglb200_moe_align_block_size(None, 1 << 25, 9, 16, None, None, None, None, 0, None) == -1
    assert L.sglb200_moe_sum_reduce(None, None, 4, 2, 100, 0, 1.0, None) == -1 and "multiple of 8" in detail()
    assert L.sglb200_moe_sum_reduce(None, None, 0, 2, 128, 0, 1.0, None) == 0
    assert L.sglb200_fp8_blockwise_scaled_masked_grouped_mm(None, None, None, None, None, None, 4, 64, 128, 128, 128, 128,
                                                            128 * 128, 128, 64, 1, 1, 1, 1, 1, 0, None) == -6
    assert "masked_m" in detail()
    assert L.sglb200_group_quant_fp8_batched(None, 2, None, None, 4, 16, 256, 128, 1e-10, -448.0, 448.0, 0, 0, None, 32, 2,
                                             1, None) == -1 and "16-bit" in detail()
    ptrs = (ctypes.c_void_p * 2)(None, None)
    assert L.sglb200_fp8_blockwise_scaled_mm_push(None, None, None, None, 64, 512, 256, 256, 256, 2, 1, 2, 1, 0, ptrs, ptrs,
                                                  0, 2, 1024, None, 0, None) == -7 and "receive slot" in detail()
    assert L.sglb200_fp8_blockwise_scaled_mm_push(None, None, None, None, 64, 512, 256, 256, 256, 2, 1, 2, 1, 0, ptrs, ptrs,
                                                  3, 2, 64 * 512, None, 0, None) == -1 and "rank" in detail()
    assert L.sglb200_peer_reduce(None, None, None, 64, 500, 512, 0, 2, 64 * 512, 0, None) == -1
    assert L.sglb200_fp8_blockwise_scaled_mm_push_scatter(None, None, None, None, 64, 128, 256, 256, 256, 2, 1, 2, 1, 0,
                                                          ptrs, ptrs, 0, 2, 64 * 128, None) == -1
    assert "fewer output tiles than ranks" in detail()
    assert L.sglb200_peer_reduce_scatter(ptrs, ptrs, None, 256, 512, 512, 0, 0, 2, 1024, 0, None) == -7
    assert L.sglb200_peer_gather(None, None, None, 256, 512, 512, 0, 0, 2, 256 * 512, 0, None) == -6
    assert L.sglb200_ep_dispatch(None, None, 2, 1, None, None, 4, 200, 2, 4, ptrs, 0, 2, 16, 16, None) == -1
    assert "multiple of 128" in detail()
    assert L.sglb200_ep_dispatch(None, None, 2, 1, None, None, 40, 256, 2, 4, ptrs, 0, 2, 16, 16, None) == -6
    assert L.sglb200_ep_dispatch_quant(None, 2, 256, None, None, 4, 256, 2, 4, ptrs, 0, 2, 16, 16, 1e-10, None) == -5
    assert L.sglb200_ep_dispatch_quant(None, 0, 100, None, None, 4, 256, 2, 4, ptrs, 0, 2, 16, 16, 1e-10, None) == -1
    assert "ldx" in detail()
    assert L.sglb200_ep_combine_reduce(ptrs, 0, 9, None, None, 0, 4, 256, 2, 4, 16, 16, 0, None) == -1
    assert L.sglb200_ep_buffer_bytes(16, 256, 2, 2, 16) > 16 * 256 and L.sglb200_ep_buffer_bytes(0, 256, 2, 2, 16) == 0
    assert L.sglb200_peer_flag_bytes() > 0 and L.sglb200_peer_recv_bytes(1024) == 2 * 8 * 1024 * 2
    assert L.sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes(129, 7168, 8192) == 0
    h = (ctypes.c_ubyte * 64)()
    assert L.sglb200_peer_alloc(0, None, h) == -6 and L.sglb200_peer_open(None, None) == -6
    assert L.sglb200_peer_close(None) == 0 and L.sglb200_peer_free(None) == 0


def test_peer_ep_exchange_refuses_a_receive_buffer_that_could_overflow():
    """capacity < world * m_max is refused before anything is allocated (no GPU needed to see the refusal)."""
    from sglang_b200.distributed.peer_ep import PeerEpExchange
    with pytest.raises(ValueError, match="capacity"):
        PeerEpExchange(capacity=10, hidden=256, topk=2, m_max=11, device="cpu")


def test_num_sms_limit_round_trip(built_lib):
    """The SM bound is plain host state: settable and readable without a GPU; a negative value is refused."""
    from sglang_b200._lib import lib
    L = lib()
    assert L.sglb200_set_num_sms(-1) == -1
    assert L.sglb200_set_num_sms(132) == 0
    assert L.sglb200_get_num_sms() == 132
    assert L.sglb200_set_num_sms(0) == 0
    assert L.sglb200_get_num_sms() != 132


def test_symm_mem_communicator_is_disabled_without_a_gpu():
    """The reference's wrapper stays disabled and declines when a prerequisite is missing
    (``device_communicators/symm_mem.py:46-47,113-123``); so does this one, and the row-parallel layer then takes the
    collective library's all-reduce."""
    import torch
    from sglang_b200.distributed import SymmMemCommunicator
    comm = SymmMemCommunicator(None, "cpu")
    assert comm.disabled and comm.all_reduce(torch.zeros(8, dtype=torch.bfloat16)) is None
    assert not comm.should_symm_mem_allreduce(torch.zeros(8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        comm.view((8,))
    comm.close()


def test_host_validation_of_the_multicast_and_few_rows_entries(built_lib):
    """The multicast all-reduce, the GEMM with the all-reduce in its launch and the kernel-selection setters refuse bad
    arguments on the host, before any device is touched."""
    import ctypes
    from sglang_b200._lib import lib
    L = lib()
    detail = lambda: L.sglb200_last_error_detail().decode()
    flags = (ctypes.c_uint64 * 8)(*([4096] * 8))
    assert L.sglb200_nvls_flag_bytes() == (2 * 8 * 128 + 128) * 4
    assert L.sglb200_nvls_all_reduce(4096, flags, 0, 1, 64, 0, 0, None) == -1 and "world" in detail()
    assert L.sglb200_nvls_all_reduce(4096, flags, 2, 2, 64, 0, 0, None) == -1 and "rank" in detail()
    assert L.sglb200_nvls_all_reduce(4096, flags, 0, 2, 60, 0, 0, None) == -1 and "multiple of 8" in detail()
    assert L.sglb200_nvls_all_reduce(4096, flags, 0, 2, 64, 2, 0, None) == -5          # fp32 is not a dtype it adds
    assert L.sglb200_nvls_all_reduce(4096, flags, 0, 2, 64, 0, 129, None) == -1 and "blocks" in detail()
    assert L.sglb200_nvls_all_reduce(4096, flags, 0, 2, 0, 0, 0, None) == 0             # nothing to add
    assert L.sglb200_nvls_all_reduce(0, flags, 0, 2, 64, 0, 0, None) == -6
    assert L.sglb200_nvls_all_reduce(4104, flags, 0, 2, 64, 0, 0, None) == -2           # not 16-byte aligned
    mm = L.sglb200_fp8_blockwise_scaled_mm_allreduce
    args = lambda **kw: [kw.get(k, v) for k, v in dict(a=None, b=None, sa=None, sb=None, out=None, mc=4096, flags=flags,
                                                       done=None, rank=0, world=2, ctas=16, M=256, N=512, K=1024, lda=1024,
                                                       ldb=1024, sam=1, sak=256, sbn=8, sbk=1, dt=0, st=None).items()]
    assert mm(*args(world=9)) == -1 and "ranks" in detail()
    assert mm(*args(ctas=0)) == -1 and "comm_ctas" in detail()
    assert mm(*args(ctas=65)) == -1
    assert mm(*args(K=1000)) == -1 and "multiple of 16" in detail()
    assert mm(*args(dt=2)) == -5
    assert mm(*args(M=0)) == 0
    assert mm(*args(M=64 * 16 * 128 + 1)) == -1 and "row blocks" in detail()
    assert mm(*args()) == -6                                                          # NULL operands
    before = L.sglb200_get_grouped_few_rows()
    assert L.sglb200_set_grouped_few_rows(65) == -1 and L.sglb200_set_grouped_few_rows(-1) == -1
    assert L.sglb200_set_grouped_few_rows(0) == 0 and L.sglb200_get_grouped_few_rows() == 0
    assert L.sglb200_set_grouped_few_rows(before) == 0 and L.sglb200_get_grouped_few_rows() == before == 20
