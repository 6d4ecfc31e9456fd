"""The UE8M0 (hardware block-scaled) GEMM against the oracle.

OFF BY DEFAULT: run with SGLB200_TEST_UE8M0=1.  The kernel gives correct results on every shape tried, but one
sustained back-to-back sequence at M=8192, N=36864, K=7168 ended in an unexplained "unspecified launch failure",
so it is kept out of the default GPU runs (each case here runs in a child process so a lost context cannot affect
other tests)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys, torch
sys.path.insert(0, %(root)r); sys.path.insert(0, %(root)r + "/tests")
import oracle
from helpers import assert_gemm_close
from sglang_b200._lib import lib
from sglang_b200.layers.quantization import (pack_ue8m0_scales, sglang_per_token_group_quant_fp8,
                                             w8a8_block_fp8_matmul_ue8m0)
M, N, K = %(M)d, %(N)d, %(K)d
g = torch.Generator().manual_seed(M + N + K)
x = (torch.randn(M, K, generator=g) * 10 ** (torch.rand(M, 1, generator=g) * 4 - 2)).bfloat16()
w = torch.randn(N, K, generator=g) * 0.02 * (10 ** (torch.rand(N, 1, generator=g) * 2 - 1))
wq, ws = oracle.block_quant_weight(w, scale_ue8m0=True)
aq_ref, as_ref = oracle.per_token_group_quant_fp8(x, 128, scale_ue8m0=True)
ref = oracle.w8a8_block_fp8_matmul(aq_ref, wq, as_ref, ws)
aq, asp = sglang_per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                           scale_ue8m0=True)
out = w8a8_block_fp8_matmul_ue8m0(aq, wq.cuda(), asp, pack_ue8m0_scales(ws.cuda()), torch.bfloat16)
torch.cuda.synchronize()
assert lib().sglb200_read_device_status() == 0
assert torch.equal(aq.cpu().view(torch.uint8), aq_ref.view(torch.uint8))
assert_gemm_close(out, ref, "ue8m0 gemm")
print("OK")
'''


@pytest.mark.skipif(os.environ.get("SGLB200_TEST_UE8M0") != "1", reason="experimental kernel: set SGLB200_TEST_UE8M0=1")
@pytest.mark.parametrize("M,N,K", [(128, 192, 128), (1, 576, 512), (200, 576, 2048), (1000, 1536, 4096),
                                   (2048, 1920, 4096)])
def test_ue8m0_gemm_matches_oracle(M, N, K):
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT, "M": M, "N": N, "K": K}], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-500:] + r.stderr[-1500:]
