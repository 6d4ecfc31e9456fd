"""Build ``sglang_b200/lib/libsgl_kernel_ops.so``: the torch registration of the ``sgl_kernel`` ops on this path
(``TORCH_LIBRARY_FRAGMENT(sgl_kernel, m)``, schemas of ``sgl-kernel/csrc/common_extension.cc``) over the C ABI of
``libsglb200.so``.

    python -m sglang_b200.build_torch_ops [--force]

One host-only translation unit, compiled with g++ against the installed torch headers and linked to ``libsglb200.so``
through ``$ORIGIN``; no kernel lives in it.  ``sglang_b200.sgl_kernel.load_torch_ops()`` loads it, after which the ops
are reachable as ``torch.ops.sgl_kernel.<name>`` like the reference's.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc", "torch_ops", "sgl_kernel_ops.cpp")
LIBDIR = os.path.join(PKG, "lib")
OUT = os.path.join(LIBDIR, "libsgl_kernel_ops.so")


def build(force: bool = False) -> str:
    import torch
    from torch.utils.cpp_extension import include_paths
    from . import build as base
    core = base.build()
    hdr = os.path.join(os.path.dirname(PKG), "include", "sglb200.h")
    newest = max(os.path.getmtime(p) for p in (SRC, hdr, core))
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= newest:
        return OUT
    cxx = os.environ.get("CXX") or shutil.which("g++")
    if not cxx:
        raise RuntimeError("g++ not found: cannot build libsgl_kernel_ops.so")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = include_paths() + [os.path.join(cuda_home, "include")]
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in incs], SRC, "-o", OUT,
           f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           f"-L{LIBDIR}", "-lsglb200", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build of libsgl_kernel_ops.so failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    print(build(ap.parse_args().force))
