"""Compile the reference's own CPU kernels for this path into ``oracle/_ref/``.

TEST / BASELINE INFRASTRUCTURE ONLY.  The sources are compiled where they lie in the
reference checkout (nothing is copied): ``sgl-kernel/csrc/cpu/{gemm,gemm_fp8,gemm_int8,moe,
moe_fp8,moe_int8}.cpp`` plus the registration shim ``oracle/ref_binding.cpp``.  They need
AVX512-BF16 and AMX at run time (``gemm_fp8.cpp:98,115`` checks).  They are W8A16 (bf16
activations, weights dequantised block-wise), so they are the timed CPU baseline and a loose
cross-check, not the bit-level oracle.

    python oracle/build_ref.py [/path/to/reference]

The result, ``oracle/_ref/libsglb200_ref.so``, is loaded with :func:`load_ref`.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libsglb200_ref.so")
FILES = ["gemm.cpp", "gemm_fp8.cpp", "gemm_int8.cpp", "moe.cpp", "moe_fp8.cpp", "moe_int8.cpp"]


def build(ref_root="/root/reference", force=False):
    src_dir = os.path.join(ref_root, "sgl-kernel", "csrc", "cpu")
    if not os.path.isdir(src_dir):
        return None
    if os.path.exists(LIB) and not force:
        return LIB
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT, exist_ok=True)
    inc = [src_dir, os.path.join(ref_root, "sgl-kernel", "include")] + ce.include_paths()
    import sysconfig
    inc.append(sysconfig.get_paths()["include"])
    flags = ["-O3", "-march=native", "-fopenmp", "-fPIC", "-std=c++17", "-Wno-unknown-pragmas",
             "-DSGLANG_CPU_FP8_CVT_FTZ", "-DTORCH_EXTENSION_NAME=libsglb200_ref",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    objs = []
    procs = []
    for f in [os.path.join(HERE, "ref_binding.cpp")] + [os.path.join(src_dir, x) for x in FILES]:
        o = os.path.join(OUT, os.path.basename(f)[:-4] + ".o")
        objs.append(o)
        procs.append(subprocess.Popen(["g++", *flags, *[f"-I{i}" for i in inc], "-c", f, "-o", o]))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("compiling the reference CPU kernels failed")
    tl = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-shared", "-o", LIB, *objs, f"-L{tl}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lgomp", f"-Wl,-rpath,{tl}"]
    subprocess.check_call(cmd)
    return LIB


def load_ref():
    """Load the prebuilt library and return ``torch.ops.sglb200_ref`` (or None if it is absent,
    does not load, or the host CPU lacks AMX / AVX512-BF16)."""
    if not os.path.exists(LIB):
        return None
    try:
        flags = open("/proc/cpuinfo").read()
        if "amx_tile" not in flags or "avx512_bf16" not in flags:
            return None
        import torch
        torch.ops.load_library(LIB)
        return torch.ops.sglb200_ref
    except Exception:
        return None


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", force="--force" in sys.argv))
