"""Compile the reference's own CPU kernels for this path into ``oracle/_ref/``.

TEST / BASELINE INFRASTRUCTURE ONLY.  The sources are compiled where they lie in the
reference checkout (nothing is copied): ``sgl-kernel/csrc/cpu/{gemm,gemm_fp8,gemm_int8,moe,
moe_fp8,moe_int8}.cpp`` plus the registration shim ``oracle/ref_binding.cpp``.  They need
AVX512-BF16 and AMX at run time (``gemm_fp8.cpp:98,115`` checks).  They are W8A16 (bf16
activations, weights dequantised block-wise), so they are the timed CPU baseline and a loose
cross-check, not the bit-level oracle.

    python oracle/build_ref.py /path/to/reference        (or SGLANG_REFERENCE_ROOT=/path/to/reference)

Without an argument :func:`build` looks for the checkout in ``$SGLANG_REFERENCE_ROOT`` and then in a directory named
``reference`` beside this repository; if there is none it returns None and the prebuilt library (if any) is used.

The result, ``oracle/_ref/libsglb200_ref.so``, is loaded with :func:`load_ref`.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libsglb200_ref.so")
FILES = ["gemm.cpp", "gemm_fp8.cpp", "gemm_int8.cpp", "moe.cpp", "moe_fp8.cpp", "moe_int8.cpp"]


def find_reference():
    """The reference checkout: ``$SGLANG_REFERENCE_ROOT``, else a directory ``reference`` beside this repository."""
    cands = [os.environ.get("SGLANG_REFERENCE_ROOT"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "sgl-kernel", "csrc", "cpu")):
            return c
    return None


def build(ref_root=None, force=False):
    ref_root = ref_root or find_reference()
    if ref_root is None:
        return LIB if os.path.exists(LIB) else None
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
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
