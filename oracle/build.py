"""Builds the test oracles.

  oracle/liboracle.so        - the CPU restatement (forge_oracle.c), gcc -O3 -fopenmp.
  oracle/_ref/libforge_ref.so - the reference's own hot-path CUDA sources, compiled where they
                                lie (never copied) for sm_100a with the reference's flags
                                (CMakeLists.txt:86-93: -O3 --use_fast_math
                                --expt-relaxed-constexpr) plus ref_shim.cu. Built only when the
                                reference tree is present; the GPU box uses the prebuilt file.

TEST INFRASTRUCTURE: nothing under forge_b200/ imports or links these.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libforge_ref.so")
# The reference source tree: $FORGE_REFERENCE_ROOT, else a directory named "reference" next to this
# repository's checkout.
REFERENCE_ROOT = os.environ.get("FORGE_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))
REF_SOURCES = [
    "src/quant/quantize.cu", "src/quant/dequantize.cu",
    "src/sparsity/prune_compress.cu", "src/sparsity/pack_metadata.cu",
    "src/gemm/int8_dense.cu", "src/gemm/int8_sparse.cu",
    "src/gemm/int8_gemm.cu", "src/gemm/int8_dp4a.cu",
    "src/nn/int8_conv2d.cu", "src/nn/int8_conv_transpose2d.cu",
]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_oracle(force=False):
    src = os.path.join(HERE, "forge_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c11",
                               src, "-o", ORACLE_SO, "-lm"])
    return ORACLE_SO


def reference_sources_present():
    return all(os.path.exists(os.path.join(REFERENCE_ROOT, s)) for s in REF_SOURCES)


def build_ref(force=False):
    """Returns the path of libforge_ref.so, or None when it is neither built nor buildable."""
    srcs = [os.path.join(REFERENCE_ROOT, s) for s in REF_SOURCES]
    if not reference_sources_present():
        return REF_SO if os.path.exists(REF_SO) else None
    shim = os.path.join(HERE, "ref_shim.cu")
    if force or _stale(REF_SO, srcs + [shim]):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        os.makedirs(REF_DIR, exist_ok=True)
        cmd = [nvcc, "-std=c++17", "-O3", "--use_fast_math", "--expt-relaxed-constexpr",
               "-gencode", "arch=compute_100a,code=sm_100a", "-Wno-deprecated-gpu-targets",
               "-Xcompiler", "-fPIC", "-shared", "-Xlinker", "-Bsymbolic",
               "-I" + os.path.join(REFERENCE_ROOT, "include"), "-I" + os.path.join(REFERENCE_ROOT, "src", "internal"),
               "-o", REF_SO] + srcs + [shim, "-lcudart"]
        subprocess.check_call(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
