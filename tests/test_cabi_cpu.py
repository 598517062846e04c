"""CPU-only checks of the boundary: libforge_b200.so loads and exports every symbol that
include/forge_b200.h declares; host-only entry points behave; no compute call is made."""
import ctypes
import os
import re

from forge_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "forge_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(forge_[a-z0-9_]+)\s*\(", text)))


def test_header_and_library_agree():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in forge_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table out of sync with the header"


def test_status_strings():
    lib = _lib.load()
    assert lib.forge_b200_status_string(0) == b"ok"
    assert b"sm_100" in lib.forge_b200_status_string(3)


def test_sparse_plan_host_logic():
    lib = _lib.load()
    t, s = ctypes.c_int(-9), ctypes.c_int(-9)
    assert lib.forge_sparse_int8_gemm_plan(4096, 4096, 11008, 0, 1, 7, ctypes.byref(t), ctypes.byref(s)) == 0
    assert 0 <= t.value < 3 and s.value == 1      # tile >= 3 means automatic (int8_sparse.cu:895)
    assert lib.forge_sparse_int8_gemm_plan(1, 64, 16, 6, 1, 2, ctypes.byref(t), ctypes.byref(s)) == 0
    assert t.value == 2
    assert lib.forge_sparse_int8_linear_fused(147456, 1280, 320) in (0, 1)


def test_public_kernel_symbols_are_exported():
    """The four kernels the reference headers declare keep their C++ names (mangled)."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    for frag in ("fused_quantize_activation_kernel", "fused_dequantize_bias_kernel", "prune_compress_kernel",
                 "pack_metadata_kernel"):
        assert frag in out


def test_cxx_face_compiles_and_links(tmp_path):
    """Reference-style C++ (namespaces, defaults, public kernels launched with <<<>>>) builds
    against include/forge/... and links against libforge_b200.so."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path / "dropin")
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cxx_dropin_check.cu"), "-o", exe, "-L" + os.path.dirname(_lib.LIB_PATH),
           "-lforge_b200", "-Xlinker", "-rpath=" + os.path.dirname(_lib.LIB_PATH)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([exe]).returncode == 0
