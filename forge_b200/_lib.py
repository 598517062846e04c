"""ctypes binding of libforge_b200.so - the C ABI declared in include/forge_b200.h.

There is no fallback: if the shared library is missing, or a call returns a non-zero
status, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libforge_b200.so")

_vp = ctypes.c_void_p
_i = ctypes.c_int
_ip = ctypes.POINTER(ctypes.c_int)

# name -> argtypes; every function returns int except where noted below
SIGNATURES = {
    "forge_fused_quantize_activation": [_vp, _vp, _vp, _i, _i, _vp],
    "forge_fused_dequantize_bias": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "forge_int8_gemm_dequant": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_int8_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_int8_dp4a_gemm_dequant": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_int8_linear": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp],
    "forge_int8_dp4a_linear": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp],
    "forge_int8_linear_static": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_get_compute_capability": [_i],
    "forge_has_wmma_int8": [_i],
    "forge_int8_gemm_s32": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_sparse_int8_gemm_plan": [_i, _i, _i, _i, _i, _i, _ip, _ip],
    "forge_sparse_int8_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _i],
    "forge_sparse_int8_linear_fused": [_i, _i, _i],
    "forge_sparse_int8_linear": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i],
    "forge_splitk_reduce": [_vp, _vp, _vp, _i, _i, _vp],
    "forge_sparse_int8_gemm_s32": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_sparse_int8_gemm_multi": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, ctypes.c_longlong, _i, _i, _i, _vp],
    "forge_int8_gated_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_sparse_int8_gated_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "forge_w8a8_gated_mlp_workspace_bytes": [_i, _i, _i],
    "forge_w8a8_gated_mlp": [_vp] * 11 + [_i, _i, _i, _vp, _vp],
    "forge_sparse_w8a8_gated_mlp": [_vp] * 14 + [_i, _i, _i, _vp, _vp],
    "forge_prune_compress_24": [_vp, _vp, _vp, _i, _i, _vp],
    "forge_pack_metadata": [_vp, _vp, _i, _i, _vp],
    "forge_prepare_weight": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "forge_int8_conv2d_workspace_size": [_i] * 12,
    "forge_int8_conv2d_forward": [_vp] * 5 + [_i] * 13 + [_vp, _vp],
    "forge_int8_conv_transpose2d_k2s2_workspace_size": [_i] * 4,
    "forge_int8_conv_transpose2d_k2s2_forward": [_vp] * 5 + [_i] * 5 + [_vp, _vp],
    "forge_b200_device_status": [_i],
    "forge_b200_device_status_raw": [_i],
    "forge_b200_status_string": [_i],
}
# exported test / tuning hooks that are not part of the public header (csrc/tuning.h)
INTERNAL_SIGNATURES = {
    "forge_b200_set_dense_tile": [_i],
    "forge_b200_set_sparse_tile": [_i],
    "forge_b200_set_tuning": [_i, _i],
    "forge_b200_get_tuning": [_i],
    "forge_b200_selftest_wait_timeout": [ctypes.c_uint, _vp],
    "forge_b200_read_probe": [_vp, _i],
    "forge_b200_probe_mma_rate": [_i, _i, _i, _i, _i],
    "forge_b200_probe_tma_ingest": [_vp, _i, _i, _i, _i],
}
_VOID_RETURN = {"forge_b200_set_dense_tile", "forge_b200_set_sparse_tile", "forge_b200_set_tuning"}

_lib = None


class ForgeError(RuntimeError):
    """A libforge_b200 entry point returned a non-zero status."""


def load():
    """Loads libforge_b200.so (once) and declares every signature. Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m forge_b200.build` (needs nvcc). "
            "forge_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in list(SIGNATURES.items()) + list(INTERNAL_SIGNATURES.items()):
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        if name in _VOID_RETURN:
            fn.restype = None
        elif name == "forge_b200_status_string":
            fn.restype = ctypes.c_char_p
        elif name.startswith("forge_b200_probe_"):
            fn.restype = ctypes.c_double
        elif name in ("forge_w8a8_gated_mlp_workspace_bytes", "forge_int8_conv2d_workspace_size",
                      "forge_int8_conv_transpose2d_k2s2_workspace_size"):
            fn.restype = ctypes.c_ulonglong
        else:
            fn.restype = ctypes.c_int
    _lib = lib
    return lib


def check(status, what):
    if status != 0:
        msg = load().forge_b200_status_string(status).decode()
        raise ForgeError(f"{what} failed: status {status} ({msg})")


def call(name, *args):
    """Calls an int-returning entry point and raises ForgeError on a non-zero status."""
    check(getattr(load(), name)(*args), name)
