"""ctypes access to the test oracles: oracle/liboracle.so (CPU restatement, numpy in/out) and
oracle/_ref/libforge_ref.so (the reference's own CUDA kernels built for sm_100a, torch CUDA
tensors in/out). Test infrastructure only."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
ORACLE_SO = os.path.join(ROOT, "oracle", "liboracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libforge_ref.so")

_vp, _i = ctypes.c_void_p, ctypes.c_int
_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import build as oracle_build  # noqa: E402
            oracle_build.build_oracle()
        lib = ctypes.CDLL(ORACLE_SO)
        lib.oracle_int8_gemm_s32.argtypes = [_vp, _vp, _vp, _i, _i, _i]
        lib.oracle_quantize.argtypes = [_vp, _vp, _vp, _i, _i]
        lib.oracle_dequantize_bias.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i]
        lib.oracle_dequantize_gemm_epilogue.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i]
        lib.oracle_gated_epilogue.argtypes = [_vp] * 8 + [_i, _i]
        lib.oracle_prune_compress_24.argtypes = [_vp, _vp, _vp, _i, _i]
        lib.oracle_prune_24_dense.argtypes = [_vp, _vp, _i, _i]
        lib.oracle_pack_metadata.argtypes = [_vp, _vp, _i, _i]
        lib.oracle_sparse_gemm_s32.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i]
        lib.oracle_float_to_half.argtypes = [ctypes.c_float]
        lib.oracle_float_to_half.restype = ctypes.c_uint16
        lib.oracle_half_to_float.argtypes = [ctypes.c_uint16]
        lib.oracle_half_to_float.restype = ctypes.c_float
        lib.oracle_im2col.argtypes = [_vp, _vp] + [_i] * 12
        lib.oracle_rows_to_nchw.argtypes = [_vp, _vp, _i, _i, _i]
        lib.oracle_int8_conv2d.argtypes = [_vp] * 5 + [_i] * 13
        lib.oracle_conv_transpose_k2s2_scatter.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i]
        lib.oracle_num_threads.restype = _i
        lib.oracle_set_num_threads.argtypes = [_i]
        _oracle = lib
    return _oracle


def _p(a):
    return None if a is None else a.ctypes.data


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def gemm_s32(A, B):
    A, B = _c(A, np.int8), _c(B, np.int8)
    M, K = A.shape
    N = B.shape[0]
    C = np.empty((M, N), np.int32)
    oracle().oracle_int8_gemm_s32(_p(A), _p(B), _p(C), M, K, N)
    return C


def quantize(x_f16):
    x = _c(x_f16, np.float16)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    oracle().oracle_quantize(_p(x), _p(q), _p(s), M, K)
    return q, s


def dequantize_bias(acc, act_scale, w_scale, bias, gemm_epilogue=False):
    acc, act_scale, w_scale = _c(acc, np.int32), _c(act_scale, np.float32), _c(w_scale, np.float16)
    bias = None if bias is None else _c(bias, np.float16)
    M, N = acc.shape
    out = np.empty((M, N), np.float16)
    fn = oracle().oracle_dequantize_gemm_epilogue if gemm_epilogue else oracle().oracle_dequantize_bias
    fn(_p(acc), _p(act_scale), _p(w_scale), _p(bias), _p(out), M, N)
    return out


def gated_epilogue(acc_g, acc_u, act_scale, wg_scale, wu_scale, bg, bu):
    acc_g, acc_u = _c(acc_g, np.int32), _c(acc_u, np.int32)
    act_scale, wg_scale, wu_scale = _c(act_scale, np.float32), _c(wg_scale, np.float16), _c(wu_scale, np.float16)
    bg = None if bg is None else _c(bg, np.float16)
    bu = None if bu is None else _c(bu, np.float16)
    M, N = acc_g.shape
    out = np.empty((M, N), np.float16)
    oracle().oracle_gated_epilogue(_p(acc_g), _p(acc_u), _p(act_scale), _p(wg_scale), _p(wu_scale), _p(bg), _p(bu),
                                   _p(out), M, N)
    return out


def half_ulp_distance(a, b):
    """Element-wise distance in fp16 units of least precision between two float16 arrays."""
    def ordered(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(ordered(np.ascontiguousarray(a)) - ordered(np.ascontiguousarray(b)))


def prune_compress_24(w):
    w = _c(w, np.int8)
    N, K = w.shape
    comp = np.empty((N, K // 2), np.int8)
    meta = np.empty((N * (K // 4),), np.uint8)
    oracle().oracle_prune_compress_24(_p(w), _p(comp), _p(meta), N, K)
    return comp, meta


def prune_24_dense(w):
    w = _c(w, np.int8)
    N, K = w.shape
    out = np.empty((N, K), np.int8)
    oracle().oracle_prune_24_dense(_p(w), _p(out), N, K)
    return out


def pack_metadata(meta_raw, N, K):
    meta_raw = _c(meta_raw, np.uint8)
    out = np.empty((N, K // 32), np.uint32)
    oracle().oracle_pack_metadata(_p(meta_raw), _p(out), N, K)
    return out


def sparse_gemm_s32(W_comp, x, w_meta):
    W_comp, x, w_meta = _c(W_comp, np.int8), _c(x, np.int8), _c(w_meta, np.uint32)
    M, K = x.shape
    N = W_comp.shape[0]
    out = np.empty((M, N), np.int32)
    oracle().oracle_sparse_gemm_s32(_p(W_comp), _p(x), _p(w_meta), _p(out), M, K, N)
    return out


def conv_out_size(size, pad, dil, k, stride):
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def im2col(x_f16, kH, kW, padH, padW, strideH, strideW, dilH, dilW):
    """(N,C,H,W) fp16 -> (N*H_out*W_out, C*kH*kW) fp16, the reference's patch-per-row layout."""
    x = _c(x_f16, np.float16)
    N, C, H, W = x.shape
    Ho, Wo = conv_out_size(H, padH, dilH, kH, strideH), conv_out_size(W, padW, dilW, kW, strideW)
    col = np.empty((N * Ho * Wo, C * kH * kW), np.float16)
    oracle().oracle_im2col(_p(x), _p(col), N, C, H, W, kH, kW, padH, padW, strideH, strideW, dilH, dilW)
    return col, Ho, Wo


def rows_to_nchw(g_f16, N, HW, C_out):
    g = _c(g_f16, np.float16)
    out = np.empty((N, C_out, HW), np.float16)
    oracle().oracle_rows_to_nchw(_p(g), _p(out), N, HW, C_out)
    return out


def int8_conv2d(x_f16, weight, w_scale, bias, kH, kW, padH, padW, strideH, strideW, dilH, dilW):
    x, weight, w_scale = _c(x_f16, np.float16), _c(weight, np.int8), _c(w_scale, np.float16)
    bias = None if bias is None else _c(bias, np.float16)
    N, C, H, W = x.shape
    C_out = weight.shape[0]
    Ho, Wo = conv_out_size(H, padH, dilH, kH, strideH), conv_out_size(W, padW, dilW, kW, strideW)
    out = np.empty((N, C_out, Ho, Wo), np.float16)
    oracle().oracle_int8_conv2d(_p(x), _p(weight), _p(w_scale), _p(bias), _p(out), N, C, H, W, C_out, kH, kW, padH,
                                padW, strideH, strideW, dilH, dilW)
    return out


def conv_transpose_k2s2_scatter(g_f16, bias, N, H, W, C_out):
    g = _c(g_f16, np.float16)
    bias = None if bias is None else _c(bias, np.float16)
    out = np.empty((N, C_out, 2 * H, 2 * W), np.float16)
    oracle().oracle_conv_transpose_k2s2_scatter(_p(g), _p(bias), _p(out), N, H, W, C_out)
    return out


# --------------------------------------------------------------------------------------------
# Reference GPU kernels (oracle/_ref). Arguments are torch CUDA tensors.

def ref_available():
    return os.path.exists(REF_SO)


def reference_sources_present():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build as oracle_build
    return oracle_build.reference_sources_present()


def require_ref():
    """Gate of every comparison against the reference's own kernels. Returns when
    oracle/_ref/libforge_ref.so is there. If it is missing although the reference sources are
    present, the test FAILS (the checker was not built: run `python oracle/build.py`); if the
    sources are absent too, the test is reported as skipped with the reason - never silently
    passed without the reference."""
    import pytest
    if ref_available():
        return True
    if reference_sources_present():
        pytest.fail("oracle/_ref/libforge_ref.so is not built although the reference sources are present; "
                    "run `python oracle/build.py`")
    pytest.skip("reference kernels unavailable: oracle/_ref/libforge_ref.so is not in this checkout and the "
                "reference sources are not here to build it (the checks against the CPU oracle above did run)")


def ref():
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(REF_SO)
        lib.ref_fused_quantize_activation.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        lib.ref_quantize_two_pass.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        lib.ref_fused_dequantize_bias.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp]
        lib.ref_int8_gemm_dequant.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        lib.ref_int8_linear.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]
        lib.ref_sparse_int8_gemm.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _i]
        lib.ref_sparse_int8_linear.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i]
        lib.ref_prune_compress_24.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        lib.ref_pack_metadata.argtypes = [_vp, _vp, _i, _i, _vp]
        lib.ref_int8_conv2d_workspace_size.argtypes = [_i] * 12
        lib.ref_int8_conv2d_workspace_size.restype = ctypes.c_ulonglong
        lib.ref_int8_conv2d_forward.argtypes = [_vp] * 5 + [_i] * 13 + [_vp, _vp]
        lib.ref_int8_conv2d_forward.restype = None
        lib.ref_int8_conv_transpose2d_k2s2_workspace_size.argtypes = [_i] * 4
        lib.ref_int8_conv_transpose2d_k2s2_workspace_size.restype = ctypes.c_ulonglong
        lib.ref_int8_conv_transpose2d_k2s2_forward.argtypes = [_vp] * 5 + [_i] * 5 + [_vp, _vp]
        lib.ref_int8_conv_transpose2d_k2s2_forward.restype = None
        lib.ref_splitk_reduce.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
        lib.ref_int8_gemm.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        lib.ref_int8_dp4a_gemm_dequant.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
        lib.ref_int8_dp4a_linear.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]
        lib.ref_get_compute_capability.argtypes = [_i]
        lib.ref_has_wmma_int8.argtypes = [_i]
        for name in ("ref_splitk_reduce", "ref_int8_gemm", "ref_int8_dp4a_gemm_dequant", "ref_int8_dp4a_linear"):
            getattr(lib, name).restype = None
        for name in ("ref_fused_quantize_activation", "ref_quantize_two_pass", "ref_fused_dequantize_bias",
                     "ref_int8_gemm_dequant", "ref_int8_linear", "ref_sparse_int8_gemm", "ref_sparse_int8_linear",
                     "ref_prune_compress_24", "ref_pack_metadata"):
            getattr(lib, name).restype = None
        _ref = lib
    return _ref


def tp(t):
    return 0 if t is None else t.data_ptr()


def cur_stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def ref_quantize(x, two_pass=False):
    import torch
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    fn = ref().ref_quantize_two_pass if two_pass else ref().ref_fused_quantize_activation
    fn(tp(x), tp(q), tp(s), M, K, cur_stream())
    return q, s


def ref_dequantize_bias(acc, act_scale, w_scale, bias):
    import torch
    M, N = acc.shape
    out = torch.empty((M, N), dtype=torch.float16, device=acc.device)
    ref().ref_fused_dequantize_bias(tp(acc), tp(act_scale), tp(w_scale), tp(bias), tp(out), M, N, cur_stream())
    return out


def ref_int8_gemm_dequant(A, B, act_scale, w_scale, bias):
    import torch
    M, K = A.shape
    N = B.shape[0]
    out = torch.empty((M, N), dtype=torch.float16, device=A.device)
    ref().ref_int8_gemm_dequant(tp(A), tp(B), tp(act_scale), tp(w_scale), tp(bias), tp(out), M, K, N, cur_stream())
    return out


def ref_sparse_int8_gemm(W_comp, x, w_meta, act_scale, w_scale, bias, tile=-1):
    import torch
    M, K = x.shape
    N = W_comp.shape[0]
    out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    ref().ref_sparse_int8_gemm(tp(W_comp), tp(x), tp(w_meta), tp(act_scale), tp(w_scale), tp(bias), tp(out), M, K, N,
                               0, 1, cur_stream(), tile)
    return out


def ref_prune_pack(w):
    import torch
    N, K = w.shape
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=w.device)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=w.device)
    packed = torch.empty((N, K // 32), dtype=torch.int32, device=w.device)
    ref().ref_prune_compress_24(tp(w), tp(comp), tp(raw), N, K, cur_stream())
    ref().ref_pack_metadata(tp(raw), tp(packed), N, K, cur_stream())
    return comp, raw, packed


def ref_int8_conv2d(x, weight, w_scale, bias, kH, kW, padH, padW, strideH, strideW, dilH, dilW):
    import torch
    N, C, H, W = x.shape
    C_out = weight.shape[0]
    Ho, Wo = conv_out_size(H, padH, dilH, kH, strideH), conv_out_size(W, padW, dilW, kW, strideW)
    out = torch.empty((N, C_out, Ho, Wo), dtype=torch.float16, device=x.device)
    ws = torch.empty(int(ref().ref_int8_conv2d_workspace_size(C, H, W, C_out, kH, kW, padH, padW, strideH, strideW,
                                                              dilH, dilW)) + 16, dtype=torch.uint8, device=x.device)
    ref().ref_int8_conv2d_forward(tp(x), tp(weight), tp(w_scale), tp(bias), tp(out), N, C, H, W, C_out, kH, kW, padH,
                                  padW, strideH, strideW, dilH, dilW, tp(ws), cur_stream())
    torch.cuda.synchronize()
    return out


def ref_int8_conv_transpose2d_k2s2(x, weight, w_scale, bias):
    import torch
    N, C, H, W = x.shape
    C_out = weight.shape[0] // 4
    out = torch.empty((N, C_out, 2 * H, 2 * W), dtype=torch.float16, device=x.device)
    ws = torch.empty(int(ref().ref_int8_conv_transpose2d_k2s2_workspace_size(C, H, W, C_out)) + 16, dtype=torch.uint8,
                     device=x.device)
    ref().ref_int8_conv_transpose2d_k2s2_forward(tp(x), tp(weight), tp(w_scale), tp(bias), tp(out), N, C, H, W, C_out,
                                                 tp(ws), cur_stream())
    torch.cuda.synchronize()
    return out
