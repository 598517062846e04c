"""Python-level mirror of the reference's `forge._forge_C` extension functions for the
quantized-inference path (reference python/forge/csrc/bindings.cpp:446-575): same names,
argument lists and return values, taking torch CUDA tensors and running on torch's current
stream. Each function forwards to the C ABI of libforge_b200.so through ctypes.
"""
import contextlib

import torch

from . import _lib

_NULL = contextlib.nullcontext()


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _on(t):
    """Context in which `t`'s GPU is the current device: the library launches on the current
    device and keys its per-device state (SM count, status word, kernel attributes) on it."""
    if t.device.index == torch.cuda.current_device():
        return _NULL
    return torch.cuda.device(t.device)


def _chk(first, **named):
    """Every tensor argument must be a contiguous CUDA tensor of the stated dtype on `first`'s device
    (None is allowed for optional ones). The C ABI takes raw pointers, so a wrong dtype or a strided
    view would be reinterpreted silently; the reference binding's typed data_ptr<T>() raises instead."""
    if not first.is_cuda:
        raise ValueError("forge_b200 runs on CUDA tensors only (there is no CPU path)")
    for name, (t, dtype) in named.items():
        if t is None:
            continue
        if t.dtype != dtype:
            raise TypeError(f"{name}: expected {dtype}, got {t.dtype}")
        if t.device != first.device:
            raise ValueError(f"{name}: on {t.device}, expected {first.device}")
        if not t.is_contiguous():
            raise ValueError(f"{name}: must be contiguous")


_f16, _f32, _i8, _i32, _u8 = torch.float16, torch.float32, torch.int8, torch.int32, torch.uint8


def fused_quantize_activation(input, M, K):
    """bindings.cpp:448-459 -> (int8 (M,K), float32 (M,))."""
    _chk(input, input=(input, _f16))
    output = torch.empty((M, K), dtype=torch.int8, device=input.device)
    scales = torch.empty((M,), dtype=torch.float32, device=input.device)
    with _on(input):
        _lib.call("forge_fused_quantize_activation", _ptr(input), _ptr(output), _ptr(scales), M, K, _stream())
    return output, scales


def fused_dequantize_bias(input, act_scale, w_scale, bias, M, N):
    """bindings.cpp:461-476 -> float16 (M,N)."""
    _chk(input, input=(input, _i32), act_scale=(act_scale, _f32), w_scale=(w_scale, _f16), bias=(bias, _f16))
    output = torch.empty((M, N), dtype=torch.float16, device=act_scale.device)
    with _on(input):
        _lib.call("forge_fused_dequantize_bias", _ptr(input), _ptr(act_scale), _ptr(w_scale), _ptr(bias),
                  _ptr(output), M, N, _stream())
    return output


def int8_linear(x, w_int8, w_scale, bias, scratch_a_int8, scratch_a_scale):
    """bindings.cpp:498-519 -> float16 (M,N)."""
    _chk(x, x=(x, _f16), w_int8=(w_int8, _i8), w_scale=(w_scale, _f16), bias=(bias, _f16),
         scratch_a_int8=(scratch_a_int8, _i8), scratch_a_scale=(scratch_a_scale, _f32))
    M, K, N = x.size(0), x.size(1), w_int8.size(0)
    output = torch.empty((M, N), dtype=x.dtype, device=x.device)
    with _on(x):
        _lib.call("forge_int8_linear", _ptr(x), _ptr(w_int8), _ptr(w_scale), _ptr(bias), _ptr(output), M, K, N,
                  _ptr(scratch_a_int8), _ptr(scratch_a_scale), _stream())
    return output


def sparse_int8_linear(x, W_comp, w_meta, w_scale, bias, scratch_x_int8, scratch_x_scale, splitk_workspace=None,
                       split_k=1, path=-1):
    """bindings.cpp:521-554 -> float16 (M,N_out). The workspace is accepted for compatibility;
    this implementation never splits K, so none is allocated."""
    _chk(x, x=(x, _f16), W_comp=(W_comp, _i8), w_meta=(w_meta, _i32), w_scale=(w_scale, _f16), bias=(bias, _f16),
         scratch_x_int8=(scratch_x_int8, _i8), scratch_x_scale=(scratch_x_scale, _f32),
         splitk_workspace=(splitk_workspace, _f32))
    M, K, N_out = x.size(0), x.size(1), W_comp.size(0)
    output = torch.empty((M, N_out), dtype=x.dtype, device=x.device)
    with _on(x):
        _lib.call("forge_sparse_int8_linear", _ptr(x), _ptr(W_comp), _ptr(w_meta), _ptr(w_scale), _ptr(bias),
                  _ptr(output), M, K, N_out, _ptr(scratch_x_int8), _ptr(scratch_x_scale), _ptr(splitk_workspace),
                  split_k, _stream(), path)
    return output


def prune_compress_24(weight, compressed, metadata_raw, N, K):
    """bindings.cpp:558-566."""
    _chk(weight, weight=(weight, _i8), compressed=(compressed, _i8), metadata_raw=(metadata_raw, _u8))
    with _on(weight):
        _lib.call("forge_prune_compress_24", _ptr(weight), _ptr(compressed), _ptr(metadata_raw), N, K, _stream())


def pack_metadata(meta_raw, meta_packed, N, K):
    """bindings.cpp:568-575."""
    _chk(meta_raw, meta_raw=(meta_raw, _u8), meta_packed=(meta_packed, _i32))
    with _on(meta_raw):
        _lib.call("forge_pack_metadata", _ptr(meta_raw), _ptr(meta_packed), N, K, _stream())


# ---- additive entry points (no counterpart in the reference extension) ----

def int8_gemm_dequant(A, B, act_scale, w_scale, bias=None):
    M, K, N = A.size(0), A.size(1), B.size(0)
    _chk(A, A=(A, _i8), B=(B, _i8), act_scale=(act_scale, _f32), w_scale=(w_scale, _f16), bias=(bias, _f16))
    output = torch.empty((M, N), dtype=torch.float16, device=A.device)
    with _on(A):
        _lib.call("forge_int8_gemm_dequant", _ptr(A), _ptr(B), _ptr(act_scale), _ptr(w_scale), _ptr(bias),
                  _ptr(output), M, K, N, _stream())
    return output


def int8_gemm_s32(A, B):
    M, K, N = A.size(0), A.size(1), B.size(0)
    _chk(A, A=(A, _i8), B=(B, _i8))
    output = torch.empty((M, N), dtype=torch.int32, device=A.device)
    with _on(A):
        _lib.call("forge_int8_gemm_s32", _ptr(A), _ptr(B), _ptr(output), M, K, N, _stream())
    return output


def sparse_int8_gemm(W_comp, x_int8, w_meta, act_scale, w_scale, bias=None, tile=-1):
    M, K, N_out = x_int8.size(0), x_int8.size(1), W_comp.size(0)
    _chk(x_int8, W_comp=(W_comp, _i8), x_int8=(x_int8, _i8), w_meta=(w_meta, _i32), act_scale=(act_scale, _f32),
         w_scale=(w_scale, _f16), bias=(bias, _f16))
    output = torch.empty((M, N_out), dtype=torch.float16, device=x_int8.device)
    with _on(x_int8):
        _lib.call("forge_sparse_int8_gemm", _ptr(W_comp), _ptr(x_int8), _ptr(w_meta), _ptr(act_scale), _ptr(w_scale),
                  _ptr(bias), _ptr(output), M, K, N_out, 0, 1, _stream(), tile)
    return output


def sparse_int8_gemm_s32(W_comp, x_int8, w_meta):
    M, K, N_out = x_int8.size(0), x_int8.size(1), W_comp.size(0)
    _chk(x_int8, W_comp=(W_comp, _i8), x_int8=(x_int8, _i8), w_meta=(w_meta, _i32))
    output = torch.empty((M, N_out), dtype=torch.int32, device=x_int8.device)
    with _on(x_int8):
        _lib.call("forge_sparse_int8_gemm_s32", _ptr(W_comp), _ptr(x_int8), _ptr(w_meta), _ptr(output), M, K, N_out,
                  _stream())
    return output


def prepare_weight(weight, sparse):
    """Float weight (N, K), fp32 or fp16, on a GPU -> (w_int8 or None, W_comp or None, w_meta or None,
    w_scale fp16) in one kernel: per-channel quantisation and, with sparse=True, 2:4 prune +
    compress + metadata pack."""
    if weight.dtype not in (torch.float32, torch.float16):
        weight = weight.to(torch.float32)
    weight = weight.contiguous()
    N, K = weight.shape
    dev = weight.device
    w_scale = torch.empty((N,), dtype=torch.float16, device=dev)
    w_int8 = None if sparse else torch.empty((N, K), dtype=torch.int8, device=dev)
    W_comp = torch.empty((N, K // 2), dtype=torch.int8, device=dev) if sparse else None
    w_meta = torch.empty((N, K // 32), dtype=torch.int32, device=dev) if sparse else None
    with _on(weight):
        _lib.call("forge_prepare_weight", _ptr(weight), 1 if weight.dtype == torch.float16 else 0, _ptr(w_int8),
                  _ptr(W_comp), _ptr(w_meta), _ptr(w_scale), N, K, _stream())
    return w_int8, W_comp, w_meta, w_scale


def int8_conv2d_forward(input, weight, w_scale, bias, kernel_size, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    """INT8 conv2d (forge::nn::int8_conv2d_forward; the reference has no Python binding for it): input
    (N,C_in,H,W) fp16, weight (C_out, C_in*kH*kW) int8, w_scale / bias (C_out) fp16 -> (N,C_out,H_out,W_out)
    fp16, each output position's patch quantized per row."""
    N, C_in, H, W = input.shape
    C_out = weight.shape[0]
    (kH, kW), (pH, pW), (sH, sW), (dH, dW) = kernel_size, padding, stride, dilation
    Ho = (H + 2 * pH - dH * (kH - 1) - 1) // sH + 1
    Wo = (W + 2 * pW - dW * (kW - 1) - 1) // sW + 1
    out = torch.empty((N, C_out, Ho, Wo), dtype=torch.float16, device=input.device)
    _chk(input, input=(input, _f16), weight=(weight, _i8), w_scale=(w_scale, _f16), bias=(bias, _f16))
    with _on(input):
        _lib.call("forge_int8_conv2d_forward", _ptr(input), _ptr(weight), _ptr(w_scale), _ptr(bias), _ptr(out), N, C_in,
                  H, W, C_out, kH, kW, pH, pW, sH, sW, dH, dW, None, _stream())
    return out


def int8_conv_transpose2d_k2s2_forward(input, weight, w_scale, bias):
    """2x2 stride-2 INT8 transposed conv (forge::nn::int8_conv_transpose2d_k2s2_forward): weight
    (4*C_out, C_in) int8 with row co*4 + kh*2 + kw -> (N,C_out,2H,2W) fp16."""
    N, C_in, H, W = input.shape
    C_out = weight.shape[0] // 4
    out = torch.empty((N, C_out, 2 * H, 2 * W), dtype=torch.float16, device=input.device)
    _chk(input, input=(input, _f16), weight=(weight, _i8), w_scale=(w_scale, _f16), bias=(bias, _f16))
    with _on(input):
        _lib.call("forge_int8_conv_transpose2d_k2s2_forward", _ptr(input), _ptr(weight), _ptr(w_scale), _ptr(bias),
                  _ptr(out), N, C_in, H, W, C_out, None, _stream())
    return out


def device_status(reset=True):
    """FORGE_B200_OK (0) unless a kernel on the current device gave up on a bounded wait since the last
    reset (then FORGE_B200_DEVICE_TIMEOUT, 5); `device_status_raw` returns the recorded code."""
    return _lib.load().forge_b200_device_status(1 if reset else 0)


def device_status_raw(reset=True):
    return _lib.load().forge_b200_device_status_raw(1 if reset else 0)
