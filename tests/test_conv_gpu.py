"""GPU parity of the fused INT8 convolution kernels, called through the C ABI.

Mirrors the reference's tests/test_int8_conv2d.cu (its six conv cases) and the transposed-conv
cases of tests/test_int8_special_conv.cu:282-284, with the tolerance tightened from the
reference's absolute 0.5 against a float conv to BIT EQUALITY against
  (1) the reference's own conv pipeline run on the same GPU (oracle/_ref), and
  (2) the composition the reference defines: CPU im2col (patch per row) -> per-row quantize (the
      quantizer kernel, itself bit-pinned to the reference's) -> exact s32 GEMM on the CPU ->
      GEMM-epilogue dequant + bias -> transpose to NCHW (or the 2x2 scatter with its second
      rounding)."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(N, C_in, H, W, rows, K, use_bias, seed, lo=-1.0, hi=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand((N, C_in, H, W), generator=g) * (hi - lo) + lo).to(torch.float16)
    w = torch.randint(-127, 128, (rows, K), generator=g, dtype=torch.int8)
    return x, w, g


def _scales(C_out, use_bias, g):
    w_scale = (torch.rand(C_out, generator=g) * 0.045 + 0.005).to(torch.float16)
    bias = (torch.rand(C_out, generator=g) - 0.5).to(torch.float16) if use_bias else None
    return w_scale, bias


def _ref_workspace_aligned(M, K):
    """The reference carves its workspace as [fp16 M*K | int8 M*K | fp32 M | ...] without padding
    (src/nn/int8_conv2d.cu:172-176), so its fp32 scales are only 4-byte aligned when M*K is a multiple
    of 4; it is not run on other shapes."""
    return (M * K) % 4 == 0


def _composed_conv(x, w, w_scale, bias, k, p, s, d):
    """(2) above; x, w, w_scale, bias are CPU tensors."""
    N, C_in = x.shape[:2]
    col, Ho, Wo = O.im2col(x.numpy(), k[0], k[1], p[0], p[1], s[0], s[1], d[0], d[1])
    M, K = col.shape
    q, a = C.fused_quantize_activation(torch.from_numpy(col).to(DEV), M, K)
    acc = O.gemm_s32(q.cpu().numpy(), w.numpy())
    gem = O.dequantize_bias(acc, a.cpu().numpy(), w_scale.numpy(), None if bias is None else bias.numpy(),
                            gemm_epilogue=True)
    return O.rows_to_nchw(gem, N, Ho * Wo, w.shape[0]).reshape(N, w.shape[0], Ho, Wo)


def _check_conv(N, C_in, H, W, C_out, k, p, s, d, use_bias, seed=42, weight_offset=0):
    K = C_in * k[0] * k[1]
    x, w, g = _inputs(N, C_in, H, W, C_out, K, use_bias, seed)
    w_scale, bias = _scales(C_out, use_bias, g)
    xd, sd = x.to(DEV), w_scale.to(DEV)
    bd = None if bias is None else bias.to(DEV)
    wbuf = torch.zeros(C_out * K + weight_offset, dtype=torch.int8, device=DEV)
    wbuf[weight_offset:] = w.reshape(-1).to(DEV)
    wd = wbuf[weight_offset:].view(C_out, K)
    out = C.int8_conv2d_forward(xd, wd, sd, bd, k, p, s, d)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    expect = _composed_conv(x, w, w_scale, bias, k, p, s, d)
    got = out.cpu().numpy()
    assert got.shape == expect.shape
    assert np.array_equal(got.view(np.uint16), expect.view(np.uint16)), \
        f"conv differs from the composed pipeline: {np.count_nonzero(got.view(np.uint16) != expect.view(np.uint16))}"
    if _ref_workspace_aligned(expect.shape[2] * expect.shape[3], K) and O.require_ref():
        # .clone(): the reference's 16-byte weight loads need an aligned matrix
        ref = O.ref_int8_conv2d(xd, wd.clone(), sd, bd, k[0], k[1], p[0], p[1], s[0], s[1], d[0], d[1])
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), "conv differs from the reference pipeline"
    return out


# tests/test_int8_conv2d.cu:206-257: (C_in, H, W, C_out, kernel, pad, stride, dilation, bias)
REFERENCE_CASES = [
    (8, 16, 16, 16, (3, 3), (1, 1), (1, 1), (1, 1), True),
    (16, 8, 8, 32, (1, 1), (0, 0), (1, 1), (1, 1), True),
    (7, 32, 32, 16, (2, 2), (0, 0), (2, 2), (1, 1), True),
    (4, 12, 12, 8, (3, 3), (1, 1), (1, 1), (1, 1), False),
    (16, 64, 64, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),
    (8, 16, 16, 8, (3, 3), (2, 2), (1, 1), (2, 2), True),
]


@pytest.mark.parametrize("C_in,H,W,C_out,k,p,s,d,use_bias", REFERENCE_CASES)
def test_conv2d_reference_cases(C_in, H, W, C_out, k, p, s, d, use_bias):
    _check_conv(1, C_in, H, W, C_out, k, p, s, d, use_bias)


@pytest.mark.parametrize("N,C_in,H,W,C_out,k,p,s,d,use_bias", [
    (3, 16, 15, 13, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),      # 195 positions per sample: tiles straddle samples
    (2, 64, 48, 40, 64, (3, 3), (1, 1), (1, 1), (1, 1), True),      # K = 576: five 128-tap slabs, ring wraps
    (2, 32, 20, 20, 320, (1, 1), (0, 0), (1, 1), (1, 1), True),     # C_out > 256: two column blocks of 160
    (1, 5, 9, 31, 3, (3, 2), (2, 0), (2, 3), (1, 2), False),        # odd everything, K = 30, C_out = 3
    (2, 3, 33, 17, 24, (5, 5), (2, 2), (1, 1), (1, 1), True),       # K = 75: weights loaded without TMA
    (1, 128, 12, 12, 48, (3, 3), (0, 0), (1, 1), (1, 1), True),     # K = 1152, no padding
    (4, 16, 7, 7, 16, (7, 7), (3, 3), (1, 1), (1, 1), True),        # kernel as large as the image
    (1, 1, 1, 1, 1, (1, 1), (0, 0), (1, 1), (1, 1), True),          # one position, one tap
    (2, 19, 21, 23, 16, (3, 3), (1, 1), (2, 2), (1, 1), True),      # C_in % 4 = 3: leftover-channel path, stride 2
    (2, 6, 30, 30, 16, (2, 2), (0, 0), (2, 2), (1, 1), False),      # 2x2 taps, C_in % 4 = 2
    (1, 130, 9, 9, 40, (1, 1), (0, 0), (1, 1), (1, 1), True),       # pointwise, K = 130: a 2-tap second stage
    (1, 57, 16, 16, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),      # K = 513: a 1-tap fifth stage
    # image widths that are multiples of 8 take the input-window (TMA) variant
    (3, 16, 21, 40, 32, (3, 3), (1, 1), (1, 1), (1, 1), True),      # ragged block rows, three samples
    (2, 12, 30, 48, 16, (3, 3), (2, 2), (1, 1), (2, 2), True),      # dilation 2, pad 2: window starts 2 columns left
    (2, 8, 33, 64, 24, (3, 3), (1, 1), (2, 2), (1, 1), False),      # stride 2
    (1, 128, 20, 24, 64, (3, 3), (1, 1), (1, 1), (1, 1), True),     # 128 channels: a 73 KB window, W_out < 32
    (1, 32, 9, 8, 16, (3, 3), (3, 3), (1, 1), (1, 1), True),        # pad 3 > kernel reach, 8-wide blocks
    (2, 20, 64, 72, 48, (1, 1), (0, 0), (1, 1), (1, 1), True),      # pointwise through the window variant
    (1, 16, 24, 32, 16, (2, 2), (0, 0), (2, 2), (1, 1), True),      # 2x2 stride 2
    (1, 16, 16, 16, 16, (3, 3), (9, 9), (1, 1), (1, 1), True),      # pad 9: xoff = 7, blocks fully outside the image
])
def test_conv2d_batches_and_shapes(N, C_in, H, W, C_out, k, p, s, d, use_bias):
    _check_conv(N, C_in, H, W, C_out, k, p, s, d, use_bias, seed=7 + C_in + C_out)


def test_conv2d_unaligned_weight_pointer():
    # K % 16 == 0 but the weight matrix starts at an odd address: the plain-load weight path
    _check_conv(1, 16, 10, 10, 16, (1, 1), (0, 0), (1, 1), (1, 1), True, weight_offset=3)


def test_conv2d_zero_image_and_outliers():
    N, C_in, H, W, C_out = 2, 8, 16, 16, 16
    g = torch.Generator().manual_seed(11)
    x = torch.randn((N, C_in, H, W), generator=g)
    x[0] = 0                      # all-zero patches: scale floor 1e-8 / 127
    x[1, 3, 5, 5] = 60000.0       # one huge pixel dominates the patches that contain it
    x = x.to(torch.float16)
    w = torch.randint(-127, 128, (C_out, C_in * 9), generator=g, dtype=torch.int8)
    w_scale, bias = _scales(C_out, True, g)
    out = C.int8_conv2d_forward(x.to(DEV), w.to(DEV), w_scale.to(DEV), bias.to(DEV), (3, 3), (1, 1))
    expect = _composed_conv(x, w, w_scale, bias, (3, 3), (1, 1), (1, 1), (1, 1))
    assert np.array_equal(out.cpu().numpy().view(np.uint16), expect.view(np.uint16))
    # a zero image gives exactly the bias
    assert torch.equal(out[0].cpu(), bias.view(C_out, 1, 1).expand(C_out, H, W))


def test_conv2d_non_finite_pixels_follow_the_quantizer():
    """Infinities and NaNs go through the same value step as the standalone quantizer (saturate, NaN -> 0):
    checked against the composed pipeline, which runs that quantizer."""
    N, C_in, H, W, C_out = 1, 8, 12, 12, 16
    g = torch.Generator().manual_seed(21)
    x = torch.randn((N, C_in, H, W), generator=g).to(torch.float16)
    x[0, 1, 2, 2] = float("inf")
    x[0, 2, 8, 8] = float("-inf")
    x[0, 5, 5, 10] = float("nan")
    w = torch.randint(-127, 128, (C_out, C_in * 9), generator=g, dtype=torch.int8)
    w_scale, bias = _scales(C_out, True, g)
    out = C.int8_conv2d_forward(x.to(DEV), w.to(DEV), w_scale.to(DEV), bias.to(DEV), (3, 3), (1, 1))
    expect = _composed_conv(x, w, w_scale, bias, (3, 3), (1, 1), (1, 1), (1, 1))
    got = out.cpu().numpy()
    # NaN outputs (0 * inf scale) carry different payloads on the CPU and the GPU; everything else bit-exact
    both_nan = np.isnan(got) & np.isnan(expect)
    assert both_nan.any() and not both_nan.all()
    assert np.array_equal(got.view(np.uint16)[~both_nan], expect.view(np.uint16)[~both_nan])
    if O.require_ref():
        ref = O.ref_int8_conv2d(x.to(DEV), w.to(DEV), w_scale.to(DEV), bias.to(DEV), 3, 3, 1, 1, 1, 1, 1, 1)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


def test_conv2d_output_fully_overwritten_and_repeatable():
    xs = (2, 16, 24, 24)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(xs, generator=g).to(torch.float16).to(DEV)
    w = torch.randint(-127, 128, (32, 16 * 9), generator=g, dtype=torch.int8).to(DEV)
    w_scale, bias = _scales(32, True, g)
    a = C.int8_conv2d_forward(x, w, w_scale.to(DEV), bias.to(DEV), (3, 3), (1, 1))
    b = C.int8_conv2d_forward(x, w, w_scale.to(DEV), bias.to(DEV), (3, 3), (1, 1))
    assert torch.equal(a, b)


def test_conv2d_empty_batch_is_a_no_op():
    from forge_b200 import _lib
    assert _lib.load().forge_int8_conv2d_forward(0, 0, 0, 0, 0, 0, 8, 4, 4, 8, 3, 3, 1, 1, 1, 1, 1, 1, 0, 0) == 0


def test_workspace_sizes_match_reference_formulas():
    from forge_b200 import _lib
    lib = _lib.load()
    # src/nn/int8_conv2d.cu:126-145 and src/nn/int8_conv_transpose2d.cu:103-117
    M, K, Co = 16 * 16, 8 * 9, 16
    assert lib.forge_int8_conv2d_workspace_size(8, 16, 16, Co, 3, 3, 1, 1, 1, 1, 1, 1) == M * K * 3 + M * 4 + M * Co * 2
    assert lib.forge_int8_conv_transpose2d_k2s2_workspace_size(32, 16, 16, 64) == \
        256 * 32 * 3 + 256 * 4 + 256 * 2 + 256 * 256 * 2
    if O.require_ref():
        assert lib.forge_int8_conv2d_workspace_size(7, 32, 32, 16, 2, 2, 0, 0, 2, 2, 1, 1) == \
            O.ref().ref_int8_conv2d_workspace_size(7, 32, 32, 16, 2, 2, 0, 0, 2, 2, 1, 1)


# ---------------------------------------------------------------- 2x2 stride-2 transposed conv

def _check_conv_transpose(N, C_in, H, W, C_out, use_bias, seed=42):
    x, w, g = _inputs(N, C_in, H, W, 4 * C_out, C_in, use_bias, seed)
    w_scale, bias = _scales(C_out, use_bias, g)
    xd, wd, sd = x.to(DEV), w.to(DEV), w_scale.to(DEV)
    bd = None if bias is None else bias.to(DEV)
    out = C.int8_conv_transpose2d_k2s2_forward(xd, wd, sd, bd)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    # composition: NHWC rows -> quantize -> GEMM with the channel scale repeated 4x, no bias -> scatter + bias
    col, _, _ = O.im2col(x.numpy(), 1, 1, 0, 0, 1, 1, 1, 1)
    q, a = C.fused_quantize_activation(torch.from_numpy(col).to(DEV), col.shape[0], C_in)
    acc = O.gemm_s32(q.cpu().numpy(), w.numpy())
    gem = O.dequantize_bias(acc, a.cpu().numpy(), np.repeat(w_scale.numpy(), 4), None, gemm_epilogue=True)
    expect = O.conv_transpose_k2s2_scatter(gem, None if bias is None else bias.numpy(), N, H, W, C_out)
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), expect.view(np.uint16))
    if _ref_workspace_aligned(H * W, C_in) and O.require_ref():
        ref = O.ref_int8_conv_transpose2d_k2s2(xd, wd, sd, bd)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


# tests/test_int8_special_conv.cu:282-284 plus batches, wide and ragged channel counts
@pytest.mark.parametrize("N,C_in,H,W,C_out,use_bias", [
    (1, 32, 16, 16, 64, True), (1, 64, 8, 8, 32, True), (1, 16, 32, 32, 16, False),
    (3, 24, 11, 9, 20, True), (2, 48, 16, 16, 80, True), (1, 7, 5, 5, 3, True), (2, 256, 8, 8, 8, False),
])
def test_conv_transpose2d_k2s2(N, C_in, H, W, C_out, use_bias):
    _check_conv_transpose(N, C_in, H, W, C_out, use_bias, seed=3 + C_in + C_out)


def test_conv2d_full_hd_frame_properties():
    """Size-independent checks on a frame-sized input (1 x 16 x 1080 x 1920 -> 32 channels, 3x3):
    sampled output positions against the composed pipeline, and translation of the image by whole
    tiles leaves interior outputs unchanged."""
    N, C_in, H, W, C_out = 1, 16, 1080, 1920, 32
    g = torch.Generator().manual_seed(99)
    x = torch.randn((N, C_in, H, W), generator=g).to(torch.float16)
    w = torch.randint(-127, 128, (C_out, C_in * 9), generator=g, dtype=torch.int8)
    w_scale, bias = _scales(C_out, True, g)
    out = C.int8_conv2d_forward(x.to(DEV), w.to(DEV), w_scale.to(DEV), bias.to(DEV), (3, 3), (1, 1)).cpu()
    assert C.device_status() == 0
    # crops: the conv of a crop equals the crop of the conv away from the crop's border
    for (h0, w0) in [(0, 0), (500, 1000), (1080 - 40, 1920 - 72)]:
        crop = x[:, :, h0:h0 + 40, w0:w0 + 72].contiguous()
        e = _composed_conv(crop, w, w_scale, bias, (3, 3), (1, 1), (1, 1), (1, 1))
        got = out[:, :, h0 + 1:h0 + 39, w0 + 1:w0 + 71].numpy()
        assert np.array_equal(got.view(np.uint16), np.ascontiguousarray(e[:, :, 1:39, 1:71]).view(np.uint16))
