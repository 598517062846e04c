"""GPU parity of the dense INT8 GEMM (tcgen05 kernel) through the C ABI.

Follows the reference's tests/test_int8_dense_gemm.cu and tests/test_int8_dp4a_gemm.cu (same
shapes, ragged K, wide N) but with the contract's tolerances: INT32 output bit-exact against the
host int32 loop; FP16 output bit-exact against the CPU oracle's epilogue (same operation order
as the reference kernel) and against the reference's own wmma kernel run on the same GPU."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (M, K, N): tests/test_int8_dense_gemm.cu:13, tests/test_int8_dp4a_gemm.cu:181-199, the 1024^3 benchmark shape,
# ragged tiles, K tails that are not a multiple of the 128-byte slab, shapes off the TMA path.
SHAPES = [(32, 128, 64), (1024, 1024, 1024), (37, 192, 208), (100, 640, 272), (129, 4096, 96), (2050, 512, 400),
          (1, 64, 16), (300, 1280, 384), (64, 256, 2112), (128, 16, 256), (257, 144, 520),
          (16, 28, 32), (5, 7, 12), (33, 64, 20)]


def _inputs(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    return A, B, a_s, w_s, bias


def _status_ok():
    torch.cuda.synchronize()
    assert C.device_status() == 0, "a kernel reported a timed-out wait"


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_s32_bit_exact(M, K, N):
    A, B, *_ = _inputs(M, K, N, 1234 + M + K + N)
    out = torch.full((M, N), 0x7B7B7B7B, dtype=torch.int32, device=DEV)   # garbage: must be overwritten
    dA, dB = A.to(DEV), B.to(DEV)
    _lib.call("forge_int8_gemm_s32", dA.data_ptr(), dB.data_ptr(), out.data_ptr(), M, K, N, 0)
    _status_ok()
    assert np.array_equal(out.cpu().numpy(), O.gemm_s32(A.numpy(), B.numpy()))


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_dequant_bit_exact(M, K, N, with_bias):
    A, B, a_s, w_s, bias = _inputs(M, K, N, 99 + M + K + N)
    if not with_bias:
        bias = None
    dA, dB, das, dws = A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV)
    dbias = None if bias is None else bias.to(DEV)
    out = C.int8_gemm_dequant(dA, dB, das, dws, dbias)
    _status_ok()
    acc = O.gemm_s32(A.numpy(), B.numpy())
    want = O.dequantize_bias(acc, a_s.numpy(), w_s.numpy(), None if bias is None else bias.numpy(),
                             gemm_epilogue=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    if O.require_ref():
        ref = O.ref_int8_gemm_dequant(dA, dB, das, dws, dbias)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), "differs from the reference wmma kernel"


@pytest.mark.parametrize("bn", [64, 80, 96, 112, 128, 256])
def test_every_tile_width(bn):
    M, K, N = 300, 1152, 784
    A, B, a_s, w_s, bias = _inputs(M, K, N, 5 + bn)
    lib = _lib.load()
    lib.forge_b200_set_dense_tile(bn)
    try:
        out = C.int8_gemm_s32(A.to(DEV), B.to(DEV))
        out16 = C.int8_gemm_dequant(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV))
        _status_ok()
    finally:
        lib.forge_b200_set_dense_tile(0)
    acc = O.gemm_s32(A.numpy(), B.numpy())
    assert np.array_equal(out.cpu().numpy(), acc)
    want = O.dequantize_bias(acc, a_s.numpy(), w_s.numpy(), bias.numpy(), gemm_epilogue=True)
    assert np.array_equal(out16.cpu().numpy().view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (300, 640, 272), (1024, 1024, 1024), (2050, 512, 400),
                                   (257, 144, 520), (512, 4096, 768)])
def test_cta_pair_kernel(M, K, N):
    """The cta_group::2 kernel (256 x 256 outputs per pair of SMs), selected with tile knob 512."""
    A, B, a_s, w_s, bias = _inputs(M, K, N, 77 + M + K + N)
    lib = _lib.load()
    lib.forge_b200_set_dense_tile(512)
    try:
        out = C.int8_gemm_s32(A.to(DEV), B.to(DEV))
        out16 = C.int8_gemm_dequant(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV))
        _status_ok()
    finally:
        lib.forge_b200_set_dense_tile(0)
    acc = O.gemm_s32(A.numpy(), B.numpy())
    assert np.array_equal(out.cpu().numpy(), acc)
    want = O.dequantize_bias(acc, a_s.numpy(), w_s.numpy(), bias.numpy(), gemm_epilogue=True)
    assert np.array_equal(out16.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_headline_8192_sampled_rows_and_determinism():
    M = K = N = 8192
    g = torch.Generator(device=DEV).manual_seed(1234)
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=DEV)
    g2 = torch.Generator(device=DEV).manual_seed(1235)
    B = torch.randint(-127, 128, (N, K), generator=g2, dtype=torch.int8, device=DEV)
    out = C.int8_gemm_s32(A, B)
    _status_ok()
    rows = [0, 1, 127, 128, 4095, 4096, 8063, 8191]
    want = O.gemm_s32(A[rows].cpu().numpy(), B.cpu().numpy())
    assert np.array_equal(out[rows].cpu().numpy(), want)
    # linearity: (A restricted to even rows) gives the same rows; repeat runs are bitwise identical
    for _ in range(3):
        again = C.int8_gemm_s32(A, B)
        assert torch.equal(again, out)
    # column checksum: sum over all rows equals (sum of A rows) x B, computed exactly in int64 on the GPU
    col_sum = out.sum(dim=0, dtype=torch.int64)
    a_sum = A.sum(dim=0, dtype=torch.int64).double()
    want_sum = (B.double() @ a_sum).round().long()
    assert torch.equal(col_sum, want_sum)


def test_int8_linear_matches_quantize_then_gemm():
    M, K, N = 512, 1024, 768
    g = torch.Generator().manual_seed(3)
    x = torch.randn((M, K), generator=g).to(torch.float16).to(DEV)
    _, B, _, w_s, bias = _inputs(M, K, N, 11)
    sa = torch.empty((M, K), dtype=torch.int8, device=DEV)
    ss = torch.empty((M,), dtype=torch.float32, device=DEV)
    out = C.int8_linear(x, B.to(DEV), w_s.to(DEV), bias.to(DEV), sa, ss)
    q, s = C.fused_quantize_activation(x, M, K)
    out2 = C.int8_gemm_dequant(q, B.to(DEV), s, w_s.to(DEV), bias.to(DEV))
    _status_ok()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    assert torch.equal(sa, q) and torch.equal(ss, s)
    if O.require_ref():
        ref = torch.empty_like(out)
        sa2, ss2 = torch.empty_like(sa), torch.empty_like(ss)
        dB, dws, dbias = B.to(DEV), w_s.to(DEV), bias.to(DEV)
        O.ref().ref_int8_linear(x.data_ptr(), dB.data_ptr(), dws.data_ptr(), dbias.data_ptr(),
                                ref.data_ptr(), M, K, N, sa2.data_ptr(), ss2.data_ptr(), O.cur_stream())
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


GEMV_SHAPES = [(1, 4096, 11008), (2, 4096, 1000), (3, 16, 8), (5, 4112, 300), (8, 8192, 520), (16, 4096, 2000),
               (16, 12288, 64), (7, 14336, 96), (1, 32, 9)]


@pytest.mark.parametrize("M,K,N", GEMV_SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_few_token_streaming_kernel_same_bits_as_the_tensor_core_kernel(M, K, N, with_bias):
    """Up to 16 tokens the dense GEMM is a weight-streaming CUDA-core kernel (dense_gemv.cu). Its INT32 output
    must equal the host loop, its FP16 output the tensor-core kernel's (pinned tile) and the reference kernel's."""
    lib = _lib.load()
    lib.forge_b200_set_tuning(9, 16)   # the kernel has instances up to 16 tokens; the default stops at 8
    try:
        _few_token_case(lib, M, K, N, with_bias)
    finally:
        lib.forge_b200_set_tuning(9, 0)


def _few_token_case(lib, M, K, N, with_bias):
    A, B, a_s, w_s, bias = _inputs(M, K, N, 500 + M + K + N)
    dA, dB, das, dws = A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV)
    dbias = bias.to(DEV) if with_bias else None
    out32 = torch.full((M, N), 0x7B7B7B7B, dtype=torch.int32, device=DEV)
    _lib.call("forge_int8_gemm_s32", dA.data_ptr(), dB.data_ptr(), out32.data_ptr(), M, K, N, 0)
    _status_ok()
    assert np.array_equal(out32.cpu().numpy(), O.gemm_s32(A.numpy(), B.numpy()))
    streamed = C.int8_gemm_dequant(dA, dB, das, dws, dbias)
    _status_ok()
    lib.forge_b200_set_dense_tile(64)        # a pinned tile keeps the tcgen05 kernel
    try:
        tensor = C.int8_gemm_dequant(dA, dB, das, dws, dbias)
        _status_ok()
    finally:
        lib.forge_b200_set_dense_tile(0)
    assert torch.equal(streamed.view(torch.int16), tensor.view(torch.int16))
    O.require_ref()
    ref = O.ref_int8_gemm_dequant(dA, dB, das, dws, dbias)
    assert torch.equal(streamed.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("M,K,N", [(1, 4096, 11008), (2, 1024, 300), (4, 4096, 1000), (16, 4096, 520), (9, 8192, 64),
                                   (3, 48, 24)])
def test_few_token_int8_linear_quantizes_inside_the_streaming_kernel(M, K, N):
    """int8_linear with a few tokens: one kernel, scratch untouched, the bytes of quantize + GEMM - also with
    non-finite activations."""
    lib = _lib.load()
    lib.forge_b200_set_tuning(9, 16)
    try:
        _few_token_linear_case(M, K, N)
    finally:
        lib.forge_b200_set_tuning(9, 0)


def _few_token_linear_case(M, K, N):
    g = torch.Generator().manual_seed(70 + M + K + N)
    x = (torch.randn((M, K), generator=g) * 3).to(torch.float16)
    x[0, :4] = torch.tensor([0.0, 65504.0, -65504.0, 6e-8], dtype=torch.float16)
    _, B, _, w_s, bias = _inputs(M, K, N, 71)
    dB, dws, dbias = B.to(DEV), w_s.to(DEV), bias.to(DEV)
    for variant in range(2):
        if variant == 1:
            x[M - 1, 1] = float("inf")
            x[0, 2] = float("nan")
        dx = x.to(DEV)
        sa = torch.full((M, K), 0x5A, dtype=torch.int8, device=DEV)
        ss = torch.full((M,), -7.0, dtype=torch.float32, device=DEV)
        out = C.int8_linear(dx, dB, dws, dbias, sa, ss)
        _status_ok()
        assert int(sa.min()) == 0x5A and int(sa.max()) == 0x5A and float(ss.max()) == -7.0   # scratch untouched
        q, s = C.fused_quantize_activation(dx, M, K)
        want = C.int8_gemm_dequant(q, dB, s, dws, dbias)
        _status_ok()
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)), f"variant {variant}"


@pytest.mark.parametrize("M,K,N", [(16, 4096, 11008), (128, 4096, 11008), (100, 1024, 28672), (37, 512, 1200),
                                   (5, 256, 176)])
def test_one_token_block_picks_a_width_that_fits_one_wave(M, K, N):
    """Calls with one block of token rows choose the tile width (64 ... 128 in steps of 16) by columns per SM; the
    narrow widths end in 16-column pieces stored by the epilogue itself. Same bits as the 64-wide tiles, the host
    loop and the reference kernel."""
    lib = _lib.load()
    lib.forge_b200_set_tuning(9, -1)          # keep the tensor-core kernel for every M here
    try:
        A, B, a_s, w_s, bias = _inputs(M, K, N, 900 + M + K + N)
        dA, dB, das, dws, dbias = A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV)
        auto16 = C.int8_gemm_dequant(dA, dB, das, dws, dbias)
        auto32 = C.int8_gemm_s32(dA, dB)
        _status_ok()
        lib.forge_b200_set_dense_tile(64)
        try:
            fixed16 = C.int8_gemm_dequant(dA, dB, das, dws, dbias)
            _status_ok()
        finally:
            lib.forge_b200_set_dense_tile(0)
    finally:
        lib.forge_b200_set_tuning(9, 0)
    assert torch.equal(auto16.view(torch.int16), fixed16.view(torch.int16))
    assert np.array_equal(auto32.cpu().numpy(), O.gemm_s32(A.numpy(), B.numpy()))
    O.require_ref()
    ref = O.ref_int8_gemm_dequant(dA, dB, das, dws, dbias)
    assert torch.equal(auto16.view(torch.int16), ref.view(torch.int16))
