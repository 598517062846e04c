"""sparse_int8_linear: the fused quantize + GEMM path against the two-pass path, through the C ABI.

Mirrors run_linear of the reference's tests/test_int8_sparse_gemm.cu:166-270: fused, two-pass and
automatic paths must be bit-identical (its contract, include/forge/gemm/int8_sparse.cuh:89), the
fused call must work without scratch buffers, and sampled rows must match the CPU chain
quantize -> pruned-weight int32 GEMM -> dequant."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TWO_PASS, FUSED, AUTO = 0, 1, -1

# tests/test_int8_sparse_gemm.cu:297-300 (the first reduced from M = 70000 to keep the CPU check
# short; 20000 x 1280 fp16 = 51 MB) plus K at the 1280 limit, ragged M, several weight tiles
SHAPES = [(20000, 1280, 320), (5000, 1024, 336), (37, 128, 16), (4096, 1280, 5120), (300, 640, 272), (129, 384, 400)]


def _prep(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    x = (torch.rand((M, K), generator=g) * 4 - 2).to(torch.float16)
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    meta = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W.to(DEV), comp, raw, N, K)
    C.pack_metadata(raw, meta, N, K)
    return W, x, w_s, bias, comp, meta


def _linear(x, comp, meta, w_s, bias, path, with_scratch=True):
    M, K = x.shape
    N = comp.shape[0]
    out = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    sq = torch.empty((M, K), dtype=torch.int8, device=DEV) if with_scratch else None
    ss = torch.empty((M,), dtype=torch.float32, device=DEV) if with_scratch else None
    _lib.call("forge_sparse_int8_linear", x.data_ptr(), comp.data_ptr(), meta.data_ptr(), w_s.data_ptr(),
              0 if bias is None else bias.data_ptr(), out.data_ptr(), M, K, N, 0 if sq is None else sq.data_ptr(),
              0 if ss is None else ss.data_ptr(), 0, 1, 0, path)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    return out, sq, ss


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_fused_two_pass_and_auto_are_bit_identical(M, K, N, with_bias):
    W, x, w_s, bias, comp, meta = _prep(M, K, N, 900 + M + K + N)
    dx, dws = x.to(DEV), w_s.to(DEV)
    dbias = bias.to(DEV) if with_bias else None
    two, sq, ss = _linear(dx, comp, meta, dws, dbias, TWO_PASS)
    fused, _, _ = _linear(dx, comp, meta, dws, dbias, FUSED, with_scratch=False)   # no scratch needed
    auto, _, _ = _linear(dx, comp, meta, dws, dbias, AUTO)
    assert torch.equal(fused.view(torch.int16), two.view(torch.int16)), "fused differs from two-pass"
    assert torch.equal(auto.view(torch.int16), two.view(torch.int16)), "automatic path differs from two-pass"
    # sampled rows against the CPU chain on the GPU's own quantized values (bit-exact downstream)
    rows = sorted({0, 1, M // 3, M // 2, M - 2 if M > 1 else 0, M - 1})
    acc = O.gemm_s32(sq[rows].cpu().numpy(), O.prune_24_dense(W.numpy()))
    want = O.dequantize_bias(acc, ss[rows].cpu().numpy(), w_s.numpy(), bias.numpy() if with_bias else None,
                             gemm_epilogue=True)
    assert np.array_equal(fused[rows].cpu().numpy().view(np.uint16), want.view(np.uint16))
    q_cpu, s_cpu = O.quantize(x[rows].numpy())
    assert np.abs(sq[rows].cpu().numpy().astype(np.int32) - q_cpu.astype(np.int32)).max() <= 1
    np.testing.assert_allclose(ss[rows].cpu().numpy(), s_cpu, rtol=1e-6)


def test_fused_needs_k_up_to_1280_else_two_pass_with_scratch():
    lib = _lib.load()
    W, x, w_s, bias, comp, meta = _prep(64, 1408, 32, 5)
    dx, dws, dbias = x.to(DEV), w_s.to(DEV), bias.to(DEV)
    out = torch.empty((64, 32), dtype=torch.float16, device=DEV)
    # K > 1280: the forced fused path falls back to two-pass, which needs the scratch buffers
    st = lib.forge_sparse_int8_linear(dx.data_ptr(), comp.data_ptr(), meta.data_ptr(), dws.data_ptr(), dbias.data_ptr(),
                                      out.data_ptr(), 64, 1408, 32, 0, 0, 0, 1, 0, FUSED)
    assert st == 2   # FORGE_B200_BAD_POINTER
    two, _, _ = _linear(dx, comp, meta, dws, dbias, TWO_PASS)
    forced, _, _ = _linear(dx, comp, meta, dws, dbias, FUSED)
    assert torch.equal(two.view(torch.int16), forced.view(torch.int16))


def test_auto_policy():
    """The automatic path fuses narrow layers (N_out <= 640, or <= 1280 with K <= 1024) with K <= 1280 whose
    FP16 activation does not fit L2 - where the fused kernel measured faster than quantize + GEMM on B200 -
    and nothing else (the reference's rule has the same form, src/gemm/int8_sparse.cu:930-938)."""
    lib = _lib.load()
    expect = {(147456, 1280, 320): 1, (147456, 512, 128): 1, (147456, 1024, 1280): 1, (147456, 1280, 1280): 0,
              (4096, 1280, 5120): 0, (5000, 1024, 336): 0, (100000, 4096, 320): 0, (32768, 1280, 320): 0}
    for shape, want in expect.items():
        assert lib.forge_sparse_int8_linear_fused(*shape) == want, shape


def test_auto_path_takes_the_fused_kernel_where_the_policy_says_so():
    """At a shape the policy fuses, the automatic path must not touch the scratch buffers (the fused kernel
    has none) and must give the two-pass bytes."""
    M, K, N = 60000, 1280, 320          # 154 MB of FP16 activations: beyond L2
    lib = _lib.load()
    assert lib.forge_sparse_int8_linear_fused(M, K, N) == 1
    W, x, w_s, bias, comp, meta = _prep(M, K, N, 77)
    dx, dws, dbias = x.to(DEV), w_s.to(DEV), bias.to(DEV)
    two, _, _ = _linear(dx, comp, meta, dws, dbias, TWO_PASS)
    out = torch.empty((M, N), dtype=torch.float16, device=DEV)
    sq = torch.full((M, K), 0x5A, dtype=torch.int8, device=DEV)
    ss = torch.full((M,), -7.0, dtype=torch.float32, device=DEV)
    _lib.call("forge_sparse_int8_linear", dx.data_ptr(), comp.data_ptr(), meta.data_ptr(), dws.data_ptr(),
              dbias.data_ptr(), out.data_ptr(), M, K, N, sq.data_ptr(), ss.data_ptr(), 0, 1, 0, AUTO)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    assert torch.equal(out.view(torch.int16), two.view(torch.int16))
    assert int(sq.min()) == 0x5A and int(sq.max()) == 0x5A and float(ss.min()) == -7.0   # scratch untouched


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("K,N", [(4096, 11008), (1024, 300), (96, 17), (4096, 1000), (2048, 8)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_one_and_two_tokens_quantize_inside_the_streaming_kernel(M, K, N, with_bias):
    """One- and two-token calls (K <= 4096) take the weight-streaming kernel with the quantizer inside it:
    no scratch is touched or needed, and the bytes are those of quantize + GEMM. Inputs include a zero row
    element pattern and large magnitudes."""
    lib = _lib.load()
    assert lib.forge_sparse_int8_linear_fused(M, K, N) == 1
    W, x, w_s, bias, comp, meta = _prep(M, K, N, 4000 + M + K + N)
    x[0, :7] = torch.tensor([0.0, -0.0, 65504.0, -65504.0, 6e-8, 1.5, -2.5], dtype=torch.float16)
    dx, dws = x.to(DEV), w_s.to(DEV)
    dbias = bias.to(DEV) if with_bias else None
    two, _, _ = _linear(dx, comp, meta, dws, dbias, TWO_PASS)
    for path in (AUTO, FUSED):
        got, _, _ = _linear(dx, comp, meta, dws, dbias, path, with_scratch=False)
        assert torch.equal(got.view(torch.int16), two.view(torch.int16)), f"path {path}"
    # non-finite activations: same bytes as the two-pass path there too
    x2 = x.clone()
    x2[M - 1, 3] = float("inf")
    x2[0, 5] = float("nan")
    d2 = x2.to(DEV)
    two2, _, _ = _linear(d2, comp, meta, dws, dbias, TWO_PASS)
    got2, _, _ = _linear(d2, comp, meta, dws, dbias, AUTO, with_scratch=False)
    assert torch.equal(got2.view(torch.int16), two2.view(torch.int16))
