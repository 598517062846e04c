"""GPU parity of the quantizer and the dequantizer, called through the C ABI.

Mirrors the reference's tests/test_quantize.cu (same case list) and tests/test_dequantize.cu,
with the tolerances tightened to the contract: int8 values and scales bit-exact against the
reference GPU kernel, +-1 against the CPU oracle (IEEE divide instead of div.approx), dequant
bit-exact against both."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# tests/test_quantize.cu:103-113 (M, K, element offset of the input pointer)
QUANT_CASES = [(32, 256, 0), (7, 8, 0), (64, 2056, 0), (16, 6144, 0), (16, 8192, 0), (5, 8200, 0), (9, 100, 0),
               (9, 256, 1), (8192, 5120, 0),
               # beyond the reference's list: MLP widths, multi-warp rows, >65536 two-pass fallback
               (33, 4096, 0), (8, 14336, 0), (3, 16384, 0), (2, 40960, 0), (2, 65536, 0), (2, 65544, 0), (1, 4096, 0)]


def _make_x(M, K, offset, seed):
    g = torch.Generator().manual_seed(seed)
    buf = torch.zeros(M * K + offset, dtype=torch.float16)
    buf[offset:] = (torch.rand(M * K, generator=g) * 6 - 3).to(torch.float16)
    dbuf = buf.to(DEV)
    return dbuf, dbuf[offset:].view(M, K)


@pytest.mark.parametrize("M,K,offset", QUANT_CASES)
def test_quantize_matches_reference_kernel_and_oracle(M, K, offset):
    _, x = _make_x(M, K, offset, 42 + M + K)
    q, s = C.fused_quantize_activation(x, M, K)
    torch.cuda.synchronize()
    if O.require_ref():
        q_ref, s_ref = O.ref_quantize(x)
        q2_ref, s2_ref = O.ref_quantize(x, two_pass=True)
        torch.cuda.synchronize()
        assert torch.equal(q, q_ref), "int8 values differ from the reference kernel"
        assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32)), "scales differ bitwise from the reference"
        assert torch.equal(q, q2_ref) and torch.equal(s.view(torch.int32), s2_ref.view(torch.int32))
    if M * K <= 4 * 1024 * 1024:
        q_cpu, s_cpu = O.quantize(x.cpu().numpy())
        assert np.abs(q.cpu().numpy().astype(np.int32) - q_cpu.astype(np.int32)).max() <= 1
        np.testing.assert_allclose(s.cpu().numpy(), s_cpu, rtol=1e-6)


def test_quantize_zero_rows_and_outliers():
    M, K = 64, 4096
    g = torch.Generator().manual_seed(7)
    x = torch.randn((M, K), generator=g)
    x[:, ::97] *= 20  # outlier channels, as in the W8A8 workload
    x[5] = 0
    x[6, 17] = 65504.0
    x = x.to(torch.float16).to(DEV)
    q, s = C.fused_quantize_activation(x, M, K)
    if O.require_ref():
        q_ref, s_ref = O.ref_quantize(x)
        assert torch.equal(q, q_ref) and torch.equal(s.view(torch.int32), s_ref.view(torch.int32))
    assert int(q[5].abs().max()) == 0
    assert q.abs().max() <= 127 or q.min() >= -128


@pytest.mark.parametrize("K", [256, 100, 4096, 14336])
def test_quantize_non_finite_inputs(K):
    """+-Inf and NaN activations (overflowed FP16 upstream). The reference's arithmetic gives: NaN is
    skipped by the row maximum (max.ftz returns the other operand) and quantizes to 0; a row holding
    an infinity gets scale = inf, reciprocal 0, and every value - the infinity included, inf * 0 = NaN
    -> 0 - quantizes to 0 (src/quant/quantize.cu:48-58,112-130). Both kernels of this library must
    reproduce the reference kernels bit for bit, including the scales."""
    M = 12
    g = torch.Generator().manual_seed(K)
    x = (torch.randn((M, K), generator=g) * 2).to(torch.float16)
    inf, nan = float("inf"), float("nan")
    x[1, 3] = inf
    x[2, K - 1] = -inf
    x[3, 0] = nan
    x[4, 5], x[4, 6] = nan, inf
    x[5, :] = nan
    x[6, ::2] = nan
    x[7, 1], x[7, 2] = inf, -inf
    x[8, K // 2] = 65504.0
    xd = x.to(DEV)
    q, s = C.fused_quantize_activation(xd, M, K)
    torch.cuda.synchronize()
    qc, sc = q.cpu(), s.cpu()
    for r in (1, 2, 4, 7):                                  # rows with an infinity
        assert torch.isinf(sc[r]) and int(qc[r].abs().max()) == 0
    assert int(qc[3, 0]) == 0 and torch.isfinite(sc[3]) and int(qc[3].abs().max()) == 127
    assert int(qc[5].abs().max()) == 0 and float(sc[5]) == pytest.approx(1e-8 / 127.0, rel=1e-6)
    assert int(qc[6, ::2].abs().max()) == 0 and int(qc[6].abs().max()) == 127
    assert int(qc[8].abs().max()) == 127 and int(qc[0].abs().max()) == 127
    if O.require_ref():
        for two_pass in (False, True):
            q_ref, s_ref = O.ref_quantize(xd, two_pass=two_pass)
            torch.cuda.synchronize()
            assert torch.equal(q, q_ref), f"values differ from the reference kernel (two_pass={two_pass})"
            assert torch.equal(s.view(torch.int32), s_ref.view(torch.int32))


def test_public_two_pass_kernel_path_is_bit_identical():
    # K % 8 != 0 forces the launcher onto the public two-pass kernel; a K % 8 == 0 prefix of the
    # same data must quantize identically when its row maximum is in the prefix.
    M, K = 12, 1000
    _, x = _make_x(M, K, 0, 99)
    x[:, 0] = 3.5  # row maximum inside the first 992 columns
    q_a, s_a = C.fused_quantize_activation(x, M, K)
    xp = x[:, :992].contiguous()
    q_b, s_b = C.fused_quantize_activation(xp, M, 992)
    assert torch.equal(q_a[:, :992], q_b) and torch.equal(s_a.view(torch.int32), s_b.view(torch.int32))


DEQUANT_CASES = [(16, 64), (1, 8), (37, 200), (5, 13), (4096, 4096), (3, 11008)]


@pytest.mark.parametrize("M,N", DEQUANT_CASES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_dequantize_bias_bit_exact(M, N, with_bias):
    g = torch.Generator().manual_seed(1000 + M + N)
    acc = torch.randint(-50000, 50001, (M, N), generator=g, dtype=torch.int32)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16) if with_bias else None
    d = [t.to(DEV) if t is not None else None for t in (acc, a_s, w_s, bias)]
    out = C.fused_dequantize_bias(d[0], d[1], d[2], d[3], M, N)
    torch.cuda.synchronize()
    if O.require_ref():
        out_ref = O.ref_dequantize_bias(*d)
        assert torch.equal(out.view(torch.int16), out_ref.view(torch.int16))
    if M * N <= 1 << 22:
        cpu = O.dequantize_bias(acc.numpy(), a_s.numpy(), w_s.numpy(), None if bias is None else bias.numpy())
        assert np.array_equal(out.cpu().numpy().view(np.uint16), cpu.view(np.uint16))


def test_empty_shapes_are_noops():
    x = torch.zeros((4, 8), dtype=torch.float16, device=DEV)
    q, s = C.fused_quantize_activation(x, 0, 8)
    assert q.numel() == 0 and s.numel() == 0
