"""Pins the CPU oracle (oracle/forge_oracle.c) against outputs of the REFERENCE's own CUDA
kernels, recorded on a B200 by tests/golden/make_golden.py into reference_vectors.npz.

Integer paths and the dequantizers must match bit for bit. The quantizer may differ by one
int8 step where the reference's approximate reciprocal moves a rounding tie (the reference's
own test allows the same, tests/test_quantize.cu:80); its scales agree to 1e-6 relative.
GEMM outputs of the reference are FP16, so the oracle chain is s32 GEMM -> epilogue dequant."""
import os

import numpy as np
import pytest

import oracle_lib as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


@pytest.mark.parametrize("case", ["q0", "q1", "q2", "q3"])
def test_quantize_within_one_step_of_reference_kernel(gold, case):
    x, q_ref, s_ref = gold[case + "_x"], gold[case + "_q"], gold[case + "_s"]
    q, s = O.quantize(x)
    diff = np.abs(q.astype(np.int32) - q_ref.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 1e-2, "more than rounding ties differ"
    np.testing.assert_allclose(s, s_ref, rtol=1e-6)


def test_dequantize_bit_exact(gold):
    args = (gold["d_acc"], gold["d_as"], gold["d_ws"])
    assert np.array_equal(O.dequantize_bias(*args, gold["d_bias"]).view(np.uint16), gold["d_out_bias"].view(np.uint16))
    assert np.array_equal(O.dequantize_bias(*args, None).view(np.uint16), gold["d_out_nobias"].view(np.uint16))


def test_prune_compress_pack_bit_exact(gold):
    w = gold["p_w"]
    comp, raw = O.prune_compress_24(w)
    assert np.array_equal(comp, gold["p_comp"])
    assert np.array_equal(raw, gold["p_raw"])
    assert np.array_equal(O.pack_metadata(raw, *w.shape), gold["p_packed"])


def test_dense_gemm_chain_bit_exact(gold):
    acc = O.gemm_s32(gold["g_A"], gold["g_B"])
    assert np.array_equal(acc, gold["g_A"].astype(np.int32) @ gold["g_B"].astype(np.int32).T)
    for bias_key, out_key in (("g_bias", "g_out_bias"), (None, "g_out_nobias")):
        bias = gold[bias_key] if bias_key else None
        got = O.dequantize_bias(acc, gold["g_as"], gold["g_ws"], bias, gemm_epilogue=True)
        assert np.array_equal(got.view(np.uint16), gold[out_key].view(np.uint16))


def test_sparse_gemm_chain_bit_exact(gold):
    W, x = gold["s_W"], gold["s_x"]
    comp, raw = O.prune_compress_24(W)
    packed = O.pack_metadata(raw, *W.shape)
    assert np.array_equal(comp, gold["s_comp"]) and np.array_equal(packed, gold["s_packed"])
    acc = O.sparse_gemm_s32(comp, x, packed)
    assert np.array_equal(acc, O.gemm_s32(x, O.prune_24_dense(W)))
    for bias_key, out_key in (("s_bias", "s_out_bias"), (None, "s_out_nobias")):
        bias = gold[bias_key] if bias_key else None
        got = O.dequantize_bias(acc, gold["s_as"], gold["s_ws"], bias, gemm_epilogue=True)
        assert np.array_equal(got.view(np.uint16), gold[out_key].view(np.uint16))


def test_prune_tie_break_order():
    # equal magnitudes: the scan drops the earliest positions first (prune_compress.cu:39-50)
    w = np.array([[5, -5, 5, 5, 1, 2, 3, 4, 4, 3, 2, 1, 0, 0, 0, 0, -7, 7, 1, -1, 2, 2, 2, 3, 3, 2, 2, 2, 9, 1, 9, 1]],
                 dtype=np.int8)
    comp, raw = O.prune_compress_24(w)
    assert raw.tolist() == [0xE, 0xE, 0x4, 0xE, 0x4, 0xE, 0xC, 0x8]
    assert comp[0].tolist() == [5, 5, 3, 4, 4, 3, 0, 0, -7, 7, 2, 3, 3, 2, 9, 9]


def test_fp16_conversion_matches_numpy():
    rng = np.random.default_rng(0)
    lib = O.oracle()
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 60000)])
    for v in vals:
        want = int(np.float32(v).astype(np.float16).view(np.uint16)) if abs(v) < 65520 else None
        if want is not None:
            assert lib.oracle_float_to_half(float(v)) == want


# ---------------------------------------------------------------- INT8 conv callers
CONV_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_conv_vectors.npz")


@pytest.fixture(scope="module")
def conv_gold():
    return np.load(CONV_GOLDEN)


@pytest.mark.parametrize("case", ["c0", "c1", "c2", "c3"])
def test_conv2d_chain_against_reference_pipeline(conv_gold, case):
    """The reference's conv pipeline ran on a B200; its int8 patches and scales were read back from
    its workspace. From those, the oracle's exact steps (s32 GEMM, GEMM-epilogue dequant + bias,
    transpose) must reproduce the reference output bit for bit; the oracle's im2col + IEEE quantizer
    must land within one int8 step of the reference's patches, and the end-to-end CPU conv within
    the output change one step can cause."""
    g = conv_gold
    Ci, H, W, Co, kH, kW, pH, pW, sH, sW, dH, dW = [int(v) for v in g[case + "_cfg"]]
    x, w, w_s, q_ref, a_ref, y_ref = (g[case + k] for k in ("_x", "_w", "_ws", "_q", "_as", "_y"))
    bias = g[case + "_bias"] if case + "_bias" in g.files else None
    col, Ho, Wo = O.im2col(x, kH, kW, pH, pW, sH, sW, dH, dW)
    assert col.shape == q_ref.shape
    acc = O.gemm_s32(q_ref, w)
    y = O.rows_to_nchw(O.dequantize_bias(acc, a_ref, w_s, bias, gemm_epilogue=True), 1, Ho * Wo, Co)
    assert np.array_equal(y.reshape(y_ref.shape).view(np.uint16), y_ref.view(np.uint16))
    q, a = O.quantize(col)
    assert np.abs(q.astype(np.int32) - q_ref.astype(np.int32)).max() <= 1
    np.testing.assert_allclose(a, a_ref, rtol=1e-6)
    y_cpu = O.int8_conv2d(x, w, w_s, bias, kH, kW, pH, pW, sH, sW, dH, dW).astype(np.float32)
    # one int8 step on every tap moves an output by at most scale * w_scale * sum|w|
    bound = (a_ref.max() * w_s.astype(np.float32) * np.abs(w.astype(np.float32)).sum(axis=1)).reshape(1, Co, 1, 1)
    assert (np.abs(y_cpu - y_ref.astype(np.float32)) <= bound + 1e-2).all()
    assert np.mean(y_cpu.astype(np.float16).view(np.uint16) == y_ref.view(np.uint16)) > 0.9


@pytest.mark.parametrize("case,H,W", [("t0", 16, 16), ("t1", 32, 32)])
def test_conv_transpose_chain_against_reference_pipeline(conv_gold, case, H, W):
    g = conv_gold
    x, w, w_s, y_ref = (g[case + k] for k in ("_x", "_w", "_ws", "_y"))
    bias = g[case + "_bias"] if case + "_bias" in g.files else None
    Co = w.shape[0] // 4
    col, _, _ = O.im2col(x, 1, 1, 0, 0, 1, 1, 1, 1)
    q, a = O.quantize(col)
    acc = O.gemm_s32(q, w)
    gem = O.dequantize_bias(acc, a, np.repeat(w_s, 4), None, gemm_epilogue=True)
    y = O.conv_transpose_k2s2_scatter(gem, bias, 1, H, W, Co)
    # the CPU quantizer may differ from the GPU's by one int8 step on a few taps
    same = np.mean(y.view(np.uint16) == y_ref.view(np.uint16))
    assert same > 0.9, same
    bound = (a.max() * w_s.astype(np.float32) * np.abs(w.astype(np.float32)).reshape(Co, -1).sum(axis=1) / 4)
    assert (np.abs(y.astype(np.float32) - y_ref.astype(np.float32)) <= bound.reshape(1, Co, 1, 1) + 1e-2).all()
