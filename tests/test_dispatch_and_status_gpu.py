"""GPU run tests of the entry points that are thin fronts for the main kernels, through the C ABI:

  forge_int8_gemm, forge_int8_dp4a_gemm_dequant, forge_int8_dp4a_linear, forge_get_compute_capability,
  forge_has_wmma_int8    the reference's dispatch front end and legacy backend (src/gemm/int8_gemm.cu:12-46,
                         src/gemm/int8_dp4a.cu:183-234), on the shapes of tests/test_int8_dp4a_gemm.cu:181-199
  forge_splitk_reduce    fp32 workspace + bias -> fp16 (src/gemm/int8_sparse.cu:99-111,945-958)
  forge_sparse_int8_gemm_plan   the plan names the kernel the GEMM's own dispatch runs
  device status          a bounded wait that runs out is reported as FORGE_B200_DEVICE_TIMEOUT and the
                         context stays usable

FP16 outputs are required bit-exact against the CPU oracle's epilogue and against the reference's own
kernels (the dp4a kernel within 1 fp16 ulp: it is a different kernel with its own rounding sequence)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TIMEOUT = 5   # FORGE_B200_DEVICE_TIMEOUT

# tests/test_int8_dp4a_gemm.cu:181-199: (M, K, N, bias)
DP4A_SHAPES = [(32, 128, 64, True), (16, 28, 16, True), (8, 7, 8, True), (64, 64, 2112, False), (256, 64, 16, True),
               (32, 64, 32, False)]


def _inputs(M, K, N, use_bias, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16) if use_bias else None
    return A, B, a_s, w_s, bias


def _want(A, B, a_s, w_s, bias):
    return O.dequantize_bias(O.gemm_s32(A.numpy(), B.numpy()), a_s.numpy(), w_s.numpy(),
                             None if bias is None else bias.numpy(), gemm_epilogue=True)


def _call_gemm(name, A, B, a_s, w_s, bias):
    M, K = A.shape
    N = B.shape[0]
    d = [t.to(DEV) if t is not None else None for t in (A, B, a_s, w_s, bias)]
    out = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    _lib.call(name, d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
              0 if d[4] is None else d[4].data_ptr(), out.data_ptr(), M, K, N, 0)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    return out, d


@pytest.mark.parametrize("M,K,N,use_bias", DP4A_SHAPES)
def test_dp4a_entry_point_runs_the_tensor_core_kernel(M, K, N, use_bias):
    A, B, a_s, w_s, bias = _inputs(M, K, N, use_bias, 42 + M + K + N)
    out, d = _call_gemm("forge_int8_dp4a_gemm_dequant", A, B, a_s, w_s, bias)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), _want(A, B, a_s, w_s, bias).view(np.uint16))
    same, _ = _call_gemm("forge_int8_gemm_dequant", A, B, a_s, w_s, bias)
    assert torch.equal(out.view(torch.int16), same.view(torch.int16))
    if O.require_ref():
        ref = torch.empty_like(out)
        O.ref().ref_int8_dp4a_gemm_dequant(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                           O.tp(d[4]), ref.data_ptr(), M, K, N, O.cur_stream())
        torch.cuda.synchronize()
        assert O.half_ulp_distance(out.cpu().numpy(), ref.cpu().numpy()).max() <= 1   # tolerance: 1 fp16 ulp


def test_unified_dispatch_and_capability_queries():
    lib = _lib.load()
    cc = lib.forge_get_compute_capability(0)
    major, minor = torch.cuda.get_device_capability(0)
    assert cc == major * 10 + minor and cc >= 100
    assert lib.forge_has_wmma_int8(0) == 1
    # test_unified_dispatch (tests/test_int8_dp4a_gemm.cu:118-170): M=32, K=128, N=64, no bias
    A, B, a_s, w_s, bias = _inputs(32, 128, 64, False, 100)
    out, d = _call_gemm("forge_int8_gemm", A, B, a_s, w_s, bias)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), _want(A, B, a_s, w_s, bias).view(np.uint16))
    if O.require_ref():
        assert O.ref().ref_get_compute_capability(0) == cc
        assert O.ref().ref_has_wmma_int8(0) == 1
        ref = torch.empty_like(out)
        O.ref().ref_int8_gemm(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), 0, ref.data_ptr(),
                              32, 128, 64, O.cur_stream())
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


def test_dp4a_linear_is_int8_linear():
    M, K, N = 48, 192, 80
    g = torch.Generator().manual_seed(8)
    x = (torch.randn((M, K), generator=g) * 3).to(torch.float16).to(DEV)
    _, B, _, w_s, bias = _inputs(M, K, N, True, 9)
    dB, dws, dbias = B.to(DEV), w_s.to(DEV), bias.to(DEV)
    outs = []
    for name in ("forge_int8_dp4a_linear", "forge_int8_linear"):
        out = torch.empty((M, N), dtype=torch.float16, device=DEV)
        sa = torch.empty((M, K), dtype=torch.int8, device=DEV)
        ss = torch.empty((M,), dtype=torch.float32, device=DEV)
        _lib.call(name, x.data_ptr(), dB.data_ptr(), dws.data_ptr(), dbias.data_ptr(), out.data_ptr(), M, K, N,
                  sa.data_ptr(), ss.data_ptr(), 0)
        torch.cuda.synchronize()
        outs.append((out, sa, ss))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    out, sa, ss = outs[0]
    want = O.dequantize_bias(O.gemm_s32(sa.cpu().numpy(), B.numpy()), ss.cpu().numpy(), w_s.numpy(), bias.numpy(),
                             gemm_epilogue=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("M,N", [(1, 16), (37, 200), (128, 4096), (2048, 11008)])
@pytest.mark.parametrize("use_bias", [True, False])
def test_splitk_reduce(M, N, use_bias):
    g = torch.Generator().manual_seed(M + N)
    ws = (torch.randn((M, N), generator=g) * 300.0).float()
    ws.view(-1)[:8] = torch.tensor([0.0, -0.0, 65504.0, -65504.0, 70000.0, 1e-8, -3e-5, 6.1e-5])[:min(8, M * N)]
    bias = (torch.randn(N, generator=g) * 2).to(torch.float16) if use_bias else None
    dws, dbias = ws.to(DEV), None if bias is None else bias.to(DEV)
    out = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    _lib.call("forge_splitk_reduce", dws.data_ptr(), O.tp(dbias), out.data_ptr(), M, N, 0)
    torch.cuda.synchronize()
    v = ws.numpy().copy()
    if use_bias:
        v = v + bias.numpy().astype(np.float32)[None, :]     # one fp32 addition, then one rounding to fp16
    with np.errstate(over="ignore"):
        want = v.astype(np.float16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    if O.require_ref():
        ref = torch.empty_like(out)
        O.ref().ref_splitk_reduce(dws.data_ptr(), O.tp(dbias), ref.data_ptr(), M, N, O.cur_stream())
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    # sizes <= 0: nothing is written
    marker = out.clone()
    _lib.call("forge_splitk_reduce", dws.data_ptr(), O.tp(dbias), out.data_ptr(), 0, N, 0)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), marker.view(torch.int16))


def _plan(M, K, N, tile=-1):
    t, s = ctypes.c_int(-9), ctypes.c_int(-9)
    assert _lib.load().forge_sparse_int8_gemm_plan(M, K, N, 1, 0, tile, ctypes.byref(t), ctypes.byref(s)) == 0
    assert s.value == 1
    return t.value


@pytest.mark.parametrize("M,K,N", [(1, 4096, 11008), (16, 4096, 11008), (40, 512, 256), (128, 4096, 11008),
                                   (200, 1024, 2048), (2048, 4096, 11008), (8192, 4096, 11008), (300, 96, 64)])
def test_planned_tile_reproduces_the_automatic_result(M, K, N):
    """forge_sparse_int8_gemm_plan names the kernel the automatic path runs; handing the planned tile back
    (the reference's calling pattern, python/forge/csrc/bindings.cpp:534-535) gives the same bytes."""
    g = torch.Generator(device=DEV).manual_seed(M + K + N)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=DEV)
    x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=DEV)
    a_s = torch.rand(M, generator=g, device=DEV) * 0.02 + 0.001
    w_s = (torch.rand(N, generator=g, device=DEV) * 0.02 + 0.001).to(torch.float16)
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    meta = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W, comp, raw, N, K)
    C.pack_metadata(raw, meta, N, K)
    tile = _plan(M, K, N)
    assert 0 <= tile <= 2
    assert _plan(M, K, N, tile) == tile          # a forced valid tile is honoured and stable
    assert _plan(M, K, N, 7) == tile             # ids >= 3 mean automatic (int8_sparse.cu:895)
    auto = C.sparse_int8_gemm(comp, x, meta, a_s, w_s, None, tile=-1)
    planned = C.sparse_int8_gemm(comp, x, meta, a_s, w_s, None, tile=tile)
    torch.cuda.synchronize()
    assert C.device_status() == 0
    assert torch.equal(auto.view(torch.int16), planned.view(torch.int16))
    want = O.dequantize_bias(O.sparse_gemm_s32(comp.cpu().numpy(), x.cpu().numpy(), meta.cpu().numpy().view(np.uint32)),
                             a_s.cpu().numpy(), w_s.cpu().numpy(), None, gemm_epilogue=True)
    assert np.array_equal(auto.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Every wait in the tcgen05 kernels is bounded; one that runs out records a code and the kernel
    returns through its normal teardown. Exercised with the library's self-test kernel: one thread waits
    one millisecond on a barrier nobody arrives at (no fault, no trap, no endless loop)."""
    lib = _lib.load()
    torch.cuda.synchronize()
    assert lib.forge_b200_device_status(1) == 0
    assert lib.forge_b200_selftest_wait_timeout(1000, 0) == 0
    torch.cuda.synchronize()
    assert lib.forge_b200_device_status(0) == TIMEOUT                 # not cleared by a plain read
    assert lib.forge_b200_device_status_raw(0) == 900
    assert b"wait" in lib.forge_b200_status_string(TIMEOUT)
    assert lib.forge_b200_device_status(1) == TIMEOUT                 # read and clear
    assert lib.forge_b200_device_status(1) == 0 and lib.forge_b200_device_status_raw(1) == 0
    # the context is intact: a GEMM right after it is bit-exact
    A, B, a_s, w_s, bias = _inputs(200, 256, 136, True, 5)
    out, _ = _call_gemm("forge_int8_gemm_dequant", A, B, a_s, w_s, bias)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), _want(A, B, a_s, w_s, bias).view(np.uint16))
