"""GPU parity of the 2:4-sparse INT8 GEMM (tcgen05.mma.sp kernel) through the C ABI.

Follows the reference's tests/test_int8_sparse_gemm.cu: the full pipeline
prune_compress_24 -> pack_metadata -> sparse GEMM at its shapes (ragged M and N_out, 1..64 K
steps), every forced tile, with and without bias and workspace. Tolerances are the contract's:
INT32 output bit-exact against the dense host loop on the pruned weights, FP16 output bit-exact
against the CPU oracle epilogue and the reference's mma.sp kernel (unsplit)."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# tests/test_int8_sparse_gemm.cu:275-284, plus K values on and off the 128 granule of the TMA path
SHAPES = [(1, 64, 16), (32, 128, 64), (37, 192, 208), (100, 640, 272), (300, 1280, 384), (1000, 1536, 512),
          (2050, 512, 400), (129, 4096, 96), (16, 256, 128), (128, 384, 256), (200, 1024, 1000)]


def _prep(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    packed = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W.to(DEV), comp, raw, N, K)
    C.pack_metadata(raw, packed, N, K)
    return W, x, a_s, w_s, bias, comp, packed


def _status_ok():
    torch.cuda.synchronize()
    assert C.device_status() == 0, "a kernel reported a timed-out wait"


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_s32_equals_dense_gemm_on_pruned_weights(M, K, N):
    W, x, _, _, _, comp, packed = _prep(M, K, N, 42 + M + K + N)
    out = torch.full((M, N), 0x7B7B7B7B, dtype=torch.int32, device=DEV)
    dx = x.to(DEV)
    _lib.call("forge_sparse_int8_gemm_s32", comp.data_ptr(), dx.data_ptr(), packed.data_ptr(), out.data_ptr(),
              M, K, N, 0)
    _status_ok()
    want = O.gemm_s32(x.numpy(), O.prune_24_dense(W.numpy()))
    assert np.array_equal(out.cpu().numpy(), want)
    # the dense tcgen05 kernel on the zero-filled weights must agree too
    dense = C.int8_gemm_s32(x.to(DEV), torch.from_numpy(O.prune_24_dense(W.numpy())).to(DEV))
    _status_ok()
    assert torch.equal(out, dense)


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("tile", [-1, 0, 1, 2])
def test_dequant_bit_exact_every_tile(M, K, N, tile):
    W, x, a_s, w_s, bias, comp, packed = _prep(M, K, N, 7 + M + K + N)
    use_bias = (tile % 2) == 0
    dx, das, dws = x.to(DEV), a_s.to(DEV), w_s.to(DEV)
    dbias = bias.to(DEV) if use_bias else None
    ws = torch.full((M, N), 0x5A5A5A5A, dtype=torch.int32, device=DEV).view(torch.float32)
    out = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    _lib.call("forge_sparse_int8_gemm", comp.data_ptr(), dx.data_ptr(), packed.data_ptr(), das.data_ptr(),
              dws.data_ptr(), 0 if dbias is None else dbias.data_ptr(), out.data_ptr(), M, K, N, ws.data_ptr(), 0,
              0, tile)
    _status_ok()
    acc = O.sparse_gemm_s32(comp.cpu().numpy(), x.numpy(), packed.cpu().numpy().view(np.uint32))
    want = O.dequantize_bias(acc, a_s.numpy(), w_s.numpy(), bias.numpy() if use_bias else None, gemm_epilogue=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    if O.require_ref():
        ref = O.ref_sparse_int8_gemm(comp, dx, packed, das, dws, dbias)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), "differs from the reference mma.sp kernel"


@pytest.mark.parametrize("bt", [128, 192, 224, 256])
@pytest.mark.parametrize("M,K,N", [(37, 256, 208), (300, 1280, 384), (1000, 1536, 512), (2050, 512, 400)])
def test_cta_pair_kernel_every_token_tile(bt, M, K, N):
    """The cta_group::2 kernel (256 weight rows x bt tokens per pair of SMs), knob 1000 + bt."""
    W, x, a_s, w_s, bias, comp, packed = _prep(M, K, N, 3 + bt + M + K + N)
    lib = _lib.load()
    dx = x.to(DEV)
    lib.forge_b200_set_sparse_tile(1000 + bt)
    try:
        out = C.sparse_int8_gemm_s32(comp, dx, packed)
        out16 = C.sparse_int8_gemm(comp, dx, packed, a_s.to(DEV), w_s.to(DEV), bias.to(DEV))
        _status_ok()
    finally:
        lib.forge_b200_set_sparse_tile(0)
    acc = O.gemm_s32(x.numpy(), O.prune_24_dense(W.numpy()))
    assert np.array_equal(out.cpu().numpy(), acc)
    want = O.dequantize_bias(acc, a_s.numpy(), w_s.numpy(), bias.numpy(), gemm_epilogue=True)
    assert np.array_equal(out16.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_every_nibble_in_every_group_position():
    """128 weight rows x K=64: each of the six valid 2:4 codes placed at each of the 16 group
    positions of a 64-deep step, against the dense host loop."""
    K, N, M = 128, 128, 32
    codes = [(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)]
    W = np.zeros((N, K), np.int8)
    rng = np.random.default_rng(0)
    for n in range(N):
        for gidx in range(K // 4):
            i0, i1 = codes[(n + gidx) % 6]
            W[n, 4 * gidx + i0] = rng.integers(1, 128) * rng.choice([-1, 1])
            W[n, 4 * gidx + i1] = rng.integers(1, 128) * rng.choice([-1, 1])
    x = torch.randint(-127, 128, (M, K), generator=torch.Generator().manual_seed(1), dtype=torch.int8)
    Wt = torch.from_numpy(W)
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * K // 4,), dtype=torch.uint8, device=DEV)
    packed = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(Wt.to(DEV), comp, raw, N, K)
    C.pack_metadata(raw, packed, N, K)
    out = C.sparse_int8_gemm_s32(comp, x.to(DEV), packed)
    _status_ok()
    assert np.array_equal(out.cpu().numpy(), O.gemm_s32(x.numpy(), W))


@pytest.mark.parametrize("M", [1, 16, 128, 2048, 8192])
def test_config3_shape_sampled(M):
    """The Llama-MLP weight shape N=11008, K=4096 over the token sweep: sparse result equals the dense GEMM on the pruned
    weights, exact, on sampled tokens; repeat runs identical."""
    N, K = 11008, 4096
    g = torch.Generator(device=DEV).manual_seed(31)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=DEV)
    x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=DEV)
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    packed = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W, comp, raw, N, K)
    C.pack_metadata(raw, packed, N, K)
    out = C.sparse_int8_gemm_s32(comp, x, packed)
    _status_ok()
    rows = sorted(set([0, M - 1, M // 2]))
    want = O.gemm_s32(x[rows].cpu().numpy(), O.prune_24_dense(W.cpu().numpy()))
    assert np.array_equal(out[rows].cpu().numpy(), want)
    assert torch.equal(C.sparse_int8_gemm_s32(comp, x, packed), out)


def test_plan_is_valid_and_honours_forced_tile():
    lib = _lib.load()
    import ctypes
    t, s = ctypes.c_int(-5), ctypes.c_int(-5)
    for (M, K, N) in [(64, 1536, 6144), (1024, 6144, 1536), (8192, 5120, 1280), (256, 4096, 14336)]:
        assert lib.forge_sparse_int8_gemm_plan(M, K, N, 0, 1, -1, ctypes.byref(t), ctypes.byref(s)) == 0
        assert 0 <= t.value < 3 and s.value >= 1
        for tile in range(3):
            lib.forge_sparse_int8_gemm_plan(M, K, N, 0, 1, tile, ctypes.byref(t), ctypes.byref(s))
            assert t.value == tile
        lib.forge_sparse_int8_gemm_plan(M, K, N, 4, 0, -1, ctypes.byref(t), ctypes.byref(s))
        assert s.value == 1   # no workspace -> unsplit (int8_sparse.cu:896)


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("K,N", [(32, 8), (96, 17), (4096, 1000), (8192, 300), (11008, 96), (4096, 11008)])
def test_one_to_four_tokens_weight_streaming_kernel(M, K, N, variant):
    """Few tokens take the CUDA-core weight-streaming kernel (PRMT selection + DP4A; by default up to two
    tokens, here every template instance: variant 1 keeps the token slices in registers, 2 in shared
    memory, 0 is the automatic choice). It must give the accumulators of the host loop on the pruned
    weights, the FP16 epilogue of the oracle, and the very bytes of the tensor-core kernel (pinned with the
    32-token tile knob where K allows it)."""
    W, x, a_s, w_s, bias, comp, packed = _prep(M, K, N, 11 + M + K + N)
    lib = _lib.load()
    dx, das, dws, dbias = x.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV)
    lib.forge_b200_set_tuning(5, variant)
    lib.forge_b200_set_tuning(6, 4 if variant else 0)
    try:
        acc = C.sparse_int8_gemm_s32(comp, dx, packed)
        out = C.sparse_int8_gemm(comp, dx, packed, das, dws, dbias)
        out_nb = C.sparse_int8_gemm(comp, dx, packed, das, dws, None, tile=2)   # the planned id of this kernel
        _status_ok()
    finally:
        lib.forge_b200_set_tuning(5, 0)
        lib.forge_b200_set_tuning(6, 0)
    want_acc = O.gemm_s32(x.numpy(), O.prune_24_dense(W.numpy()))
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    want = O.dequantize_bias(want_acc, a_s.numpy(), w_s.numpy(), bias.numpy(), gemm_epilogue=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    want_nb = O.dequantize_bias(want_acc, a_s.numpy(), w_s.numpy(), None, gemm_epilogue=True)
    assert np.array_equal(out_nb.cpu().numpy().view(np.uint16), want_nb.view(np.uint16))
    if K % 128 == 0 and variant == 0:
        lib.forge_b200_set_sparse_tile(32)
        try:
            tc = C.sparse_int8_gemm(comp, dx, packed, das, dws, dbias)
            _status_ok()
        finally:
            lib.forge_b200_set_sparse_tile(0)
        assert torch.equal(out.view(torch.int16), tc.view(torch.int16))
