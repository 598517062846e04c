"""GPU parity of 2:4 prune+compress and metadata packing, through the C ABI. Mirrors the
reference's tests/test_prune_compress.cu and tests/test_pack_metadata.cu (exact match on
compressed values, nibbles and packed words, plus the decompress round trip) over more shapes,
including ones that take the scalar path."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHAPES = [(32, 128), (16, 64), (1, 32), (7, 96), (5, 36), (3, 100), (208, 192), (11008, 4096)]


def _prune_pack(w):
    N, K = w.shape
    comp = torch.full((N, K // 2), 0x7B, dtype=torch.int8, device=DEV)
    raw = torch.full((N * (K // 4),), 0x7B, dtype=torch.uint8, device=DEV)
    packed = torch.full((N, K // 32), 0x5A5A5A5A, dtype=torch.int32, device=DEV)
    C.prune_compress_24(w, comp, raw, N, K)
    if K // 32 > 0:
        C.pack_metadata(raw, packed, N, K)
    torch.cuda.synchronize()
    return comp, raw, packed


@pytest.mark.parametrize("N,K", SHAPES)
def test_prune_compress_pack_exact(N, K):
    g = torch.Generator().manual_seed(42 + N + K)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    w[0, :4] = torch.tensor([9, -9, 9, 9], dtype=torch.int8)   # ties: first two are dropped
    comp, raw, packed = _prune_pack(w.to(DEV))
    comp_cpu, raw_cpu = O.prune_compress_24(w.numpy())
    assert np.array_equal(comp.cpu().numpy(), comp_cpu)
    assert np.array_equal(raw.cpu().numpy(), raw_cpu)
    if K % 32 == 0:
        packed_cpu = O.pack_metadata(raw_cpu, N, K)
        assert np.array_equal(packed.cpu().numpy().view(np.uint32), packed_cpu)
    if K % 32 == 0 and O.require_ref():
        comp_r, raw_r, packed_r = O.ref_prune_pack(w.to(DEV))
        assert torch.equal(comp, comp_r) and torch.equal(raw, raw_r) and torch.equal(packed, packed_r)


def test_prune_every_order_and_tie_pattern():
    """Every group of four over an alphabet of 21 byte values (0, +-1, +-2, +-3, +-63, +-64, +-126, +-127,
    -128 and a few in between: all magnitude orders, every tie shape, both signs, the -128 whose
    magnitude does not fit a signed byte): 194481 groups, vector and scalar kernels, against the
    oracle and the reference kernel."""
    vals = np.array([0, 1, -1, 2, -2, 3, -3, 63, -63, 64, -64, 100, -100, 126, -126, 127, -127, -128, 5, -5, 90], np.int8)
    grid = np.stack(np.meshgrid(vals, vals, vals, vals, indexing="ij"), axis=-1).reshape(-1, 4)
    n_groups = grid.shape[0]
    pad = (-n_groups) % 8
    grid = np.concatenate([grid, np.zeros((pad, 4), np.int8)])
    for K in (32, 36):                                   # 36: rows that are not a multiple of 16 bytes
        rows = (grid.size // K)
        w = torch.from_numpy(grid.reshape(-1)[:rows * K].reshape(rows, K).copy())
        comp, raw, _ = _prune_pack(w.to(DEV))
        comp_cpu, raw_cpu = O.prune_compress_24(w.numpy())
        assert np.array_equal(comp.cpu().numpy(), comp_cpu)
        assert np.array_equal(raw.cpu().numpy(), raw_cpu)
        if K % 32 == 0 and O.require_ref():
            comp_r, raw_r, _ = O.ref_prune_pack(w.to(DEV))
            assert torch.equal(comp, comp_r) and torch.equal(raw, raw_r)
    # the scalar kernel (misaligned compressed output)
    w = torch.from_numpy(grid.reshape(-1, 32).copy())
    N, K = w.shape
    buf = torch.zeros(N * K // 2 + 1, dtype=torch.int8, device=DEV)
    comp = buf[1:].view(N, K // 2)
    raw = torch.zeros(N * K // 4, dtype=torch.uint8, device=DEV)
    C.prune_compress_24(w.to(DEV), comp, raw, N, K)
    comp_cpu, raw_cpu = O.prune_compress_24(w.numpy())
    assert np.array_equal(comp.cpu().numpy(), comp_cpu) and np.array_equal(raw.cpu().numpy(), raw_cpu)


def test_round_trip_decompress():
    N, K = 64, 256
    g = torch.Generator().manual_seed(5)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    comp, raw, _ = _prune_pack(w.to(DEV))
    comp, raw = comp.cpu().numpy(), raw.cpu().numpy().reshape(N, K // 4)
    dense = np.zeros((N, K), np.int8)
    for r in range(N):
        for gidx in range(K // 4):
            nib = raw[r, gidx]
            i0, i1 = nib & 3, nib >> 2
            assert i0 < i1
            dense[r, 4 * gidx + i0] = comp[r, 2 * gidx]
            dense[r, 4 * gidx + i1] = comp[r, 2 * gidx + 1]
    assert np.array_equal(dense, O.prune_24_dense(w.numpy()))
    # every group keeps its two largest magnitudes
    wa = np.abs(w.numpy().astype(np.int32)).reshape(N, K // 4, 4)
    da = np.abs(dense.astype(np.int32)).reshape(N, K // 4, 4)
    assert np.array_equal(np.sort(wa, axis=2)[:, :, 2:].sum(2), da.sum(2))


def test_pack_accepts_any_nibble():
    # tests/test_pack_metadata.cu:14-18 packs arbitrary 4-bit values, not only valid 2:4 codes
    N, K = 16, 128
    g = torch.Generator().manual_seed(42)
    raw = torch.randint(0, 16, (N * K // 4,), generator=g, dtype=torch.uint8)
    packed = torch.zeros((N, K // 32), dtype=torch.int32, device=DEV)
    C.pack_metadata(raw.to(DEV), packed, N, K)
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), O.pack_metadata(raw.numpy(), N, K))
