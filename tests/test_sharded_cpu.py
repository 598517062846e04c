"""Host logic of the multi-GPU sharding (forge_b200/sharded.py) on two gloo ranks, CPU only.

The local GEMM is injected (the CPU oracle chain quantize -> sparse s32 GEMM -> epilogue), so the
test exercises exactly the partitioning, the all-gather and the column interleave; the CUDA
kernels themselves are covered by the -m gpu tests."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def _oracle_linear(x, w):
    import oracle_lib as O
    q, s = O.quantize(x.numpy())
    acc = O.sparse_gemm_s32(w.W_comp.numpy(), q, w.w_meta.numpy().view(np.uint32))
    bias = None if w.bias is None else w.bias.numpy()
    return torch.from_numpy(O.dequantize_bias(acc, s, w.w_scale.numpy(), bias, gemm_epilogue=True))


def _make(M, K, N):
    import oracle_lib as O
    from forge_b200.sharded import SparseWeights
    g = torch.Generator().manual_seed(123)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    comp, raw = O.prune_compress_24(W.numpy())
    meta = O.pack_metadata(raw, N, K)
    w_scale = (torch.rand(N, generator=g) * 0.01 + 0.001).to(torch.float16)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.float16)
    x = torch.randn((M, K), generator=g).to(torch.float16)
    return x, SparseWeights(torch.from_numpy(comp), torch.from_numpy(meta.view(np.int32)), w_scale, bias)


def _worker(rank, world, port, M, K, N, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from forge_b200.sharded import ShardedSparseLinear
        x, w = _make(M, K, N)
        full = _oracle_linear(x, w)
        rows = ShardedSparseLinear(w, "rows", local_linear=_oracle_linear)
        r0, n = rows.rows_of(M)
        y_rows = rows(x[r0:r0 + n])
        ok_rows = torch.equal(y_rows.view(torch.int16), full[r0:r0 + n].view(torch.int16))
        cols = ShardedSparseLinear(w, "columns", chunks=3, local_linear=_oracle_linear)
        y_cols = cols(x)
        ok_cols = torch.equal(y_cols.view(torch.int16), full.view(torch.int16))
        results[rank] = (ok_rows, ok_cols, n, tuple(cols.weights.W_comp.shape))
    finally:
        dist.destroy_process_group()


def test_partition_is_balanced_and_covers_everything():
    from forge_b200.sharded import partition
    for total in (0, 1, 7, 64, 65536, 1001):
        for world in (1, 2, 3, 8):
            spans = [partition(total, world, r) for r in range(world)]
            assert sum(n for _, n in spans) == total
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(n for _, n in spans) - min(n for _, n in spans) <= 1


@pytest.mark.timeout(300)
def test_rows_and_columns_sharding_match_single_process_bitwise():
    world, M, K, N = 2, 75, 128, 96
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29500 + (os.getpid() % 2000)
        procs = [ctx.Process(target=_worker, args=(r, world, port, M, K, N, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
        assert all(p.exitcode == 0 for p in procs)
        got = dict(results)
    assert set(got) == {0, 1}
    for r in range(world):
        ok_rows, ok_cols, n_rows, w_shape = got[r]
        assert ok_rows and ok_cols
        assert w_shape == (N // world, K // 2)
    assert got[0][2] + got[1][2] == M


def test_columns_mode_requires_divisible_channels():
    from forge_b200.sharded import ShardedSparseLinear, SparseWeights
    w = SparseWeights(torch.zeros((6, 32), dtype=torch.int8), torch.zeros((6, 2), dtype=torch.int32),
                      torch.ones(6, dtype=torch.float16))
    layer = ShardedSparseLinear(w, "columns", local_linear=lambda x, ww: None)   # world size 1: trivially fine
    assert layer.weights.W_comp.shape[0] == 6
