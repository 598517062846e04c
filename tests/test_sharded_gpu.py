"""Multi-GPU check of forge_b200/sharded.py (the sharded 2:4-sparse W8A8 layer at a reduced size): rows- and
columns-sharded 2:4-sparse W8A8 linear on 2 GPUs must equal the single-GPU result bit for bit.
Spawns one process per GPU (NCCL over 127.0.0.1); skipped on single-GPU boxes."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from forge_b200 import _forge_C as C
        from forge_b200.sharded import ShardedSparseLinear, SparseWeights
        M, K, N = 3000, 1024, 2048
        g = torch.Generator(device=dev)
        g.manual_seed(2024)   # same seed on every rank: replicated inputs
        W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=dev)
        x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float16)
        w_scale = (torch.rand(N, generator=g, device=dev) * 0.01 + 0.001).to(torch.float16)
        bias = (torch.randn(N, generator=g, device=dev) * 0.01).to(torch.float16)
        comp = torch.empty((N, K // 2), dtype=torch.int8, device=dev)
        raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=dev)
        meta = torch.empty((N, K // 32), dtype=torch.int32, device=dev)
        C.prune_compress_24(W, comp, raw, N, K)
        C.pack_metadata(raw, meta, N, K)
        w = SparseWeights(comp, meta, w_scale, bias)
        single = ShardedSparseLinear(w, "rows", group=None)
        single.world, single.rank = 1, 0
        full = single(x)
        rows = ShardedSparseLinear(w, "rows")
        r0, n = rows.rows_of(M)
        ok_rows = torch.equal(rows(x[r0:r0 + n]).view(torch.int16), full[r0:r0 + n].view(torch.int16))
        ok_cols = True
        for exchange in ("nccl", "fused"):
            cols = ShardedSparseLinear(w, "columns", chunks=3, exchange=exchange)
            for _ in range(2):   # twice: the fused path reuses its peer-mapped output buffer
                y = cols(x)
                torch.cuda.synchronize()
                ok_cols = ok_cols and torch.equal(y.view(torch.int16), full.view(torch.int16))
            # a smaller batch afterwards reuses the leading rows of the same mapping
            y = cols(x[:1100].contiguous())
            torch.cuda.synchronize()
            ok_cols = ok_cols and torch.equal(y.view(torch.int16), full[:1100].view(torch.int16))
        results[rank] = (bool(ok_rows), bool(ok_cols), C.device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_sharding_bit_exact():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = 29700 + (os.getpid() % 2000)
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(500)
        assert all(p.exitcode == 0 for p in procs)
        got = dict(results)
    assert got == {0: (True, True, 0), 1: (True, True, 0)}
