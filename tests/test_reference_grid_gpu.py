"""The reference's own benchmark grid (benchmarks/bench_int8_sparse.cu:113-114: four (K, N) weight
shapes x M in {64, 1024, 4096, 8192}), run through both libraries on the same GPU with the same inputs.

Two requirements per grid point: the FP16 outputs are the same bytes (the reference's unsplit,
deterministic path: split_k = 1, no workspace), and this library's 2:4-sparse GEMM is not slower than
the reference's mma.sp kernel compiled for the same GPU. Timing: one call between CUDA events, 256 MiB
written between calls so that operands come from HBM, median of 7 after 3 warm-ups, for both sides.

When FORGE_B200_GRID_TABLE names a file, the measured table (markdown) is written there."""
import os
import statistics

import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GRID = [(K, N, M) for (K, N) in [(1536, 6144), (6144, 1536), (1280, 5120), (5120, 1280)]
        for M in [64, 1024, 4096, 8192]]


def _median_ms(fn, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(7):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def test_reference_benchmark_grid_same_bytes_and_not_slower():
    O.require_ref()
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(0)
    rows, slower = [], []
    for (K, N, M) in GRID:
        W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=DEV)
        comp, _, meta = O.ref_prune_pack(W)
        x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=DEV)
        a_s = torch.rand(M, generator=g, device=DEV) * 0.02 + 0.001
        w_s = (torch.rand(N, generator=g, device=DEV) * 0.02 + 0.001).to(torch.float16)
        bias = (torch.randn(N, generator=g, device=DEV) * 0.01).to(torch.float16)
        ours = C.sparse_int8_gemm(comp, x, meta, a_s, w_s, bias)
        theirs = O.ref_sparse_int8_gemm(comp, x, meta, a_s, w_s, bias)
        torch.cuda.synchronize()
        assert C.device_status() == 0
        assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16)), f"K={K} N={N} M={M}: outputs differ"
        t_ref = _median_ms(lambda: O.ref_sparse_int8_gemm(comp, x, meta, a_s, w_s, bias), flush)
        t_new = _median_ms(lambda: C.sparse_int8_gemm(comp, x, meta, a_s, w_s, bias), flush)
        tops = lambda ms: 2.0 * M * N * K / (ms * 1e-3) / 1e12
        rows.append(f"| {K} x {N} | {M} | {t_ref:.4f} | {tops(t_ref):.0f} | {t_new:.4f} | {tops(t_new):.0f} | "
                    f"{t_ref / t_new:.1f}x |")
        if t_new > t_ref:
            slower.append((K, N, M, t_ref, t_new))
    table = "\n".join(["| K x N | M | reference ms | dense-equiv TOP/s | this library ms | dense-equiv TOP/s | ratio |",
                       "|---|---|---|---|---|---|---|"] + rows)
    print("\n" + table)
    path = os.environ.get("FORGE_B200_GRID_TABLE")
    if path:
        with open(path, "w") as f:
            f.write(table + "\n")
    assert not slower, f"slower than the reference kernel at {slower}"
