"""Every entry point of the path next to the reference's own kernel for it (compiled for this GPU under
oracle/_ref): same inputs, outputs compared bit for bit, then both timed with one harness - CUDA events
around a single call, 256 MiB written between calls so that operands come from HBM, median of 7 calls
after three warm-ups. The test fails if an output differs or if this library is slower than the
reference kernel (10 % tolerance, 30 % for rows under 30 microseconds, which are launch-bound on both sides).

FORGE_B200_SPEED_TABLE names a file for the measured table (markdown); FORGE_B200_CPU_TABLE one for the
CPU oracle's rates on this host (the second test)."""
import os
import statistics

import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ITERS = 7


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def rand_i8(shape, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randint(-127, 128, shape, dtype=torch.int8, device=DEV, generator=g)


def scales(M, N, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    a = torch.rand(M, device=DEV, generator=g) * 0.02 + 0.001
    w = (torch.rand(N, device=DEV, generator=g) * 0.02 + 0.001).half()
    b = (torch.randn(N, device=DEV, generator=g) * 0.01).half()
    return a, w, b


@pytest.mark.timeout(900)
def test_every_entry_point_same_bits_and_not_slower_than_the_reference_kernel():
    O.require_ref()
    torch.cuda.set_device(0)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=DEV)
    rows = []

    def report(case, shape, unit, work, t_ref, t_new, same):
        # work is scaled so that work / milliseconds is already in the stated unit
        rows.append({"case": case, "shape": shape, "reference_ms": t_ref, "b200_ms": t_new,
                     "reference": work / t_ref, "b200": work / t_new, "unit": unit,
                     "speedup": t_ref / t_new, "bit_identical": bool(same)})

    # Dense INT8 GEMM + dequant (wmma kernel of the reference).
    for (M, N, K) in [(4096, 4096, 4096), (8192, 8192, 8192)]:
        A, B = rand_i8((M, K), 1234), rand_i8((N, K), 1235)
        a, w, b = scales(M, N, 1)
        o_ref = O.ref_int8_gemm_dequant(A, B, a, w, b)
        o_new = C.int8_gemm_dequant(A, B, a, w, b)
        t_ref = timed(lambda: O.ref_int8_gemm_dequant(A, B, a, w, b), ITERS, flush)
        t_new = timed(lambda: C.int8_gemm_dequant(A, B, a, w, b), ITERS, flush)
        report("int8_gemm_dequant", f"M={M} N={N} K={K}", "TOP/s", 2.0 * M * N * K / 1e9, t_ref, t_new,
               torch.equal(o_ref, o_new))
        del A, B, o_ref, o_new

    # 2:4-sparse INT8 GEMM (mma.sp kernel of the reference, its own plan), dense-equivalent rate.
    for (M, N, K) in [(1, 11008, 4096), (16, 11008, 4096), (128, 11008, 4096), (2048, 11008, 4096),
                      (8192, 11008, 4096), (8192, 8192, 8192)]:
        W = rand_i8((N, K), 77)
        comp, _, meta = O.ref_prune_pack(W)
        x = rand_i8((M, K), 78)
        a, w, b = scales(M, N, 2)
        o_ref = O.ref_sparse_int8_gemm(comp, x, meta, a, w, b)
        o_new = C.sparse_int8_gemm(comp, x, meta, a, w, b)
        t_ref = timed(lambda: O.ref_sparse_int8_gemm(comp, x, meta, a, w, b), ITERS, flush)
        t_new = timed(lambda: C.sparse_int8_gemm(comp, x, meta, a, w, b), ITERS, flush)
        report("sparse_int8_gemm", f"M={M} N={N} K={K}", "TOP/s (dense-equivalent)", 2.0 * M * N * K / 1e9,
               t_ref, t_new, torch.equal(o_ref, o_new))
        del W, comp, meta, x, o_ref, o_new

    # Per-token quantize.
    for (M, K) in [(4096, 4096), (16384, 8192)]:
        g = torch.Generator(device=DEV).manual_seed(5)
        x = torch.randn((M, K), device=DEV, generator=g).half()
        q_ref, s_ref = O.ref_quantize(x)
        q_new, s_new = C.fused_quantize_activation(x, M, K)
        t_ref = timed(lambda: O.ref_quantize(x), ITERS, flush)
        t_new = timed(lambda: C.fused_quantize_activation(x, M, K), ITERS, flush)
        report("fused_quantize_activation", f"M={M} K={K}", "GB/s", (3.0 * M * K + 4 * M) / 1e6, t_ref,
               t_new, torch.equal(q_ref, q_new) and torch.equal(s_ref, s_new))
        del x

    # Dequant + bias.
    for (M, N) in [(4096, 4096), (8192, 8192)]:
        g = torch.Generator(device=DEV).manual_seed(6)
        acc = torch.randint(-(1 << 20), 1 << 20, (M, N), dtype=torch.int32, device=DEV, generator=g)
        a, w, b = scales(M, N, 3)
        o_ref = O.ref_dequantize_bias(acc, a, w, b)
        o_new = C.fused_dequantize_bias(acc, a, w, b, M, N)
        t_ref = timed(lambda: O.ref_dequantize_bias(acc, a, w, b), ITERS, flush)
        t_new = timed(lambda: C.fused_dequantize_bias(acc, a, w, b, M, N), ITERS, flush)
        report("fused_dequantize_bias", f"M={M} N={N}", "GB/s", (6.0 * M * N + 4 * (M + N)) / 1e6, t_ref,
               t_new, torch.equal(o_ref, o_new))
        del acc

    # Prune + compress and metadata pack.
    N, K = 28672, 8192
    W = rand_i8((N, K), 9)
    comp_r, raw_r, packed_r = O.ref_prune_pack(W)
    comp = torch.empty_like(comp_r)
    raw = torch.empty_like(raw_r)
    packed = torch.empty_like(packed_r)
    C.prune_compress_24(W, comp, raw, N, K)
    C.pack_metadata(raw, packed, N, K)
    same_prune = torch.equal(comp, comp_r) and torch.equal(raw, raw_r)
    same_pack = torch.equal(packed, packed_r)
    st = O.cur_stream()
    t_ref = timed(lambda: O.ref().ref_prune_compress_24(O.tp(W), O.tp(comp_r), O.tp(raw_r), N, K, st),
                  ITERS, flush)
    t_new = timed(lambda: C.prune_compress_24(W, comp, raw, N, K), ITERS, flush)
    report("prune_compress_24", f"N={N} K={K}", "GB/s", 1.75 * N * K / 1e6, t_ref, t_new, same_prune)
    t_ref = timed(lambda: O.ref().ref_pack_metadata(O.tp(raw_r), O.tp(packed_r), N, K, st), ITERS, flush)
    t_new = timed(lambda: C.pack_metadata(raw, packed, N, K), ITERS, flush)
    report("pack_metadata", f"N={N} K={K}", "GB/s", 0.375 * N * K / 1e6, t_ref, t_new, same_pack)

    # INT8 conv callers (the reference runs im2col / quantize / GEMM / transpose per sample).
    for (N, Ci, H, W, Co) in [(1, 16, 540, 960, 32), (1, 16, 1080, 1920, 32), (4, 64, 128, 128, 64)]:
        g = torch.Generator(device=DEV).manual_seed(12)
        x = torch.randn((N, Ci, H, W), device=DEV, generator=g).half()
        wq = rand_i8((Co, Ci * 9), 13)
        _, w, b = scales(1, Co, 4)
        o_ref = O.ref_int8_conv2d(x, wq, w, b, 3, 3, 1, 1, 1, 1, 1, 1)
        o_new = C.int8_conv2d_forward(x, wq, w, b, (3, 3), (1, 1))
        ws = torch.empty(int(O.ref().ref_int8_conv2d_workspace_size(Ci, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1)) + 16,
                         dtype=torch.uint8, device=DEV)
        st = O.cur_stream()
        t_ref = timed(lambda: O.ref().ref_int8_conv2d_forward(O.tp(x), O.tp(wq), O.tp(w), O.tp(b), O.tp(o_ref), N,
                                                               Ci, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1, O.tp(ws), st),
                      ITERS, flush)
        t_new = timed(lambda: C.int8_conv2d_forward(x, wq, w, b, (3, 3), (1, 1)), ITERS, flush)
        report("int8_conv2d_forward 3x3", f"N={N} C_in={Ci} {H}x{W} C_out={Co}", "GB/s (input + output bytes)",
               (2.0 * x.numel() + 2.0 * o_new.numel() + wq.numel()) / 1e6, t_ref, t_new, torch.equal(o_ref, o_new))
        wt = rand_i8((4 * Co, Ci), 14)
        o_ref = O.ref_int8_conv_transpose2d_k2s2(x, wt, w, b)
        o_new = C.int8_conv_transpose2d_k2s2_forward(x, wt, w, b)
        ws = torch.empty(int(O.ref().ref_int8_conv_transpose2d_k2s2_workspace_size(Ci, H, W, Co)) + 16,
                         dtype=torch.uint8, device=DEV)
        t_ref = timed(lambda: O.ref().ref_int8_conv_transpose2d_k2s2_forward(O.tp(x), O.tp(wt), O.tp(w), O.tp(b),
                                                                              O.tp(o_ref), N, Ci, H, W, Co, O.tp(ws),
                                                                              st), ITERS, flush)
        t_new = timed(lambda: C.int8_conv_transpose2d_k2s2_forward(x, wt, w, b), ITERS, flush)
        report("int8_conv_transpose2d_k2s2", f"N={N} C_in={Ci} {H}x{W} C_out={Co}", "GB/s (input + output bytes)",
               (2.0 * x.numel() + 2.0 * o_new.numel() + wt.numel()) / 1e6, t_ref, t_new, torch.equal(o_ref, o_new))
        del x, o_ref, o_new, ws


    lines = ["| entry point | shape | reference kernel on B200 | this library | unit | speed-up | bit-identical |",
             "|---|---|---|---|---|---|---|"]
    for r in rows:
        lines.append(f"| {r['case']} | {r['shape']} | {r['reference']:.1f} ({r['reference_ms']:.4f} ms) | "
                     f"{r['b200']:.1f} ({r['b200_ms']:.4f} ms) | {r['unit']} | {r['speedup']:.1f}x | "
                     f"{'yes' if r['bit_identical'] else 'NO'} |")
    table = "\n".join(lines)
    print("\n" + table)
    path = os.environ.get("FORGE_B200_SPEED_TABLE")
    if path:
        with open(path, "w") as f:
            f.write(table + "\n")
    assert C.device_status() == 0
    assert all(r["bit_identical"] for r in rows), [r["case"] + " " + r["shape"] for r in rows if not r["bit_identical"]]
    # rows of a few tens of microseconds are launch-bound on both sides and noisy: wider margin there
    slower = [(r["case"], r["shape"], r["reference_ms"], r["b200_ms"]) for r in rows
              if r["b200_ms"] > (1.3 if r["reference_ms"] < 0.03 else 1.1) * r["reference_ms"]]
    assert not slower, f"slower than the reference kernel: {slower}"


def _cpu_baselines():
    """The CPU oracle (OpenMP C restatement of the reference's host loops) on this machine's cores, best of
    five: the 1024^3 INT32 GEMM in full, per-token quantize and dequant + bias of a 4096 x 4096 activation in
    full, and a 64-row slice of the 8192^3 GEMM with its linear extrapolation. A reported baseline, not a target."""
    import time

    import numpy as np
    rng = np.random.default_rng(1234)
    threads = O.oracle().oracle_num_threads()
    out = [f"| CPU oracle case ({threads} host threads) | best of 5 | rate |", "|---|---|---|"]

    def best(fn):
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    A = rng.integers(-127, 128, (1024, 1024), dtype=np.int8)
    B = rng.integers(-127, 128, (1024, 1024), dtype=np.int8)
    t = best(lambda: O.gemm_s32(A, B))
    out.append(f"| INT32 GEMM 1024^3 (full) | {t * 1e3:.2f} ms | {2 * 1024 ** 3 / t / 1e12:.4f} TOP/s |")
    x = rng.standard_normal((4096, 4096)).astype(np.float16)
    t = best(lambda: O.quantize(x))
    out.append(f"| quantize 4096 x 4096 (full) | {t * 1e3:.2f} ms | {(3 * 4096 * 4096 + 4 * 4096) / t / 1e9:.2f} GB/s |")
    acc = rng.integers(-(1 << 20), 1 << 20, (4096, 4096), dtype=np.int32)
    a_s = rng.random(4096, dtype=np.float32)
    w_s = rng.random(4096, dtype=np.float32).astype(np.float16)
    b = rng.random(4096, dtype=np.float32).astype(np.float16)
    t = best(lambda: O.dequantize_bias(acc, a_s, w_s, b))
    out.append(f"| dequant + bias 4096 x 4096 (full) | {t * 1e3:.2f} ms | {6 * 4096 * 4096 / t / 1e9:.2f} GB/s |")
    A = rng.integers(-127, 128, (64, 8192), dtype=np.int8)
    B = rng.integers(-127, 128, (8192, 8192), dtype=np.int8)
    t = best(lambda: O.gemm_s32(A, B))
    out.append(f"| INT32 GEMM 8192^3, 64-row slice | {t * 1e3:.1f} ms | {2 * 64 * 8192 ** 2 / t / 1e12:.4f} TOP/s "
               f"(whole GEMM extrapolated linearly: {t * 128:.1f} s) |")
    return out




def test_cpu_oracle_rates_on_this_host():
    rows = _cpu_baselines()
    print("\n" + "\n".join(rows))
    path = os.environ.get("FORGE_B200_CPU_TABLE")
    if path:
        with open(path, "w") as f:
            f.write("\n".join(rows) + "\n")
    assert len(rows) == 6
