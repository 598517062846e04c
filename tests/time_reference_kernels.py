"""Times the reference's own CUDA kernels (built for sm_100a under oracle/_ref, test
infrastructure) next to this library's kernels with one harness: CUDA events around a single
call, 256 MiB written between calls so operands come from HBM, median of `--iters` calls after
three warm-ups. Not a pytest file; run it on a B200:

    python tests/time_reference_kernels.py [--iters 10] [--out table.md]

Prints one JSON line per case and, at the end, a markdown table. The two sides of every row are
first compared bit for bit on the same inputs (the parity tests do that at more shapes)."""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import oracle_lib as ol  # noqa: E402
from forge_b200 import _forge_C as C  # noqa: E402

DEV = "cuda:0"


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


def cpu_baselines():
    """The CPU oracle (OpenMP C restatement of the reference's host loops) on this machine's cores, best of
    five: the 1024^3 INT32 GEMM in full, per-token quantize and dequant + bias of a 4096 x 4096 activation in
    full, and a 64-row slice of the 8192^3 GEMM with its linear extrapolation. A reported baseline, not a target."""
    import time

    import numpy as np
    rng = np.random.default_rng(1234)
    threads = ol.oracle().oracle_num_threads()
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
    t = best(lambda: ol.gemm_s32(A, B))
    out.append(f"| INT32 GEMM 1024^3 (full) | {t * 1e3:.2f} ms | {2 * 1024 ** 3 / t / 1e12:.4f} TOP/s |")
    x = rng.standard_normal((4096, 4096)).astype(np.float16)
    t = best(lambda: ol.quantize(x))
    out.append(f"| quantize 4096 x 4096 (full) | {t * 1e3:.2f} ms | {(3 * 4096 * 4096 + 4 * 4096) / t / 1e9:.2f} GB/s |")
    acc = rng.integers(-(1 << 20), 1 << 20, (4096, 4096), dtype=np.int32)
    a_s = rng.random(4096, dtype=np.float32)
    w_s = rng.random(4096, dtype=np.float32).astype(np.float16)
    b = rng.random(4096, dtype=np.float32).astype(np.float16)
    t = best(lambda: ol.dequantize_bias(acc, a_s, w_s, b))
    out.append(f"| dequant + bias 4096 x 4096 (full) | {t * 1e3:.2f} ms | {6 * 4096 * 4096 / t / 1e9:.2f} GB/s |")
    A = rng.integers(-127, 128, (64, 8192), dtype=np.int8)
    B = rng.integers(-127, 128, (8192, 8192), dtype=np.int8)
    t = best(lambda: ol.gemm_s32(A, B))
    out.append(f"| INT32 GEMM 8192^3, 64-row slice | {t * 1e3:.1f} ms | {2 * 64 * 8192 ** 2 / t / 1e12:.4f} TOP/s "
               f"(whole GEMM extrapolated linearly: {t * 128:.1f} s) |")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    ap.add_argument("--cpu", type=int, default=1, help="also time the CPU oracle on this host (reported baseline)")
    ap.add_argument("--only-cpu", type=int, default=0, help="print the CPU oracle timings and stop")
    args = ap.parse_args()
    if args.only_cpu:
        print("\n".join(cpu_baselines()))
        return
    if not ol.ref_available():
        raise SystemExit("oracle/_ref/libforge_ref.so is not built")
    torch.cuda.set_device(0)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=DEV)
    rows = []

    def report(case, shape, unit, work, t_ref, t_new, same):
        # work is scaled so that work / milliseconds is already in the stated unit
        r = {"case": case, "shape": shape, "reference_ms": t_ref, "b200_ms": t_new,
             "reference": work / t_ref, "b200": work / t_new, "unit": unit,
             "speedup": t_ref / t_new, "bit_identical": bool(same)}
        rows.append(r)
        print(json.dumps(r), flush=True)

    # Dense INT8 GEMM + dequant (wmma kernel of the reference).
    for (M, N, K) in [(4096, 4096, 4096), (8192, 8192, 8192)]:
        A, B = rand_i8((M, K), 1234), rand_i8((N, K), 1235)
        a, w, b = scales(M, N, 1)
        o_ref = ol.ref_int8_gemm_dequant(A, B, a, w, b)
        o_new = C.int8_gemm_dequant(A, B, a, w, b)
        t_ref = timed(lambda: ol.ref_int8_gemm_dequant(A, B, a, w, b), args.iters, flush)
        t_new = timed(lambda: C.int8_gemm_dequant(A, B, a, w, b), args.iters, flush)
        report("int8_gemm_dequant", f"M={M} N={N} K={K}", "TOP/s", 2.0 * M * N * K / 1e9, t_ref, t_new,
               torch.equal(o_ref, o_new))
        del A, B, o_ref, o_new

    # 2:4-sparse INT8 GEMM (mma.sp kernel of the reference, its own plan), dense-equivalent rate.
    for (M, N, K) in [(1, 11008, 4096), (16, 11008, 4096), (128, 11008, 4096), (2048, 11008, 4096),
                      (8192, 11008, 4096), (8192, 8192, 8192)]:
        W = rand_i8((N, K), 77)
        comp, _, meta = ol.ref_prune_pack(W)
        x = rand_i8((M, K), 78)
        a, w, b = scales(M, N, 2)
        o_ref = ol.ref_sparse_int8_gemm(comp, x, meta, a, w, b)
        o_new = C.sparse_int8_gemm(comp, x, meta, a, w, b)
        t_ref = timed(lambda: ol.ref_sparse_int8_gemm(comp, x, meta, a, w, b), args.iters, flush)
        t_new = timed(lambda: C.sparse_int8_gemm(comp, x, meta, a, w, b), args.iters, flush)
        report("sparse_int8_gemm", f"M={M} N={N} K={K}", "TOP/s (dense-equivalent)", 2.0 * M * N * K / 1e9,
               t_ref, t_new, torch.equal(o_ref, o_new))
        del W, comp, meta, x, o_ref, o_new

    # Per-token quantize.
    for (M, K) in [(4096, 4096), (16384, 8192)]:
        g = torch.Generator(device=DEV).manual_seed(5)
        x = torch.randn((M, K), device=DEV, generator=g).half()
        q_ref, s_ref = ol.ref_quantize(x)
        q_new, s_new = C.fused_quantize_activation(x, M, K)
        t_ref = timed(lambda: ol.ref_quantize(x), args.iters, flush)
        t_new = timed(lambda: C.fused_quantize_activation(x, M, K), args.iters, flush)
        report("fused_quantize_activation", f"M={M} K={K}", "GB/s", (3.0 * M * K + 4 * M) / 1e6, t_ref,
               t_new, torch.equal(q_ref, q_new) and torch.equal(s_ref, s_new))
        del x

    # Dequant + bias.
    for (M, N) in [(4096, 4096), (8192, 8192)]:
        g = torch.Generator(device=DEV).manual_seed(6)
        acc = torch.randint(-(1 << 20), 1 << 20, (M, N), dtype=torch.int32, device=DEV, generator=g)
        a, w, b = scales(M, N, 3)
        o_ref = ol.ref_dequantize_bias(acc, a, w, b)
        o_new = C.fused_dequantize_bias(acc, a, w, b, M, N)
        t_ref = timed(lambda: ol.ref_dequantize_bias(acc, a, w, b), args.iters, flush)
        t_new = timed(lambda: C.fused_dequantize_bias(acc, a, w, b, M, N), args.iters, flush)
        report("fused_dequantize_bias", f"M={M} N={N}", "GB/s", (6.0 * M * N + 4 * (M + N)) / 1e6, t_ref,
               t_new, torch.equal(o_ref, o_new))
        del acc

    # Prune + compress and metadata pack.
    N, K = 28672, 8192
    W = rand_i8((N, K), 9)
    comp_r, raw_r, packed_r = ol.ref_prune_pack(W)
    comp = torch.empty_like(comp_r)
    raw = torch.empty_like(raw_r)
    packed = torch.empty_like(packed_r)
    C.prune_compress_24(W, comp, raw, N, K)
    C.pack_metadata(raw, packed, N, K)
    same_prune = torch.equal(comp, comp_r) and torch.equal(raw, raw_r)
    same_pack = torch.equal(packed, packed_r)
    st = ol.cur_stream()
    t_ref = timed(lambda: ol.ref().ref_prune_compress_24(ol.tp(W), ol.tp(comp_r), ol.tp(raw_r), N, K, st),
                  args.iters, flush)
    t_new = timed(lambda: C.prune_compress_24(W, comp, raw, N, K), args.iters, flush)
    report("prune_compress_24", f"N={N} K={K}", "GB/s", 1.75 * N * K / 1e6, t_ref, t_new, same_prune)
    t_ref = timed(lambda: ol.ref().ref_pack_metadata(ol.tp(raw_r), ol.tp(packed_r), N, K, st), args.iters, flush)
    t_new = timed(lambda: C.pack_metadata(raw, packed, N, K), args.iters, flush)
    report("pack_metadata", f"N={N} K={K}", "GB/s", 0.375 * N * K / 1e6, t_ref, t_new, same_pack)

    # INT8 conv callers (the reference runs im2col / quantize / GEMM / transpose per sample).
    for (N, Ci, H, W, Co) in [(1, 16, 540, 960, 32), (1, 16, 1080, 1920, 32), (4, 64, 128, 128, 64)]:
        g = torch.Generator(device=DEV).manual_seed(12)
        x = torch.randn((N, Ci, H, W), device=DEV, generator=g).half()
        wq = rand_i8((Co, Ci * 9), 13)
        _, w, b = scales(1, Co, 4)
        o_ref = ol.ref_int8_conv2d(x, wq, w, b, 3, 3, 1, 1, 1, 1, 1, 1)
        o_new = C.int8_conv2d_forward(x, wq, w, b, (3, 3), (1, 1))
        ws = torch.empty(int(ol.ref().ref_int8_conv2d_workspace_size(Ci, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1)) + 16,
                         dtype=torch.uint8, device=DEV)
        st = ol.cur_stream()
        t_ref = timed(lambda: ol.ref().ref_int8_conv2d_forward(ol.tp(x), ol.tp(wq), ol.tp(w), ol.tp(b), ol.tp(o_ref), N,
                                                               Ci, H, W, Co, 3, 3, 1, 1, 1, 1, 1, 1, ol.tp(ws), st),
                      args.iters, flush)
        t_new = timed(lambda: C.int8_conv2d_forward(x, wq, w, b, (3, 3), (1, 1)), args.iters, flush)
        report("int8_conv2d_forward 3x3", f"N={N} C_in={Ci} {H}x{W} C_out={Co}", "GB/s (input + output bytes)",
               (2.0 * x.numel() + 2.0 * o_new.numel() + wq.numel()) / 1e6, t_ref, t_new, torch.equal(o_ref, o_new))
        wt = rand_i8((4 * Co, Ci), 14)
        o_ref = ol.ref_int8_conv_transpose2d_k2s2(x, wt, w, b)
        o_new = C.int8_conv_transpose2d_k2s2_forward(x, wt, w, b)
        ws = torch.empty(int(ol.ref().ref_int8_conv_transpose2d_k2s2_workspace_size(Ci, H, W, Co)) + 16,
                         dtype=torch.uint8, device=DEV)
        t_ref = timed(lambda: ol.ref().ref_int8_conv_transpose2d_k2s2_forward(ol.tp(x), ol.tp(wt), ol.tp(w), ol.tp(b),
                                                                              ol.tp(o_ref), N, Ci, H, W, Co, ol.tp(ws),
                                                                              st), args.iters, flush)
        t_new = timed(lambda: C.int8_conv_transpose2d_k2s2_forward(x, wt, w, b), args.iters, flush)
        report("int8_conv_transpose2d_k2s2", f"N={N} C_in={Ci} {H}x{W} C_out={Co}", "GB/s (input + output bytes)",
               (2.0 * x.numel() + 2.0 * o_new.numel() + wt.numel()) / 1e6, t_ref, t_new, torch.equal(o_ref, o_new))
        del x, o_ref, o_new, ws

    if args.cpu:
        cpu_rows = cpu_baselines()
        print("\n".join(cpu_rows))
        if args.out:
            with open(args.out + ".cpu.md", "w") as f:
                f.write("\n".join(cpu_rows) + "\n")

    lines = ["| entry point | shape | reference kernel on B200 | this library | unit | speed-up | bit-identical |",
             "|---|---|---|---|---|---|---|"]
    for r in rows:
        lines.append(f"| {r['case']} | {r['shape']} | {r['reference']:.1f} ({r['reference_ms']:.4f} ms) | "
                     f"{r['b200']:.1f} ({r['b200_ms']:.4f} ms) | {r['unit']} | {r['speedup']:.1f}x | "
                     f"{'yes' if r['bit_identical'] else 'NO'} |")
    table = "\n".join(lines)
    print(table)
    if args.out:
        with open(args.out, "w") as f:
            f.write(table + "\n")


if __name__ == "__main__":
    main()
