#!/usr/bin/env python
"""Benchmark of the forge_b200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (every N): the headline of the metric, the dense INT8 GEMM with fused dequant + bias
at M = N = K = 8192 per GPU (forge::gemm::int8_gemm_dequant), int8 operands uniform in
[-127,127] from seeded Philox streams. A "step" is one call on one batch of activations.
  value : whole-job INT8 TOPS (2*M*N*K per step per GPU) with inputs resident in HBM.
  e2e   : the same call through the C ABI with HOST buffers: the step's activations and
          their scales are copied from pinned host memory and the FP16 result is copied back,
          inside the timed region (three streams, copies overlapped with the kernel);
          copy_only_ms_per_step is the same loop with the kernel call removed.
  sustained : the same kernel back to back for >= 0.6 s with the SM clock sampled, as TOPS and as
          operations per clock per SM.
  extras : the other figures of the metric on one GPU - 2:4-sparse GEMM at 8192^3, the W8A8 gated
          MLP block (tokens/s, dense and 2:4), quantize / dequant GB/s.
With N > 1 (torchrun, one rank per GPU) token rows are sharded: every rank runs the same
per-GPU workload on its own rows, no collective on the data path ("weak" scaling), and
  sharded : the sharded workloads on the N GPUs - the gated MLP block with token rows sharded
          (tokens/s), the 65536 x 8192 -> 28672 2:4-sparse layer sharded by token rows and by output
          channels (all-gather done by the GEMM epilogue's peer stores), with a bitwise check of
          sampled rows against a local recomputation.

--impl reference times the reference's host int32 GEMM + dequant loop (the CPU restatement in
oracle/, all host threads) on a bounded row sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
OPS_PER_STEP = 2.0 * M * N * K
METRIC = "int8_gemm_dequant_tops_m8192_n8192_k8192"
UNIT = "TOPS"
CPU_SAMPLE_ROWS = 256
NOMINAL_DENSE_TOPS = 4500.0    # datasheet dense INT8 rate of a B200; 2:4-sparse is twice that
HEADLINE_KERNEL_PROFILE = "dense_pair_kernel_8192.md"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


def _traffic_from_profile(name):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu summary of the
    headline kernel (mean over the captured launches); None when the summary is not there."""
    import re
    path = os.path.join(ROOT, "profiles", name)
    if not os.path.exists(path):
        return None
    total = 0.0
    for metric in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"\|\s*`" + re.escape(metric) + r"`\s*\|(.*)\|", open(path).read())
        if m is None:
            return None
        vals = [float(v) * {"Mbyte": 1e6, "Gbyte": 1e9, "Kbyte": 1e3}[u]
                for v, u in re.findall(r"([0-9.]+)\s*(Mbyte|Gbyte|Kbyte)", m.group(1))]
        if not vals:
            return None
        total += sum(vals) / len(vals)
    return total


def _config(world):
    return {"workload": "int8_gemm_dequant M=N=K=8192 per GPU (headline shape of the metric)",
            "operands": "int8 uniform [-127,127], seeded Philox; fp32 token scales, fp16 channel scales + bias",
            "sharding": "token rows, one shard per GPU, no collective" if world > 1 else "single GPU",
            "l2": "3 rotating activation/output buffer sets, 256 MiB touched per step (L2 is 126 MB)"}


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons through NVML (read-only) while `active` is set."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.active = threading.Event()
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
                getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._halt.is_set():
                # wakes up as soon as the timed region starts (a region of 20 steps lasts a few milliseconds)
                if not self.active.wait(timeout=0.02):
                    continue
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = get_reasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.0005)
        except Exception as e:  # clocks are evidence, not the product: report the failure, keep benchmarking
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._halt.set()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": sorted(self.reasons)}


def _cpu_baseline(rows, reps):
    """Reference host loop (int32 GEMM + dequant) on `rows` token rows of the workload."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    # all the cores this process may run on, whatever OMP_NUM_THREADS a launcher exported
    O.oracle().oracle_set_num_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(1234)
    A = rng.integers(-127, 128, (rows, K), dtype=np.int8)
    B = rng.integers(-127, 128, (N, K), dtype=np.int8)
    a_s = rng.random(rows, dtype=np.float32) * 0.05
    w_s = (rng.random(N, dtype=np.float32) * 0.05).astype(np.float16)
    bias = (rng.random(N, dtype=np.float32) - 0.5).astype(np.float16)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        acc = O.gemm_s32(A, B)
        O.dequantize_bias(acc, a_s, w_s, bias, gemm_epilogue=True)
        times.append(time.perf_counter() - t0)
    return times, O.oracle().oracle_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # size the per-step row sample so that warmup + steps take about a minute of host time
    probe, _ = _cpu_baseline(8, 2)
    rows_per_s = 8 / min(probe)
    budget_s = float(os.environ.get("FORGE_B200_REFERENCE_SECONDS", "60"))   # host time for warmup + steps
    rows = int(max(1, min(CPU_SAMPLE_ROWS, rows_per_s * budget_s / (args.warmup + args.steps))))
    times, cores = _cpu_baseline(rows, args.warmup + args.steps)
    timed = times[args.warmup:]
    total = sum(timed)
    tops = 2.0 * rows * N * K * len(timed) / total / 1e12
    sample = f"{rows} of {M} token rows per step (int32 GEMM + dequant host loop, OpenMP)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(timed), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": _config(int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def _median_ms(fn, steps, warmup, flush=None):
    """Median CUDA-event time of `steps` single calls after `warmup` calls; `flush` (a buffer larger
    than L2) is rewritten before each timed call so operands come from HBM."""
    import torch
    for _ in range(warmup):
        assert fn() == 0
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        assert fn() == 0
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def _ceilings(lib, dev, sm_mhz):
    """The two rates that bound the GEMM kernels, measured on this GPU by the library's built-in probes:
    clocks per tcgen05.mma kind::i8 instruction with operands resident in shared memory (dense and
    2:4-sparse, in the tile shapes the pair kernels use, with their one commit per four instructions), and
    the bytes per clock one SM receives from L2 through TMA when every SM pulls at once. TOP/s figures are
    at `sm_mhz` (the clock sampled during the timed region)."""
    import torch
    n_sms = torch.cuda.get_device_properties(dev).multi_processor_count
    out = {}
    try:
        dense = lib.forge_b200_probe_mma_rate(1, 256, 0, 1, n_sms)
        sparse = lib.forge_b200_probe_mma_rate(1, 224, 1, 1, n_sms)
        out["dense_pair_n256_clocks_per_mma"] = dense
        out["sparse_pair_n224_clocks_per_mma"] = sparse
        out["dense_ops_per_clock_per_sm"] = 2.0 * 128 * 256 * 32 / dense
        out["sparse_dense_equiv_ops_per_clock_per_sm"] = 2.0 * 128 * 224 * 64 / sparse
        buf = torch.randint(-127, 128, (8192, 4096), dtype=torch.int8, device=dev)   # 32 MB: L2 resident
        out["tma_ingest_bytes_per_clock_one_sm"] = lib.forge_b200_probe_tma_ingest(buf.data_ptr(), 8192, 4096, 4, 1)
        out["tma_ingest_bytes_per_clock_per_sm_all_sms"] = lib.forge_b200_probe_tma_ingest(buf.data_ptr(), 8192, 4096,
                                                                                           4, n_sms)
        if sm_mhz:
            out["dense_tensor_ceiling_tops_at_sampled_clock"] = out["dense_ops_per_clock_per_sm"] * n_sms * sm_mhz * 1e6 / 1e12
            out["sparse_tensor_ceiling_tops_at_sampled_clock"] = (out["sparse_dense_equiv_ops_per_clock_per_sm"] * n_sms *
                                                                 sm_mhz * 1e6 / 1e12)
            out["l2_to_sm_TBps_at_sampled_clock"] = (out["tma_ingest_bytes_per_clock_per_sm_all_sms"] * n_sms * sm_mhz *
                                                     1e6 / 1e12)
        if lib.forge_b200_device_status(1) != 0:
            out["error"] = "a probe gave up on a bounded wait"
    except Exception as e:
        out["error"] = f"{type(e).__name__}: {e}"
    return out


def _single_gpu_extras(lib, dev, peaks):
    """The other figures of the metric, measured in the same run on this rank's GPU: 2:4-sparse GEMM at
    8192^3, the W8A8 gated MLP block (8192 tokens, 4096 -> 14336 -> 4096, dense and 2:4), and the
    quantize / dequant kernels against the measured HBM copy bandwidth. Each is the median of 10 single
    launches with a 256 MiB L2 flush in between (the protocol of the --case runs)."""
    import types

    import torch
    from forge_b200 import _forge_C as C
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    S = [torch.cuda.current_stream().cuda_stream]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {}

    def case(name, **kw):
        a = types.SimpleNamespace(m=0, n=0, k=0, height=1080, width=1920, ksize=3)
        a.__dict__.update(kw)
        fn, work, unit, bound, shape = _build_case(name, a, lib, C, dev, g, S)
        ms = _median_ms(fn, 10, 3, flush)
        torch.cuda.synchronize()
        return ms, work / (ms * 1e-3), shape

    try:
        ms, rate, _ = case("sparse")
        out["sparse_8192"] = {
            "ms": ms, "dense_equiv_tops": rate, "executed_tops": rate / 2.0,
            "frac_of_2x_measured_bf16_burst": rate / (2.0 * peaks["bf16_burst"]),
            "frac_of_nominal_sparse_9000": rate / (2.0 * NOMINAL_DENSE_TOPS),
            "kernel": "sparse_pair_kernel<224,1> (tcgen05.mma.sp cta_group::2 kind::i8, 256 weight rows x 224 tokens)"}
        for name in ("mlp", "mlp_sparse"):
            ms, rate, shape = case(name)
            out[name] = {"ms": ms, "tokens_per_s": shape["tokens"] / (ms * 1e-3), "dense_equiv_tops": rate,
                         "shape": shape}
        for key, name, kw in (("quantize_4096x4096", "quantize", {"m": 4096, "k": 4096}),
                              ("quantize_16384x8192", "quantize", {"m": 16384, "k": 8192}),
                              ("dequant_4096x4096", "dequant", {"m": 4096, "n": 4096}),
                              ("dequant_16384x8192", "dequant", {"m": 16384, "n": 8192})):
            ms, rate, _ = case(name, **kw)
            out[key] = {"ms": ms, "GBps": rate, "frac_of_measured_hbm": rate / peaks["hbm"],
                        "frac_of_nominal_8000": rate / 8000.0}
        out["peak_source"] = peaks["source"]
    except Exception as e:   # the headline line must survive a failure here; the failure is reported
        out["error"] = f"{type(e).__name__}: {e}"
    del flush
    torch.cuda.empty_cache()
    return out


def run_b200(args):
    import datetime

    import torch
    import torch.distributed as dist
    from forge_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    lib = _lib.load()   # raises if libforge_b200.so is missing: there is no fallback
    n_sms = torch.cuda.get_device_properties(dev).multi_processor_count

    NSETS = 3   # activation/output buffer sets rotated between steps: 256 MiB touched per step > 126 MB L2
    g = torch.Generator(device=dev)
    g.manual_seed(1235)
    B = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=dev)
    w_s = (torch.rand(N, generator=g, device=dev) * 0.02 + 0.001).to(torch.float16)
    bias = (torch.randn(N, generator=g, device=dev) * 0.01).to(torch.float16)
    A, a_s, out = [], [], []
    for i in range(NSETS):
        g.manual_seed(1234 + 100 * rank + i)
        A.append(torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=dev))
        a_s.append(torch.rand(M, generator=g, device=dev) * 0.05 + 0.001)
        out.append(torch.empty((M, N), dtype=torch.float16, device=dev))
    stream = torch.cuda.current_stream()

    def step(i, s=None):
        j = i % NSETS
        st = lib.forge_int8_gemm_dequant(A[j].data_ptr(), B.data_ptr(), a_s[j].data_ptr(), w_s.data_ptr(),
                                         bias.data_ptr(), out[j].data_ptr(), M, K, N,
                                         (s or stream).cuda_stream)
        if st != 0:
            raise RuntimeError(f"forge_int8_gemm_dequant returned {st}")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()

    # ---- device-resident throughput: exactly `steps` calls
    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.active.set()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    sampler.active.clear()
    ms = e0.elapsed_time(e1)
    if lib.forge_b200_device_status(1) != 0:
        raise RuntimeError("a forge_b200 kernel gave up on a bounded wait")
    clocks = sampler.summary()

    # ---- the same kernel back to back for at least 0.6 s: the power-capped regime, with the SM clock
    # sampled every 20 ms so that work per clock can be told apart from the clock itself
    sus_steps = max(args.steps, int(600.0 / max(ms / args.steps, 1e-3)) + 1)
    sus = ClockSampler(local)
    sus.start()
    barrier()
    e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sus.active.set()
    e4.record(stream)
    for i in range(sus_steps):
        step(i)
    e5.record(stream)
    barrier()
    sus.active.clear()
    sus.stop()
    sus_ms = e4.elapsed_time(e5)
    sus_clk = sus.summary()

    # ---- end to end: host buffers in, host buffers out, every step
    hA = [torch.randint(-127, 128, (M, K), dtype=torch.int8).pin_memory() for _ in range(2)]
    h_as = [torch.rand(M).pin_memory() for _ in range(2)]
    h_out = [torch.empty((M, N), dtype=torch.float16).pin_memory() for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(NSETS)]
    ev_run = [torch.cuda.Event() for _ in range(NSETS)]
    ev_out = [torch.cuda.Event() for _ in range(NSETS)]

    def e2e_loop(n, with_kernel=True):
        for i in range(n):
            j = i % NSETS
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_run[j])          # the kernel that last read this set is done
                A[j].copy_(hA[i % 2], non_blocking=True)
                a_s[j].copy_(h_as[i % 2], non_blocking=True)
                ev_in[j].record(s_in)
            s_run.wait_event(ev_in[j])
            s_run.wait_event(ev_out[j])             # the copy-out that last read this output is done
            if with_kernel:
                step(i, s_run)
            ev_run[j].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[j])
                h_out[i % 2].copy_(out[j], non_blocking=True)
                ev_out[j].record(s_out)

    def timed_e2e(n, with_kernel):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(s_in)
        e2e_loop(n, with_kernel)
        s_out.synchronize()
        b.record(s_out)
        barrier()
        return a.elapsed_time(b)

    e2e_warm = min(args.warmup, 5)
    e2e_steps = min(args.steps, 200)   # each step moves 192 MiB over PCIe; bounded so defaults stay in minutes
    e2e_loop(e2e_warm)
    e2e_ms = timed_e2e(e2e_steps, True)
    copy_ms = timed_e2e(e2e_steps, False)   # the same loop without the kernel: the floor set by the copies
    sampler.stop()

    times = torch.tensor([ms, e2e_ms, sus_ms, copy_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, sus_ms, copy_ms = times.tolist()

    peaks = _peaks()
    extras = _single_gpu_extras(lib, dev, peaks) if rank == 0 else None
    ceilings = _ceilings(lib, dev, clocks["sm_mhz"]) if rank == 0 else None
    sharded = None
    if world > 1:
        barrier()
        sharded = _sharded_extras(world, rank, dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    value = OPS_PER_STEP * args.steps * world / (ms * 1e-3) / 1e12
    e2e_value = OPS_PER_STEP * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
    launch_ms = ms / args.steps
    sustained_region = ms > 250.0
    peak_bf16 = peaks["bf16_sustained"] if sustained_region else peaks["bf16_burst"]
    achieved = OPS_PER_STEP / (launch_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": 2.0 * peak_bf16, "unit": "TOP/s",
        "frac": achieved / (2.0 * peak_bf16), "traffic": _traffic_from_profile(HEADLINE_KERNEL_PROFILE),
        "kernel": "dense_pair_kernel<1> (tcgen05.mma cta_group::2 kind::i8, 256x256 tiles per SM pair)",
        "peak_basis": f"2 x {'sustained' if sustained_region else 'burst'} cuBLAS bf16 TFLOP/s of {peaks['source']} "
                      "(kind::i8 issues at twice the bf16 rate); nominal dense int8 is 4500",
        "frac_of_nominal_4500": achieved / NOMINAL_DENSE_TOPS,
        # the tensor pipe's own rate on this GPU (built-in probe) at the clock sampled during the timed region
        "frac_of_measured_tensor_ceiling": (achieved / ceilings["dense_tensor_ceiling_tops_at_sampled_clock"])
        if ceilings and ceilings.get("dense_tensor_ceiling_tops_at_sampled_clock") else None,
    }
    sus_tops = OPS_PER_STEP * sus_steps / (sus_ms * 1e-3) / 1e12
    sustained = {
        "steps": sus_steps, "seconds": sus_ms * 1e-3, "tops_per_gpu": sus_tops,
        "frac_of_2x_measured_bf16_sustained": sus_tops / (2.0 * peaks["bf16_sustained"]),
        "frac_of_nominal_4500": sus_tops / NOMINAL_DENSE_TOPS, "clocks": sus_clk,
        # 2*M*N*K per launch / (launch time x median SM clock x SMs); the tensor pipe's own limit is
        # 16384 per clock per SM (8192 MACs), measured 15060 with operands resident in shared memory
        "ops_per_clock_per_sm": (OPS_PER_STEP * sus_steps / (sus_ms * 1e-3) / (sus_clk["sm_mhz"] * 1e6) / n_sms)
        if sus_clk["sm_mhz"] else None,
        "burst_ops_per_clock_per_sm": (OPS_PER_STEP / (launch_ms * 1e-3) / (clocks["sm_mhz"] * 1e6) / n_sms)
        if clocks["sm_mhz"] else None,
    }
    cpu = None
    if world == 1:
        times_cpu, cores = _cpu_baseline(CPU_SAMPLE_ROWS, 3)
        best = min(times_cpu)
        cpu = {"value": 2.0 * CPU_SAMPLE_ROWS * N * K / best / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{CPU_SAMPLE_ROWS} of {M} token rows, best of 3 (int32 GEMM + dequant host loop, OpenMP)"}
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": launch_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic", "config": _config(world),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M * K + 4 * M, "d2h_bytes_per_step": 2 * M * N,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "copy_only_ms_per_step": copy_ms / e2e_steps,
                "note": "weights resident; activations+scales copied in and FP16 result copied out every step; "
                        "copy_only = the same three-stream loop with the kernel call removed"},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": roofline,
        "sustained": sustained,
        "cpu_baseline": cpu,
        "extras": extras,
        "ceilings": ceilings,
        "sharded": sharded,
    }))
    if world > 1:
        dist.destroy_process_group()


def _build_case(name, args, lib, C, dev, g, S):
    """One complete operand set on `dev` + the call on it, for the single-kernel case `name`:
    returns (fn, work per call, unit of work/s, bound, shape). S[0] is the stream handle the call uses."""
    import torch

    def ri8(*shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8, device=dev)

    work, unit, bound = None, None, None
    if name in ("dense", "dense_s32", "sparse", "sparse_s32"):
        m, n, k = args.m or 8192, args.n or 8192, args.k or 8192
        a_s = torch.rand(m, generator=g, device=dev) * 0.05 + 0.001
        w_s = (torch.rand(n, generator=g, device=dev) * 0.02 + 0.001).half()
        bias = (torch.randn(n, generator=g, device=dev) * 0.01).half()
        x, W = ri8(m, k), ri8(n, k)
        out = torch.empty((m, n), dtype=torch.int32 if name.endswith("s32") else torch.float16, device=dev)
        work, unit, bound = 2.0 * m * n * k / 1e12, "TOP/s", "tensor"
        if name.startswith("sparse"):
            comp = torch.empty((n, k // 2), dtype=torch.int8, device=dev)
            raw = torch.empty((n * (k // 4),), dtype=torch.uint8, device=dev)
            meta = torch.empty((n, k // 32), dtype=torch.int32, device=dev)
            C.prune_compress_24(W, comp, raw, n, k)
            C.pack_metadata(raw, meta, n, k)
            if name == "sparse":
                fn = lambda: lib.forge_sparse_int8_gemm(comp.data_ptr(), x.data_ptr(), meta.data_ptr(), a_s.data_ptr(),
                                                        w_s.data_ptr(), bias.data_ptr(), out.data_ptr(), m, k, n, 0, 1,
                                                        S[0], -1)
            else:
                fn = lambda: lib.forge_sparse_int8_gemm_s32(comp.data_ptr(), x.data_ptr(), meta.data_ptr(),
                                                            out.data_ptr(), m, k, n, S[0])
        elif name == "dense":
            fn = lambda: lib.forge_int8_gemm_dequant(x.data_ptr(), W.data_ptr(), a_s.data_ptr(), w_s.data_ptr(),
                                                     bias.data_ptr(), out.data_ptr(), m, k, n, S[0])
        else:
            fn = lambda: lib.forge_int8_gemm_s32(x.data_ptr(), W.data_ptr(), out.data_ptr(), m, k, n, S[0])
        shape = {"M": m, "N": n, "K": k}
    elif name == "linear":
        # the W8A8 linear call itself (per-token quantize + dense GEMM + dequant + bias); default = config 2
        m, n, k = args.m or 4096, args.n or 4096, args.k or 4096
        x = torch.randn((m, k), generator=g, device=dev, dtype=torch.float16)
        W = ri8(n, k)
        w_s = (torch.rand(n, generator=g, device=dev) * 0.02 + 0.001).half()
        bias = (torch.randn(n, generator=g, device=dev) * 0.01).half()
        q = torch.empty((m, k), dtype=torch.int8, device=dev)
        sc = torch.empty((m,), dtype=torch.float32, device=dev)
        out = torch.empty((m, n), dtype=torch.float16, device=dev)
        fn = lambda: lib.forge_int8_linear(x.data_ptr(), W.data_ptr(), w_s.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                           m, k, n, q.data_ptr(), sc.data_ptr(), S[0])
        work, unit, bound, shape = 2.0 * m * n * k / 1e12, "TOP/s", "tensor", {"M": m, "N": n, "K": k}
    elif name == "quantize":
        m, k = args.m or 16384, args.k or 8192
        x = torch.randn((m, k), generator=g, device=dev, dtype=torch.float16)
        q = torch.empty((m, k), dtype=torch.int8, device=dev)
        sc = torch.empty((m,), dtype=torch.float32, device=dev)
        fn = lambda: lib.forge_fused_quantize_activation(x.data_ptr(), q.data_ptr(), sc.data_ptr(), m, k, S[0])
        work, unit, bound, shape = (3.0 * m * k + 4.0 * m) / 1e9, "GB/s", "hbm", {"M": m, "K": k}
    elif name == "dequant":
        m, n = args.m or 8192, args.n or 8192
        acc = torch.randint(-50000, 50000, (m, n), generator=g, dtype=torch.int32, device=dev)
        a_s = torch.rand(m, generator=g, device=dev)
        w_s = torch.rand(n, generator=g, device=dev).half()
        bias = torch.rand(n, generator=g, device=dev).half()
        out = torch.empty((m, n), dtype=torch.float16, device=dev)
        fn = lambda: lib.forge_fused_dequantize_bias(acc.data_ptr(), a_s.data_ptr(), w_s.data_ptr(), bias.data_ptr(),
                                                     out.data_ptr(), m, n, S[0])
        work, unit, bound, shape = (6.0 * m * n + 4.0 * m + 4.0 * n) / 1e9, "GB/s", "hbm", {"M": m, "N": n}
    elif name in ("prune", "pack"):
        n, k = args.n or 28672, args.k or 8192
        W = ri8(n, k)
        comp = torch.empty((n, k // 2), dtype=torch.int8, device=dev)
        raw = torch.empty((n * (k // 4),), dtype=torch.uint8, device=dev)
        meta = torch.empty((n, k // 32), dtype=torch.int32, device=dev)
        C.prune_compress_24(W, comp, raw, n, k)
        if name == "prune":
            fn = lambda: lib.forge_prune_compress_24(W.data_ptr(), comp.data_ptr(), raw.data_ptr(), n, k, S[0])
            work = 1.75 * n * k / 1e9
        else:
            fn = lambda: lib.forge_pack_metadata(raw.data_ptr(), meta.data_ptr(), n, k, S[0])
            work = 0.375 * n * k / 1e9
        unit, bound, shape = "GB/s", "hbm", {"N": n, "K": k}
    elif name in ("sparse_linear_fused", "sparse_linear_two_pass"):
        # fp16 in -> quantize -> 2:4 GEMM -> fp16 out; the reference's showcase shape for its fused path
        # (include/forge/gemm/int8_sparse.cuh:82) by default
        m, k, n = args.m or 147456, args.k or 1280, args.n or 320
        x = torch.randn((m, k), generator=g, device=dev, dtype=torch.float16)
        W = ri8(n, k)
        comp = torch.empty((n, k // 2), dtype=torch.int8, device=dev)
        raw = torch.empty((n * (k // 4),), dtype=torch.uint8, device=dev)
        meta = torch.empty((n, k // 32), dtype=torch.int32, device=dev)
        C.prune_compress_24(W, comp, raw, n, k)
        C.pack_metadata(raw, meta, n, k)
        w_s = (torch.rand(n, generator=g, device=dev) * 0.02 + 0.001).half()
        bias = (torch.randn(n, generator=g, device=dev) * 0.01).half()
        out = torch.empty((m, n), dtype=torch.float16, device=dev)
        sq = torch.empty((m, k), dtype=torch.int8, device=dev)
        ss = torch.empty((m,), dtype=torch.float32, device=dev)
        path = 1 if name == "sparse_linear_fused" else 0
        fn = lambda: lib.forge_sparse_int8_linear(x.data_ptr(), comp.data_ptr(), meta.data_ptr(), w_s.data_ptr(),
                                                  bias.data_ptr(), out.data_ptr(), m, k, n, sq.data_ptr(),
                                                  ss.data_ptr(), 0, 1, S[0], path)
        # minimum traffic: read x (fp16) and the compressed weight once, write the fp16 output
        work, unit, bound = (2.0 * m * k + 0.625 * n * k + 2.0 * m * n) / 1e9, "GB/s", "hbm"
        shape = {"M": m, "K": k, "N": n}
    elif name in ("conv", "conv_transpose"):
        # INT8 conv2d 3x3 pad 1 (or the 2x2 stride-2 transposed conv) on a frame: --m = batch,
        # --k = C_in, --n = C_out, --height / --width
        nb, ci, co = args.m or 1, args.k or 16, args.n or 32
        hh, ww = args.height, args.width
        x = torch.randn((nb, ci, hh, ww), generator=g, device=dev, dtype=torch.float16)
        w_s = (torch.rand(co, generator=g, device=dev) * 0.02 + 0.001).half()
        bias = (torch.randn(co, generator=g, device=dev) * 0.01).half()
        if name == "conv":
            ks = args.ksize            # 3: 3x3 pad 1; 1: pointwise; 2: 2x2 stride 2
            pad, st = (1, 1) if ks == 3 else (0, 1) if ks == 1 else (0, 2)
            ho, wo = (hh + 2 * pad - ks) // st + 1, (ww + 2 * pad - ks) // st + 1
            wq = ri8(co, ci * ks * ks)
            out = torch.empty((nb, co, ho, wo), dtype=torch.float16, device=dev)
            fn = lambda: lib.forge_int8_conv2d_forward(x.data_ptr(), wq.data_ptr(), w_s.data_ptr(), bias.data_ptr(),
                                                       out.data_ptr(), nb, ci, hh, ww, co, ks, ks, pad, pad, st, st,
                                                       1, 1, 0, S[0])
        else:
            wq = ri8(4 * co, ci)
            out = torch.empty((nb, co, 2 * hh, 2 * ww), dtype=torch.float16, device=dev)
            fn = lambda: lib.forge_int8_conv_transpose2d_k2s2_forward(x.data_ptr(), wq.data_ptr(), w_s.data_ptr(),
                                                                      bias.data_ptr(), out.data_ptr(), nb, ci, hh,
                                                                      ww, co, 0, S[0])
        # minimum traffic: the input and the weight read once, the output written once
        work, unit, bound = (2.0 * x.numel() + wq.numel() + 2.0 * out.numel()) / 1e9, "GB/s", "hbm"
        shape = {"N": nb, "C_in": ci, "H": hh, "W": ww, "C_out": co, "kernel": args.ksize if name == "conv" else 2}
    elif name in ("mlp", "mlp_sparse"):
        # W8A8 gated MLP block (Llama-style), default 8192 tokens, d_model 4096, d_ffn 14336
        m, dm, df = args.m or 8192, args.k or 4096, args.n or 14336
        x = torch.randn((m, dm), generator=g, device=dev, dtype=torch.float16)

        def qweight(rows, cols):
            w = torch.randn((rows, cols), generator=g, device=dev) * 0.02
            sc = w.abs().amax(dim=1).clamp(min=1e-8) / 127.0
            wq = torch.clamp(torch.round(w / sc[:, None]), -127, 127).to(torch.int8)
            return wq, sc.to(torch.float16)

        (Wg, sg), (Wu, su), (Wd, sd) = qweight(df, dm), qweight(df, dm), qweight(dm, df)
        outp = torch.empty((m, dm), dtype=torch.float16, device=dev)
        ws = torch.empty(lib.forge_w8a8_gated_mlp_workspace_bytes(m, dm, df), dtype=torch.uint8, device=dev)
        if name == "mlp":
            fn = lambda: lib.forge_w8a8_gated_mlp(x.data_ptr(), Wg.data_ptr(), Wu.data_ptr(), Wd.data_ptr(),
                                                  sg.data_ptr(), su.data_ptr(), sd.data_ptr(), 0, 0, 0, outp.data_ptr(),
                                                  m, dm, df, ws.data_ptr(), S[0])
        else:
            packs = []
            for W in (Wg, Wu, Wd):
                n_, k_ = W.shape
                comp = torch.empty((n_, k_ // 2), dtype=torch.int8, device=dev)
                raw = torch.empty((n_ * (k_ // 4),), dtype=torch.uint8, device=dev)
                meta = torch.empty((n_, k_ // 32), dtype=torch.int32, device=dev)
                C.prune_compress_24(W, comp, raw, n_, k_)
                C.pack_metadata(raw, meta, n_, k_)
                packs += [comp, meta]
            fn = lambda: lib.forge_sparse_w8a8_gated_mlp(x.data_ptr(), *[t.data_ptr() for t in packs], sg.data_ptr(),
                                                         su.data_ptr(), sd.data_ptr(), 0, 0, 0, outp.data_ptr(), m, dm,
                                                         df, ws.data_ptr(), S[0])
        work, unit, bound = 3 * 2.0 * m * dm * df / 1e12, "TOP/s", "tensor"
        shape = {"tokens": m, "d_model": dm, "d_ffn": df}
    else:
        raise SystemExit(f"unknown case {name}")
    return fn, work, unit, bound, shape


def run_case(args):
    """Single-kernel timing cases (also the commands the ncu summaries under profiles/ were made
    with). Prints one JSON line: kernel time from CUDA events, achieved rate, roofline fraction."""
    import torch
    from forge_b200 import _forge_C as C
    from forge_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    lib = _lib.load()
    lib.forge_b200_set_dense_tile(args.tile)
    lib.forge_b200_set_sparse_tile(args.tile)
    for kv in args.knob:   # library-internal tuning knobs (forge_b200/csrc/tuning.h), "key=value"
        key, value = kv.split("=")
        lib.forge_b200_set_tuning(int(key), int(value))
    peaks = _peaks()
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    name = args.case
    S = [torch.cuda.current_stream().cuda_stream]   # the stream the calls go to (swapped for graph capture)

    # --rotate builds several operand sets so that back-to-back calls inside a CUDA graph each read
    # operands that are not in L2
    sets = [_build_case(name, args, lib, C, dev, g, S) for _ in range(max(1, args.rotate))]
    fn, work, unit, bound, shape = sets[0]
    fns = [s[0] for s in sets]

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if args.flush_l2 else None
    for _ in range(args.warmup):
        for f in fns:
            assert f() == 0
    torch.cuda.synchronize()
    if args.graph:
        # the reference's protocol (benchmarks/bench_int8_sparse.cu:41-85): `reps` calls captured in
        # a CUDA graph, replays timed with events - device time without host launch latency
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            S[0] = side.cuda_stream
            with torch.cuda.graph(graph, stream=side):
                for r in range(args.reps):
                    assert fns[r % len(fns)]() == 0
        S[0] = torch.cuda.current_stream().cuda_stream
        fn = lambda: (graph.replay(), 0)[1]
        reps_in_fn, args.reps = args.reps, 1
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
    else:
        reps_in_fn = 1
    times = []
    for _ in range(args.steps):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            assert fn() == 0
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / (args.reps * reps_in_fn))
    assert lib.forge_b200_device_status(1) == 0
    probe = None
    if any(kv.startswith("3=") and int(kv[2:]) & 4 for kv in args.knob):
        import ctypes
        buf = (ctypes.c_ulonglong * 8)()
        lib.forge_b200_read_probe(ctypes.addressof(buf), 8)
        probe = list(buf)[:5]
    ms = statistics.median(times)
    achieved = work / (ms * 1e-3)
    peak = 2.0 * peaks["bf16_burst"] if bound == "tensor" else peaks["hbm"]
    extra = {"tokens_per_s": shape["tokens"] / (ms * 1e-3)} if name.startswith("mlp") else {}
    print(json.dumps({"case": name, "shape": shape, **extra, "ms": ms, "ms_min": min(times), "achieved": achieved,
                      "unit": unit,
                      "bound": bound, "peak": peak, "frac": achieved / peak, "peak_source": peaks["source"],
                      "l2_flush_between_launches": bool(args.flush_l2), "steps": args.steps, "tile": args.tile, "reps": args.reps * reps_in_fn, "cuda_graph": bool(args.graph),
                      "rotating_operand_sets": len(fns), "knobs": args.knob, "probe": probe,
                      "cta_pairs": lib.forge_b200_get_tuning(4)}))


def _init_ranks(timeout_s=300):
    import datetime

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=timeout_s))
    return world, rank, dev


def _rank_barrier(world):
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(ms, world, dev):
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sharded_sparse_layer(mode, m, k, n, steps, warmup, exchange, world, rank, dev, check_rows=0):
    """The sharded 2:4-sparse W8A8 linear layer, M tokens x K -> N, on the ranks of a torchrun launch.
    mode "rows": token rows split, weights replicated, no collective. mode "columns": output channels
    split, every rank ends with the full FP16 output (all-gather over NVLink, by the GEMM epilogue's
    peer stores with exchange="fused", by NCCL with "nccl"). Device time per call, max over ranks.
    check_rows > 0: that many sampled rows of the result are compared, bit for bit, against this
    rank's own computation of the whole layer on those rows (all ranks; the flag is the AND)."""
    import torch
    import torch.distributed as dist
    from forge_b200 import _forge_C as C
    from forge_b200.sharded import ShardedSparseLinear, SparseWeights, _forge_sparse_linear

    g = torch.Generator(device=dev)
    g.manual_seed(55)   # replicated weights: same seed on every rank
    W = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8, device=dev)
    comp = torch.empty((n, k // 2), dtype=torch.int8, device=dev)
    raw = torch.empty((n * (k // 4),), dtype=torch.uint8, device=dev)
    meta = torch.empty((n, k // 32), dtype=torch.int32, device=dev)
    C.prune_compress_24(W, comp, raw, n, k)
    C.pack_metadata(raw, meta, n, k)
    del W, raw
    w = SparseWeights(comp, meta, (torch.rand(n, generator=g, device=dev) * 0.01 + 0.001).half(), None)
    layer = ShardedSparseLinear(w, mode, chunks=8, exchange=exchange)
    if mode == "rows":
        r0, rows = layer.rows_of(m)
        g.manual_seed(1000 + rank)
        x = torch.randn((rows, k), generator=g, device=dev, dtype=torch.float16)
    else:
        g.manual_seed(1000)
        x = torch.randn((m, k), generator=g, device=dev, dtype=torch.float16)   # replicated activations

    for _ in range(max(warmup, 1)):
        y = layer(x)
    _rank_barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        y = layer(x)
    e1.record()
    _rank_barrier(world)
    ms = _max_over_ranks(e0.elapsed_time(e1) / steps, world, dev)
    line = {"case": "shard_" + ("rows" if mode == "rows" else "cols"), "n_gpus": world,
            "shape": {"M": m, "K": k, "N": n}, "ms": ms, "tokens_per_s": m / (ms * 1e-3),
            "dense_equiv_tops": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
            "includes": "per-token quantize + 2:4-sparse GEMM + dequant" + (" + FP16 all-gather" if mode == "columns" else ""),
            "steps": steps, "exchange": layer.exchange if mode == "columns" else None}
    if mode == "columns" and world > 1:
        recv = (world - 1) / world * 2.0 * m * n
        line["allgather_bytes_received_per_gpu"] = recv
        line["received_GBps_per_gpu"] = recv / (ms * 1e-3) / 1e9
        line["link_bound_ms_at_770GBs"] = recv / 770e9 * 1e3
        line["frac_of_nominal_900GBps_per_direction"] = recv / (ms * 1e-3) / 900e9
    if check_rows > 0:
        rows_total = y.shape[0]
        idx = torch.linspace(0, rows_total - 1, check_rows, device=dev).long()
        local = _forge_sparse_linear(x[idx].contiguous(), w)          # all N channels, computed here
        ok = torch.equal(y[idx].view(torch.int16), local.view(torch.int16))
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        line["bitwise_equal_to_local_recompute"] = bool(flag.item())
        line["rows_checked_per_rank"] = check_rows
    del layer, y, x
    torch.cuda.empty_cache()
    return line


def run_sharded_case(args):
    """--case shard_rows / shard_cols: prints one JSON line from rank 0."""
    import torch.distributed as dist
    world, rank, dev = _init_ranks()
    mode = "rows" if args.case == "shard_rows" else "columns"
    line = sharded_sparse_layer(mode, args.m or 65536, args.k or 8192, args.n or 28672, args.steps, args.warmup,
                                args.exchange, world, rank, dev, check_rows=16)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def sharded_mlp(sparse, m, dm, df, steps, warmup, world, rank, dev):
    """W8A8 gated MLP block (m tokens per GPU) on every rank: token rows sharded, weights replicated, no
    collective on the data path (weak scaling). Aggregate tokens/s from the device time, max over ranks."""
    import torch
    from forge_b200 import _forge_C as C
    from forge_b200 import _lib
    lib = _lib.load()
    g = torch.Generator(device=dev)
    g.manual_seed(77)   # replicated weights: same seed on every rank

    def qweight(rows, cols):
        w = torch.randn((rows, cols), generator=g, device=dev) * 0.02
        return C.prepare_weight(w, sparse=sparse)

    packs = [qweight(df, dm), qweight(df, dm), qweight(dm, df)]
    g.manual_seed(2000 + rank)
    x = torch.randn((m, dm), generator=g, device=dev, dtype=torch.float16)
    out = torch.empty((m, dm), dtype=torch.float16, device=dev)
    ws = torch.empty(lib.forge_w8a8_gated_mlp_workspace_bytes(m, dm, df), dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    scales = [p[3].data_ptr() for p in packs]
    if not sparse:
        fn = lambda: lib.forge_w8a8_gated_mlp(x.data_ptr(), packs[0][0].data_ptr(), packs[1][0].data_ptr(),
                                              packs[2][0].data_ptr(), *scales, 0, 0, 0, out.data_ptr(), m, dm, df,
                                              ws.data_ptr(), st)
    else:
        wm = []
        for p in packs:
            wm += [p[1].data_ptr(), p[2].data_ptr()]
        fn = lambda: lib.forge_sparse_w8a8_gated_mlp(x.data_ptr(), *wm, *scales, 0, 0, 0, out.data_ptr(), m, dm, df,
                                                     ws.data_ptr(), st)
    for _ in range(max(warmup, 3)):
        assert fn() == 0
    _rank_barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        assert fn() == 0
    e1.record()
    _rank_barrier(world)
    ms = _max_over_ranks(e0.elapsed_time(e1) / steps, world, dev)
    assert lib.forge_b200_device_status(1) == 0
    line = {"case": "shard_mlp_sparse" if sparse else "shard_mlp", "n_gpus": world, "scaling": "weak",
            "shape": {"tokens_per_gpu": m, "d_model": dm, "d_ffn": df}, "ms": ms,
            "tokens_per_s": world * m / (ms * 1e-3),
            "dense_equiv_tops": world * 3 * 2.0 * m * dm * df / (ms * 1e-3) / 1e12,
            "includes": "quantize -> gate/up GEMM + SiLU gate -> re-quantize -> down GEMM + dequant",
            "steps": steps}
    del packs, x, out, ws
    torch.cuda.empty_cache()
    return line


def run_sharded_mlp(args):
    """--case shard_mlp (dense weights) / shard_mlp_sparse (2:4): prints one JSON line from rank 0."""
    import torch.distributed as dist
    world, rank, dev = _init_ranks()
    line = sharded_mlp(args.case == "shard_mlp_sparse", args.m or 8192, args.k or 4096, args.n or 14336, args.steps,
                       args.warmup, world, rank, dev)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _sharded_extras(world, rank, dev):
    """The sharded workloads of the metric on the ranks of this launch (called by every rank): the gated
    MLP block with token rows sharded, and the 65536 x 8192 -> 28672 2:4-sparse layer sharded by token rows
    and by output channels (fused exchange), each with its bitwise check. A failure is reported in place
    of the figures; a failure on one rank only ends the launch at the next collective's time-out."""
    out = {}
    try:
        out["mlp"] = sharded_mlp(False, 8192, 4096, 14336, 10, 3, world, rank, dev)
        out["mlp_sparse"] = sharded_mlp(True, 8192, 4096, 14336, 10, 3, world, rank, dev)
        out["sparse_layer_rows"] = sharded_sparse_layer("rows", 65536, 8192, 28672, 5, 2, "auto", world, rank, dev,
                                                        check_rows=16)
        out["sparse_layer_cols"] = sharded_sparse_layer("columns", 65536, 8192, 28672, 5, 2, "fused", world, rank, dev,
                                                        check_rows=16)
        cols, rows = out["sparse_layer_cols"], out["sparse_layer_rows"]
        out["sharded_parity"] = bool(cols.get("bitwise_equal_to_local_recompute") and
                                     rows.get("bitwise_equal_to_local_recompute"))
    except Exception as e:
        out["error"] = f"{type(e).__name__}: {e}"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="headline",
                    help="headline (the contract line) or one kernel: dense, dense_s32, sparse, sparse_s32, "
                         "linear, quantize, dequant, prune, pack, conv, conv_transpose, mlp, mlp_sparse (for mlp: --m tokens --k d_model --n d_ffn); "
                         "under torchrun: shard_rows, shard_cols, shard_mlp, shard_mlp_sparse")
    ap.add_argument("--m", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--tile", type=int, default=0,
                    help="--case runs: pin the kernel tile (dense 64/128/256, 512 = CTA pair; sparse 32/64/128, "
                         "1000+BT = CTA pair with BT tokens); 0 = automatic")
    ap.add_argument("--reps", type=int, default=1,
                    help="--case runs: back-to-back calls per timed region (hides host launch latency of "
                         "microsecond-sized kernels; inputs then stay in L2 after the first call)")
    ap.add_argument("--ksize", type=int, default=3, choices=[1, 2, 3],
                    help="conv case: 3 = 3x3 pad 1, 1 = pointwise, 2 = 2x2 stride 2")
    ap.add_argument("--height", type=int, default=1080, help="conv cases: input height")
    ap.add_argument("--width", type=int, default=1920, help="conv cases: input width")
    ap.add_argument("--rotate", type=int, default=1,
                    help="--case runs with --graph: number of separate operand sets the captured calls cycle through "
                         "(sets x bytes per set above the L2 size makes every call read from HBM)")
    ap.add_argument("--graph", type=int, default=0, help="--case runs: capture --reps calls in a CUDA graph and time replays")
    ap.add_argument("--knob", action="append", default=[],
                    help="--case runs: library-internal tuning knob as key=value (2 = cap on CTA pairs, 3 = pair-kernel "
                         "measurement variant: 1 operands resident after the first ring fill, 4 clock probe, 32 no epilogue, "
                         "128 stores issued by the epilogue warps ...; 7 = dense raster band)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "nccl"],
                    help="shard_cols: all-gather by the GEMM epilogue's peer stores (fused) or by NCCL")
    ap.add_argument("--flush-l2", type=int, default=1, help="write 256 MiB between launches of a --case run")
    args = ap.parse_args()
    if args.case in ("shard_rows", "shard_cols"):
        run_sharded_case(args)
        return
    if args.case in ("shard_mlp", "shard_mlp_sparse"):
        if args.steps == 1000:
            args.steps = 50
        run_sharded_mlp(args)
        return
    if args.case == "probe":
        import torch
        from forge_b200 import _lib
        torch.cuda.set_device(0)
        lib = _lib.load()
        dev = torch.device("cuda", 0)
        n_sms = torch.cuda.get_device_properties(dev).multi_processor_count
        rows = {}
        for pair in (1, 0):
            for sparse in (0, 1):
                for n in (64, 128, 192, 224, 256):
                    for commits in (0, 1, 2):
                        if commits == 2 and not pair:
                            continue
                        key = f"{'pair M=256' if pair else 'one CTA M=128'} {'sparse K=64' if sparse else 'dense K=32'} N={n} commits={commits}"
                        rows[key] = lib.forge_b200_probe_mma_rate(pair, n, sparse, commits, n_sms)
        buf = torch.randint(-127, 128, (8192, 4096), dtype=torch.int8, device=dev)
        for producers in (1, 2, 4):
            for ctas in (1, n_sms // 2, n_sms):
                rows[f"tma ingest B/clk/SM producers={producers} ctas={ctas}"] = lib.forge_b200_probe_tma_ingest(
                    buf.data_ptr(), 8192, 4096, producers, ctas)
        print(json.dumps({"case": "probe", "sms": n_sms, "clocks_per_mma_and_bytes_per_clock": rows,
                          "status": lib.forge_b200_device_status(1)}))
        return
    if args.case != "headline":
        run_case(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
