#!/usr/bin/env python
"""Benchmark of the ternary sparse product hot path on B200.

Workload (the configuration the headline metric is quoted on): decode ternary SpMV, Llama-7B
up-projection shape -- x [M=1, 4096] fp16 ~ N(0,1), W [4096, 11008] ternary with 75 % zeros and +-1
equiprobable, per-tensor fp16 scale ~ U(0.01, 0.05), seeded synthetic data.

One step = one decode token pushed through R distinct packed weights of that shape (R*bytes is several
times the L2 capacity, so every launch streams its weight from HBM).  `value` is algorithmic GB/s
(B_alg per launch / average launch time): B_alg = 2*nnz + 16*N*ceil(K/512) + e*M*(K+N) + 4 bytes, the
bytes of the reference's own layout.  `e2e` is the same metric through the host-buffer C-ABI entry point
(tllm_spmm_host): pinned host x -> device, kernel, y -> host, every call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--rows M] [--sparsity S]

With --impl reference the reference's own CPU GEMV kernels (compiled in place into oracle/_ref) are timed
on the host cores for the same workload; that arm launches no GPU kernel.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ternaryllm_b200.synthetic import make_weight  # noqa: E402

K_IN, N_OUT = 4096, 11008
L2_BYTES = 126 * 1024 * 1024
METRIC = "ternary_spmv_algorithmic_hbm_gbps"
# DRAM bytes per launch of the decode kernel from an ncu capture of this workload at one row
# (dram__bytes_read.sum + dram__bytes_write.sum = 23.70 MB + 0; profiles/tstream_spmm_decode_4096x11008_s75_m1.md).
NCU_TRAFFIC_BYTES = 23.70e6


def algorithmic_bytes(nnz: int, K: int, N: int, M: int, e: int) -> int:
    return 2 * nnz + 16 * N * (-(-K // 512)) + e * M * (K + N) + 4


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._n = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._n = None

    def _run(self):
        n = self._n
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                try:
                    r = n.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self._n:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def measured_peak(key="hbm_gbs", fallback=6650.0):
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))[key]), "measured"
        except Exception:
            pass
    return fallback, "fallback"


def graph_time_us(torch, fn, reps, warmup=3):
    """Average time of fn() in microseconds over `reps` replays of a CUDA graph of one call (plain launches if the
    capture fails), CUDA events on the current stream."""
    fn()
    torch.cuda.synchronize()
    run = fn
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        run = g.replay
    except Exception:
        torch.cuda.synchronize()
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def other_configs(torch, device, packed, nnz, K, N, peak_hbm):
    """Short measurements of the neighbouring configurations (each a few hundred replays): the same weights at
    4 and 16 rows, the fused MLP block of the same shape at 60 % zeros, and the 13B-shape QKV prefill product on
    the tensor cores.  Reported beside the headline, not part of it."""
    from ternaryllm_b200 import PackedMLP, PackedWeight, _lib

    L = _lib.lib()
    out = []
    R = len(packed)
    for M in (4, 16):
        X = torch.randn((M, K), device=device).to(torch.float16)
        Y = torch.empty((M, N), dtype=torch.float16, device=device)
        n0, m0 = L.tllm_launch_count(), L.tllm_mma_launch_count()

        def fn():
            for w in packed:
                w.matmul(X, out=Y)

        us = graph_time_us(torch, fn, 50) / R
        tensor = L.tllm_mma_launch_count() > m0
        balg = algorithmic_bytes(nnz, K, N, M, 2)
        out.append({"workload": f"same weights, {M} rows fp16", "kernel": "tensor-core" if tensor else "gather", "us_per_launch": us,
                    "algorithmic_GBps": balg / us / 1e3, "frac_of_hbm_peak": balg / us / 1e3 / peak_hbm,
                    "GOPs": M * nnz / us / 1e3})
    # fused MLP 4096 -> 11008 -> 4096, 60 % zeros, fp16
    hidden, inter, S = 4096, 11008, 0.6
    mlps, rng = [], np.random.default_rng(777)
    for i in range(3):
        sg, su, sd = (float(np.float16(v)) for v in rng.uniform(0.01, 0.05, 3))
        mlps.append(PackedMLP(make_weight(50 + 3 * i, hidden, inter, S), make_weight(51 + 3 * i, hidden, inter, S),
                              make_weight(52 + 3 * i, inter, hidden, S), sg, su, sd, device))
    infos = mlps[0].info
    balg_w = sum(i["algorithmic_bytes"] for i in infos)
    for M in (1, 8, 32):
        X = torch.randn((M, hidden), device=device).to(torch.float16)
        Y = torch.empty((M, hidden), dtype=torch.float16, device=device)
        H = torch.empty((M, inter), dtype=torch.float16, device=device)
        m0 = L.tllm_mma_launch_count()

        def fn():
            for m in mlps:
                m.forward(X, out=Y, h=H)

        us = graph_time_us(torch, fn, 50) / len(mlps)
        balg = balg_w + 2 * M * 2 * hidden
        out.append({"workload": f"fused MLP block {hidden}->{inter}->{hidden}, 60% zeros, {M} rows fp16 (two launches)",
                    "kernel": "tensor-core" if L.tllm_mma_launch_count() > m0 else "gather", "us_per_block": us,
                    "algorithmic_GBps": balg / us / 1e3, "frac_of_hbm_peak": balg / us / 1e3 / peak_hbm})
    for m in mlps:
        m.close()
    # attention-projection prefill, 13B shape: X [2048, 5120] bf16, W [5120, 15360] at 50 % zeros
    Kp, Np, Mp = 5120, 15360, 2048
    wq = PackedWeight.from_dense(make_weight(90, Kp, Np, 0.5), scale=0.02, device=device)
    X = torch.randn((Mp, Kp), device=device).to(torch.bfloat16)
    Y = torch.empty((Mp, Np), dtype=torch.bfloat16, device=device)
    m0 = L.tllm_mma_launch_count()
    us = graph_time_us(torch, lambda: wq.matmul(X, out=Y), 20)
    peak_tc, kind = measured_peak("bf16_tflops", 1590.0)
    tf = 2.0 * Mp * Kp * Np / us / 1e6
    out.append({"workload": f"QKV prefill, X[{Mp},{Kp}] bf16, W[{Kp},{Np}] 50% zeros", "kernel": "tensor-core" if L.tllm_mma_launch_count() > m0 else "gather",
                "us_per_launch": us, "dense_equivalent_TFLOPs": tf, "frac_of_bf16_peak": tf / peak_tc, "bf16_peak_TFLOPs": peak_tc, "peak_source": kind})
    wq.close()
    return out


# ------------------------------------------------------------------------------------------------------
# reference CPU arm
# ------------------------------------------------------------------------------------------------------
GEMV_CANDIDATES = [   # (group, kernel name, simd chunk of the format)
    (64, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G64_AVX512_OpenMP", 0),
    (128, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G128_CS16_AVX512_OpenMP", 16),
    (32, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G32_AVX512_OpenMP", 0),
    (64, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G64_AVX2_OpenMP", 0),
]


def cpu_reference_run(weights, x_rows, steps, warmup, budget_s=25.0):
    """Times the reference's CPU kernels (oracle/_ref: its GEMV family, GEMM_CPU_FP32.cpp:14879-16838) on the
    given dense weights; falls back to the C restatement when the compiled reference cannot run here.
    Returns (seconds per product, description dict)."""
    import oracle

    K, N = weights[0].shape
    M = x_rows.shape[0]
    r = oracle.ref()
    cores = os.cpu_count() or 1
    if r is None:
        # C restatement, single thread: dense walk of the ternary matrix (oracle.c, orc_dense_f64)
        w = weights[0]
        t0 = time.perf_counter()
        oracle.dense_f64(x_rows.astype(np.float64), w, 1.0)
        dt = time.perf_counter() - t0
        return dt, {"kind": "port", "cores": 1, "kernel": "orc_dense_f64", "sample": f"1 product of {M}x{K}x{N}, 1 thread"}
    r.ref_set_threads(cores)
    x32 = np.ascontiguousarray(x_rows.astype(np.float32))
    best = None
    t_begin = time.perf_counter()
    for G, name, simd in GEMV_CANDIDATES:
        if N % G or time.perf_counter() - t_begin > budget_s:
            continue
        fmts = []
        for w in weights:
            meta, ri = oracle.ref_merged_group(w, G, "min", False, simd)
            fmts.append((meta, np.concatenate([ri.astype(np.int32), np.zeros(64, np.int32)])))
        y = np.zeros(N, np.float32)

        def one_pass():
            for meta, ri32 in fmts:
                for m in range(M):          # the reference's decode path is one GEMV per row
                    oracle.ref_call("F4", name, x32[m], meta, ri32, y, N, K)

        try:
            for _ in range(max(1, warmup)):
                one_pass()
        except KeyError:
            continue
        n = 0
        t0 = time.perf_counter()
        while n < steps and time.perf_counter() - t0 < budget_s / len(GEMV_CANDIDATES):
            one_pass()
            n += 1
        dt = (time.perf_counter() - t0) / (n * len(fmts))
        if best is None or dt < best[0]:
            best = (dt, name, n)
    dt, name, n = best
    return dt, {"kind": "reference", "cores": cores, "kernel": name,
                "sample": f"{n} passes over {len(weights)} distinct weights of {K}x{N}, {M} row(s), best of {len(GEMV_CANDIDATES)} reference GEMV kernels"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--sparsity", type=float, default=0.75)
    ap.add_argument("--inners", type=int, default=K_IN, help="rows of W (K); the headline workload is 4096")
    ap.add_argument("--columns", type=int, default=N_OUT, help="columns of W (N); the headline workload is 11008")
    ap.add_argument("--copies", type=int, default=0, help="distinct packed weights per step (0 = enough to exceed 3x L2)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the short measurements of the neighbouring configurations")
    ap.add_argument("--prefill", action="store_true",
                    help="time only the 13B-shape QKV prefill product on the tensor cores (X [2048,5120] bf16, W [5120,15360], 50 %% zeros)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    M, K, N, S = a.rows, a.inners, a.columns, a.sparsity
    shape_name = "Llama-7B up-projection shape" if (K, N) == (K_IN, N_OUT) else "custom shape"
    workload = f"decode ternary SpMV, {shape_name}: x[{M},{K}] fp16 N(0,1), W[{K},{N}] ternary {S:.0%} zeros, fp16 scale U(0.01,0.05)"

    if a.impl == "reference":
        if rank != 0:
            return 0
        weights = [make_weight(1000 + i, K, N, S) for i in range(4)]
        nnz = int(np.mean([(w != 0).sum() for w in weights]))
        rng = np.random.default_rng(12345)
        x = rng.standard_normal((M, K)).astype(np.float16)
        dt, desc = cpu_reference_run(weights, x, a.steps, a.warmup, budget_s=120.0)
        balg = algorithmic_bytes(nnz, K, N, M, 2)
        gbps = balg / dt / 1e9
        line = {"impl": "reference", "metric": METRIC, "value": gbps, "unit": "GB/s", "n_gpus": a.gpus, "steps": a.steps,
                "warmup": a.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload, "step": "one product on the host cores", "algorithmic_bytes_per_product": balg},
                "cpu_baseline": {"value": gbps, "unit": "GB/s", **desc},
                "e2e": {"value": gbps, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    import torch

    from ternaryllm_b200 import PackedWeight, _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in this library)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    if a.prefill:
        Kp, Np, Mp = 5120, 15360, 2048
        wq = PackedWeight.from_dense(make_weight(90, Kp, Np, 0.5), scale=0.02, device=device)
        Xp = torch.randn((Mp, Kp), device=device).to(torch.bfloat16)
        Yp = torch.empty((Mp, Np), dtype=torch.bfloat16, device=device)
        for _ in range(a.warmup):
            wq.matmul(Xp, out=Yp)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            wq.matmul(Xp, out=Yp)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / a.steps
        ref = (Xp[:64].double() @ torch.tensor(make_weight(90, Kp, Np, 0.5), device=device).double()) * 0.02
        err = float((Yp[:64].double() - ref).abs().max() / ref.abs().max())
        peak_tc, kind = measured_peak("bf16_tflops", 1590.0)
        tf = 2.0 * Mp * Kp * Np / us / 1e6
        print(json.dumps({"metric": "ternary_prefill_dense_equivalent_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": a.steps,
                          "warmup": a.warmup, "ms_per_step": us / 1e3, "higher_is_better": True, "dtype": "bf16 x ternary, fp32 accumulate",
                          "data": "synthetic", "config": {"workload": f"QKV prefill, X[{Mp},{Kp}] bf16, W[{Kp},{Np}] 50% zeros", "check_rel_err": err},
                          "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_tc, "unit": "TFLOP/s", "frac": tf / peak_tc, "peak_source": kind,
                                       "traffic": None},
                          "gpu_launches": a.steps}))
        return 0

    peak, peak_kind = measured_peak()
    R = a.copies or max(4, -(-3 * L2_BYTES // (2 * int(K * N * (1 - S)))) + 1)
    rng = np.random.default_rng(12345)
    scales = [float(np.float16(v)) for v in rng.uniform(0.01, 0.05, R)]
    packed, nnzs, w0 = [], [], None
    for i in range(R):
        w = make_weight(1000 + 100 * rank + i, K, N, S)
        nnzs.append(int((w != 0).sum()))
        packed.append(PackedWeight.from_dense(w, scale=scales[i], device=device))
        if i == 0:
            w0 = w
    nnz = int(np.mean(nnzs))
    info = packed[0].info
    balg = algorithmic_bytes(nnz, K, N, M, 2)
    bphys = info["stream_bytes"] + info["meta_bytes"] + 2 * M * (K + N)

    x_host = torch.tensor(rng.standard_normal((M, K)), dtype=torch.float16).pin_memory()
    X = x_host.to(device)
    Y = [torch.empty((M, N), dtype=torch.float16, device=device) for _ in range(R)]

    def step():
        for i in range(R):
            packed[i].matmul(X, out=Y[i])

    # correctness guard inside the benchmark: compare one product with a dense fp64 product on the device
    step()
    torch.cuda.synchronize()
    ref = (X.double() @ torch.tensor(w0, device=device).double()) * scales[0]
    err = float((Y[0].double() - ref).abs().max() / ref.abs().max())
    if not err <= 1e-3 + 2.0 ** -11:
        raise SystemExit(f"benchmark output differs from the dense product (rel err {err})")

    graph = None
    if not a.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        except Exception as e:      # keep measuring with plain launches
            sys.stderr.write(f"[bench] CUDA graph capture failed ({e}); timing plain launches\n")
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else step

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        run()
    barrier()
    launches0 = _lib.lib().tllm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        e0.record()
        for _ in range(a.steps):
            run()
        e1.record()
        barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / a.steps
    us_launch = ms_step * 1e3 / R
    gpu_launches = a.steps * R            # R kernel launches per step (replayed from a graph when one was captured)
    value = world * R * balg / (ms_step * 1e-3) / 1e9
    achieved = balg / (us_launch * 1e-6) / 1e9
    for p in packed:
        p.check()

    # ---- end to end through the host-buffer entry point ----
    y_host = [np.empty((M, N), np.float16) for _ in range(R)]
    y_pin = [torch.from_numpy(y).pin_memory() for y in y_host]
    e2e_steps = max(3, min(a.steps, 100))

    def e2e_step():
        for i in range(R):
            _lib.check(_lib.lib().tllm_spmm_host(packed[i]._h, x_host.data_ptr(), _lib.F16, _lib.ROW_MAJOR, M, y_pin[i].data_ptr(),
                                                 _lib.F16, _lib.ROW_MAJOR))

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    dt_e2e = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([dt_e2e], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_e2e = float(t.item())
    e2e_val = world * R * balg / dt_e2e / 1e9
    err2 = float((y_pin[0].to(device).double() - ref).abs().max() / ref.abs().max())
    if not err2 <= 1e-3 + 2.0 ** -11:
        raise SystemExit(f"host-buffer path differs from the dense product (rel err {err2})")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "step": f"one decode token through {R} distinct packed weights ({R} launches)",
                   "l2": f"inputs larger than L2: {R} weights x {bphys / 1e6:.1f} MB rotate through a {L2_BYTES >> 20} MiB L2",
                   "algorithmic_bytes_per_launch": balg, "physical_bytes_per_launch": bphys, "nnz": nnz,
                   "us_per_launch": us_launch, "cuda_graph": graph is not None, "pdl": os.environ.get("TLLM_PDL", "1") != "0",
                   "accumulate": "fp32", "check_rel_err": err,
                   "pack": {k: info[k] for k in ("tile_rows", "tiles", "col_blocks", "k_splits", "num_ctas", "units")}},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_physical": (bphys / (us_launch * 1e-6) / 1e9) / peak, "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                     "traffic": NCU_TRAFFIC_BYTES if (M == 1 and S == 0.75 and (K, N) == (K_IN, N_OUT)) else None},
        "clocks": clk.summary(),
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": R * 2 * M * K, "d2h_bytes_per_step": R * 2 * M * N,
                "us_per_call": dt_e2e * 1e6 / R, "steps": e2e_steps},
        "gpu_launches": gpu_launches,
    }
    if world == 1 and not a.no_cpu_baseline:
        try:
            cw = [w0] + [make_weight(1000 + i, K, N, S) for i in range(1, 4)]
            dt, desc = cpu_reference_run(cw, x_host.numpy(), 10, 3, budget_s=20.0)
            line["cpu_baseline"] = {"value": balg / dt / 1e9, "unit": "GB/s", "us_per_product": dt * 1e6, **desc}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    if world == 1 and not a.no_other_configs:
        try:
            line["other_configs"] = other_configs(torch, device, packed, nnz, K, N, peak)
        except Exception as e:
            line["other_configs"] = [{"failed": str(e)}]
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
