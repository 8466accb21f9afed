#!/usr/bin/env python
"""Benchmark of the ternary sparse product hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --gpus N ...

One JSON line on rank 0.

Headline (`metric`, `value`): decode tokens/s of the tensor-parallel ternary Llama-70B-shaped decoder stack
(hidden 8192, FFN 28672, 64 query / 8 KV heads of 128, 80 layers, 50 % zeros, bf16 activations, KV length 1024) at
decode batch 1, on N GPUs of one node -- strong scaling: the same model at every N.  Every rank packs its shards of
the same seeded weights; before anything is timed, one layer's output on the N ranks is compared with the same
layer computed with dense fp32 matrices on rank 0.  A step is one token through all layers, replayed from a CUDA
graph; batches 16 and 64, the other sparsities and a per-layer breakdown are reported beside the headline.

`roofline` is that of the kernel that dominates the step, the decode product on one activation row, measured in
the same run on its own headline workload: x [1, 4096] fp16 ~ N(0,1), W [4096, 11008] ternary with 75 % zeros, fp16
scale ~ U(0.01, 0.05), R distinct packed weights replayed back to back from a CUDA graph (R weights exceed the L2
capacity several times).  achieved = B_alg / average launch time, B_alg = 2*nnz + 16*N*ceil(K/512) + e*M*(K+N) + 4
bytes (the reference layout's bytes); `spmv` carries the same for 50..90 % zeros and the neighbouring configurations.

`e2e` is the headline metric through host buffers: the token's activations start in pinned host memory and the
step's result is read back to the host, every step.

With --impl reference the reference's own CPU kernels (compiled in place into oracle/_ref) are timed on the host
cores on a bounded sample of the same step (one layer's linears, scaled to the layer count); no GPU kernel runs.
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

from ternaryllm_b200.synthetic import block_weight, make_weight  # noqa: E402

K_IN, N_OUT = 4096, 11008
L2_BYTES = 126 * 1024 * 1024
METRIC = "ternary_llama70b_shape_decode_tokens_per_s"
DEC = dict(hidden=8192, ffn=28672, heads=64, kv_heads=8, head_dim=128, layers=80, kv_len=1024)
# DRAM bytes per launch of the decode kernel from an ncu capture of the headline product (dram__bytes_read.sum +
# dram__bytes_write.sum); refreshed whenever the kernel or the format changes
NCU_TRAFFIC = {"bytes": 14.03e6, "source": "ncu, profiles/bstream_spmm_decode_4096x11008_s75_m1.md"}


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


def capture(torch, fn):
    """fn() captured into a CUDA graph (after one eager run on a side stream); returns the graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        fn()
    return g


def timed_us(torch, run, min_seconds=0.2, warmup=3, max_reps=200000):
    """Average time of run() in microseconds: CUDA events on the current stream around enough back-to-back calls to
    fill `min_seconds`."""
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    one = max(e0.elapsed_time(e1) * 1e-3, 1e-6)
    reps = int(min(max_reps, max(3, min_seconds / one)))
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps, reps


# ------------------------------------------------------------------------------------------------------
# the decode product on its own workloads (roofline of the dominant kernel, sparsity sweep, neighbours)
# ------------------------------------------------------------------------------------------------------
def spmv_records(torch, device, peak_hbm, quick=False):
    from ternaryllm_b200 import PackedMLP, PackedWeight, _lib

    L = _lib.lib()
    rng = np.random.default_rng(12345)
    out = {"sweep": [], "other_configs": []}

    KERNELS = {"gather": "gather (index lists)", "mma": "tensor core (two-bit tiles)", "nibble": "decode tensor core (four-bit planes by TMA)"}

    def pin(which):
        """auto = the library's cost model; gather / nibble = that kernel for every call it can take"""
        L.tllm_set_mma_min_rows(0 if which == "gather" else -1)
        L.tllm_set_nibble_max_rows({"auto": -1, "gather": 0, "nibble": 64}[which])

    def counters():
        return L.tllm_mma_launch_count(), L.tllm_nibble_launch_count()

    def ran_since(c0):
        m1, n1 = counters()
        names = ([KERNELS["mma"]] if m1 > c0[0] else []) + ([KERNELS["nibble"]] if n1 > c0[1] else [])
        return " + ".join(names) if names else KERNELS["gather"]

    def product(K, N, S, M, dtype=torch.float16, seed0=1000, check=True, pins=("auto",)):
        """R distinct weights of one shape replayed from a graph, once per kernel choice in `pins`; returns the record of
        pins[0] with the others' times under "by_kernel" """
        e = torch.empty((), dtype=dtype).element_size()
        bytes_one = min(int(K * N * (1 - S)) * 1.1 + 1, K * N / 2)     # the fewest bytes any kernel reads per weight
        R = min(32, max(3, int(-(-3 * L2_BYTES // bytes_one)) + 1))     # small weights stay (and are marked) L2-resident
        scales = [float(np.float16(v)) for v in rng.uniform(0.01, 0.05, R)]
        packed, nnzs, w0 = [], [], None
        for i in range(R):
            w = make_weight(seed0 + i, K, N, S)
            nnzs.append(int((w != 0).sum()))
            packed.append(PackedWeight.from_dense(w, scale=scales[i], device=device))
            if i == 0:
                w0 = w
        nnz = int(np.mean(nnzs))
        info = packed[0].info
        X = torch.tensor(rng.standard_normal((M, K)), dtype=dtype, device=device)
        Y = [torch.empty((M, N), dtype=dtype, device=device) for _ in range(R)]
        balg = algorithmic_bytes(nnz, K, N, M, e)

        def step():
            for i in range(R):
                packed[i].matmul(X, out=Y[i])

        recs = []
        for which in pins:
            pin(which)
            m0, n0 = L.tllm_mma_launch_count(), L.tllm_nibble_launch_count()
            step()
            torch.cuda.synchronize()
            kern = "mma" if L.tllm_mma_launch_count() > m0 else ("nibble" if L.tllm_nibble_launch_count() > n0 else "gather")
            err = None
            if check:
                ref = (X.double() @ torch.tensor(w0, device=device).double()) * scales[0]
                err = float((Y[0].double() - ref).abs().max() / ref.abs().max())
                if not err <= 1e-3 + 2.0 ** -8:
                    raise SystemExit(f"benchmark output differs from the dense product (rel err {err}) at {K}x{N} S={S} M={M} ({which})")
            g = capture(torch, step)
            us, reps = timed_us(torch, g.replay, 0.05 if quick else 0.2)
            us /= R
            for p in packed:
                p.check()
            wbytes = {"mma": info["bit_tile_bytes"], "nibble": info["nibble_bytes"], "gather": info["stream_bytes"] + info["meta_bytes"]}[kern]
            bphys = wbytes + e * M * (K + N)
            recs.append({"K": K, "N": N, "zeros": S, "rows": M, "choice": which, "kernel": KERNELS[kern], "us_per_launch": us,
                         "algorithmic_GBps": balg / us / 1e3, "frac": balg / us / 1e3 / peak_hbm, "physical_bytes": int(bphys),
                         "frac_physical": bphys / us / 1e3 / peak_hbm, "GOPs": M * nnz / us / 1e3, "weights_in_rotation": R,
                         "rotation_exceeds_l2": bool(R * bytes_one > 2 * L2_BYTES), "graph_replays_timed": reps, "check_rel_err": err,
                         "algorithmic_bytes": balg, "nnz": nnz})
        pin("auto")
        rec = recs[0]
        rec["pack"] = {k: info[k] for k in ("tile_rows", "tiles", "col_blocks", "k_splits", "num_ctas", "units", "stream_bytes", "meta_bytes",
                                             "nibble_bytes", "bit_tile_bytes")}
        if len(recs) > 1:
            rec["by_kernel"] = [{k: r[k] for k in ("choice", "kernel", "us_per_launch", "algorithmic_GBps", "frac", "physical_bytes", "frac_physical")}
                                for r in recs[1:]]
        for p in packed:
            p.close()
        return rec

    both = ("auto", "gather", "nibble")
    out["headline"] = product(K_IN, N_OUT, 0.75, 1, pins=both)
    for S in ((0.5, 0.9) if quick else (0.5, 0.6, 0.7, 0.8, 0.9)):
        out["sweep"].append(product(K_IN, N_OUT, S, 1, seed0=2000 + int(S * 100), pins=both))
    if quick:
        return out
    for M in (4, 16):
        out["other_configs"].append(dict(product(K_IN, N_OUT, 0.75, M, seed0=1000, pins=both if M == 4 else ("auto",)), workload=f"C2 up-projection shape, {M} rows fp16"))
    out["other_configs"].append(dict(product(8192, 28672, 0.5, 1, dtype=torch.bfloat16, seed0=3000, pins=both), workload="70B up-projection shape, 1 row bf16"))
    # C1: the reference's own CPU case, M = 8, K = N = 2048, fp32 N(0,1), 50 % zeros
    out["other_configs"].append(dict(product(2048, 2048, 0.5, 8, dtype=torch.float32, seed0=0), workload="C1: X[8,2048] fp32, W[2048,2048] 50% zeros"))
    # C3: fused MLP 4096 -> 11008 -> 4096, 60 % zeros, fp16 (two launches per block: gate|up with SiLU*mul, then down)
    import oracle

    hidden, inter, S = 4096, 11008, 0.6
    mlps, mrng = [], np.random.default_rng(777)
    wsets = []
    for i in range(3):
        sg, su, sd = (float(np.float16(v)) for v in mrng.uniform(0.01, 0.05, 3))
        ws = (make_weight(50 + 3 * i, hidden, inter, S), make_weight(51 + 3 * i, hidden, inter, S), make_weight(52 + 3 * i, inter, hidden, S))
        mlps.append(PackedMLP(*ws, sg, su, sd, device))
        wsets.append((ws, (sg, su, sd)))
    balg_w = sum(i["algorithmic_bytes"] for i in mlps[0].info)
    for M in (1, 8, 32):
        X = torch.tensor(mrng.standard_normal((M, hidden)), dtype=torch.float16, device=device)
        Y = torch.empty((M, hidden), dtype=torch.float16, device=device)
        H = torch.empty((M, inter), dtype=torch.float16, device=device)
        c0 = counters()
        mlps[0].forward(X, out=Y, h=H)
        torch.cuda.synchronize()
        (wg, wu, wd), (sg, su, sd) = wsets[0]
        rows = min(M, 2)          # the fp64 oracle on two rows of the full-size block
        ref = oracle.mlp_f64(X[:rows].double().cpu().numpy(), wg, wu, wd, sg, su, sd, h_round=1)
        err = float(np.max(np.abs(Y[:rows].double().cpu().numpy() - ref)) / np.max(np.abs(ref)))
        if not err <= 1e-3 + 2.0 ** -9:
            raise SystemExit(f"fused MLP differs from the oracle (rel err {err}) at {M} rows")

        def fn():
            for m in mlps:
                m.forward(X, out=Y, h=H)

        g = capture(torch, fn)
        us, _ = timed_us(torch, g.replay, 0.1)
        us /= len(mlps)
        balg = balg_w + 2 * M * 2 * hidden
        out["other_configs"].append({"workload": f"C3: MLP block {hidden}->{inter}->{hidden}, 60% zeros, {M} rows fp16 (two launches)",
                                     "kernel": ran_since(c0), "us_per_block": us,
                                     "algorithmic_GBps": balg / us / 1e3, "frac": balg / us / 1e3 / peak_hbm, "check_rel_err": err})
    for m in mlps:
        m.close()
    # C4: attention projections, 13B shape prefill, X [2048, 5120] bf16 against W [5120, 15360] and W [5120, 5120], 50 % zeros
    peak_tc, kind = measured_peak("bf16_tflops", 1590.0)
    for Np, name in ((15360, "QKV"), (5120, "O")):
        Kp, Mp = 5120, 2048
        w = make_weight(90 + Np, Kp, Np, 0.5)
        wq = PackedWeight.from_dense(w, scale=0.02, device=device)
        X = torch.randn((Mp, Kp), device=device).to(torch.bfloat16)
        Y = torch.empty((Mp, Np), dtype=torch.bfloat16, device=device)
        c0 = counters()
        wq.matmul(X, out=Y)
        ref = (X[:128].double() @ torch.tensor(w, device=device).double()) * 0.02
        err = float((Y[:128].double() - ref).abs().max() / ref.abs().max())
        if not err <= 1e-3 + 2.0 ** -8:
            raise SystemExit(f"prefill product differs from the dense product (rel err {err})")
        us, _ = timed_us(torch, lambda: wq.matmul(X, out=Y), 0.1)
        tf = 2.0 * Mp * Kp * Np / us / 1e6
        out["other_configs"].append({"workload": f"C4: {name} prefill, X[{Mp},{Kp}] bf16, W[{Kp},{Np}] 50% zeros",
                                     "kernel": ran_since(c0), "us_per_launch": us,
                                     "dense_equivalent_TFLOPs": tf, "frac_of_bf16_peak": tf / peak_tc, "bf16_peak_TFLOPs": peak_tc,
                                     "peak_source": kind, "check_rel_err": err})
        wq.close()
    return out


# ------------------------------------------------------------------------------------------------------
# the tensor-parallel decoder
# ------------------------------------------------------------------------------------------------------
def decoder_bench(torch, dist, world, rank, device, steps, warmup, sparsities, batches, reduce, quick=False):
    from ternaryllm_b200 import _lib
    from ternaryllm_b200.tensor_parallel import PeerReduce, TernaryDecoderLayerTP, reference_decoder_layer

    L = _lib.lib()
    d = DEC
    t_begin = time.time()

    def note(msg):
        sys.stderr.write(f"[bench rank {rank} +{time.time() - t_begin:6.1f}s] {msg}\n")
        sys.stderr.flush()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peer = PeerReduce(max(batches), d["hidden"], device) if reduce == "peer" else None
    records, clocks, headline = [], None, None
    for S in sparsities:
        # enough distinct layer weight sets per rank that a step streams every set from HBM (3x the L2 capacity)
        layers = [TernaryDecoderLayerTP(d["hidden"], d["ffn"], d["heads"], d["kv_heads"], d["head_dim"], S, world, rank, device,
                                        kv_len=d["kv_len"], max_batch=max(batches), seed=100, reduce=reduce, peer=peer)]
        per_set = sum(i["stream_bytes"] + i["meta_bytes"] for i in (layers[0].qkv.info, layers[0].o.info, *layers[0].mlp.info))
        nsets = 1 if quick else max(1, min(8, int(-(-3 * L2_BYTES // per_set))))
        for i in range(1, nsets):
            layers.append(TernaryDecoderLayerTP(d["hidden"], d["ffn"], d["heads"], d["kv_heads"], d["head_dim"], S, world, rank, device,
                                                kv_len=d["kv_len"], max_batch=max(batches), seed=100 + 50 * i, reduce=reduce, peer=peer))
        alg_local = float(np.mean([l.alg_bytes_local for l in layers])) * d["layers"]
        note(f"{S:.0%} zeros: {nsets} layer weight set(s) packed ({per_set / 1e6:.0f} MB per set and rank)")

        barrier()     # packing takes a different time on every rank; the peer reduce waits for a peer about a second, not longer
        # ---- parity before timing: one layer on the N ranks against the dense fp32 layer on rank 0 ----
        g = torch.Generator(device="cpu").manual_seed(7)
        Mc = min(4, max(batches))
        xc = torch.randn((Mc, d["hidden"]), generator=g).to(device, torch.bfloat16)
        xs, pending = layers[0](xc.clone())
        got = layers[0].finish(xs, pending).float()
        torch.cuda.synchronize()
        parity = None
        if rank == 0:
            want = reference_decoder_layer(layers[0].weights, xc.float(), d["kv_len"], max(batches), 100)
            parity = float((got - want).abs().max() / want.abs().max())
            del want
            torch.cuda.empty_cache()
            if not parity < 2e-2:
                raise SystemExit(f"TP-{world} layer differs from the dense layer: rel err {parity}")
            note(f"TP-{world} layer vs dense fp32 layer: rel err {parity:.2e}")
        barrier()

        for batch in batches:
            g = torch.Generator(device="cpu").manual_seed(1)
            x_host = torch.randn((batch, d["hidden"]), generator=g).to(torch.bfloat16).pin_memory()
            x0 = x_host.to(device)
            xw = torch.empty_like(x0)
            y_host = torch.empty((batch, d["hidden"]), dtype=torch.bfloat16).pin_memory()

            result = {}

            def step():
                xw.copy_(x0)                          # the layers update the residual stream in place
                x, pending = xw, None
                for i in range(d["layers"]):
                    x, pending = layers[i % nsets](x, pending)
                result["y"] = layers[0].finish(x, pending)

            n0, m0, d0 = L.tllm_launch_count(), L.tllm_mma_launch_count(), L.tllm_nibble_launch_count()
            step()
            torch.cuda.synchronize()
            launches, tensor_launches = L.tllm_launch_count() - n0, L.tllm_mma_launch_count() - m0
            decode_tc_launches = L.tllm_nibble_launch_count() - d0
            assert torch.isfinite(result["y"].float()).all()
            graph = capture(torch, step)
            y = result["y"]                           # the tensor the captured step writes
            for _ in range(max(3, warmup)):
                graph.replay()
            barrier()
            nsteps = steps if steps > 0 else (10 if quick else 20)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(device.index) as clk:
                e0.record()
                for _ in range(nsteps):
                    graph.replay()
                e1.record()
                barrier()
            ms = e0.elapsed_time(e1) / nsteps
            # end to end: the token's activations come from pinned host memory and the result goes back, every step
            def e2e_step():
                x0.copy_(x_host, non_blocking=True)
                graph.replay()
                y_host.copy_(y, non_blocking=True)
                torch.cuda.current_stream().synchronize()

            for _ in range(2):
                e2e_step()
            barrier()
            t0 = time.perf_counter()
            n_e2e = max(3, nsteps // 2)
            for _ in range(n_e2e):
                e2e_step()
            dt_e2e = (time.perf_counter() - t0) / n_e2e
            if world > 1:
                t = torch.tensor([ms, dt_e2e], device=device, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms, dt_e2e = float(t[0]), float(t[1])
            rec = {"zeros": S, "batch": batch, "tokens_per_s": batch / (ms * 1e-3), "ms_per_step": ms, "steps": nsteps,
                   "e2e_tokens_per_s": batch / dt_e2e, "launches_per_step": int(launches), "tensor_core_launches_per_step": int(tensor_launches),
                   "decode_tensor_core_launches_per_step": int(decode_tc_launches),
                   "weight_sets": nsets, "algorithmic_weight_GBps_per_rank": alg_local / (ms * 1e-3) / 1e9, "parity_rel_err": parity,
                   "h2d_bytes_per_step": batch * d["hidden"] * 2, "d2h_bytes_per_step": batch * d["hidden"] * 2}
            if headline is None:
                headline, clocks = rec, clk.summary()
                rec["breakdown_us_per_layer"] = layer_breakdown(torch, layers[0], x0, reduce)
                us_launch, per_layer = products_only(torch, layers[:nsets], x0)
                balg_launch = layers[0].alg_bytes_local / per_layer
                rec["products_only"] = {"us_per_launch": us_launch, "launches_per_layer": per_layer, "algorithmic_bytes_per_launch": balg_launch,
                                        "algorithmic_GBps": balg_launch / us_launch / 1e3,
                                        "kernel": "nibble_spmm_kernel" if decode_tc_launches else ("mma_spmm_kernel" if tensor_launches else "bstream_spmm_kernel")}
            records.append(rec)
            note(f"{S:.0%} zeros, batch {batch}: {rec['tokens_per_s']:.1f} tokens/s ({ms:.2f} ms/step)")
            del graph
            torch.cuda.synchronize()
        for l in layers:
            l.qkv.close(), l.o.close(), l.mlp.close()
        del layers
        torch.cuda.empty_cache()
    if peer is not None:
        peer.check()
    return headline, records, clocks


def layer_breakdown(torch, layer, x0, reduce, reps=20):
    """CUDA-event times of the phases of one layer (eager launches, averaged): where a step's time goes."""
    M = x0.shape[0]
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(reps)]
    x = x0.clone()
    pending = layer._part2[:M].zero_() if reduce == "peer" else torch.zeros_like(x)
    from ternaryllm_b200.tensor_parallel import add_rms_norm, all_reduce_sum

    for r in range(reps):
        e = ev[r]
        e[0].record()
        h = layer.peer.reduce(pending, x) if reduce == "peer" else add_rms_norm(x, all_reduce_sum(pending))
        e[1].record()
        qkv = layer.qkv.matmul(h)
        e[2].record()
        a = layer.attention(qkv, M)
        e[3].record()
        o = layer.o.matmul(a, out=layer._part[:M]) if reduce == "peer" else layer.o.matmul(a)
        e[4].record()
        h2 = layer.peer.reduce(o, x) if reduce == "peer" else add_rms_norm(x, all_reduce_sum(o))
        e[5].record()
        pending = layer.mlp.forward(h2, out=layer._part2[:M]) if reduce == "peer" else layer.mlp.forward(h2)
        e[6].record()
    torch.cuda.synchronize()
    names = ["reduce+add+norm (MLP)", "QKV product", "attention core and cache write (stock)", "O product", "reduce+add+norm (attention)", "MLP products"]
    return {n: float(np.median([ev[r][i].elapsed_time(ev[r][i + 1]) for r in range(3, reps)])) * 1e3 for i, n in enumerate(names)}


def products_only(torch, layers, x0, reps=10):
    """The four ternary products of a layer (QKV, O, gate|up + down) back to back over the distinct weight sets, from one
    CUDA graph, no glue in between: (mean microseconds per launch, launches per layer).  The dominant kernel of the
    decoder step timed on its own, live."""
    M = x0.shape[0]
    h = x0.clone()
    a = torch.randn((M, layers[0].hq * layers[0].hd), device=x0.device).to(x0.dtype)      # stands for the attention output

    def step():
        for layer in layers:
            layer.qkv.matmul(h)
            layer.o.matmul(a, out=layer._part[:M])
            layer.mlp.forward(h, out=layer._part2[:M])

    from ternaryllm_b200 import _lib

    L = _lib.lib()
    n0 = L.tllm_launch_count()
    step()
    torch.cuda.synchronize()
    launches = (L.tllm_launch_count() - n0) // len(layers)
    g = capture(torch, step)
    us, _ = timed_us(torch, g.replay, 0.1)
    return us / (launches * len(layers)), int(launches)


# ------------------------------------------------------------------------------------------------------
# reference CPU arm: the reference's own kernels on the host cores, bounded sample
# ------------------------------------------------------------------------------------------------------
GEMV_CANDIDATES = [   # (group, kernel name, simd chunk of the format)
    (64, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G64_AVX512_OpenMP", 0),
    (128, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G128_CS16_AVX512_OpenMP", 16),
    (64, "GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G64_AVX2_OpenMP", 0),
]


def cpu_decoder_sample(budget_s=25.0, sparsity=0.5, slice_div=8):
    """Tokens/s of the decoder step at batch 1 on the host cores with the reference's GEMV kernels (oracle/_ref:
    GEMM_CPU_FP32.cpp:14879-16838), from a bounded sample: a 1/slice_div column slice of each of one layer's five
    linears (same rows, same sparsity), timed and scaled to the full width and to the layer count.  The attention core
    and the norms are left out (they are not the reference's ternary path).  Falls back to the C restatement's dense
    walk when the compiled reference cannot run on this host."""
    import oracle

    d = DEC
    cores = os.cpu_count() or 1
    shapes = [(d["hidden"], (d["heads"] + 2 * d["kv_heads"]) * d["head_dim"]), (d["heads"] * d["head_dim"], d["hidden"]),
              (d["hidden"], d["ffn"]), (d["hidden"], d["ffn"]), (d["ffn"], d["hidden"])]
    r = oracle.ref()
    rng = np.random.default_rng(3)
    if r is None:
        K, N = shapes[0][0], shapes[0][1] // slice_div
        w = make_weight(1, K, N, sparsity)
        x = rng.standard_normal((1, K))
        t0 = time.perf_counter()
        oracle.dense_f64(x, w, 1.0)
        dt = (time.perf_counter() - t0) * slice_div
        total = dt * sum(k * n for k, n in shapes) / (shapes[0][0] * shapes[0][1]) * d["layers"]
        return 1.0 / total, {"kind": "port", "cores": 1, "kernel": "orc_dense_f64",
                             "sample": f"one {K}x{N} slice, 1 thread, scaled to the five linears of {d['layers']} layers"}
    r.ref_set_threads(cores)
    best = None
    t_begin = time.perf_counter()
    for G, name, simd in GEMV_CANDIDATES:
        if time.perf_counter() - t_begin > budget_s:
            break
        per_layer, ok = 0.0, True
        for (K, N) in shapes:
            Ns = max(G, N // slice_div // G * G)
            w = make_weight(K + N, K, Ns, sparsity)
            meta, ri = oracle.ref_merged_group(w, G, "min", False, simd)
            ri32 = np.concatenate([ri.astype(np.int32), np.zeros(64, np.int32)])
            x = np.ascontiguousarray(rng.standard_normal(K).astype(np.float32))
            y = np.zeros(Ns, np.float32)
            try:
                oracle.ref_call("F4", name, x, meta, ri32, y, Ns, K)
            except KeyError:
                ok = False
                break
            n, t0 = 0, time.perf_counter()
            while n < 3 or (time.perf_counter() - t0 < 0.5 and n < 50):
                oracle.ref_call("F4", name, x, meta, ri32, y, Ns, K)
                n += 1
            per_layer += (time.perf_counter() - t0) / n * (N / Ns)
        if ok and (best is None or per_layer < best[0]):
            best = (per_layer, name)
    per_layer, name = best
    return 1.0 / (per_layer * d["layers"]), {
        "kind": "reference", "cores": cores, "kernel": name,
        "sample": f"1/{slice_div} column slice of each of one layer's five linears ({sparsity:.0%} zeros), best of the reference GEMV kernels, "
                  f"scaled to full width and {d['layers']} layers; attention core and norms not included"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed decoder steps per configuration (0 = 20)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reduce", default="peer", choices=["peer", "nccl"], help="how the row-sharded products are summed over the ranks")
    ap.add_argument("--quick", action="store_true", help="one weight set, 50 %% zeros only, short product sweep (for smoke runs)")
    ap.add_argument("--no-spmv", action="store_true", help="skip the stand-alone product measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--spmv-only", action="store_true", help="only the stand-alone headline product (for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    d = DEC
    workload = (f"tensor-parallel ternary Llama-70B-shaped decoder: hidden {d['hidden']}, FFN {d['ffn']}, {d['heads']}q/{d['kv_heads']}kv x {d['head_dim']}, "
                f"{d['layers']} layers, 50% zeros, bf16 activations, KV length {d['kv_len']}, decode batch 1")

    if a.impl == "reference":
        if rank != 0:
            return 0
        tps, desc = cpu_decoder_sample(budget_s=120.0)
        line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": 1e3 / tps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload, "step": "one token through the linears of all layers on the host cores (sampled)"},
                "cpu_baseline": {"value": tps, "unit": "tokens/s", **desc},
                "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    import torch

    from ternaryllm_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in this library)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    peak, peak_kind = measured_peak()

    if a.spmv_only:
        rec = spmv_records(torch, device, peak, quick=True)["headline"]
        print(json.dumps(rec))
        return 0

    sparsities = (0.5,) if (a.quick or world > 1) else (0.5, 0.7, 0.9)
    batches = (1, 16, 64)
    headline, records, clocks = decoder_bench(torch, dist, world, rank, device, a.steps, a.warmup, sparsities, batches, a.reduce, quick=a.quick)

    spmv = None
    if rank == 0 and not a.no_spmv:
        spmv = spmv_records(torch, device, peak, quick=a.quick or world > 1)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()

    if rank == 0:
        line = {
            "metric": METRIC, "value": headline["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": headline["steps"], "warmup": a.warmup,
            "ms_per_step": headline["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 activations, ternary weights, fp32 sums", "data": "synthetic",
            "config": {"workload": workload, "parallelism": f"tp{world}", "reduce": a.reduce,
                       "step": f"one token through {d['layers']} layers ({headline['launches_per_step']} kernel launches of this library, one CUDA graph)",
                       "l2": f"inputs larger than L2: {headline['weight_sets']} distinct layer weight set(s) per rank, cycled through the layers",
                       "parity_rel_err_vs_dense_layer": headline["parity_rel_err"]},
            "clocks": clocks,
            "e2e": {"value": headline["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": headline["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": headline["d2h_bytes_per_step"]},
            "gpu_launches": int(headline["launches_per_step"]) * int(headline["steps"]),
            "decoder": records,
        }
        if spmv is not None:
            h = spmv["headline"]
            line["roofline"] = {"bound": "hbm", "achieved": h["algorithmic_GBps"], "peak": peak, "unit": "GB/s", "frac": h["frac"],
                                "frac_physical": h["frac_physical"], "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                                "kernel": "nibble_spmm_kernel" if h["kernel"].startswith("decode") else "bstream_spmm_kernel<float,1>",
                                "kernel_choice": "the library's cost model (the times of the gather and the decode tensor-core kernel, each pinned, are under spmv.headline.by_kernel)",
                                "us_per_launch": h["us_per_launch"],
                                "workload": f"decode product x[1,{K_IN}] fp16, W[{K_IN},{N_OUT}] 75% zeros, {h['weights_in_rotation']} weights in rotation (larger than L2)",
                                "algorithmic_bytes_per_launch": h["algorithmic_bytes"], "physical_bytes_per_launch": h["physical_bytes"],
                                "traffic": NCU_TRAFFIC["bytes"], "traffic_source": NCU_TRAFFIC["source"]}
            line["spmv"] = spmv
        po = headline.get("products_only")
        if po:
            line["roofline_decoder"] = {"bound": "hbm", "achieved": po["algorithmic_GBps"], "peak": peak, "unit": "GB/s", "frac": po["algorithmic_GBps"] / peak,
                                        "kernel": po["kernel"], "us_per_launch": po["us_per_launch"],
                                        "workload": f"the {po['launches_per_layer']} ternary products of one decoder layer per rank (QKV, O, gate|up, down), "
                                                    "mean over launches, weights streamed from HBM",
                                        "algorithmic_bytes_per_launch": po["algorithmic_bytes_per_launch"],
                                        "note": "the dominant kernel of the timed decoder step (about three quarters of its GPU time); algorithmic bytes = "
                                                "the reference layout's 2 B per non-zero + 16 B per (column, 512 rows)"}
        if world == 1 and not a.no_cpu_baseline:
            try:
                tps, desc = cpu_decoder_sample(budget_s=25.0)
                line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", **desc}
            except Exception as e:
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group right after graph replays that
        # used peer-mapped memory is not needed, and the processes end here anyway.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
