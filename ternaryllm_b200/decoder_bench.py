"""Decode throughput of a tensor-parallel ternary Llama-shaped decoder stack (tokens/s at 1/2/4/8 GPUs).

    python -m ternaryllm_b200.decoder_bench --batch 1 --sparsity 0.5                       # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
           -m ternaryllm_b200.decoder_bench --batch 16 --sparsity 0.7                        # one rank per GPU

Default shape: Llama-70B-like (hidden 8192, FFN 28672, 64 query / 8 KV heads of 128, 80 layers), random ternary
linears at the given sparsity, bf16 activations, unit RMSNorm weights, a synthetic KV cache of --kv-len entries
per head.  To keep host-side packing time bounded, --distinct layer weight sets are built and cycled through the
80 layers; two sets of this shape already exceed the L2 capacity several times over, so every layer streams its
weights from HBM.  One JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--distinct", type=int, default=2)
    ap.add_argument("--batch", default="1", help="decode batch, or a comma-separated list measured one after the other on the same weights")
    ap.add_argument("--sparsity", type=float, default=0.5)
    ap.add_argument("--kv-len", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--stall-dump", type=int, default=120, help="seconds between stack dumps to stderr while the run is alive (0 = off)")
    a = ap.parse_args()

    import torch.distributed as dist

    from ternaryllm_b200.synthetic import make_weight, measured_peak
    from ternaryllm_b200 import _lib
    from ternaryllm_b200.tensor_parallel import TernaryDecoderLayerTP

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    t_begin = time.time()
    if a.stall_dump > 0:            # where every rank stands if the run stalls
        faulthandler.dump_traceback_later(a.stall_dump, repeat=True, file=sys.stderr)

    def note(msg):
        sys.stderr.write(f"[decoder_bench rank {rank} +{time.time() - t_begin:6.1f}s] {msg}\n")
        sys.stderr.flush()

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        note("process group up")

    batches = [int(b) for b in str(a.batch).split(",")]
    layers = [TernaryDecoderLayerTP(a.hidden, a.ffn, a.heads, a.kv_heads, a.head_dim, a.sparsity, world, rank, device,
                                    kv_len=a.kv_len, max_batch=max(batches), seed=100 * i, make_weight=make_weight)
              for i in range(a.distinct)]
    alg_local = float(np.mean([l.alg_bytes_local for l in layers])) * a.layers
    note(f"{a.distinct} layer weight set(s) packed")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for batch in batches:
        g = torch.Generator(device="cpu").manual_seed(1)
        x0 = torch.randn((batch, a.hidden), generator=g).to(device, torch.bfloat16)

        def step():
            x, delta = x0.clone(), None              # the layers update the residual stream in place
            for i in range(a.layers):
                x, delta = layers[i % a.distinct](x, delta)
            return x + delta

        y = step()
        torch.cuda.synchronize()
        assert torch.isfinite(y.float()).all()
        note(f"batch {batch}: first step done")
        graph = None
        if not a.no_graph:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    step()
                note(f"batch {batch}: step captured in a CUDA graph")
            except Exception as e:
                sys.stderr.write(f"[decoder_bench] graph capture failed ({e}); timing eager launches\n")
                graph = None
                torch.cuda.synchronize()
        run = graph.replay if graph is not None else step
        for _ in range(max(3, a.warmup)):
            run()
        barrier()
        m0 = _lib.lib().tllm_mma_launch_count()
        step()                                   # one eager step, only to see which kernels the dispatch picks
        tensor_launches = _lib.lib().tllm_mma_launch_count() - m0
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            run()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / a.steps
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        if rank == 0:
            peak, kind = measured_peak()
            gbps_rank = alg_local / (ms * 1e-3) / 1e9
            print(json.dumps({
                "metric": "ternary_llama_decode_tokens_per_s", "value": batch / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "ms_per_step": ms, "steps": a.steps, "warmup": max(3, a.warmup), "scaling": "strong", "dtype": "bf16 activations, fp32 sums",
                "data": "synthetic",
                "config": {"workload": f"tensor-parallel ternary Llama-shaped decoder, hidden {a.hidden}, FFN {a.ffn}, {a.heads}q/{a.kv_heads}kv x {a.head_dim}, "
                                       f"{a.layers} layers ({a.distinct} distinct weight sets cycled), {a.sparsity:.0%} zeros, decode batch {batch}, KV length {a.kv_len}",
                           "parallelism": f"tp{world}", "cuda_graph": graph is not None,
                           "tensor_core_launches_per_step": tensor_launches, "linear_launches_per_step": 4 * a.layers,
                           "algorithmic_weight_bytes_per_rank_per_step": alg_local},
                "roofline": {"bound": "hbm", "achieved": gbps_rank, "peak": peak, "unit": "GB/s", "frac": gbps_rank / peak, "peak_source": kind,
                             "note": "per rank: reference-layout weight bytes of the rank's shards / step time (the step includes attention, norms and all-reduces)"},
            }), flush=True)
        del graph, run
        torch.cuda.synchronize()
    faulthandler.cancel_dump_traceback_later()
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group while CUDA graphs that captured
        # its collectives were alive hung here, and the processes end right after this anyway.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
