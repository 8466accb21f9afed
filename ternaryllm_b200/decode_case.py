"""One decode product on synthetic weights, a few launches: the smallest program that runs a chosen kernel of the library.

    python -m ternaryllm_b200.decode_case --kernel gather --K 4096 --N 11008 --zeros 0.75 --rows 1 --weights 10 --rounds 2

Packs `--weights` distinct seeded ternary matrices (more bytes than the L2 holds, so every launch streams its weight
from HBM), runs `--rounds` rounds of one product per weight, checks the last result against a dense fp64 product on
the device and prints the mean time per launch from CUDA events.  `--kernel` pins the choice the library would
otherwise make from its cost model: gather (index lists), nibble (four-bit planes streamed by TMA into the tensor
cores), mma (two-bit tiles expanded in shared memory for the tensor cores; fp16 / bf16, any row count) or auto.  Meant for profilers: `ncu -k regex:<kernel> -s <weights> -c 2 ...` captures launches of the second
round.
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--kernel", choices=("auto", "gather", "nibble", "mma"), default="auto")
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=11008)
    ap.add_argument("--zeros", type=float, default=0.75)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--dtype", choices=("f16", "bf16", "f32"), default="f16")
    ap.add_argument("--weights", type=int, default=10)
    ap.add_argument("--rounds", type=int, default=2)
    a = ap.parse_args(argv)

    import torch

    from . import PackedWeight, _lib
    from .synthetic import make_weight

    if not torch.cuda.is_available():
        print("decode_case needs a CUDA device", file=sys.stderr)
        return 2
    L = _lib.lib()
    L.tllm_set_mma_min_rows({"auto": -1, "gather": 0, "nibble": -1, "mma": 1}[a.kernel])
    L.tllm_set_nibble_max_rows({"auto": -1, "gather": 0, "nibble": 64, "mma": 0}[a.kernel])
    dev = torch.device("cuda", 0)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[a.dtype]
    ws = [make_weight(100 + i, a.K, a.N, a.zeros) for i in range(a.weights)]
    packed = [PackedWeight.from_dense(w, scale=0.03125, device=dev, no_bit_tiles=0 if a.kernel in ("auto", "mma") else 1) for w in ws]
    X = torch.randn((a.rows, a.K), device=dev).to(dt)
    Y = torch.empty((a.rows, a.N), device=dev, dtype=torch.float32 if a.rows <= 64 else dt)
    n0, g0, m0 = L.tllm_nibble_launch_count(), L.tllm_launch_count(), L.tllm_mma_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for r in range(a.rounds):
        if r == a.rounds - 1:
            e0.record()
        for p in packed:
            p.matmul(X, out=Y)
    e1.record()
    torch.cuda.synchronize()
    for p in packed:
        p.check()
    rows_checked = min(a.rows, 64)
    ref = (X[:rows_checked].double() @ torch.tensor(ws[-1], device=dev).double()) * 0.03125
    err = float((Y[:rows_checked].double() - ref).abs().max() / ref.abs().max())
    info = packed[0].info
    which = "nibble" if L.tllm_nibble_launch_count() > n0 else ("mma" if L.tllm_mma_launch_count() > m0 else "gather")
    print(f"{which} kernel, {L.tllm_launch_count() - g0} launches, x[{a.rows},{a.K}] {a.dtype}, W[{a.K},{a.N}] {a.zeros:.0%} zeros: "
          f"{e0.elapsed_time(e1) * 1e3 / len(packed):.2f} us per launch (eager, last round), rel err {err:.2e}; per weight: "
          f"index stream {info['stream_bytes'] + info['meta_bytes']} B, four-bit planes {info['nibble_bytes']} B, "
          f"reference layout {info['algorithmic_bytes']} B")
    return 0 if err <= 1e-3 + 2.0 ** -8 else 1


if __name__ == "__main__":
    sys.exit(main())
