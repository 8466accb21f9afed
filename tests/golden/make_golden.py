"""Generate the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Run in a container that has the reference checkout (default location given by --ref) after
`python oracle/build_ref.py`.  Two sources:

  1. the reference's pure-Python packers, ternaryLLM_GPU/TernaryLLM/TernaryCSC.py
     (convert_to_ter_csc :17-48, convert_to_ter_tiled_csc :50-94, convert_to_ter_tiled_mcsc :97-156),
     imported straight from the checkout;
  2. the reference's CPU format builders and kernels (ternaryLLM_CPU/src/TCSC.hpp, GEMM_CPU_FP32.cpp,
     GEMM_CPU_INT8.cpp) compiled in place into oracle/_ref/libtllm_ref.so.

The fixtures are small (a few tens of KB, compressed) and are what `pytest -m "not gpu"` pins the C
oracle against, and what `pytest -m gpu` pins the CUDA path against.  Inputs follow the reference's own
verification regime (main.cpp:1403, :1893): integer-valued activations, so every sum is exact.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def random_ternary(rng, K, N, sparsity):
    """i.i.d. P(0)=s, P(-1)=P(+1)=(1-s)/2 -- TernaryLinear.py:79-83."""
    r = rng.random((K, N))
    w = np.zeros((K, N), np.int32)
    w[(r >= sparsity) & (r < (sparsity + 1) / 2)] = -1
    w[r >= (sparsity + 1) / 2] = 1
    return w


def aligned_ternary(rng, K, N, sparsity, uniform):
    """Equal #(+1) and #(-1) per column (sparseWeight Aligned / Uniformed, initData.hpp:40-130)."""
    w = np.zeros((K, N), np.int8)
    base = int(K * (1 - sparsity)) // 2
    for n in range(N):
        h = base if uniform else max(1, base + int(rng.integers(-base // 4, base // 4 + 1)))
        rows = rng.permutation(K)[: 2 * h]
        w[rows[:h], n] = 1
        w[rows[h:], n] = -1
    return w


def gen_python_packers(ref_root, out):
    import torch

    path = os.path.join(ref_root, "ternaryLLM_GPU", "TernaryLLM", "TernaryCSC.py")
    spec = importlib.util.spec_from_file_location("ref_TernaryCSC", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(20240601)
    cases = {}
    for name, (K, N, T, s) in {
        "a": (64, 24, 16, 0.5),
        "b": (128, 16, 32, 0.75),
        "c": (96, 8, 32, 0.9),
        "d": (64, 8, 64, 0.0),
    }.items():
        w = random_ternary(rng, K, N, s)
        if name == "c":
            w[:, 3] = 0          # an empty column
            w[32:64, 5] = 0      # an empty tile
            w[:, 6] = 1          # an all +1 column
        wt = torch.tensor(w)
        ni, no, pi, po = mod.convert_to_ter_csc(wt)
        tni, tno, tpi, tpo = mod.convert_to_ter_tiled_csc(wt, T)
        mi, mo = mod.convert_to_ter_tiled_mcsc(wt, T)
        cases[name] = dict(
            w=w.astype(np.int8), T=np.int32(T),
            csc_neg_idx=np.array(ni, np.int32), csc_neg_off=np.array(no, np.int32),
            csc_pos_idx=np.array(pi, np.int32), csc_pos_off=np.array(po, np.int32),
            tcsc_neg_idx=tni.numpy().astype(np.int32), tcsc_neg_off=tno.numpy().astype(np.int32),
            tcsc_pos_idx=tpi.numpy().astype(np.int32), tcsc_pos_off=tpo.numpy().astype(np.int32),
            mcsc_idx=mi.numpy().astype(np.int32), mcsc_off=mo.numpy().astype(np.int32),
        )
    gen_cpp_packers(cases)
    flat = {f"{c}.{k}": v for c, d in cases.items() for k, v in d.items()}
    np.savez_compressed(out, **flat)
    print("wrote", out, os.path.getsize(out), "bytes")


def gen_cpp_packers(cases):
    """Adds to every case what the reference's C++ packers return for its matrix (the host side of
    ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu: convert_to_ter_csc :9-72, convert_to_ter_tiled_csc :75-153,
    convert_to_ter_tiled_mcsc :156-315 -- the one with the truncating step :277-291), without padding and with
    padding to 4 and to 8.  Needs oracle/_ref/gpu_ext (python oracle/build_ref.py --gpu-ext); two further matrices
    at a tile size the reference uses (256) are added so that the truncation and the tile order are exercised on
    tiles with tens of entries."""
    import glob

    import torch

    ext = glob.glob(os.path.join(ROOT, "oracle", "_ref", "gpu_ext", "ter_spmm*.so"))
    assert ext, "run python oracle/build_ref.py --gpu-ext first"
    spec = importlib.util.spec_from_file_location("ter_spmm", ext[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(20250101)
    for name, (K, N, T, s) in {"e": (512, 12, 256, 0.5), "f": (1024, 6, 256, 0.8)}.items():
        w = random_ternary(rng, K, N, s)
        if name == "f":
            w[256:512, 2] = 0
            w[:, 4] = -1
        cases[name] = dict(w=w.astype(np.int8), T=np.int32(T))
    for name, c in cases.items():
        w = torch.tensor(c["w"].astype(np.int32)).contiguous()
        K, N = w.shape
        T = int(c["T"])
        pos, neg = int((w == 1).sum()), int((w == -1).sum())
        ni, no, pi, po = mod.convert_to_ter_csc(w, N, K, pos, neg)
        c.update(cpp_csc_neg_idx=np.array(ni, np.int32), cpp_csc_neg_off=np.array(no, np.int32),
                 cpp_csc_pos_idx=np.array(pi, np.int32), cpp_csc_pos_off=np.array(po, np.int32))
        ni, no, pi, po = mod.convert_to_ter_tiled_csc(w, N, K, pos, neg, T)
        c.update(cpp_tcsc_neg_idx=np.array(ni, np.int32), cpp_tcsc_neg_off=np.array(no, np.int32),
                 cpp_tcsc_pos_idx=np.array(pi, np.int32), cpp_tcsc_pos_off=np.array(po, np.int32))
        for tag, pad, padsz in (("nopad", False, 4), ("pad4", True, 4), ("pad8", True, 8)):
            idx, off, til = mod.convert_to_ter_tiled_mcsc(w, N, K, pos, neg, T, pad, padsz)
            c[f"cpp_mcsc_{tag}_idx"] = np.array(idx, np.int32)
            c[f"cpp_mcsc_{tag}_off"] = np.array(off, np.int32)
            c[f"cpp_mcsc_{tag}_til"] = np.array(til, np.int32)
    print("reference C++ packers:", ext[0])


def gen_cpu(out):
    import oracle

    r = oracle.ref()
    assert r is not None, "run python oracle/build_ref.py first (and this host needs AVX-512)"
    r.ref_set_threads(2)
    rng = np.random.default_rng(7)
    K, N, M = 96, 64, 64
    W = random_ternary(rng, K, N, 0.6).astype(np.int8)
    Wal = aligned_ternary(rng, K, N, 0.6, uniform=False)
    Wun = aligned_ternary(rng, K, N, 0.6, uniform=True)
    X = rng.integers(-512, 513, size=(M, K)).astype(np.float32)       # initX<float>(…, 512)
    X8 = rng.integers(-10, 11, size=(M, K)).astype(np.int8)           # initX<int8_t>(…, 10)
    XT = np.ascontiguousarray(X.T)                                    # [K][M] "colMajor"
    X8T = np.ascontiguousarray(X8.T)
    fx = dict(W=W, Wal=Wal, Wun=Wun, X=X, X8=X8)

    # --- formats ---
    csp, csn, rip, rin = oracle.ref_sparse_format(W)
    fx.update(sf_csp=csp, sf_csn=csn, sf_rip=rip, sf_rin=rin)
    meta, ri = oracle.ref_merged_tcsc(W)
    fx.update(merged_meta=meta, merged_ri=ri)
    groups = []
    for (wname, Wm) in (("W", W), ("Wal", Wal), ("Wun", Wun)):
        for G in (1, 4, 8, 16, 32):
            for method in ("min", "mid", "max", "uniform"):
                if wname == "W" and method in ("max", "uniform"):
                    continue
                if wname != "W" and method in ("min", "mid") and G != 4:
                    continue
                for inter, simd in ((1, 0), (0, 0), (0, 8), (0, 16)):
                    if simd and (G % simd or method == "mid"):
                        continue
                    if G == 1 and not inter:
                        continue
                    m, r_i = oracle.ref_merged_group(Wm, G, method, bool(inter), simd)
                    key = f"grp.{wname}.G{G}.{method}.i{inter}.s{simd}"
                    fx[key + ".meta"] = m
                    fx[key + ".ri"] = r_i
                    groups.append(key)
    print(len(groups), "group formats")

    # --- kernels: dense ground truth by the reference's own Direct kernels ---
    def direct_col(Xt, Wm):
        out_ = np.zeros((N, M), np.float32)
        oracle.ref_call("FD", "GEMM_CPU_FP32_colMajor_Direct_OpenMP", Xt.copy(), Wm, out_, M, N, K)
        return out_

    Yd = {"W": direct_col(XT, W), "Wal": direct_col(XT, Wal), "Wun": direct_col(XT, Wun)}
    for k, v in Yd.items():
        fx[f"direct_col.{k}"] = v                                     # [N][M]
        assert np.array_equal(v.T.astype(np.float64), X.astype(np.float64) @ fx[k].astype(np.float64))

    def try_formats(run, wname, cands):
        """run(meta, ri) -> output; return the first candidate format whose output equals Direct."""
        for key in cands:
            y = run(fx[key + ".meta"], fx[key + ".ri"])
            if y is not None and np.array_equal(y, Yd[wname]):
                return key, y
        return None, None

    kern = {}
    import re

    for name in oracle.ref_names("F1"):
        mG = re.search(r"xG(\d+)_", name)
        mrow = re.search(r"_(\d+)x", name)
        rows = int(mrow.group(1)) if mrow else 8
        if M % rows:
            continue

        def run(meta_, ri_, name=name):
            y = np.zeros((N, M), np.float32)
            oracle.ref_call("F1", name, XT, meta_, ri_, y, M, N, K)
            return y

        if "GroupMin" in name or "GroupMid" in name or "GroupMax" in name:
            G = int(mG.group(1))
            if N % G:
                continue
            method = "min" if "GroupMin" in name else "mid" if "GroupMid" in name else "max"
            wname = "Wal" if method == "max" else "W"
            cands = [k for k in groups if k.startswith(f"grp.{wname}.G{G}.{method}.")]
            key, y = try_formats(run, wname, cands)
        else:
            y = run(fx["merged_meta"], fx["merged_ri"])
            key = "merged" if np.array_equal(y, Yd["W"]) else None
        if key:
            kern[name] = key
    for name in oracle.ref_names("F2"):
        mG = re.search(r"xG(\d+)_", name)
        G = int(mG.group(1))
        rows = int(re.search(r"_(\d+)x", name).group(1))
        if M % rows or N % G:
            continue

        def run(meta_, ri_, name=name):
            y = np.zeros((N, M), np.float32)
            oracle.ref_call("F2", name, XT, int(meta_[0]), ri_, y, M, N, K)
            return y

        key, y = try_formats(run, "Wun", [k for k in groups if k.startswith(f"grp.Wun.G{G}.uniform.")])
        if key:
            kern[name] = key
    # GEMV (row-major x, int32 ids): first row of X only
    x0 = np.ascontiguousarray(X[0])
    y0 = {k: np.ascontiguousarray(v[:, 0]) for k, v in Yd.items()}
    for fam in ("F4", "F4U"):
        for name in oracle.ref_names(fam):
            G = int(re.search(r"_G(\d+)_", name).group(1))
            if N % G:
                continue
            wname = "Wun" if fam == "F4U" else "W"
            method = "uniform" if fam == "F4U" else "min"
            for key in [k for k in groups if k.startswith(f"grp.{wname}.G{G}.{method}.")]:
                ri32 = fx[key + ".ri"].astype(np.int32)
                ri32 = np.concatenate([ri32, np.zeros(64, np.int32)])     # vector loads may over-read the tail
                y = np.zeros(N, np.float32)
                if fam == "F4":
                    oracle.ref_call(fam, name, x0, fx[key + ".meta"], ri32, y, N, K)
                else:
                    oracle.ref_call(fam, name, x0, int(fx[key + ".meta"][0]), ri32, y, N, K)
                if np.array_equal(y, y0[wname]):
                    kern[name] = key
                    break
    # row-major GEMM (int32 ids)
    for name in oracle.ref_names("F3"):
        mG = re.search(r"xG(\d+)_", name)
        G = int(mG.group(1))
        rows = int(re.search(r"_(\d+)x", name).group(1))
        if M % rows or N % G:
            continue
        for key in [k for k in groups if k.startswith(f"grp.W.G{G}.min.")]:
            ri32 = np.concatenate([fx[key + ".ri"].astype(np.int32), np.zeros(64, np.int32)])
            y = np.zeros((M, N), np.float32)
            oracle.ref_call("F3", name, X.copy(), fx[key + ".meta"].copy(), ri32, y, M, N, K)
            if np.array_equal(y.T, Yd["W"]):
                kern[name] = key
                break
    # naive split CSC
    for name in oracle.ref_names("F5"):
        col = "colMajor" in name
        y = np.zeros((N, M) if col else (M, N), np.float32)
        oracle.ref_call("F5", name, (XT if col else X).copy(), rin.copy(), csn.copy(), rip.copy(), csp.copy(), y, M, N, K)
        if np.array_equal(y if col else y.T, Yd["W"]):
            kern[name] = "naive"
    # int8 (wrap-around)
    y8 = {}
    for name in oracle.ref_names("F6") + oracle.ref_names("F6U"):
        uni = "Uniform" in name
        G = int(re.search(r"xG(\d+)_", name).group(1))
        rows = int(re.search(r"_(\d+)x", name).group(1))
        if M % rows or N % G:
            continue
        wname = "Wun" if uni else "W"
        want = (X8.astype(np.int64) @ fx[wname].astype(np.int64)).astype(np.int8).T     # wraps mod 256
        for key in [k for k in groups if k.startswith(f"grp.{wname}.G{G}.{'uniform' if uni else 'min'}.")]:
            y = np.zeros((N, M), np.int8)
            if uni:
                oracle.ref_call("F6U", name, X8T, int(fx[key + ".meta"][0]), fx[key + ".ri"], y, M, N, K)
            else:
                oracle.ref_call("F6", name, X8T, fx[key + ".meta"], fx[key + ".ri"], y, M, N, K)
            if np.array_equal(y, want):
                kern[name] = key
                y8[wname] = y
                break
    for k, v in y8.items():
        fx[f"int8_col.{k}"] = v
    fx["kernel_names"] = np.array(sorted(kern), dtype="U128")
    fx["kernel_formats"] = np.array([kern[k] for k in sorted(kern)], dtype="U64")
    print(len(kern), "reference kernels reproduce their Direct product; formats used:")
    for k in sorted(kern):
        print("   ", k, "<-", kern[k])
    # drop formats that no kernel and no builder test needs?  keep all: they pin the builders.
    np.savez_compressed(out, **fx)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="checkout of the reference project (default: $TLLM_REFERENCE_ROOT, else ../reference)")
    a = ap.parse_args()
    if a.ref is None:
        import oracle

        a.ref = oracle.reference_root()
    gen_python_packers(a.ref, os.path.join(HERE, "gpu_packers.npz"))
    gen_cpu(os.path.join(HERE, "cpu_reference.npz"))
