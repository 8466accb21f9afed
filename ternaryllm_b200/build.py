"""Build libtllm.so (the C-ABI shared library) in-tree with nvcc for sm_100a.

    python -m ternaryllm_b200.build [--force] [--verbose]

The library has no dependency on torch; the Python modules of this package bind it with ctypes.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtllm.so")
SOURCES = ["capi.cu", "comm.cu", "packer.cpp", "bstream_pack.cpp", "ssr_format.cpp"]
DEPS = ["kernels.cuh", "mma_kernel.cuh", "bstream_kernel.cuh", "nibble_kernel.cuh", "nibble_rows_kernel.cuh", "nibble_format.h", "bstream_format.h", "bittile_format.h", "column_lists.h", "util.h", os.path.join("..", "..", "include", "tllm.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O2", "--shared", "-Xptxas", "-v",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log = os.path.join(HERE, "build.log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("nvcc failed; see " + log)
    if verbose:
        print(r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
