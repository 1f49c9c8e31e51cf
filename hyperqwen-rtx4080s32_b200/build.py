"""Build the CUDA library in-tree for sm_100a: hyperqwen-rtx4080s32_b200/libgq_b200.so.

nvcc cross-compiles without a GPU.  The format tables are generated first from the installed gguf
package (csrc/gen_tables.py).  `python -m hyperqwen_rtx4080s32_b200.build` or build() from Python.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB = os.path.join(_HERE, "libgq_b200.so")
SOURCES = ["gq_b200.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))) + [os.path.join("..", "..", "include", "gq_b200.h")]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--expt-relaxed-constexpr", "-diag-suppress", "177",
              "-shared", "-Xcompiler", "-fPIC"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths if os.path.exists(p))


def build(force: bool = False, verbose: bool = False) -> str:
    sys.path.insert(0, CSRC)
    try:
        import gen_tables
    finally:
        sys.path.pop(0)
    table_h = gen_tables.generate()
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS] + [table_h]
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(deps):
        return LIB
    nvcc = os.environ.get("NVCC") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + srcs
    subprocess.check_call(cmd, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
