"""Build libturboquant_b200.so in-tree with nvcc for sm_100a.

    python turboquant-pytorch_b200/build.py [--force] [--verbose]

The library lands next to the Python package (turboquant/libturboquant_b200.so)
so that it is found without installation.  The CUDA runtime is linked
statically; the driver API is resolved at run time, so the library loads on a
machine without a GPU.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "turboquant", "libturboquant_b200.so")
SOURCES = ["tq_api.cu", "tq_simt.cu", "tq_umma.cu", "tq_qjl_umma.cu", "tq_v2_umma.cu", "tq_score_static.cu", "tq_copy.cu", "tq_attn_mma.cu", "tq_qjl_packed.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return exe


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "turboquant_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, ablate: bool = False, out: str = OUT, defines=()) -> str:
    """Compile the library.  `ablate` adds -DTQ_ABLATION: the timing-only switches that skip parts of the
    tensor-core kernels (environment variable TQ_ABLATE) exist only in such a build; give it its own `out`
    path and load it through TURBOQUANT_B200_LIB, never as the in-tree library."""
    if ablate and os.path.abspath(out) == os.path.abspath(OUT):
        raise ValueError("an ablation build must not replace the in-tree library: pass --out")
    if not force and out == OUT and not stale():
        return OUT
    # --fmad=false: products that the reference rounds before adding (k_mse before the
    # residual, for one) must not be contracted; the kernels call fmaf() where they want one.
    cmd = [nvcc_path(), *ARCH, "-lineinfo", "-O3", "-std=c++17", "--fmad=false", "--threads", "0", "-shared",
           "-Xcompiler", "-fPIC", "-Xcompiler", "-ffp-contract=off", "-o", out, *sources()]
    if ablate:
        cmd.insert(1, "-DTQ_ABLATION")
    for d in defines:
        cmd.insert(1, "-D" + d)
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ablate", action="store_true", help="profiling build with the TQ_ABLATE switches (needs --out)")
    ap.add_argument("--out", default=OUT)
    ap.add_argument("-D", dest="defines", action="append", default=[], help="extra preprocessor definitions")
    a = ap.parse_args()
    print(build(force=a.force or a.out != OUT, verbose=a.verbose, ablate=a.ablate, out=a.out, defines=a.defines))
