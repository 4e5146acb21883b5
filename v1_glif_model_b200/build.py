"""Builds ``libv1g.so`` (the C-ABI library) for sm_100a with nvcc, in-tree.

    python -m v1_glif_model_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects and the library land in
``v1_glif_model_b200/csrc/build/`` and ``v1_glif_model_b200/libv1g.so``.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libv1g.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

# -fmad=false: every float operation rounds on its own, as the reference's separate TensorFlow
# ops do, so the dense update reproduces a NumPy/PyTorch fp32 restatement bit for bit.
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
# Gradient kernels are held to 1e-4, not to bit-equality, so they may contract multiply-adds; so
# may the LGN filters, whose sums run in another order than the reference's convolutions anyway.
FMAD_OK = {"v1g_rollout_bwd.cu", "v1g_lgn.cu"}


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_dep():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(INCLUDE, "v1g.h"))
    deps.append(os.path.abspath(__file__))
    return max(os.path.getmtime(d) for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    out_dir = os.path.join(CSRC, "build")
    os.makedirs(out_dir, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(out_dir, src[:-3] + ".o")
        fmad = [] if src in FMAD_OK else ["-fmad=false"]
        cmd = [NVCC, *FLAGS, *fmad, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        results = list(ex.map(compile_one, sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs,
           "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
