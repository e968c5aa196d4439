"""Builds ``tnsr_b200/csrc/libtnsr_b200.so`` in-tree with nvcc for sm_100a.

    python -m tnsr_b200.build [--force] [--verbose]

Every ``.cu`` file is compiled with ``-gencode arch=compute_100a,code=sm_100a``
and linked into one shared library whose only exports are the ``extern "C"``
entry points of ``include/tnsr_b200.h``.  ``strict.cu`` and ``encoder.cu`` are
compiled with ``--fmad=false``: their kernels must round every product before
adding it.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(CSRC, "libtnsr_b200.so")

SOURCES = ["decoder.cu", "ops_api.cu", "elementwise.cu", "strict.cu", "gemm.cu", "gemm_skinny.cu", "attention.cu", "prefill.cu", "prefill_tc.cu",
           "decode_attention_static.cu", "sampler.cu", "encoder.cu", "decode_tail.cu", "gemm_stream.cu"]
EXTRA = {"strict.cu": ["--fmad=false"], "encoder.cu": ["--fmad=false"]}

BASE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build tnsr_b200")
    return path


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = list(SOURCES)
    # every object depends on every header of the library: editing any .cuh (or the public header) rebuilds all
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(HERE, "..", "include", "tnsr_b200.h")]
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            cmd = [nvcc(), "-c", os.path.join(CSRC, src), "-o", obj] + BASE_FLAGS + EXTRA.get(src, [])
            if verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, res

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, res in pool.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {cmd[2]}")
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in sources]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                        "-Xcompiler", "-fPIC"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libtnsr_b200.so failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.force, args.verbose))
