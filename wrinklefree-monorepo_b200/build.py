"""Compiles the CUDA sources of this package into libwf_b200.so (in-tree, sm_100a only)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libwf_b200.so")
SOURCES = ["wf_capi.cu", "wf_pack.cu", "wf_actquant.cu", "wf_decode.cu", "wf_prefill.cu", "wf_elementwise.cu",
           "wf_allreduce.cu", "wf_probe.cu", "wf_attention.cu", "wf_linear.cu"]
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _host_compiler() -> str:
    """The distribution's g++ when it exists (some images put a wrapper without OpenMP first on PATH)."""
    cand = os.path.join(os.sep, "usr", "bin", "g++")
    return os.environ.get("CXX") or (cand if os.path.exists(cand) else "g++")


def _nvcc() -> str:
    if os.environ.get("NVCC"):
        return os.environ["NVCC"]
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or os.path.join(os.sep, "usr", "local", "cuda")
    cand = os.path.join(home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
           [os.path.join(HERE, "..", "include", "wf_b200.h")]


def _newer(target: str, deps) -> bool:
    """True when `target` is missing or older than one of `deps`."""
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles the sources whose object is older than the source or a header, links libwf_b200.so when an object
    changed; returns its path."""
    nvcc, cxx = _nvcc(), _host_compiler()
    objs, procs = [], []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    hdrs = _headers()
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        objs.append(obj)
        if not force and not _newer(obj, [os.path.join(CSRC, src), *hdrs]):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-ccbin", cxx, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    if procs or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-ccbin", cxx]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
