"""In-tree build of the native libraries (no torch, no JIT cache).

libyuuka_cuda.so   hand-written sm_100a kernels + the C ABI (include/yuuka_cuda.h)
libyuuka_synth.so  host-only synthetic-weight generator and quantizers
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
CUDA_LIB = os.path.join(HERE, "libyuuka_cuda.so")
SYNTH_LIB = os.path.join(HERE, "libyuuka_synth.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2,-Wall",
    "--expt-relaxed-constexpr",
]


def _host_cc() -> str:
    for cand in ("/usr/bin/gcc", shutil.which("gcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("no host C compiler found")


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_synth(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "synth_quant.c")
    if force or _stale(SYNTH_LIB, [src]):
        cmd = [_host_cc(), "-O2", "-fopenmp", "-fPIC", "-fvisibility=hidden", "-std=c11", "-Wall",
               "-shared", "-o", SYNTH_LIB, src, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return SYNTH_LIB


def cuda_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build_cuda(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> str:
    srcs = cuda_sources()
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not (force or _stale(CUDA_LIB, deps)):
        return CUDA_LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and not _stale(o, [s] + [d for d in deps if not d.endswith(".cu")]):
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", s, "-o", o]
        if ptxas_v:
            cmd.insert(1, "-Xptxas=-v")
        if verbose:
            print(" ".join(cmd))
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or ptxas_v or (verbose and out.strip()):
            print(f"--- {os.path.basename(s)}\n{out}")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-shared", "-o", CUDA_LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined",
           "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return CUDA_LIB


def build_all(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> None:
    build_synth(force, verbose)
    build_cuda(force, verbose, ptxas_v)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True, ptxas_v="--ptxas-v" in sys.argv)
