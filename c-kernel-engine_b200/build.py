"""Builds libckb200.so in-tree: nvcc for the .cu kernels (sm_100a only), gcc for the C host code.

Usage:  python c-kernel-engine_b200/build.py [--verbose] [--force]
The object files go to c-kernel-engine_b200/build/, the library next to this file.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libckb200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
NVCC_FLAGS += os.environ.get("CKB_NVCC_EXTRA", "").split()       # e.g. -DCKB_TC_TRACE or -DCKB_STEP_TRACE for the in-kernel timeline recorders
CC_FLAGS = ["-O2", "-fPIC", "-std=c11", "-Wall", "-Wextra", "-Wno-unused-parameter", f"-I{CUDA_HOME}/include"]


def _newer(src: str, dst: str, deps: list[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src, *deps])


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(PKG, "..", "include", f) for f in os.listdir(os.path.join(PKG, "..", "include"))]
    headers.append(os.path.abspath(__file__))
    jobs = []
    objs = []
    for f in sorted(os.listdir(CSRC)):
        src = os.path.join(CSRC, f)
        if f.endswith(".cu"):
            obj = os.path.join(OBJ, f[:-3] + ".o")
            cmd = [NVCC, *NVCC_FLAGS, "-c", src, "-o", obj]
        elif f.endswith(".c"):
            obj = os.path.join(OBJ, f[:-2] + ".o")
            cmd = ["gcc", *CC_FLAGS, "-c", src, "-o", obj]
        else:
            continue
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append((f, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, r in ex.map(run, jobs):
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"compile failed: {name}")
            if verbose:
                sys.stderr.write(f"--- {name}\n{r.stderr}")
            with open(os.path.join(OBJ, name + ".ptxas.txt"), "w") as fh:
                fh.write(r.stderr)
    if jobs or not os.path.exists(LIB):
        link = [NVCC, "-shared", "-o", LIB, *objs, "-cudart", "static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    # the two thin model-ABI libraries (same symbol names, different signatures: they cannot share one library)
    for name, src in (("libckb200_model_v7.so", "model_v7.c"), ("libckb200_model_api.so", "model_handle.c")):
        out = os.path.join(PKG, name)
        srcp = os.path.join(CSRC, "abi", src)
        if force or _newer(srcp, out, headers + [LIB]):
            cmd = ["gcc", *CC_FLAGS, "-shared", "-fvisibility=hidden", srcp, "-o", out, f"-L{PKG}", "-lckb200", "-Wl,-rpath,$ORIGIN"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"compile failed: {src}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
