"""Builds libaxiom_b200.so (CUDA kernels + C ABI) and libaxiom_b200_backend.so
(the C host layer that fills axiom's backend vtable) in-tree for sm_100a.

    python -m axiom_b200.build          # incremental
    python -m axiom_b200.build --force  # rebuild everything

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is
installed.  Objects land in axiom_b200/build/, libraries in axiom_b200/lib/.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "lib")
ENGINE_SO = os.path.join(LIB, "libaxiom_b200.so")
BACKEND_SO = os.path.join(LIB, "libaxiom_b200_backend.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + cmd[0])
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    cus = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    for f in cus:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".o")
        if force or not _newer(obj, [src] + headers):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=8) as ex:
            for out in ex.map(_run, jobs):
                if verbose or ptxas_info:
                    sys.stderr.write(out)
    objs = [os.path.join(OBJ, f[:-3] + ".o") for f in cus]
    if force or jobs or not _newer(ENGINE_SO, objs):
        _run(["nvcc", "-shared", "-o", ENGINE_SO] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                             "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lrt", "-lpthread"])
    # C host layer (vtable adapter); plain gcc, links against the engine
    host_srcs = sorted(os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".c")) if os.path.isdir(HOST) else []
    if host_srcs and (force or jobs or not _newer(BACKEND_SO, host_srcs + headers + [ENGINE_SO])):
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-fvisibility=hidden",
              "-I" + os.path.join(ROOT, "include"), "-o", BACKEND_SO] + host_srcs +
             ["-L" + LIB, "-laxiom_b200", "-Wl,-rpath,$ORIGIN"])
    return ENGINE_SO


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(ENGINE_SO)
