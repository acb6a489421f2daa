"""Builds libqx_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libqx_b200.so")
OBJ = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]
# developer switch: extra -D defines for experiments
NVCC_FLAGS += os.environ.get("QX_B200_DEFINES", "").split()


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "qx_b200.h"))
    objects = []
    procs = []
    for src in sources():
        obj = os.path.join(OBJ, src[:-3] + ".o")
        objects.append(obj)
        path = os.path.join(CSRC, src)
        if _newer(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
                ["-DQX_BUILDING=1", "-c", path, "-o", obj]
            if verbose:
                print(" ".join(cmd))
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        text = out.decode()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src}\n{text}\n")
        elif text.strip() and (verbose or ptxas_info):
            print(f"--- {src}\n{text}")
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or _newer(LIB, objects):
        cmd = [nvcc, "-shared", "-o", LIB] + objects + ["-cudart", "static", "-ldl"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
