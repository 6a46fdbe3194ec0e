"""Build libjitllm_b200.so in-tree with nvcc for sm_100a.

    python -m jitllm_b200.build [--force] [--verbose]

Cross-compiles without a GPU. Objects are rebuilt only when their source (or a
header) is newer; the shared library lands beside this file.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libjitllm_b200.so")
SOURCES = ["ctx.cu", "formats.cu", "gemv.cu", "gemv_q8.cu", "gemv_mxfp4.cu", "gemm_tc5.cu", "moe.cu", "aux.cu", "block.cu", "packed.cu", "tune.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-DJL_BUILD",
]


def _nvcc() -> str:
    n = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(n):
        raise RuntimeError("nvcc not found: libjitllm_b200.so cannot be built")
    return n


def _newer(dst: str, srcs: list[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "jitllm_b200.h"))
    nvcc = _nvcc()
    # the build's identity: persisted selection verdicts are keyed on it (a changed kernel is measured again)
    h = hashlib.sha1()
    for f in sorted(headers + [os.path.join(CSRC, s) for s in SOURCES]):
        h.update(open(f, "rb").read())
    build_id = h.hexdigest()[:16]
    stamp = os.path.join(OBJ, "build_id.txt")
    if not os.path.exists(stamp) or open(stamp).read() != build_id:
        open(stamp, "w").write(build_id)
    objs = []
    procs = []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s.replace(".cu", ".o"))
        objs.append(obj)
        extra = [stamp] if s == "tune.cu" else []
        if force or _newer(obj, [src] + headers + extra):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if s == "tune.cu":
                cmd.insert(-4, f'-DJL_BUILD_ID="{build_id}"')
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stdout.write(out)
        if p.returncode != 0:
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
