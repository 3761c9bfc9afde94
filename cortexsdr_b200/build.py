"""Builds libcortexsdr_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcortexsdr_b200.so")

SOURCES = [
    "capi.cu",
    "kernels/matmul.cu",
    "kernels/decode.cu",
    "kernels/gemv_fused.cu",
    "kernels/gemv_queue.cu",
    "kernels/decoder_ops.cu",
    "kernels/gemm_tcgen05.cu", "kernels/gemm_tma.cu",
    "decoder.cu",
    "kernels/encode.cu",
    "encoder.cu",
    "host/format.cpp",
    "host/archive.cpp",
    "host/sdk_capi.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unknown-pragmas",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for root, _, files in os.walk(CSRC):
        for f in files:
            if os.path.getmtime(os.path.join(root, f)) > t:
                return True
    inc = os.path.join(HERE, "..", "include")
    return any(os.path.getmtime(os.path.join(inc, f)) > t for f in os.listdir(inc))


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    objs = []
    procs = []
    for s in sources:
        obj = os.path.join(objdir, s.replace("/", "_") + ".o")
        objs.append(obj)
        cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", os.path.join(CSRC, s), "-o", obj]
        if ptxas_verbose:
            cmd += ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for s, p in procs:
        out = p.communicate()[0].decode()
        if out.strip() and (verbose or ptxas_verbose or p.returncode):
            print(f"--- {s}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "-ldl"]
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_verbose="--ptxas" in sys.argv)
    print(LIB)
