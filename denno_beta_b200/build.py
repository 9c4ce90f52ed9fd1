"""Build libdnb200.so (the CUDA library with the C ABI of include/dnb200.h) in-tree.

    python -m denno_beta_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The shared object is written next
to this file; it links the CUDA runtime statically and needs nothing from Python.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdnb200.so")
OBJ = os.path.join(HERE, "build")
SOURCES = ["api.cu", "router_tc.cu", "seg_matmul.cu", "gemv_bulk.cu", "gemv_mma.cu", "decode_fused.cu", "grouped_umma.cu", "grouped_exact.cu", "grouped_q4k_int.cu", "moe_kernels.cu", "synth.cu", "ep_p2p.cu", "ep_decode.cu", "gguf_loader.cu", "hc_mix.cu"]
NVCC = os.environ.get("DNB_NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-ccbin", "g++",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _deps():
    d = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    d += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return d


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    dep_m = max(os.path.getmtime(p) for p in _deps())
    objs = []
    jobs = []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), dep_m):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in jobs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("---- %s\n%s\n" % (s, out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or force or not os.path.exists(OUT):
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++"]
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
