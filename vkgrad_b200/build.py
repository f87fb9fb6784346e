"""Builds libvkgrad_b200.so in-tree with nvcc for sm_100a.

    python -m vkgrad_b200.build [--force] [--verbose]

The shared object lands next to this file so it travels with the source tree;
nothing is installed into site-packages and nothing is JIT-compiled at import.
"""

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libvkgrad_b200.so")
STAMP = os.path.join(HERE, "csrc", ".build_stamp")
SOURCES = ["runtime.cu", "gemm_sm100.cu", "attn_sm100.cu", "ops.cu", "comm.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _digest():
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + ["../../include/vkgrad_b200.h"]
    for name in names:
        path = os.path.join(CSRC, name)
        if name.startswith(".") or not os.path.isfile(path) or name.endswith(".o"):
            continue        # sources and headers only: object files are products
        h.update(name.encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compile every .cu into one shared library. Returns the library path."""
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(STAMP):
        with open(STAMP) as f:
            if f.read().strip() == digest:
                return LIB
    objs = []
    for src in _sources():
        obj = os.path.join(CSRC, src[:-3] + ".o")
        cmd = [_nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
               "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objs.append(obj)
    cmd = [_nvcc(), *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static", "-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    with open(STAMP, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
