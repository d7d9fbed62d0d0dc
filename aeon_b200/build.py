"""In-tree build of libaeon_b200.so (CUDA kernels + host C++ behind the C ABI) for sm_100a.

Usage: ``python -m aeon_b200.build [--force] [--verbose]``.
The library is built next to this file so that it travels with the source tree.
"""
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaeon_b200.so")
OBJ = os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread", "-Xcompiler", "-Wall"]
# Exact OpenCV parity needs IEEE single operations: no implicit FMA contraction in device code.
CUDA_FLAGS = ["-fmad=false"]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers():
    out = [os.path.join(os.path.dirname(HERE), "include", "aeon_b200.h")]
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".hpp", ".cuh", ".h")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build aeon_b200")
    return exe


def build(force=False, verbose=False):
    """Compile every source for sm_100a and link the shared library.  Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    hdr = _digest(_headers(), " ".join(ARCH + COMMON + CUDA_FLAGS))
    objs = []
    rebuilt = False
    for src in sources():
        tag = _digest([src], hdr)
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_") + "." + tag + ".o")
        objs.append(obj)
        if os.path.exists(obj) and not force:
            continue
        cmd = [nvcc()] + ARCH + COMMON
        if src.endswith(".cu"):
            cmd += CUDA_FLAGS
            if verbose:
                cmd += ["-Xptxas", "-v"]
        else:
            cmd += ["-x", "cu"] if False else []
        cmd += ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        rebuilt = True
    # drop objects of older source versions
    for f in os.listdir(OBJ):
        p = os.path.join(OBJ, f)
        if p.endswith(".o") and p not in objs:
            os.remove(p)
    if rebuilt or force or not os.path.exists(LIB):
        cmd = [nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart", "-lpthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
