"""In-tree build of libgrab_anns.so (hand-written CUDA for sm_100a + the C ABI).

`python grab-anns_b200/build.py` or `build()` from Python.  The library is written next to
this file so that it travels with the source tree; nothing is installed anywhere else.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libgrab_anns.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fopenmp",
    "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", CSRC, "-I", HOST,
] + os.environ.get("GRAB_EXTRA_NVCC_FLAGS", "").split()


def _sources():
    out = []
    for d in (CSRC, HOST):
        if os.path.isdir(d):
            for f in sorted(os.listdir(d)):
                if f.endswith((".cu", ".cpp")):
                    out.append(os.path.join(d, f))
    return out


def _headers_digest():
    h = hashlib.sha256()
    for d in (CSRC, HOST, INCLUDE):
        if os.path.isdir(d):
            for f in sorted(os.listdir(d)):
                if f.endswith((".cuh", ".h", ".hpp")):
                    with open(os.path.join(d, f), "rb") as fh:
                        h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src, hdig, verbose):
    with open(src, "rb") as fh:
        dig = hashlib.sha256(fh.read() + hdig.encode()).hexdigest()[:16]
    obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
    stamp = obj + ".stamp"
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, ""
    cmd = ["nvcc", *NVCC_FLAGS, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as fh:
        fh.write(dig)
    return obj, r.stderr


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    srcs = _sources()
    hdig = _headers_digest()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, hdig, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = ["nvcc", "-shared", "-o", LIB, *objs, "-Xcompiler", "-fopenmp", "-lcudart", "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
