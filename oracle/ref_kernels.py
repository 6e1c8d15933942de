"""ctypes wrapper of oracle/_ref/libgrab_ref.so: the REFERENCE's own search kernels compiled for
sm_100a from its sources (see oracle/Makefile, target `ref`).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libgrab_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
    return _lib


def search(mode, dataset, graph, queries, k, itopk, width, max_iter, hash_bitlen, ts=None, lo=0, hi=0,
           active_deg=None, seeds=None, xor_mask=0x9E3779B97F4A7C15):
    """mode 0 search_kernel, 1 search_kernel_bucket, 2 search_kernel_range (one range per launch).
    All arrays are torch CUDA tensors.  Returns (ids int64 tensor, dists, kernel milliseconds)."""
    import torch
    n, dim = dataset.shape
    nq = queries.shape[0]
    deg = graph.shape[1]
    ids = torch.empty((nq, k), dtype=torch.int32, device=dataset.device)
    dists = torch.empty((nq, k), dtype=torch.float32, device=dataset.device)
    ms = C.c_float(0)
    p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    rc = lib().ref_search(C.c_int(mode), p(dataset), C.c_uint32(dim), C.c_uint64(n), p(graph), C.c_uint32(deg),
                          C.c_uint32(active_deg if active_deg is not None else deg), p(ts), C.c_uint64(lo),
                          C.c_uint64(hi), p(queries), C.c_int64(nq), C.c_uint32(k), C.c_uint32(itopk),
                          C.c_uint32(width), C.c_uint32(max_iter), C.c_uint32(hash_bitlen), p(seeds),
                          C.c_uint32(seeds.shape[1] if seeds is not None else 0), C.c_uint64(xor_mask), p(ids),
                          p(dists), C.byref(ms))
    if rc != 0:
        raise RuntimeError(f"reference kernel harness returned {rc}")
    return ids.to(torch.int64), dists, ms.value
