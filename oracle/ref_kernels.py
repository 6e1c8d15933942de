"""ctypes wrapper of oracle/_ref/libgrab_ref.so: the REFERENCE's own search and insert kernels compiled
for sm_100a from its sources (see oracle/Makefile, target `ref`).  Test infrastructure only."""
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


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference {what} returned {rc}")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def update_topology_v1(graph, found, num_existing, search_k):
    """update_topology_gpu_v1 (src/index/insert.cu:372-440) in place on `graph` (int32 CUDA tensor [n, deg] holding
    uint32 bits); found int64 [num_new, search_k]."""
    import torch
    torch.cuda.synchronize()
    _check(lib().ref_update_topology_v1(_ptr(graph), _ptr(found), C.c_uint64(num_existing),
                                        C.c_uint64(found.shape[0]), C.c_uint32(graph.shape[1]),
                                        C.c_uint32(search_k)), "update_topology_gpu_v1")


def insert_opt_fill(graph, ts, local_knn, global_knn, num_existing, local_deg):
    """fill_new_nodes_kernel_opt (insert.cu:448-577) in place; local candidates must be valid ids (the kernel
    reads d_ts[candidate] before it tests the candidate's sign)."""
    import torch
    torch.cuda.synchronize()
    _check(lib().ref_insert_opt_fill(_ptr(graph), _ptr(ts), _ptr(local_knn), _ptr(global_knn),
                                     C.c_uint64(num_existing), C.c_uint64(local_knn.shape[0]),
                                     C.c_uint32(graph.shape[1]), C.c_uint32(local_deg),
                                     C.c_uint32(local_knn.shape[1]), C.c_uint32(global_knn.shape[1])), "fill kernel")


def insert_opt_generate(graph, ts, num_existing, target_ts, local_deg):
    """generate_update_requests_kernel_opt (insert.cu:579-640): returns (lcount, llist, rcount, rlist) CUDA tensors;
    the order inside a list and, past the capacity, which senders were kept are an atomics race."""
    import torch
    n, total = graph.shape
    lmax, rmax = local_deg // 2, (total - local_deg) // 2
    dev = graph.device
    lc = torch.zeros(n, dtype=torch.int32, device=dev)
    rc = torch.zeros(n, dtype=torch.int32, device=dev)
    ll = torch.full((n, max(lmax, 1)), -1, dtype=torch.int32, device=dev)
    rl = torch.full((n, max(rmax, 1)), -1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    _check(lib().ref_insert_opt_generate(_ptr(graph), _ptr(lc), _ptr(ll), _ptr(rc), _ptr(rl),
                                         C.c_uint64(num_existing), C.c_uint64(n - num_existing),
                                         C.c_uint64(target_ts), _ptr(ts), C.c_uint32(total), C.c_uint32(local_deg)),
           "generate kernel")
    return lc, ll[:, :lmax], rc, rl[:, :rmax]


def insert_opt_apply(graph, ts, num_existing, local_deg, lcount, llist, rcount, rlist):
    """apply_topology_updates_kernel_opt (insert.cu:653-765) in place on `graph` with the given mailboxes
    (lists contiguous [n, local/2] and [n, remote/2])."""
    import torch
    ll = llist.contiguous() if llist.numel() else torch.zeros(1, dtype=torch.int32, device=graph.device)
    rl = rlist.contiguous() if rlist.numel() else torch.zeros(1, dtype=torch.int32, device=graph.device)
    torch.cuda.synchronize()
    _check(lib().ref_insert_opt_apply(_ptr(graph), _ptr(lcount), _ptr(ll), _ptr(rcount), _ptr(rl), _ptr(ts),
                                      C.c_uint64(num_existing), C.c_uint32(graph.shape[1]), C.c_uint32(local_deg)),
           "apply kernel")


def update_topology_opt(graph, data, ts, local_knn, global_knn, num_existing, target_ts, local_deg):
    """update_topology_gpu_opt (insert.cu:1398-1573) as the reference's insert calls it, in place."""
    import torch
    nn_, kl = local_knn.shape
    kg = global_knn.shape[1]
    ld = torch.zeros((nn_, kl), dtype=torch.float32, device=graph.device)
    gd = torch.zeros((nn_, kg), dtype=torch.float32, device=graph.device)
    torch.cuda.synchronize()
    _check(lib().ref_update_topology_opt(_ptr(graph), _ptr(data), C.c_uint64(data.shape[1]), C.c_uint64(target_ts),
                                         _ptr(ts), _ptr(local_knn), _ptr(ld), _ptr(global_knn), _ptr(gd),
                                         C.c_uint64(num_existing), C.c_uint64(nn_), C.c_uint32(graph.shape[1]),
                                         C.c_uint32(local_deg), C.c_uint32(kl), C.c_uint32(kg)),
           "update_topology_gpu_opt")


def find_near_nodes(data, num_existing, new, graph, search_k, itopk, width, max_iter, hash_bitlen):
    """find_near_nodes (insert.cu:140-219): (ids int64 [num_new, search_k], exact dists ascending)."""
    import torch
    nn_ = new.shape[0]
    ids = torch.empty((nn_, search_k), dtype=torch.int64, device=data.device)
    dists = torch.empty((nn_, search_k), dtype=torch.float32, device=data.device)
    torch.cuda.synchronize()
    _check(lib().ref_find_near_nodes(_ptr(data), C.c_uint32(data.shape[1]), C.c_uint64(num_existing),
                                     C.c_uint64(nn_), _ptr(new), _ptr(graph), C.c_uint32(graph.shape[1]),
                                     C.c_uint32(search_k), C.c_uint32(itopk), C.c_uint32(width),
                                     C.c_uint32(max_iter), C.c_uint32(hash_bitlen), _ptr(ids), _ptr(dists)),
           "find_near_nodes")
    return ids, dists


# ---------------------------------------------------------------------------------------------------------
# Graph optimisation (src/index/cagra.cu compiled with the FAISS declaration shim, oracle/ref_build_harness.cu).
# Host numpy arrays in and out, as the reference's functions take them; they launch their own kernels.
# ---------------------------------------------------------------------------------------------------------
def _np_u32(a):
    import numpy as np
    return np.ascontiguousarray(a, dtype=np.uint32)


def optimize_prune(knn, out_deg):
    """optimize_prune (src/index/cagra.cu:286-401): [n, in_deg] uint32 kNN graph -> [n, out_deg] pruned graph."""
    import numpy as np
    knn = _np_u32(knn)
    n, in_deg = knn.shape
    out = np.empty((n, out_deg), dtype=np.uint32)
    _check(lib().ref_optimize_prune(knn.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_uint64(n),
                                    C.c_uint32(in_deg), C.c_uint32(out_deg)), "optimize_prune")
    return out


def optimize_reverse(graph):
    """optimize_create_reverse_graph (src/index/cagra.cu:455-548): -> (rev [n, deg], counts [n])."""
    import numpy as np
    graph = _np_u32(graph)
    n, deg = graph.shape
    rev = np.full((n, deg), 0xFFFFFFFF, dtype=np.uint32)
    cnt = np.zeros(n, dtype=np.uint32)
    _check(lib().ref_optimize_reverse(graph.ctypes.data_as(C.c_void_p), rev.ctypes.data_as(C.c_void_p),
                                      cnt.ctypes.data_as(C.c_void_p), C.c_uint64(n), C.c_uint32(deg)),
           "optimize_create_reverse_graph")
    return rev, cnt


def optimize_merge(graph, rev, counts):
    """optimize_merge_graphs (src/index/cagra.cu:574-650): returns the merged copy of `graph`."""
    graph = _np_u32(graph).copy()
    rev, counts = _np_u32(rev), _np_u32(counts)
    n, deg = graph.shape
    _check(lib().ref_optimize_merge(graph.ctypes.data_as(C.c_void_p), rev.ctypes.data_as(C.c_void_p),
                                    counts.ctypes.data_as(C.c_void_p), C.c_uint64(n), C.c_uint32(deg)),
           "optimize_merge_graphs")
    return graph


def build(data, raw_knn, deg):
    """build (src/index/cagra.cu:665-711): device dataset [n, dim] and raw kNN graph (int32 CUDA tensor [n, inter]
    holding uint32 bits) -> final graph, int32 CUDA tensor [n, deg]."""
    import torch
    n, inter = raw_knn.shape
    out = torch.empty((n, deg), dtype=torch.int32, device=raw_knn.device)
    torch.cuda.synchronize()
    _check(lib().ref_build(_ptr(data), C.c_uint64(n), _ptr(raw_knn), C.c_uint32(inter), C.c_uint32(deg), _ptr(out)),
           "build")
    return out


# ---------------------------------------------------------------------------------------------------------
# Remote edges, reverse injection and the reference's own launchers (src/index/cagra_opt.cu compiled with the
# FAISS / RAFT / RMM declaration shims, oracle/ref_opt_harness.cu).  torch CUDA tensors (int32 holding uint32 bits).
# ---------------------------------------------------------------------------------------------------------
def update_remote_edges(graph, ts, cand, local_deg):
    """update_remote_edges_kernel (cagra_opt.cu:209-303) in place on `graph` [n, total]; `cand` [n, gk] is consumed."""
    n, total = graph.shape
    _check(lib().ref_update_remote_edges(_ptr(graph), _ptr(ts), _ptr(cand), C.c_uint64(n), C.c_uint32(total),
                                         C.c_uint32(local_deg), C.c_uint32(cand.shape[1])), "update_remote_edges_kernel")


def make_global_rev(graph, local_deg, max_rev=32):
    """kern_make_global_rev_graph (cagra_opt.cu:457-482) -> (rev [n, max_rev], counts [n]); racy order inside a list."""
    import torch
    n, total = graph.shape
    rev = torch.full((n, max_rev), -1, dtype=torch.int32, device=graph.device)
    cnt = torch.zeros(n, dtype=torch.int32, device=graph.device)
    _check(lib().ref_make_global_rev(_ptr(graph), _ptr(rev), _ptr(cnt), C.c_uint64(n), C.c_uint32(total),
                                     C.c_uint32(local_deg), C.c_uint32(max_rev)), "kern_make_global_rev_graph")
    return rev, cnt


def inject_global_rev(graph, rev, cnt, local_deg):
    """kern_inject_global_reverse_edges (cagra_opt.cu:487-600) in place on `graph`."""
    n, total = graph.shape
    _check(lib().ref_inject_global_rev(_ptr(graph), _ptr(rev), _ptr(cnt), C.c_uint64(n), C.c_uint32(total),
                                       C.c_uint32(local_deg), C.c_uint32(rev.shape[1])),
           "kern_inject_global_reverse_edges")


def enhance_global_connectivity(graph, local_deg):
    """enhance_global_connectivity (cagra_opt.cu:739-793): both kernels in a row, in place (racy through the lists)."""
    n, total = graph.shape
    _check(lib().ref_enhance_global_connectivity(C.c_uint64(n), _ptr(graph), C.c_uint32(total), C.c_uint32(local_deg)),
           "enhance_global_connectivity")


def search_launcher(mode, dataset, graph, queries, k, itopk, width, max_iter, hash_bitlen, local_deg=None, ts=None,
                    lo=0, hi=0, seeds=None):
    """The reference's own launchers: mode 0 search_opt, 1 search_bucket_opt, 2 search_bucket_range."""
    import torch
    n, dim = dataset.shape
    nq = queries.shape[0]
    total = graph.shape[1]
    ids = torch.empty((nq, k), dtype=torch.int64, device=dataset.device)
    dists = torch.empty((nq, k), dtype=torch.float32, device=dataset.device)
    torch.cuda.synchronize()
    _check(lib().ref_search_launcher(C.c_int(mode), _ptr(dataset), C.c_uint32(dim), C.c_uint64(n), _ptr(graph),
                                     C.c_uint32(total), C.c_uint32(local_deg if local_deg is not None else total),
                                     _ptr(ts), C.c_uint64(lo), C.c_uint64(hi), _ptr(queries), C.c_int64(nq),
                                     C.c_int64(k), C.c_uint32(itopk), C.c_uint32(width), C.c_uint32(max_iter),
                                     C.c_uint32(hash_bitlen), _ptr(seeds),
                                     C.c_uint32(seeds.shape[1] if seeds is not None else 0), _ptr(ids), _ptr(dists)),
           "search launcher")
    return ids, dists
