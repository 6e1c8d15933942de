"""ctypes wrapper of the CPU oracle (libgrab_oracle.so).  TEST INFRASTRUCTURE ONLY: imported
by tests/, the smoke check and the benchmark's CPU-baseline / reference arm, never by the
product package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgrab_oracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", HERE, "libgrab_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = C.CDLL(LIB_PATH)
        _lib.orc_dist.restype = C.c_float
        _lib.orc_make_key.restype = C.c_uint64
        _lib.orc_wang_hash.restype = C.c_uint32
    return _lib


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads():
    return lib().orc_num_threads()


def dist(q, x, metric=0):
    q, x = _f32(q), _f32(x)
    return float(lib().orc_dist(_p(q), _p(x), C.c_uint32(q.size), C.c_int(metric)))


def exact_search(data, queries, k, ts=None, lo=None, hi=None, labels=None, masks=None, metric=0,
                 canonical=True):
    data, queries = _f32(data), _f32(queries)
    n, dim = data.shape
    nq = queries.shape[0]
    ids = np.empty((nq, k), dtype=np.int64)
    dists = np.empty((nq, k), dtype=np.float32)
    if ts is not None:
        ts = np.ascontiguousarray(ts, dtype=np.uint64)
        lo = np.ascontiguousarray(np.broadcast_to(np.asarray(lo, dtype=np.uint64), (nq,)))
        hi = np.ascontiguousarray(np.broadcast_to(np.asarray(hi, dtype=np.uint64), (nq,)))
    if labels is not None:
        labels = np.ascontiguousarray(labels, dtype=np.uint8)
        masks = np.ascontiguousarray(np.broadcast_to(np.asarray(masks, dtype=np.uint32), (nq,)))
    lib().orc_exact_search(_p(data), C.c_uint64(n), C.c_uint32(dim), _p(ts), _p(labels), _p(queries),
                           C.c_uint64(nq), C.c_uint32(k), _p(lo), _p(hi), _p(masks), C.c_int(metric),
                           C.c_int(int(canonical)), _p(ids), _p(dists))
    return ids, dists


def warp_sort(keys, vals, asc=True):
    keys = _f32(keys).copy()
    vals = np.ascontiguousarray(vals, dtype=np.uint32).copy()
    lib().orc_warp_sort(_p(keys), _p(vals), C.c_uint32(keys.size), C.c_int(int(asc)))
    return keys, vals


def hash_insert(table, bitlen, key):
    return int(lib().orc_hash_insert(_p(table), C.c_uint32(bitlen), C.c_uint32(key)))


def knn_block(data, k, metric=0):
    data = _f32(data)
    n, dim = data.shape
    out = np.empty((n, k), dtype=np.uint32)
    lib().orc_knn_block(_p(data), C.c_uint64(n), C.c_uint32(dim), C.c_uint32(k), C.c_int(metric), _p(out))
    return out


def prune(knn, out_deg, want_detour=False):
    knn = np.ascontiguousarray(knn, dtype=np.uint32)
    n, in_deg = knn.shape
    out = np.empty((n, out_deg), dtype=np.uint32)
    det = np.empty((n, in_deg), dtype=np.uint8) if want_detour else None
    lib().orc_prune(_p(knn), _p(out), C.c_uint64(n), C.c_uint32(in_deg), C.c_uint32(out_deg), _p(det))
    return (out, det) if want_detour else out


def reverse_graph(graph):
    graph = np.ascontiguousarray(graph, dtype=np.uint32)
    n, deg = graph.shape
    rev = np.empty((n, deg), dtype=np.uint32)
    cnt = np.empty(n, dtype=np.uint32)
    lib().orc_reverse_graph(_p(graph), _p(rev), _p(cnt), C.c_uint64(n), C.c_uint32(deg))
    return rev, cnt


def merge_graphs(graph, rev, cnt):
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    n, deg = graph.shape
    lib().orc_merge_graphs(_p(graph), _p(np.ascontiguousarray(rev, dtype=np.uint32)),
                           _p(np.ascontiguousarray(cnt, dtype=np.uint32)), C.c_uint64(n), C.c_uint32(deg))
    return graph


def remote_edges(graph, bucket, cand, local_deg):
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    cand = np.ascontiguousarray(cand, dtype=np.uint32).copy()
    bucket = np.ascontiguousarray(bucket, dtype=np.uint64)
    n, total = graph.shape
    lib().orc_remote_edges(_p(graph), _p(bucket), _p(cand), C.c_uint64(n), C.c_uint32(total),
                           C.c_uint32(local_deg), C.c_uint32(cand.shape[1]))
    return graph, cand


def inject_reverse_remote(graph, local_deg, max_rev=32):
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    n, total = graph.shape
    lib().orc_inject_reverse_remote(_p(graph), C.c_uint64(n), C.c_uint32(total), C.c_uint32(local_deg),
                                    C.c_uint32(max_rev))
    return graph


def graph_search(data, graph, queries, k, itopk, width, max_iter, hash_bitlen, mode=0, ts=None, lo=None,
                 hi=None, active_deg=None, seeds=None, xor_mask=0x9E3779B97F4A7C15, metric=0,
                 want_stats=False):
    """mode 0 plain, 1 bucket prefix, 2 timestamp range (the reference's three kernels)."""
    data, queries = _f32(data), _f32(queries)
    graph = np.ascontiguousarray(graph, dtype=np.uint32)
    n, dim = data.shape
    nq = queries.shape[0]
    deg = graph.shape[1]
    ids = np.empty((nq, k), dtype=np.int64)
    dists = np.empty((nq, k), dtype=np.float32)
    stats = np.zeros(5, dtype=np.uint64)
    if ts is not None:
        ts = np.ascontiguousarray(ts, dtype=np.uint64)
        lo = np.ascontiguousarray(np.broadcast_to(np.asarray(lo, dtype=np.uint64), (nq,)))
        hi = np.ascontiguousarray(np.broadcast_to(np.asarray(hi, dtype=np.uint64), (nq,)))
    spq = 0
    if seeds is not None:
        seeds = np.ascontiguousarray(seeds, dtype=np.uint32)
        spq = seeds.shape[1]
    lib().orc_graph_search(_p(data), C.c_uint64(n), C.c_uint32(dim), _p(graph), C.c_uint32(deg),
                           C.c_uint32(active_deg if active_deg is not None else deg), _p(ts), _p(lo), _p(hi),
                           C.c_int(mode), _p(queries), C.c_uint64(nq), _p(seeds), C.c_uint32(spq),
                           C.c_uint64(xor_mask), C.c_uint32(k), C.c_uint32(itopk), C.c_uint32(width),
                           C.c_uint32(max_iter), C.c_uint32(hash_bitlen), C.c_int(metric), _p(ids), _p(dists),
                           _p(stats))
    return (ids, dists, stats) if want_stats else (ids, dists)


def insert_v1(graph, found, num_existing, search_k):
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    found = np.ascontiguousarray(found, dtype=np.int64)
    num_new = found.shape[0]
    lib().orc_insert_v1(_p(graph), _p(found), C.c_uint64(num_existing), C.c_uint64(num_new),
                        C.c_uint32(graph.shape[1]), C.c_uint32(search_k))
    return graph


def insert_opt(graph, bucket, local_knn, global_knn, num_existing, target_bucket, local_deg):
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    bucket = np.ascontiguousarray(bucket, dtype=np.uint64)
    local_knn = np.ascontiguousarray(local_knn, dtype=np.int64).copy()
    global_knn = np.ascontiguousarray(global_knn, dtype=np.int64).copy()
    num_new = local_knn.shape[0]
    lib().orc_insert_opt(_p(graph), _p(bucket), _p(local_knn), _p(global_knn), C.c_uint64(num_existing),
                         C.c_uint64(num_new), C.c_uint64(target_bucket), C.c_uint32(graph.shape[1]),
                         C.c_uint32(local_deg), C.c_uint32(local_knn.shape[1]), C.c_uint32(global_knn.shape[1]))
    return graph


def insert_opt_fill(graph, bucket, local_knn, global_knn, num_existing, local_deg):
    """Stage 1 of insert_opt alone: (graph with the new rows written, consumed local_knn, consumed global_knn)."""
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    bucket = np.ascontiguousarray(bucket, dtype=np.uint64)
    local_knn = np.ascontiguousarray(local_knn, dtype=np.int64).copy()
    global_knn = np.ascontiguousarray(global_knn, dtype=np.int64).copy()
    lib().orc_insert_opt_fill(_p(graph), _p(bucket), _p(local_knn), _p(global_knn), C.c_uint64(num_existing),
                              C.c_uint64(local_knn.shape[0]), C.c_uint32(graph.shape[1]), C.c_uint32(local_deg),
                              C.c_uint32(local_knn.shape[1]), C.c_uint32(global_knn.shape[1]))
    return graph, local_knn, global_knn


def insert_opt_mailboxes(graph, bucket, num_existing, target_bucket, local_deg):
    """Stage 2: (local counts, local lists [n, local/2], remote counts, remote lists [n, remote/2]); counts are
    the true request counts, lists keep the first `max` senders in ascending (new id, column) order; unused list
    entries are 0xFFFFFFFF."""
    graph = np.ascontiguousarray(graph, dtype=np.uint32)
    bucket = np.ascontiguousarray(bucket, dtype=np.uint64)
    n, total = graph.shape
    lmax, rmax = local_deg // 2, (total - local_deg) // 2
    lcnt, rcnt = np.zeros(n, dtype=np.uint32), np.zeros(n, dtype=np.uint32)
    llist = np.full((n, max(lmax, 1)), 0xFFFFFFFF, dtype=np.uint32)
    rlist = np.full((n, max(rmax, 1)), 0xFFFFFFFF, dtype=np.uint32)
    lib().orc_insert_opt_mailboxes(_p(graph), _p(bucket), C.c_uint64(num_existing), C.c_uint64(n - num_existing),
                                   C.c_uint64(target_bucket), C.c_uint32(total), C.c_uint32(local_deg), _p(lcnt),
                                   _p(llist), _p(rcnt), _p(rlist))
    return lcnt, llist[:, :lmax], rcnt, rlist[:, :rmax]


def insert_opt_apply(graph, bucket, num_existing, local_deg, lcnt, llist, rcnt, rlist):
    """Stage 3 on given mailboxes (lists [n, local/2] and [n, remote/2])."""
    graph = np.ascontiguousarray(graph, dtype=np.uint32).copy()
    bucket = np.ascontiguousarray(bucket, dtype=np.uint64)
    lcnt, rcnt = np.ascontiguousarray(lcnt, dtype=np.uint32), np.ascontiguousarray(rcnt, dtype=np.uint32)
    llist, rlist = np.ascontiguousarray(llist, dtype=np.uint32), np.ascontiguousarray(rlist, dtype=np.uint32)
    if llist.size == 0:
        llist = np.zeros(1, dtype=np.uint32)
    if rlist.size == 0:
        rlist = np.zeros(1, dtype=np.uint32)
    lib().orc_insert_opt_apply(_p(graph), _p(bucket), C.c_uint64(num_existing), C.c_uint32(graph.shape[1]),
                               C.c_uint32(local_deg), _p(lcnt), _p(llist), _p(rcnt), _p(rlist))
    return graph


def merge_topk(dists, ids, k):
    dists = _f32(dists)
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    nq, parts, _ = dists.shape
    oi = np.empty((nq, k), dtype=np.int64)
    od = np.empty((nq, k), dtype=np.float32)
    lib().orc_merge_topk(_p(dists), _p(ids), C.c_uint64(nq), C.c_uint32(parts), C.c_uint32(k), _p(oi), _p(od))
    return oi, od


def recall(result_ids, gt_ids):
    """|res ∩ gt| / min(|gt|, k), averaged over queries (tests/test_cagra_auto.cu:196)."""
    tot, cnt = 0.0, 0
    for r, g in zip(np.asarray(result_ids), np.asarray(gt_ids)):
        g = set(int(x) for x in g if x >= 0)
        if not g:
            continue
        tot += len(g.intersection(int(x) for x in r)) / len(g)
        cnt += 1
    return tot / max(cnt, 1)


class HNSW:
    """CPU HNSW baseline (oracle/hnsw_baseline.c): the published algorithm with the parameters of
    the reference's FAISS harness (tests/test_faiss_hnsw_insert.cpp: M 32, efConstruction 128,
    efSearch 64).  Not FAISS; parity unpinned."""

    def __init__(self, data, M=32, ef_construction=128, seed=1):
        self.data = _f32(data)            # the index borrows this array: keep it alive
        n, dim = self.data.shape
        L = lib()
        L.orc_hnsw_new.restype = C.c_void_p
        self.h = L.orc_hnsw_new(_p(self.data), C.c_uint64(n), C.c_uint32(dim), C.c_uint32(M),
                                C.c_uint32(ef_construction), C.c_uint64(seed))
        self.dim = dim

    def add(self, count):
        lib().orc_hnsw_add(C.c_void_p(self.h), C.c_uint64(count))

    def search(self, queries, k, ef=64):
        q = _f32(queries)
        ids = np.empty((q.shape[0], k), dtype=np.int64)
        d = np.empty((q.shape[0], k), dtype=np.float32)
        lib().orc_hnsw_search(C.c_void_p(self.h), _p(q), C.c_uint64(q.shape[0]), C.c_uint32(k), C.c_uint32(ef),
                              _p(ids), _p(d))
        return ids, d

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_hnsw_free(C.c_void_p(self.h))
            self.h = None


# ------------------------------------------------------------------ entry-point router
def nearest_centroids(rows, cen, cnorm, metric=0, probes=1):
    rows, cen, cnorm = _f32(rows), _f32(cen), _f32(cnorm)
    m, dim = rows.shape
    out = np.empty((m, probes), dtype=np.uint32)
    lib().orc_nearest_centroids(_p(rows), C.c_uint64(m), C.c_uint32(dim), _p(cen), _p(cnorm),
                                C.c_uint32(cen.shape[0]), C.c_int(metric), C.c_uint32(probes), _p(out))
    return out


def group_by_centroid(assign, num_centroids):
    assign = np.ascontiguousarray(assign, dtype=np.uint32).reshape(-1)
    offsets = np.empty(num_centroids + 1, dtype=np.uint32)
    members = np.empty(assign.shape[0], dtype=np.uint32)
    lib().orc_group_by_centroid(_p(assign), C.c_uint64(assign.shape[0]), C.c_uint32(num_centroids),
                                _p(offsets), _p(members))
    return offsets, members


def router_build(data, num_centroids, metric=0, iterations=10, max_sample=0):
    """k-means on the strided sample, then assignment and member lists: (cen, cnorm, offsets, members)."""
    data = _f32(data)
    n, dim = data.shape
    nc = num_centroids
    m = min(n, max_sample if max_sample else 64 * nc)
    m = max(m, nc)
    sample = np.ascontiguousarray(data[(np.arange(m, dtype=np.uint64) * np.uint64(n)) // np.uint64(m)])
    cen = np.ascontiguousarray(sample[(np.arange(nc, dtype=np.uint64) * np.uint64(m)) // np.uint64(nc)]).copy()
    cnorm = np.empty(nc, dtype=np.float32)
    empty = np.zeros(nc + 1, dtype=np.uint32)
    none = np.zeros(1, dtype=np.uint32)
    L = lib()
    L.orc_centroid_update(_p(sample), C.c_uint32(dim), _p(empty), _p(none), C.c_int(0), C.c_uint32(nc), _p(cen),
                          _p(cnorm))
    for _ in range(iterations):
        a = nearest_centroids(sample, cen, cnorm, metric, 1)
        offs, mem = group_by_centroid(a, nc)
        L.orc_centroid_update(_p(sample), C.c_uint32(dim), _p(offs), _p(mem), C.c_int(metric), C.c_uint32(nc),
                              _p(cen), _p(cnorm))
    a = nearest_centroids(data, cen, cnorm, metric, 1)
    offs, mem = group_by_centroid(a, nc)
    return cen, cnorm, offs, mem


def route_seeds(probes, n, offsets, members, seeds_per_query, seed=0x1234ABCD, ts=None, lo=None, hi=None,
                ts_sorted=True, labels=None, masks=None, label_offsets=None):
    """Seeds [nq, seeds_per_query] (0xFFFFFFFF = none); lo/hi and masks scalar or per query."""
    probes = np.ascontiguousarray(probes, dtype=np.uint32)
    nq, p = probes.shape
    offsets = np.ascontiguousarray(offsets, dtype=np.uint32)
    members = np.ascontiguousarray(members, dtype=np.uint32)
    kind, lo1, hi1, mask1 = 0, 0, 0, 0
    lo_a = hi_a = masks_a = None
    if ts is not None:
        kind = 1
        ts = np.ascontiguousarray(ts, dtype=np.uint64)
        if np.ndim(lo) == 0:
            lo1, hi1 = int(lo), int(hi)
        else:
            lo_a = np.ascontiguousarray(lo, dtype=np.uint64)
            hi_a = np.ascontiguousarray(hi, dtype=np.uint64)
    elif labels is not None:
        kind = 2
        labels = np.ascontiguousarray(labels, dtype=np.uint8)
        if np.ndim(masks) == 0:
            mask1 = int(masks)
        else:
            masks_a = np.ascontiguousarray(masks, dtype=np.uint32)
        if label_offsets is not None:
            label_offsets = np.ascontiguousarray(label_offsets, dtype=np.uint32)
    out = np.empty((nq, seeds_per_query), dtype=np.uint32)
    lib().orc_route_seeds(_p(probes), C.c_uint32(p), C.c_uint64(nq), C.c_uint64(n), C.c_uint32(offsets.shape[0] - 1),
                          _p(offsets), _p(members), C.c_int(kind), C.c_int(1 if ts_sorted else 0), _p(ts), _p(lo_a),
                          _p(hi_a), C.c_uint64(lo1), C.c_uint64(hi1), _p(labels), _p(masks_a), C.c_uint32(mask1),
                          _p(label_offsets), C.c_uint32(seeds_per_query), C.c_uint64(seed), _p(out))
    return out
