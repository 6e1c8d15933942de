"""grab-anns_b200: B200-native hot path of GRAB-ANNS behind a C ABI.

This module is the thin Python binding (ctypes) used by the tests and the benchmark.
All compute lives in ``libgrab_anns.so`` (hand-written CUDA for sm_100a); there is no
Python or CPU fallback: importing the bindings without the built library raises.

Import with ``importlib.import_module("grab-anns_b200")`` (the directory name carries a
hyphen).
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgrab_anns.so")

METRIC_L2, METRIC_IP = 0, 1
FILTER_NONE, FILTER_TS_RANGE, FILTER_LABELS, FILTER_PREFIX = 0, 1, 2, 3
KNN_EXACT_SCAN, KNN_TC_BF16, KNN_TC_SPLIT = 0, 1, 2
ROUTER_EXACT_SCAN = 1
GLOBAL_AUTO, GLOBAL_ALL_PAIRS, GLOBAL_ROUTED_SEARCH = 0, 1, 2


class GrabError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"grab status {status}: {msg}")
        self.status = status


class BuildParams(C.Structure):
    _fields_ = [("intermediate_degree", C.c_uint32), ("graph_degree", C.c_uint32)]


class SearchParams(C.Structure):
    """Mirror of the reference's SearchParams (src/index/cagra.cuh:36-42)."""
    _fields_ = [("itopk_size", C.c_uint32), ("search_width", C.c_uint32),
                ("min_iterations", C.c_uint32), ("max_iterations", C.c_uint32),
                ("hash_bitlen", C.c_uint32)]

    def __init__(self, itopk_size=64, search_width=5, min_iterations=0, max_iterations=20,
                 hash_bitlen=12):
        super().__init__(itopk_size, search_width, min_iterations, max_iterations, hash_bitlen)


class Filter(C.Structure):
    _fields_ = [("kind", C.c_int32), ("ts_sorted", C.c_int32), ("d_ts", C.c_void_p),
                ("d_lo", C.c_void_p), ("d_hi", C.c_void_p), ("lo", C.c_uint64), ("hi", C.c_uint64),
                ("d_labels", C.c_void_p), ("d_masks", C.c_void_p), ("mask", C.c_uint32),
                ("active_degree", C.c_uint32), ("d_label_offsets", C.c_void_p), ("d_id_windows", C.c_void_p)]


class SearchStats(C.Structure):
    _fields_ = [("iterations", C.c_uint64), ("parents", C.c_uint64), ("edges", C.c_uint64),
                ("distances", C.c_uint64), ("seeds", C.c_uint64), ("hash_resets", C.c_uint64)]


class SearchArgs(C.Structure):
    _fields_ = [("d_dataset", C.c_void_p), ("n", C.c_uint64), ("dim", C.c_uint32),
                ("metric", C.c_int32), ("d_graph", C.c_void_p), ("graph_degree", C.c_uint32),
                ("d_queries", C.c_void_p), ("nq", C.c_uint64), ("k", C.c_uint32),
                ("params", SearchParams), ("filter", Filter), ("d_seeds", C.c_void_p),
                ("seeds_per_query", C.c_uint32), ("seed", C.c_uint64), ("d_out_ids", C.c_void_p),
                ("d_out_dists", C.c_void_p), ("id_scale", C.c_uint64), ("id_offset", C.c_uint64),
                ("d_stats", C.c_void_p), ("d_ws", C.c_void_p), ("ws_bytes", C.c_size_t),
                ("stream", C.c_void_p), ("d_out_keys", C.c_void_p), ("ctas_per_query", C.c_uint32)]


CTAS_AUTO = 0xFFFFFFFF


class RouterStruct(C.Structure):
    _fields_ = [("num_centroids", C.c_uint32), ("dim", C.c_uint32), ("metric", C.c_int32),
                ("d_centroids", C.c_void_p), ("d_centroid_norms", C.c_void_p),
                ("d_member_offsets", C.c_void_p), ("d_members", C.c_void_p), ("flags", C.c_uint32)]


_lib = None


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile libgrab_anns.so in-tree (nvcc, sm_100a)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_grab_build", os.path.join(HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=verbose, force=force)


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise GrabError(-1, f"{LIB_PATH} is missing: run `python grab-anns_b200/build.py` "
                                "(the CUDA extension is the only implementation)")
        _lib = C.CDLL(LIB_PATH)
        _lib.grab_last_error.restype = C.c_char_p
        _lib.grab_status_string.restype = C.c_char_p
        _lib.grab_exact_search_workspace_bytes.restype = C.c_size_t
        _lib.grab_exact_search_workspace_bytes.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32]
        _lib.grab_graph_search_workspace_bytes.restype = C.c_size_t
        _lib.grab_graph_search_workspace_bytes.argtypes = [C.c_uint64, C.c_uint32]
        _lib.grab_graph_search_workspace_bytes_for.restype = C.c_size_t
        _lib.grab_graph_search_workspace_bytes_for.argtypes = [C.c_void_p]
        _lib.grab_route_seeds_workspace_bytes.restype = C.c_size_t
        _lib.grab_route_seeds_workspace_bytes.argtypes = [C.c_uint64, C.c_uint32]
    return _lib


def check(status: int):
    if status != 0:
        raise GrabError(status, lib().grab_last_error().decode())


def _p(t):
    """Device (or host) pointer of a torch tensor / numpy array, None -> NULL."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        assert t.is_contiguous()
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_filter(kind=FILTER_NONE, ts=None, lo=None, hi=None, ts_sorted=False, labels=None,
                masks=None, active_degree=0, label_offsets=None, id_windows=None) -> Filter:
    """id_windows: optional int32 tensor [nq, 4] shared by route_seeds (writes every query's id window) and a
    graph_search with the same queries and ranges (reads it instead of searching the timestamps again)."""
    f = Filter()
    f.kind = kind
    f.ts_sorted = int(ts_sorted)
    f.d_ts = _p(ts)
    if hasattr(lo, "data_ptr"):
        f.d_lo, f.d_hi = _p(lo), _p(hi)
    elif lo is not None:
        f.lo, f.hi = int(lo), int(hi)
    f.d_labels = _p(labels)
    if hasattr(masks, "data_ptr"):
        f.d_masks = _p(masks)
    elif masks is not None:
        f.mask = int(masks)
    f.active_degree = active_degree
    f.d_label_offsets = _p(label_offsets)
    f.d_id_windows = _p(id_windows)
    # the struct only holds raw pointers: keep the tensors alive as long as the filter is
    f._keepalive = (ts, lo, hi, labels, masks, label_offsets, id_windows)
    return f


def exact_search(dataset, queries, k, metric=METRIC_L2, flt: Filter | None = None):
    """Exact filtered top-k on the GPU (bit-exact ids against the CPU oracle)."""
    import torch
    n, dim = dataset.shape
    nq = queries.shape[0]
    ids = torch.empty((nq, k), dtype=torch.int64, device=dataset.device)
    dists = torch.empty((nq, k), dtype=torch.float32, device=dataset.device)
    ws_bytes = lib().grab_exact_search_workspace_bytes(n, nq, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dataset.device)
    check(lib().grab_exact_search(_p(dataset), C.c_uint64(n), C.c_uint32(dim), C.c_int(metric),
                                  C.byref(flt) if flt is not None else None, _p(queries),
                                  C.c_uint64(nq), C.c_uint32(k), _p(ids), _p(dists), _p(ws),
                                  C.c_size_t(ws_bytes), _stream()))
    return ids, dists


def search_args(dataset, graph, queries, k, params: SearchParams, metric=METRIC_L2, flt: Filter | None = None,
                seeds=None, ctas_per_query=0) -> SearchArgs:
    """A grab_search_args with the inputs filled in (no outputs, no workspace): what
    grab_graph_search_workspace_bytes_for() needs."""
    a = SearchArgs()
    a.d_dataset, a.n, a.dim, a.metric = _p(dataset), dataset.shape[0], dataset.shape[1], metric
    a.d_graph, a.graph_degree = _p(graph), graph.shape[1]
    a.d_queries, a.nq, a.k = _p(queries), queries.shape[0], k
    a.params = params
    if flt is not None:
        a.filter = flt
    if seeds is not None:
        a.d_seeds, a.seeds_per_query = _p(seeds), seeds.shape[1]
    a.ctas_per_query = ctas_per_query
    return a


def search_workspace_bytes(args: SearchArgs) -> int:
    """grab_graph_search_workspace_bytes_for: bytes of d_ws this request needs (covers ctas_per_query > 1)."""
    return lib().grab_graph_search_workspace_bytes_for(C.byref(args))


def graph_search(dataset, graph, queries, k, params: SearchParams, metric=METRIC_L2,
                 flt: Filter | None = None, seeds=None, seed=0x1234ABCD, id_scale=1, id_offset=0,
                 stats=False, out=None, ws=None, out_keys=None, ctas_per_query=0):
    """Filtered graph search; returns (ids, dists[, SearchStats]).  out_keys: optional int64 tensor [nq, k] that
    receives the results as (ordered distance << 32 | result id) keys for the sharded exchange step; with
    out=(None, None) only the keys are written.  ctas_per_query: 0/1 = one CTA per query (the reference's walk),
    n >= 2 = n co-operating CTAs per query, CTAS_AUTO = as many as fill the GPU (small batches)."""
    import torch
    n, dim = dataset.shape
    nq = queries.shape[0]
    if out is None:
        ids = torch.empty((nq, k), dtype=torch.int64, device=dataset.device)
        dists = torch.empty((nq, k), dtype=torch.float32, device=dataset.device)
    else:
        ids, dists = out
    a = SearchArgs()
    a.d_dataset, a.n, a.dim, a.metric = _p(dataset), n, dim, metric
    a.d_graph, a.graph_degree = _p(graph), graph.shape[1]
    a.d_queries, a.nq, a.k = _p(queries), nq, k
    a.params = params
    if flt is not None:
        a.filter = flt
    if seeds is not None:
        a.d_seeds, a.seeds_per_query = _p(seeds), seeds.shape[1]
    a.seed = seed
    a.d_out_ids, a.d_out_dists = _p(ids), _p(dists)
    a.d_out_keys = _p(out_keys)
    a.id_scale, a.id_offset = id_scale, id_offset
    st = None
    if stats:
        st = torch.zeros(6, dtype=torch.int64, device=dataset.device)
        a.d_stats = _p(st)
    a.ctas_per_query = ctas_per_query
    if ws is None:
        ws_bytes = search_workspace_bytes(a)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dataset.device)
    a.d_ws, a.ws_bytes = _p(ws), ws.numel()
    a.stream = _stream()
    check(lib().grab_graph_search(C.byref(a)))
    if stats:
        v = st.cpu().tolist()
        return ids, dists, SearchStats(*v)
    return ids, dists


def knn_graph_blocks(dataset, block_offsets, k, mode=0, metric=METRIC_L2, want_dists=False,
                     precision=KNN_EXACT_SCAN):
    import numpy as np
    import torch
    n, dim = dataset.shape
    offs = np.ascontiguousarray(np.asarray(block_offsets, dtype=np.uint64))
    out = torch.empty((n, k), dtype=torch.int32, device=dataset.device)
    dists = torch.empty((n, k), dtype=torch.float32, device=dataset.device) if want_dists else None
    check(lib().grab_knn_graph_blocks(_p(dataset), C.c_uint64(n), C.c_uint32(dim), C.c_int(metric),
                                      _p(offs), C.c_uint32(len(offs) - 1), C.c_uint32(k),
                                      C.c_int(mode), C.c_int(precision), _p(out), _p(dists), _stream()))
    return (out, dists) if want_dists else out


class TpBuildOptions(C.Structure):
    _fields_ = [("knn_precision", C.c_int32), ("global_candidates", C.c_int32),
                ("search_iterations", C.c_uint32), ("search_width", C.c_uint32)]


def build_time_partitioned_graph(dataset, bucket, bucket_sizes, total_degree, local_degree,
                                 metric=METRIC_L2, knn_precision=KNN_TC_SPLIT, global_candidates=GLOBAL_AUTO,
                                 search_iterations=0, search_width=0):
    """grab_build_time_partitioned_graph_ex; global_candidates: GLOBAL_AUTO / _ALL_PAIRS / _ROUTED_SEARCH."""
    import numpy as np
    import torch
    n, dim = dataset.shape
    sizes = np.ascontiguousarray(np.asarray(bucket_sizes, dtype=np.uint64))
    graph = torch.full((n, total_degree), -1, dtype=torch.int32, device=dataset.device)
    torch.cuda.synchronize()
    opt = TpBuildOptions(knn_precision, global_candidates, search_iterations, search_width)
    check(lib().grab_build_time_partitioned_graph_ex(_p(dataset), C.c_uint64(n), C.c_uint32(dim),
                                                     C.c_int(metric), _p(graph), _p(bucket), _p(sizes),
                                                     C.c_uint32(len(sizes)), C.c_uint32(total_degree),
                                                     C.c_uint32(local_degree), C.byref(opt)))
    return graph


def merge_topk(dists, ids, k):
    import torch
    nq, parts, kk = dists.shape
    assert kk == k
    out_ids = torch.empty((nq, k), dtype=torch.int64, device=dists.device)
    out_d = torch.empty((nq, k), dtype=torch.float32, device=dists.device)
    check(lib().grab_merge_topk(_p(dists), _p(ids), C.c_uint64(nq), C.c_uint32(parts), C.c_uint32(k),
                                _p(out_ids), _p(out_d), _stream()))
    return out_ids, out_d


def merge_sorted_keys(keys, k, out=None):
    """grab_merge_sorted_keys: keys int64 tensor [parts, nq, run_length] (uint64 bits, runs ascending) -> (ids, dists)."""
    import torch
    parts, nq, kp = keys.shape
    if out is None:
        out = (torch.empty((nq, k), dtype=torch.int64, device=keys.device),
               torch.empty((nq, k), dtype=torch.float32, device=keys.device))
    check(lib().grab_merge_sorted_keys(_p(keys), C.c_uint64(nq), C.c_uint32(parts), C.c_uint32(kp), C.c_uint32(k),
                                       _p(out[0]), _p(out[1]), _stream()))
    return out


class Comm:
    """grab_comm: the communicator of the id-sharded search (NCCL inside the C library).  `broadcast_bytes(buf)`
    must hand rank 0's 128-byte buffer to every rank (torch.distributed, MPI, a file -- any side channel)."""

    def __init__(self, world: int, rank: int, broadcast_bytes):
        import numpy as np
        self.world, self.rank = world, rank
        uid = np.zeros(128, dtype=np.uint8)
        if rank == 0:
            check(lib().grab_comm_unique_id(_p(uid), C.c_size_t(128)))
        uid = np.ascontiguousarray(broadcast_bytes(uid), dtype=np.uint8)
        h = C.c_void_p()
        check(lib().grab_comm_create(_p(uid), C.c_int(world), C.c_int(rank), C.byref(h)))
        self.handle = h

    def gather_merge(self, keys, k, gather=None, out=None):
        """All-gather of this rank's keys [nq, run_length] + G-way merge, on the current stream -> (ids, dists)."""
        import torch
        nq, kp = keys.shape
        if gather is None:
            gather = torch.empty((self.world, nq, kp), dtype=torch.int64, device=keys.device)
        if out is None:
            out = (torch.empty((nq, k), dtype=torch.int64, device=keys.device),
                   torch.empty((nq, k), dtype=torch.float32, device=keys.device))
        check(lib().grab_sharded_gather_merge(self.handle, _p(keys), C.c_uint64(nq), C.c_uint32(kp), C.c_uint32(k),
                                              _p(gather), C.c_size_t(gather.numel() * 8), _p(out[0]), _p(out[1]),
                                              _stream()))
        return out

    def close(self):
        if self.handle:
            lib().grab_comm_destroy(self.handle)
            self.handle = None


def torch_broadcast_bytes(buf):
    """Side channel for Comm over an initialised torch.distributed group (any backend)."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(buf.copy())
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.broadcast(t, src=0)
    return t.cpu().numpy()


class Router:
    """Entry-point router (grab_router): centroids plus the ids grouped by nearest centroid."""

    def __init__(self, centroids, norms, offsets, members, metric, exact_scan=False):
        self.centroids, self.norms, self.offsets, self.members, self.metric = centroids, norms, offsets, members, metric
        self.struct = RouterStruct(centroids.shape[0], centroids.shape[1], metric, _p(centroids), _p(norms),
                                   _p(offsets), _p(members), ROUTER_EXACT_SCAN if exact_scan else 0)

    def exact(self, on=True):
        """Rank centroids with the exact fp32 scan (True) or on the tensor cores (False)."""
        self.struct.flags = ROUTER_EXACT_SCAN if on else 0
        return self


def router_build(dataset, num_centroids, metric=METRIC_L2, iterations=10, max_sample=0, centroids=None, norms=None):
    """grab_router_build; with `centroids`/`norms` given and iterations=0 only re-assigns."""
    import torch
    n, dim = dataset.shape
    dev = dataset.device
    if centroids is None:
        centroids = torch.empty((num_centroids, dim), dtype=torch.float32, device=dev)
        norms = torch.empty(num_centroids, dtype=torch.float32, device=dev)
    offsets = torch.empty(num_centroids + 1, dtype=torch.int32, device=dev)
    members = torch.empty(n, dtype=torch.int32, device=dev)
    check(lib().grab_router_build(_p(dataset), C.c_uint32(dim), C.c_uint64(n), C.c_int(metric),
                                  C.c_uint32(num_centroids), C.c_uint32(iterations), C.c_uint64(max_sample),
                                  _p(centroids), _p(norms), _p(offsets), _p(members), _stream()))
    return Router(centroids, norms, offsets, members, metric)


def nearest_centroids(router: Router, rows, probes=1):
    import torch
    out = torch.empty((rows.shape[0], probes), dtype=torch.int32, device=rows.device)
    check(lib().grab_nearest_centroids(C.byref(router.struct), _p(rows), C.c_uint64(rows.shape[0]),
                                       C.c_uint32(probes), _p(out), _stream()))
    return out


def route_seeds(router: Router, queries, n, flt: Filter | None = None, probes=2, seeds_per_query=64,
                seed=0x1234ABCD, out=None, ws=None):
    """grab_route_seeds: int32 tensor [nq, seeds_per_query] (-1 = no seed found) for `seeds=`."""
    import torch
    nq = queries.shape[0]
    if out is None:
        out = torch.empty((nq, seeds_per_query), dtype=torch.int32, device=queries.device)
    if ws is None:
        ws = torch.empty(lib().grab_route_seeds_workspace_bytes(nq, probes), dtype=torch.uint8, device=queries.device)
    check(lib().grab_route_seeds(C.byref(router.struct), _p(queries), C.c_uint64(nq), C.c_uint64(n),
                                 C.byref(flt) if flt is not None else None, C.c_uint32(probes),
                                 C.c_uint32(seeds_per_query), C.c_uint64(seed), _p(out), _p(ws),
                                 C.c_size_t(ws.numel()), _stream()))
    return out


def search_bytes(stats: SearchStats, nq: int, dim: int, deg: int, k: int, filter_bytes: int) -> int:
    """Algorithmic bytes of one search launch: vectors that had to be read (queries, seeds,
    distance-evaluated neighbours), graph rows of expanded parents, filter values of examined
    neighbours (filter_bytes = 8 for gathered uint64 timestamps, 1 for labels, 0 when sorted
    timestamps make the range an id window), results written."""
    return (4 * dim * (nq + stats.seeds + stats.distances) + 4 * deg * stats.parents +
            filter_bytes * stats.edges + 12 * k * nq)
