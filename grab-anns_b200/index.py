"""Python view of the three index classes (through the C handles of include/grab_index.h).
Host numpy arrays in and out, exactly like the C++ classes they forward to."""
from __future__ import annotations

import ctypes as C
import importlib

import numpy as np

_g = importlib.import_module("grab-anns_b200")


def _lib():
    lib = _g.lib()
    if not getattr(lib, "_index_api_ready", False):
        for name in ("grab_index_opt_create", "grab_index_create", "grab_tsindex_create",
                     "grab_index_opt_create_on", "grab_index_create_on", "grab_tsindex_create_on"):
            getattr(lib, name).restype = C.c_void_p
        for name in ("grab_index_opt_size", "grab_index_size", "grab_tsindex_size"):
            getattr(lib, name).restype = C.c_size_t
            getattr(lib, name).argtypes = [C.c_void_p]
        lib._index_api_ready = True
    return lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint64)


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


class _Base:
    _prefix = ""

    def _call(self, name, *args):
        _g.check(getattr(_lib(), self._prefix + name)(C.c_void_p(self.h), *args))

    def __del__(self):
        try:
            if getattr(self, "h", None):
                getattr(_lib(), self._prefix + "destroy")(C.c_void_p(self.h))
                self.h = None
        except Exception:      # interpreter shutdown: the library module may already be gone
            pass

    def _out(self, nq, k):
        return np.empty((nq, k), dtype=np.int64), np.empty((nq, k), dtype=np.float32)

    def size(self):
        return getattr(_lib(), self._prefix + "size")(C.c_void_p(self.h))

    def save(self, path):
        self._call("save", C.c_char_p(str(path).encode()))

    def load(self, path):
        self._call("load", C.c_char_p(str(path).encode()))

    def set_small_batch_mode(self, ctas_per_query=0xFFFFFFFF, exact_below=1024):
        """ctas_per_query: CTAs co-operating on one query (0xFFFFFFFF = as many as fill the GPU, 1 = the reference's
        one per query); single-range queries over at most exact_below vectors are answered by an exact scan."""
        self._call("set_small_batch_mode", C.c_uint32(ctas_per_query), C.c_size_t(exact_below))

    def set_query_params(self, itopk=256, width=6, min_iter=1, max_iter=50, hash_bitlen=13):
        self._call("set_query_params", C.c_uint32(itopk), C.c_uint32(width), C.c_uint32(min_iter),
                   C.c_uint32(max_iter), C.c_uint32(hash_bitlen))


class CagraIndexOpt(_Base):
    """cagra::CagraIndexOpt (reference: src/cagraIndexOpt.cuh:13-155)."""
    _prefix = "grab_index_opt_"

    def __init__(self, dim, graph_degree=32, local_degree=16, vmm_max_bytes=4 << 30, bucket_width=1, metric=0,
                 knn_precision=2, seed=0x9E3779B97F4A7C15, insert_batch=4096, device=-1):
        """device: the GPU the index lives on (-1 = the calling thread's current device); every later call runs
        there whatever the current device is."""
        self.dim, self.graph_degree = dim, graph_degree
        self.h = _lib().grab_index_opt_create_on(C.c_int(device), C.c_uint32(dim), C.c_uint32(graph_degree),
                                                 C.c_uint32(local_degree), C.c_size_t(vmm_max_bytes))
        if not self.h:
            raise _g.GrabError(1, _lib().grab_last_error().decode())
        self._call("configure", C.c_uint64(bucket_width), C.c_int(metric), C.c_int(knn_precision), C.c_uint64(seed),
                   C.c_size_t(insert_batch))

    def add(self, vectors, timestamps):
        v, t = _f32(vectors), _u64(timestamps)
        self._call("add", C.c_size_t(v.shape[0]), _ptr(v), _ptr(t))

    def build(self):
        self._call("build")

    def insert(self, vectors, timestamps):
        v, t = _f32(vectors), _u64(timestamps)
        self._call("insert", C.c_size_t(v.shape[0]), _ptr(v), _ptr(t))

    def query(self, queries, k):
        q = _f32(queries)
        ids, d = self._out(q.shape[0], k)
        self._call("query", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), _ptr(ids), _ptr(d))
        return ids, d

    def set_router(self, centroids=0xFFFFFFFF, probes=2, seeds_per_query=64):
        """Entry-point router for searches without caller seeds: 0 = off, 0xFFFFFFFF = about sqrt(n)."""
        self._call("set_router", C.c_uint32(centroids), C.c_uint32(probes), C.c_uint32(seeds_per_query))

    def set_insert_mode(self, routed=True, repair_mode=1):
        """Routed insert searches; repair_mode 0 = the reference's pseudo-random slot, 1 = every request takes the
        farthest weak-half slot, 2 = only closer requests replace the farthest neighbour.  (False, 0) = the
        reference's rules."""
        self._call("set_insert_mode", C.c_int(int(routed)), C.c_int(int(repair_mode)))

    def set_insert_search_params(self, itopk=128, width=4, max_iter=16, hash_bitlen=12):
        self._call("set_insert_search_params", C.c_uint32(itopk), C.c_uint32(width), C.c_uint32(max_iter),
                   C.c_uint32(hash_bitlen))

    def query_local(self, queries, k, target_timestamp):
        q = _f32(queries)
        ids, d = self._out(q.shape[0], k)
        self._call("query_local", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), C.c_uint64(target_timestamp),
                   _ptr(ids), _ptr(d))
        return ids, d

    def query_range(self, queries, k, start, end):
        q = _f32(queries)
        ids, d = self._out(q.shape[0], k)
        self._call("query_range", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), C.c_uint64(start), C.c_uint64(end),
                   _ptr(ids), _ptr(d))
        return ids, d

    def query_range_batch(self, queries, k, start, end, out=None):
        """out: optional (ids int64 [nq, k], dists float32 [nq, k]) arrays of the caller's, as the C call takes them;
        fresh arrays are allocated otherwise."""
        q, s, e = _f32(queries), _u64(start), _u64(end)
        ids, d = out if out is not None else self._out(q.shape[0], k)
        self._call("query_range_batch", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), _ptr(s), _ptr(e), _ptr(ids),
                   _ptr(d))
        return ids, d

    def get_graph(self):
        out = np.empty((self.size(), self.graph_degree), dtype=np.uint32)
        self._call("get_graph", _ptr(out), C.c_size_t(out.size))
        return out


class CagraIndex(_Base):
    """cagra::CagraIndex (reference: src/cagraIndex.hpp:12-119)."""
    _prefix = "grab_index_"

    def __init__(self, dim, graph_degree=64, vmm_max_bytes=4 << 30, metric=0, knn_precision=2,
                 seed=0x9E3779B97F4A7C15, insert_batch=64, device=-1):
        self.dim, self.graph_degree = dim, graph_degree
        self.h = _lib().grab_index_create_on(C.c_int(device), C.c_uint32(dim), C.c_uint32(graph_degree),
                                             C.c_size_t(vmm_max_bytes))
        if not self.h:
            raise _g.GrabError(1, _lib().grab_last_error().decode())
        self._call("configure", C.c_int(metric), C.c_int(knn_precision), C.c_uint64(seed), C.c_size_t(insert_batch))

    def add(self, vectors, timestamps=None):
        v, t = _f32(vectors), _u64(timestamps)
        self._call("add", C.c_size_t(v.shape[0]), _ptr(v), _ptr(t))

    def build(self):
        self._call("build")

    def insert(self, vectors, timestamps=None):
        v, t = _f32(vectors), _u64(timestamps)
        self._call("insert", C.c_size_t(v.shape[0]), _ptr(v), _ptr(t))

    def query(self, queries, k):
        q = _f32(queries)
        ids, d = self._out(q.shape[0], k)
        self._call("query", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), _ptr(ids), _ptr(d))
        return ids, d

    def query_range(self, queries, k, range_radius, start, end):
        q = _f32(queries)
        ids, d = self._out(q.shape[0], k)
        self._call("query_range", _ptr(q), C.c_size_t(q.shape[0]), C.c_int(k), C.c_float(range_radius),
                   C.c_uint64(start), C.c_uint64(end), _ptr(ids), _ptr(d))
        return ids, d

    def get_graph(self):
        out = np.empty((self.size(), self.graph_degree), dtype=np.uint32)
        self._call("get_graph", _ptr(out), C.c_size_t(out.size))
        return out


class TimeStampIndex(_Base):
    """timestamp::TimeStampIndex (reference: src/timeStampIndex.cuh:39-95)."""
    _prefix = "grab_tsindex_"

    def __init__(self, dim, degree=32, cluster_ratio=1000, device=-1):
        self.dim = dim
        self.h = _lib().grab_tsindex_create_on(C.c_int(device), C.c_uint32(dim), C.c_uint32(degree),
                                               C.c_size_t(cluster_ratio))

    def insert(self, vectors, timestamps):
        v, t = _f32(vectors), _u64(timestamps)
        first = C.c_uint64(0)
        self._call("insert", _ptr(v), _ptr(t), C.c_size_t(v.shape[0]), C.byref(first))
        return first.value

    def build_virtual_index(self):
        self._call("build_virtual_index")

    def query(self, query, topk, probe_buckets=5):
        q = _f32(query).reshape(-1)
        ids, d = np.empty(topk, dtype=np.int64), np.empty(topk, dtype=np.float32)
        self._call("query", _ptr(q), C.c_size_t(topk), _ptr(ids), _ptr(d), C.c_int(probe_buckets))
        return ids, d

    def query_by_timestamp(self, query, topk, timestamp):
        q = _f32(query).reshape(-1)
        ids, d = np.empty(topk, dtype=np.int64), np.empty(topk, dtype=np.float32)
        self._call("query_by_timestamp", _ptr(q), C.c_size_t(topk), C.c_uint64(timestamp), _ptr(ids), _ptr(d))
        return ids, d
