"""Failure paths that never reach the GPU: every entry point validates its arguments on the host
and answers with a status and a message instead of exiting (the reference calls exit(1) on CUDA
errors, src/index/cagra.cuh:9-17, and prints from the device for unsupported shapes)."""
import ctypes as C
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def lib():
    grab = importlib.import_module("grab-anns_b200")
    grab.build()
    return grab.lib()


def _err(lib):
    return lib.grab_last_error().decode()


def test_null_and_shape_errors_return_status(lib):
    null = None
    one = C.c_void_p(16)          # a non-null dummy: validation fails before it is dereferenced
    assert lib.grab_exact_search(null, C.c_uint64(10), 8, 0, null, null, C.c_uint64(1), 1, null, null, null,
                                 C.c_size_t(0), null) == 1
    assert "null pointer" in _err(lib)
    assert lib.grab_exact_search(one, C.c_uint64(10), 6, 0, null, one, C.c_uint64(1), 1, one, one, null,
                                 C.c_size_t(0), null) == 1
    assert "multiple of 4" in _err(lib)
    assert lib.grab_exact_search(one, C.c_uint64(10), 8, 0, null, one, C.c_uint64(1), 5000, one, one, null,
                                 C.c_size_t(0), null) == 1
    assert lib.grab_exact_search(one, C.c_uint64(10), 8, 7, null, one, C.c_uint64(1), 5, one, one, null,
                                 C.c_size_t(0), null) == 1
    assert "metric" in _err(lib)
    assert lib.grab_graph_search(null) == 1
    assert lib.grab_optimize_prune_device(null, null, C.c_uint64(4), 8, 4, null, null) == 1
    assert lib.grab_optimize_prune_device(one, one, C.c_uint64(4), 600, 4, null, null) == 1     # > 512, as the reference
    assert "512" in _err(lib)
    assert lib.grab_optimize_prune_device(one, one, C.c_uint64(4), 8, 9, null, null) == 1       # out > in
    assert lib.grab_merge_topk(one, one, C.c_uint64(4), 100, 100, one, one, null) == 1          # parts*k > 8192
    assert lib.grab_update_topology_opt(one, one, one, one, C.c_uint64(4), C.c_uint64(1), C.c_uint64(0), 8, 8, 4, 4,
                                        null) == 1
    offs = np.array([0, 5], dtype=np.uint64)
    assert lib.grab_knn_graph_blocks(one, C.c_uint64(10), 8, 0, C.c_void_p(offs.ctypes.data), 1, 4, 0, 0, one, null,
                                     null) == 1
    assert "span" in _err(lib)
    assert lib.grab_knn_graph_blocks(one, C.c_uint64(5), 8, 0, C.c_void_p(offs.ctypes.data), 1, 300, 0, 1, one, null,
                                     null) == 1                                                 # k too wide for the tensor-core path
    assert lib.grab_build_time_partitioned_graph(one, C.c_uint64(10), 8, 0, one, one, C.c_void_p(offs.ctypes.data), 2,
                                                 2, 2, 0) == 1
    assert lib.grab_exact_search_noalloc(one, C.c_uint64(10), 8, 0, null, one, C.c_uint64(10**7), 10, one, one,
                                         null) == 4                                             # scratch too small
    assert lib.grab_status_string(4) == b"workspace too small"


def test_search_argument_checks(lib):
    grab = importlib.import_module("grab-anns_b200")
    a = grab.SearchArgs()
    a.d_dataset = a.d_graph = a.d_queries = a.d_out_ids = a.d_out_dists = 16
    a.n, a.dim, a.graph_degree, a.nq, a.k = 100, 8, 4, 1, 2
    a.params = grab.SearchParams(64, 4, 0, 10, 30)
    assert lib.grab_graph_search(C.byref(a)) == 1 and "hash_bitlen" in _err(lib)
    a.params = grab.SearchParams(64, 0, 0, 10, 12)
    assert lib.grab_graph_search(C.byref(a)) == 1 and "search_width" in _err(lib)
    a.params = grab.SearchParams(64, 4, 0, 10, 12)
    a.filter.kind = grab.FILTER_TS_RANGE
    assert lib.grab_graph_search(C.byref(a)) == 1 and "d_ts" in _err(lib)
    a.filter.kind = grab.FILTER_PREFIX
    a.filter.active_degree = 9
    assert lib.grab_graph_search(C.byref(a)) == 1 and "active_degree" in _err(lib)
    a.filter.kind = 42
    assert lib.grab_graph_search(C.byref(a)) == 1
    a.filter.kind = grab.FILTER_NONE
    a.n = 1 << 31
    assert lib.grab_graph_search(C.byref(a)) == 1 and "2^31" in _err(lib)


def test_router_argument_checks(lib):
    grab = importlib.import_module("grab-anns_b200")
    null = None
    one = C.c_void_p(16)
    build = lib.grab_router_build
    assert build(null, 8, C.c_uint64(100), 0, 4, 2, C.c_uint64(0), one, one, one, one, null) == 1
    assert "null pointer" in _err(lib)
    assert build(one, 6, C.c_uint64(100), 0, 4, 2, C.c_uint64(0), one, one, one, one, null) == 1
    assert "multiple of 4" in _err(lib)
    assert build(one, 8, C.c_uint64(100), 0, 0, 2, C.c_uint64(0), one, one, one, one, null) == 1      # no centroids
    assert build(one, 8, C.c_uint64(100), 0, 101, 2, C.c_uint64(0), one, one, one, one, null) == 1    # more than vectors
    assert "num_centroids" in _err(lib)
    assert build(one, 8, C.c_uint64(100), 5, 4, 2, C.c_uint64(0), one, one, one, one, null) == 1
    assert "metric" in _err(lib)
    assert build(one, 8, C.c_uint64(1 << 31), 0, 4, 2, C.c_uint64(0), one, one, one, one, null) == 1

    r = grab.RouterStruct(16, 8, 0, 16, 16, 16, 16, 0)
    route = lib.grab_route_seeds
    args = lambda probes, seeds: (C.byref(r), one, C.c_uint64(4), C.c_uint64(100), null, probes, seeds,
                                  C.c_uint64(1), one, null, C.c_size_t(0), null)
    assert route(*args(0, 32)) == 1 and "probes" in _err(lib)
    assert route(*args(17, 32)) == 1
    assert route(*args(4, 0)) == 1 and "seeds_per_query" in _err(lib)
    assert route(*args(4, 5000)) == 1
    assert route(null, one, C.c_uint64(4), C.c_uint64(100), null, 4, 32, C.c_uint64(1), one, null, C.c_size_t(0),
                 null) == 1
    assert "router" in _err(lib)
    empty = grab.RouterStruct(16, 8, 0, 16, 16, None, 16, 0)          # no member offsets
    assert route(C.byref(empty), one, C.c_uint64(4), C.c_uint64(100), null, 4, 32, C.c_uint64(1), one, null,
                 C.c_size_t(0), null) == 1
    f = grab.Filter()
    f.kind = grab.FILTER_TS_RANGE                                      # range filter without timestamps
    assert route(C.byref(r), one, C.c_uint64(4), C.c_uint64(100), C.byref(f), 4, 32, C.c_uint64(1), one, null,
                 C.c_size_t(0), null) == 1
    assert "d_ts" in _err(lib)
    f.kind = 9
    assert route(C.byref(r), one, C.c_uint64(4), C.c_uint64(100), C.byref(f), 4, 32, C.c_uint64(1), one, null,
                 C.c_size_t(0), null) == 1
    # an empty batch is a success and touches nothing
    assert route(C.byref(r), one, C.c_uint64(0), C.c_uint64(100), null, 4, 32, C.c_uint64(1), one, null,
                 C.c_size_t(0), null) == 0
    assert lib.grab_nearest_centroids(C.byref(r), one, C.c_uint64(4), 0, one, null) == 1
    assert lib.grab_route_seeds_workspace_bytes(1000, 4) >= 256 + 8 * 1000 * 8 * 8

    # build options: unknown cross-bucket candidate mode
    offs = np.array([5, 5], dtype=np.uint64)
    opt = grab.TpBuildOptions(1, 7, 0, 0)
    assert lib.grab_build_time_partitioned_graph_ex(one, C.c_uint64(10), 8, 0, one, one, C.c_void_p(offs.ctypes.data),
                                                    2, 4, 2, C.byref(opt)) == 1
    assert "global_candidates" in _err(lib)


def test_sharded_and_selftest_entry_points_validate_on_the_host(lib):
    """The exchange step, the communicator and the device-level test entry points reject bad arguments with a
    status before any GPU work; a communicator is never created from a null id."""
    null = None
    one = C.c_void_p(16)
    assert lib.grab_merge_sorted_keys(null, C.c_uint64(4), 2, 10, 10, one, one, null) == 1
    assert "null pointer" in _err(lib)
    assert lib.grab_merge_sorted_keys(one, C.c_uint64(4), 0, 10, 10, one, one, null) == 1      # no runs
    assert lib.grab_merge_sorted_keys(one, C.c_uint64(4), 2, 5000, 10, one, one, null) == 1     # run too long
    assert lib.grab_merge_sorted_keys(one, C.c_uint64(0), 2, 10, 10, one, one, null) == 0       # nothing to do
    assert lib.grab_sharded_gather_merge(null, null, C.c_uint64(4), 10, 10, null, C.c_size_t(0), one, one, null) == 1
    buf = (C.c_uint8 * 64)()
    assert lib.grab_comm_unique_id(buf, C.c_size_t(64)) == 1                                    # needs 128 bytes
    assert "128" in _err(lib)
    h = C.c_void_p()
    assert lib.grab_comm_create(null, 2, 0, C.byref(h)) == 1
    uid = (C.c_uint8 * 128)()
    assert lib.grab_comm_create(uid, 2, 5, C.byref(h)) == 1                                     # rank outside the world
    assert lib.grab_comm_destroy(null) == 0
    assert lib.grab_comm_world(null) == 1 and lib.grab_comm_rank(null) == 0
    assert lib.grab_route_status(null, null) == 1
    assert lib.grab_selftest_sort_merge(one, one, C.c_uint64(1), 48, 4, 4, 0, one, null) == 1   # m not a power of two
    assert lib.grab_selftest_sort_merge(one, one, C.c_uint64(1), 64, 40, 40, 2, one, null) == 1  # rank merge: <= 32
    assert lib.grab_selftest_hash_insert(one, 2, one, 4, 64, one, null) == 1
    assert lib.grab_selftest_hash_insert(one, 8, one, 4, 48, one, null) == 1                    # threads % 32


def test_search_workspace_plan_is_host_arithmetic(lib):
    """grab_graph_search_workspace_bytes_for() plans a request without touching the GPU: one CTA per query needs the
    id windows only (plus a global table above 2^13), several CTAs per query add the shared table and the per-CTA
    result runs, and AUTO falls back to one CTA for batches that fill the GPU or walks too short to split."""
    grab = importlib.import_module("grab-anns_b200")
    lib.grab_graph_search_workspace_bytes_for.restype = C.c_size_t
    lib.grab_graph_search_workspace_bytes.restype = C.c_size_t

    def need(nq, k, itopk, width, iters, bitlen, ctas):
        a = grab.SearchArgs()
        a.n, a.dim, a.graph_degree, a.nq, a.k = 100000, 128, 32, nq, k
        a.params = grab.SearchParams(itopk, width, 0, iters, bitlen)
        a.ctas_per_query = ctas
        return lib.grab_graph_search_workspace_bytes_for(C.byref(a))

    single = lib.grab_graph_search_workspace_bytes(C.c_uint64(64), C.c_uint32(13))
    assert need(64, 10, 256, 6, 50, 13, 0) == single == need(64, 10, 256, 6, 50, 13, 1)
    multi = need(64, 10, 256, 6, 50, 13, 8)
    # 8 runs of k keys per query + a shared table of at least 2 x (seeds + 8 CTAs x iterations x width x degree) slots
    assert multi >= single + 8 * 64 * 10 * 8 + 4 * 64 * 2 * (8 * 38 * 1 * 32)
    assert need(64, 10, 256, 6, 50, 13, grab.CTAS_AUTO) > single          # small batch, long walk: split
    assert need(10000, 10, 256, 6, 50, 13, grab.CTAS_AUTO) == lib.grab_graph_search_workspace_bytes(
        C.c_uint64(10000), C.c_uint32(13))                                  # the batch fills the GPU: one CTA each
    assert need(64, 10, 64, 3, 5, 11, grab.CTAS_AUTO) == lib.grab_graph_search_workspace_bytes(
        C.c_uint64(64), C.c_uint32(11))                                     # 15 expansions: nothing to split
    assert need(64, 200, 256, 6, 50, 13, grab.CTAS_AUTO) == single          # k above the per-CTA list: one CTA each
    assert lib.grab_graph_search_workspace_bytes_for(None) == 0
