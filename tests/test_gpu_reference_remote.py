"""Live three-way check of cross-bucket edge selection and reverse injection -- the reference's OWN kernels
(src/index/cagra_opt.cu in oracle/_ref/libgrab_ref.so), the CPU restatement and the new CUDA code on the same inputs
-- and of the reference's own search LAUNCHERS against this library's search on the same graph and seeds."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_remote_golden as gen  # noqa: E402
from conftest import clustered  # noqa: E402

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def ref():
    import ref_kernels
    if not ref_kernels.available() or not hasattr(ref_kernels.lib(), "ref_update_remote_edges"):
        pytest.skip("oracle/_ref/libgrab_ref.so lacks the cagra_opt harness (make -C oracle ref REF=...)")
    return ref_kernels


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("ci", range(len(gen.CASES)))
def test_three_way_remote_edges_and_injection(grab, oracle, ref, ci):
    import torch
    case = gen.CASES[ci]
    n, total, local, gk = case[0], case[1], case[2], case[3]
    g, bucket, cand = gen.inputs(case)
    L, C = grab.lib(), grab.C
    # selection: reference == restatement == CUDA
    r_g, r_c = _t(g.view(np.int32)), _t(cand.view(np.int32))
    d_ts = _t(bucket.view(np.int64))
    ref.update_remote_edges(r_g, d_ts, r_c, local)
    o_g, o_c = oracle.remote_edges(g, bucket, cand, local)
    assert np.array_equal(_u32(r_g), o_g) and np.array_equal(_u32(r_c), o_c)
    m_g, m_c = _t(g.view(np.int32)), _t(cand.view(np.int32))
    grab.check(L.grab_remote_edges_device(grab._p(m_g), grab._p(d_ts), grab._p(m_c), C.c_uint64(n), total, local, gk,
                                          None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(m_g), o_g)
    # injection on the canonical lists: reference kernel == restatement == CUDA (which builds the same lists itself)
    crev, ccnt = gen.canonical_global_rev(o_g, local)
    r_inj = _t(o_g.view(np.int32).copy())
    ref.inject_global_rev(r_inj, _t(crev.view(np.int32)), _t(ccnt.view(np.int32)), local)
    o_inj = oracle.inject_reverse_remote(o_g, local, gen.MAX_REV)
    assert np.array_equal(_u32(r_inj), o_inj)
    grab.check(L.grab_inject_reverse_remote_device(grab._p(m_g), C.c_uint64(n), total, local, gen.MAX_REV, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(m_g), o_inj)
    # the reference's racy lists: same counts as the canonical ones
    rev, cnt = ref.make_global_rev(_t(o_g.view(np.int32)), local, gen.MAX_REV)
    assert np.array_equal(_u32(cnt), ccnt)


def test_reference_launchers_against_this_search(grab, oracle, ref):
    """search_opt / search_bucket_opt / search_bucket_range AS THE REFERENCE LAUNCHES THEM (cagra_opt.cu:1108-1442,
    their own queue sizes, seed counts and shared-memory arithmetic) on a graph built here, the same seeds handed to
    both sides: recall of this library's search within 0.5 points of the reference's, and no result outside the
    filter on either side."""
    n, dim, total, local, nq, k = 20000, 128, 32, 24, 256, 10   # 128: a dimension the reference's refine kernel has
    rng = np.random.default_rng(91)
    data = clustered(n, dim, 40, 1.0, 92)
    nb = 8
    bucket = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    d_data = _t(data)
    graph = grab.build_time_partitioned_graph(d_data, _t(bucket.view(np.int64)), [n // nb] * nb, total, local,
                                              knn_precision=grab.KNN_EXACT_SCAN)
    q = data[rng.integers(0, n, nq)] + 0.1 * rng.standard_normal((nq, dim)).astype(np.float32)
    d_q, d_ts = _t(q), _t(bucket.view(np.int64))
    # mode 2: buckets [2, 5)
    lo, hi = 2, 5
    ts_full = bucket
    gt, _ = oracle.exact_search(data, q, k, ts=ts_full, lo=np.full(nq, lo, np.uint64), hi=np.full(nq, hi, np.uint64))
    seeds = rng.integers(lo * (n // nb), hi * (n // nb), size=(nq, 32)).astype(np.uint32)
    r_ids, _ = ref.search_launcher(2, d_data, graph, d_q, k, 64, 4, 40, 13, local_deg=local, ts=d_ts, lo=lo, hi=hi,
                                   seeds=_t(seeds.view(np.int32)))
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=lo, hi=hi)
    m_ids, _ = grab.graph_search(d_data, graph, d_q, k, grab.SearchParams(64, 4, 0, 40, 13), flt=f,
                                 seeds=_t(seeds.view(np.int32)))
    r_ids, m_ids = r_ids.cpu().numpy(), m_ids.cpu().numpy()
    for ids in (r_ids, m_ids):
        v = ids[ids >= 0]
        assert np.all((bucket[v] >= lo) & (bucket[v] < hi))
    r_rec, m_rec = oracle.recall(r_ids, gt), oracle.recall(m_ids, gt)
    assert m_rec >= r_rec - 0.005 and r_rec > 0.85, (r_rec, m_rec)
    # mode 0: unfiltered
    gt0, _ = oracle.exact_search(data, q, k)
    seeds0 = rng.integers(0, n, size=(nq, 32)).astype(np.uint32)
    r0, _ = ref.search_launcher(0, d_data, graph, d_q, k, 64, 4, 40, 13, seeds=_t(seeds0.view(np.int32)))
    m0, _ = grab.graph_search(d_data, graph, d_q, k, grab.SearchParams(64, 4, 0, 40, 13), seeds=_t(seeds0.view(np.int32)))
    r0_rec, m0_rec = oracle.recall(r0.cpu().numpy(), gt0), oracle.recall(m0.cpu().numpy(), gt0)
    assert m0_rec >= r0_rec - 0.005 and r0_rec > 0.85, (r0_rec, m0_rec)
    # mode 1: one bucket through the local columns
    b = 3
    gtb, _ = oracle.exact_search(data[b * (n // nb):(b + 1) * (n // nb)], q, k)
    gtb = gtb + b * (n // nb)
    seedsb = rng.integers(b * (n // nb), (b + 1) * (n // nb), size=(nq, 32)).astype(np.uint32)
    r1, _ = ref.search_launcher(1, d_data, graph, d_q, k, 128, 4, 40, 13, local_deg=local, seeds=_t(seedsb.view(np.int32)))
    fb = grab.make_filter(grab.FILTER_PREFIX, active_degree=local)
    m1, _ = grab.graph_search(d_data, graph, d_q, k, grab.SearchParams(128, 4, 0, 40, 13), flt=fb,
                              seeds=_t(seedsb.view(np.int32)))
    r1, m1 = r1.cpu().numpy(), m1.cpu().numpy()
    assert np.all(bucket[m1[m1 >= 0]] == b) and np.all(bucket[r1[r1 >= 0]] == b)
    r1_rec, m1_rec = oracle.recall(r1, gtb), oracle.recall(m1, gtb)
    assert m1_rec >= r1_rec - 0.005 and r1_rec > 0.85, (r1_rec, m1_rec)
