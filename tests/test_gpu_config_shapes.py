"""Parity at the shape of a benchmark configuration (not a scaled-down stand-in): C1 in full -- 100 000 x 128
Gaussian mixture, 1 000 queries with their own 10 % timestamp ranges, L2, k 10, degree 32, itopk 64.
(a) the GPU exact filtered kernel returns the CPU oracle's ids and fp32 bits for every query, within 1e-4 of
float64; how tie-sensitive that comparison is gets reported (k-th / (k+1)-th gap below 1e-6 relative, ids that
differ between the canonical summation order and the reference's sequential one, tests/test_cagra_auto.cu:48-50);
(b) the filtered graph search on the configuration's graph reaches recall@10 >= 0.95 and stays within 0.5 points
of the REFERENCE's own range kernel on the same graph, seeds, itopk and width."""
import importlib
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def c1(datasets):
    return datasets.config("C1", 1.0)


def test_c1_exact_ids_match_the_cpu_oracle(grab, oracle, c1):
    bench = importlib.import_module("bench")
    w = dict(c1)
    w["n"] = w["base"].shape[0]
    assert w["base"].shape == (100_000, 128) and w["queries"].shape[0] == 1000
    d_base, d_q = _t(w["base"]), _t(w["queries"])
    flt = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(w["ts"].view(np.int64)), lo=_t(w["lo"].view(np.int64)),
                           hi=_t(w["hi"].view(np.int64)), ts_sorted=True)
    gi, gd = grab.exact_search(d_base, d_q, w["k"], flt=flt)
    rep = bench.parity_at_config_shape(w, gi.cpu().numpy(), gd.cpu().numpy(), sample=1000)
    assert rep["queries"] == 1000 and rep["base_vectors"] == 100_000
    assert rep["exact_ids_match"] and rep["exact_dist_bits_match"], rep      # bit-exact: ids and fp32 distances
    assert rep["max_rel_dist_err_vs_fp64"] <= 1e-4, rep                      # the tolerance the target states
    # reported, not asserted to be zero: how many queries sit on a near-tie, and what the other summation order does
    assert rep["tie_sensitive_queries"] >= 0 and rep["ids_differing_canonical_vs_sequential_order"] <= 20, rep
    print("C1 parity report:", rep)


def test_c1_graph_search_recall_and_reference_kernel(grab, oracle, c1):
    import torch
    w = c1
    n, dim, k, deg = 100_000, 128, w["k"], w["degree"]
    d_base, d_q = _t(w["base"]), _t(w["queries"])
    d_ts = _t(w["ts"].view(np.int64))
    buckets = 20
    bsize = n // buckets
    d_bucket = d_ts // bsize
    sizes = torch.bincount(d_bucket).cpu().tolist()
    graph = grab.build_time_partitioned_graph(d_base, d_bucket.contiguous(), sizes, deg, deg * 3 // 4, knn_precision=2)
    d_lo, d_hi = _t(w["lo"].view(np.int64)), _t(w["hi"].view(np.int64))
    flt = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=d_lo, hi=d_hi, ts_sorted=True)
    gt, _ = grab.exact_search(d_base, d_q, k, flt=flt)
    gt = gt.cpu().numpy()
    # the configuration as stated: itopk 64, per-query ranges, routed seeds
    router = grab.router_build(d_base, 256)
    seeds = grab.route_seeds(router, d_q, n, flt, probes=2, seeds_per_query=64)
    ids, _ = grab.graph_search(d_base, graph, d_q, k, grab.SearchParams(64, 3, 0, 6, 11), flt=flt, seeds=seeds)
    res = ids.cpu().numpy()
    assert (((res >= w["lo"][:, None].astype(np.int64)) & (res < w["hi"][:, None].astype(np.int64))) | (res < 0)).all()
    rec = oracle.recall(res, gt)
    assert rec >= 0.95, rec
    # against the reference's own range kernel: one range for all queries (the only form it has), same seeds
    import ref_kernels
    if not ref_kernels.available():
        pytest.skip("oracle/_ref/libgrab_ref.so not built")
    lo, hi = 40_000, 50_000
    rng = np.random.default_rng(5)
    sd = _t(rng.integers(lo, hi, size=(1000, 32)).astype(np.uint32).view(np.int32))
    f1 = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=lo, hi=hi, ts_sorted=True)
    gt1 = grab.exact_search(d_base, d_q, k, flt=f1)[0].cpu().numpy()
    ri, _, _ = ref_kernels.search(2, d_base, graph, d_q, k, 64, 4, 24, 12, ts=d_ts, lo=lo, hi=hi, seeds=sd)
    gi, _ = grab.graph_search(d_base, graph, d_q, k, grab.SearchParams(64, 4, 0, 24, 12), flt=f1, seeds=sd)
    r_ref, r_new = oracle.recall(ri.cpu().numpy(), gt1), oracle.recall(gi.cpu().numpy(), gt1)
    assert r_new >= r_ref - 0.005, (r_new, r_ref)
