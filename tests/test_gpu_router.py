"""Entry-point router: CUDA path (through the C ABI) against the CPU oracle.  Needs a B200."""
import numpy as np
import pytest

from conftest import clustered

pytestmark = pytest.mark.gpu


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("dim,metric,nc", [(64, 0, 48), (100, 0, 33), (768, 1, 40)])
def test_router_build_bit_exact(grab, oracle, dim, metric, nc):
    n = 9000 if dim < 768 else 5000
    data = clustered(n, dim, 16, 0.6, dim + 1)
    if metric == 1:
        data /= np.linalg.norm(data, axis=1, keepdims=True)
    r = grab.router_build(_t(data), nc, metric=metric, iterations=4, max_sample=3000)
    cen, cnorm, offs, mem = oracle.router_build(data, nc, metric, iterations=4, max_sample=3000)
    assert np.array_equal(r.centroids.cpu().numpy().view(np.uint32), cen.view(np.uint32))   # same fp32 bits
    assert np.array_equal(r.norms.cpu().numpy().view(np.uint32), cnorm.view(np.uint32))
    assert np.array_equal(_u32(r.offsets), offs)
    assert np.array_equal(_u32(r.members), mem)
    # ragged row count, several probes
    q = data[:1001] + np.float32(0.01)
    got = _u32(grab.nearest_centroids(r, _t(q), probes=5))
    assert np.array_equal(got, oracle.nearest_centroids(q, cen, cnorm, metric, 5))
    # re-assignment only (the path used after inserts) gives the same lists
    r2 = grab.router_build(_t(data), nc, metric=metric, iterations=0, centroids=r.centroids, norms=r.norms)
    assert np.array_equal(_u32(r2.members), mem) and np.array_equal(_u32(r2.offsets), offs)


def test_router_more_probes_than_centroids_and_tiny_inputs(grab, oracle):
    data = clustered(70, 16, 3, 0.5, 5)
    r = grab.router_build(_t(data), 3, iterations=2)
    cen, cnorm, offs, mem = oracle.router_build(data, 3, 0, iterations=2)
    assert np.array_equal(_u32(r.members), mem)
    got = _u32(grab.nearest_centroids(r, _t(data[:5]), probes=6))
    assert (got[:, 3:] == 0xFFFFFFFF).all()
    assert np.array_equal(got, oracle.nearest_centroids(data[:5], cen, cnorm, 0, 6))
    seeds = _u32(grab.route_seeds(r, _t(data[:5]), 70, probes=6, seeds_per_query=16))
    probes = oracle.nearest_centroids(data[:5], cen, cnorm, 0, 3)
    assert np.array_equal(seeds, oracle.route_seeds(probes, 70, offs, mem, 16))
    with pytest.raises(grab.GrabError):
        grab.route_seeds(r, _t(data[:5]), 70, probes=17)
    with pytest.raises(grab.GrabError):
        grab.router_build(_t(data), 71)


def test_route_seeds_bit_exact_all_filters(grab, oracle):
    rng = np.random.default_rng(8)
    n, dim, nc, nq, S, P = 12000, 64, 64, 333, 32, 4
    data = clustered(n, dim, 20, 0.6, 9)
    q = data[rng.integers(0, n, nq)] + np.float32(0.02)
    r = grab.router_build(_t(data), nc, iterations=3)
    cen, cnorm, offs, mem = (r.centroids.cpu().numpy(), r.norms.cpu().numpy(), _u32(r.offsets), _u32(r.members))
    probes = oracle.nearest_centroids(q, cen, cnorm, 0, P)
    d_q = _t(q)
    # no filter
    assert np.array_equal(_u32(grab.route_seeds(r, d_q, n, probes=P, seeds_per_query=S)),
                          oracle.route_seeds(probes, n, offs, mem, S))
    # timestamp ranges: sorted (id windows), unsorted (predicate tests), per query and call-wide, empty
    ts = np.arange(n, dtype=np.uint64) * 3
    lo = rng.integers(0, 3 * n - 6000, nq).astype(np.uint64)
    hi = lo + 6000
    hi[5] = lo[5]
    d_ts, d_lo, d_hi = _t(ts.view(np.int64)), _t(lo.view(np.int64)), _t(hi.view(np.int64))
    for srt in (True, False):
        f = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=d_lo, hi=d_hi, ts_sorted=srt)
        got = _u32(grab.route_seeds(r, d_q, n, f, probes=P, seeds_per_query=S, seed=77))
        assert np.array_equal(got, oracle.route_seeds(probes, n, offs, mem, S, seed=77, ts=ts, lo=lo, hi=hi,
                                                      ts_sorted=srt))
        assert (got[5] == 0xFFFFFFFF).all()
        v = got != 0xFFFFFFFF
        tv = ts[np.where(v, got, 0)]
        assert ((tv >= lo[:, None]) & (tv < hi[:, None]))[v].all()
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=3000, hi=9000, ts_sorted=True)
    assert np.array_equal(_u32(grab.route_seeds(r, d_q, n, f, probes=P, seeds_per_query=S)),
                          oracle.route_seeds(probes, n, offs, mem, S, ts=ts, lo=3000, hi=9000))
    # labels: grouped by label (id ranges) and scattered (predicate tests)
    labels = np.sort(rng.integers(0, 6, n)).astype(np.uint8)
    loff = np.searchsorted(labels, np.arange(33), side="left").astype(np.uint32)
    masks = rng.integers(0, 64, nq).astype(np.uint32)
    d_lab, d_m, d_off = _t(labels), _t(masks.view(np.int32)), _t(loff.view(np.int32))
    f = grab.make_filter(grab.FILTER_LABELS, labels=d_lab, masks=d_m, label_offsets=d_off)
    got = _u32(grab.route_seeds(r, d_q, n, f, probes=P, seeds_per_query=S))
    assert np.array_equal(got, oracle.route_seeds(probes, n, offs, mem, S, labels=labels, masks=masks,
                                                  label_offsets=loff))
    v = got != 0xFFFFFFFF
    assert (((masks[:, None] >> labels[np.where(v, got, 0)]) & 1) == 1)[v].all()
    scattered = rng.integers(0, 6, n).astype(np.uint8)
    d_sc = _t(scattered)
    f = grab.make_filter(grab.FILTER_LABELS, labels=d_sc, masks=d_m)
    got = _u32(grab.route_seeds(r, d_q, n, f, probes=P, seeds_per_query=S))
    assert np.array_equal(got, oracle.route_seeds(probes, n, offs, mem, S, labels=scattered, masks=masks))


def test_routed_seeds_reach_separated_clusters(grab, oracle):
    """Well-separated clusters: the kNN graph falls apart into one component per cluster, uniform
    seeds miss the query's cluster, routed seeds start inside it."""
    rng = np.random.default_rng(12)
    n, dim, total, local, nq, k = 32000, 64, 32, 24, 300, 10
    data = clustered(n, dim, 160, 0.15, 13)
    ts = np.arange(n, dtype=np.uint64)
    nb = 4
    sizes = [n // nb] * nb
    bucket = (ts // np.uint64(n // nb)).astype(np.int64)
    d_data = _t(data)
    graph = grab.build_time_partitioned_graph(d_data, _t(bucket), sizes, total, local)
    q = data[rng.integers(0, n, nq)] + np.float32(0.01)
    lo = rng.integers(0, n - n // 4, nq).astype(np.uint64)
    hi = lo + np.uint64(n // 4)
    gt, _ = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi)
    d_q, d_ts, d_lo, d_hi = _t(q), _t(ts.view(np.int64)), _t(lo.view(np.int64)), _t(hi.view(np.int64))
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=d_lo, hi=d_hi, ts_sorted=True)
    p = grab.SearchParams(64, 2, 0, 8, 11)
    plain, _ = grab.graph_search(d_data, graph, d_q, k, p, flt=f)
    r = grab.router_build(d_data, 256, iterations=5)
    seeds = grab.route_seeds(r, d_q, n, f, probes=4, seeds_per_query=32)
    routed, _ = grab.graph_search(d_data, graph, d_q, k, p, flt=f, seeds=seeds)
    routed = routed.cpu().numpy()
    assert ((routed >= lo[:, None].astype(np.int64)) & (routed < hi[:, None].astype(np.int64)) | (routed < 0)).all()
    r_plain, r_routed = oracle.recall(plain.cpu().numpy(), gt), oracle.recall(routed, gt)
    assert r_routed > 0.95 and r_routed > r_plain + 0.1, (r_plain, r_routed)
    # the id windows handed from the router to the search: the windows themselves, and the same results bit for bit
    import torch
    win = torch.full((nq, 4), -1, dtype=torch.int32, device="cuda")
    fw = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=d_lo, hi=d_hi, ts_sorted=True, id_windows=win)
    seeds_w = grab.route_seeds(r, d_q, n, fw, probes=4, seeds_per_query=32)
    assert torch.equal(seeds_w, seeds)
    w = win.cpu().numpy()
    assert np.array_equal(w[:, 0], np.searchsorted(ts, lo, side="left"))
    assert np.array_equal(w[:, 1], np.searchsorted(ts, hi, side="left"))
    shared, shared_d = grab.graph_search(d_data, graph, d_q, k, p, flt=fw, seeds=seeds_w)
    again, again_d = grab.graph_search(d_data, graph, d_q, k, p, flt=f, seeds=seeds)
    assert torch.equal(shared, again) and torch.equal(shared_d, again_d)


@pytest.mark.parametrize("dim,metric,nc,nq", [(128, 0, 256, 1000), (100, 0, 200, 300), (768, 1, 384, 513)])
def test_tensor_core_routing_matches_exact_scan(grab, oracle, dim, metric, nc, nq):
    """Centroid ranking on the tensor cores (tf32, probes + 4 candidates re-scored exactly) gives the
    seeds of the exact fp32 scan, which are the oracle's: ragged row, column and K tiles included."""
    rng = np.random.default_rng(dim + nc)
    n = 30000 if dim < 768 else 12000
    data = clustered(n, dim, 60, 0.7, dim + 7)
    if metric == 1:
        data /= np.linalg.norm(data, axis=1, keepdims=True)
    q = data[rng.integers(0, n, nq)] + np.float32(0.02) * rng.standard_normal((nq, dim)).astype(np.float32)
    d_data, d_q = _t(data), _t(q)
    r = grab.router_build(d_data, nc, metric=metric, iterations=3, max_sample=8000)
    cen, cnorm, offs, mem = (r.centroids.cpu().numpy(), r.norms.cpu().numpy(), _u32(r.offsets), _u32(r.members))
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n // 2, nq).astype(np.uint64)
    hi = lo + np.uint64(n // 3)
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                         hi=_t(hi.view(np.int64)), ts_sorted=True)
    for P, S in [(4, 32), (1, 8), (12, 48)]:
        tc = _u32(grab.route_seeds(r.exact(False), d_q, n, f, probes=P, seeds_per_query=S))
        ex = _u32(grab.route_seeds(r.exact(True), d_q, n, f, probes=P, seeds_per_query=S))
        probes = oracle.nearest_centroids(q, cen, cnorm, metric, P)
        want = oracle.route_seeds(probes, n, offs, mem, S, ts=ts, lo=lo, hi=hi)
        assert np.array_equal(ex, want)
        assert np.array_equal(tc, want)
    r.exact(False)
    # 13 probes and more: no room for 4 spare candidates, the exact scan runs
    tc = _u32(grab.route_seeds(r, d_q, n, f, probes=14, seeds_per_query=56))
    probes = oracle.nearest_centroids(q, cen, cnorm, metric, 14)
    assert np.array_equal(tc, oracle.route_seeds(probes, n, offs, mem, 56, ts=ts, lo=lo, hi=hi))
