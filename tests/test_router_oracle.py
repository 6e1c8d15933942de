"""Properties of the oracle's entry-point router restatement (CPU only)."""
import numpy as np

from conftest import clustered


def test_group_by_centroid_is_a_stable_partition(oracle):
    rng = np.random.default_rng(3)
    a = rng.integers(0, 17, 5000).astype(np.uint32)
    offs, mem = oracle.group_by_centroid(a, 17)
    assert offs[0] == 0 and offs[-1] == 5000
    assert np.array_equal(np.diff(offs.astype(np.int64)), np.bincount(a, minlength=17))
    for c in range(17):
        run = mem[offs[c]:offs[c + 1]]
        assert (a[run] == c).all() and (np.diff(run.astype(np.int64)) > 0).all()
    assert np.array_equal(np.sort(mem), np.arange(5000, dtype=np.uint32))


def test_nearest_centroids_matches_float64(oracle):
    rng = np.random.default_rng(4)
    cen = rng.standard_normal((40, 32)).astype(np.float32)
    x = cen[rng.integers(0, 40, 300)] + 0.1 * rng.standard_normal((300, 32)).astype(np.float32)
    cn = (cen.astype(np.float64) ** 2).sum(1).astype(np.float32)
    got = oracle.nearest_centroids(x, cen, cn, 0, 3)
    d = ((x[:, None, :].astype(np.float64) - cen[None].astype(np.float64)) ** 2).sum(2)
    assert np.array_equal(got[:, 0], d.argmin(1).astype(np.uint32))
    assert np.array_equal(got, np.argsort(d, axis=1, kind="stable")[:, :3].astype(np.uint32))
    got_ip = oracle.nearest_centroids(x, cen, cn, 1, 1)
    assert np.array_equal(got_ip[:, 0], (-(x.astype(np.float64) @ cen.T.astype(np.float64))).argmin(1))


def test_router_build_and_seeds(oracle):
    n, dim, nc = 6000, 32, 24
    data = clustered(n, dim, 12, 0.5, 11)
    cen, cnorm, offs, mem = oracle.router_build(data, nc, 0, iterations=4)
    assert np.allclose(cnorm, (cen.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    # every vector sits in the list of its nearest centroid
    a = oracle.nearest_centroids(data, cen, cnorm, 0, 1)[:, 0]
    for c in range(nc):
        assert (a[mem[offs[c]:offs[c + 1]]] == c).all()
    # Lloyd made the clustering tighter than the initial centroids
    init = data[(np.arange(nc) * min(n, 64 * nc) // nc) * n // min(n, 64 * nc)]
    cost = lambda cc: ((data[:, None, :] - cc[None]) ** 2).sum(2).min(1).mean()
    assert cost(cen) < cost(init)

    q = data[::600].copy()
    probes = oracle.nearest_centroids(q, cen, cnorm, 0, 4)
    ts = np.arange(n, dtype=np.uint64)
    lo = np.arange(q.shape[0], dtype=np.uint64) * 100
    hi = lo + 2500
    for ts_sorted in (True, False):
        s = oracle.route_seeds(probes, n, offs, mem, 32, ts=ts, lo=lo, hi=hi, ts_sorted=ts_sorted)
        for i in range(q.shape[0]):
            v = s[i][s[i] != 0xFFFFFFFF]
            assert v.size >= 8
            assert ((v >= lo[i]) & (v < hi[i])).all()               # inside the filter
            assert np.isin(a[v], probes[i]).all()                    # members of the probed centroids
            if ts_sorted:
                assert np.unique(v).size == v.size                   # no seed twice
    # empty range -> no seeds
    s = oracle.route_seeds(probes, n, offs, mem, 32, ts=ts, lo=7, hi=7)
    assert (s == 0xFFFFFFFF).all()
    # labels as id ranges
    labels = np.repeat(np.arange(4, dtype=np.uint8), n // 4)
    lo_off = np.zeros(33, np.uint32)
    lo_off[1:5] = np.cumsum([n // 4] * 4)
    lo_off[5:] = n
    masks = np.full(q.shape[0], 0b0110, np.uint32)
    s = oracle.route_seeds(probes, n, offs, mem, 32, labels=labels, masks=masks, label_offsets=lo_off)
    v = s[s != 0xFFFFFFFF]
    assert np.isin(labels[v], [1, 2]).all() and (labels[v] == 1).any() and (labels[v] == 2).any()
    s2 = oracle.route_seeds(probes, n, offs, mem, 32, labels=labels, masks=masks)      # predicate tests
    v2 = s2[s2 != 0xFFFFFFFF]
    assert v2.size and np.isin(labels[v2], [1, 2]).all()
