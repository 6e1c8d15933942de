"""Parity of the CUDA path (through the C ABI) against the CPU oracle.  Needs a B200."""
import numpy as np
import pytest

from conftest import clustered

pytestmark = pytest.mark.gpu


def _t(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


# ------------------------------------------------------------------ exact filtered search
@pytest.mark.parametrize("dim,metric", [(128, 0), (96, 0), (64, 0), (768, 1), (100, 0)])
def test_exact_range_bit_exact(grab, oracle, dim, metric):
    rng = np.random.default_rng(dim)
    n, nq, k = 20000, 64, 10
    data = clustered(n, dim, 50, 0.5, dim)
    q = data[rng.integers(0, n, nq)] + 0.05 * rng.standard_normal((nq, dim)).astype(np.float32)
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n - 2000, nq).astype(np.uint64)
    hi = lo + 2000
    oi, od = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi, metric=metric)
    for sorted_flag in (True, False):
        f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                             hi=_t(hi.view(np.int64)), ts_sorted=sorted_flag)
        gi, gd = grab.exact_search(_t(data), _t(q), k, metric=metric, flt=f)
        assert np.array_equal(gi.cpu().numpy(), oi)                      # ids bit-exact
        assert np.array_equal(gd.cpu().numpy().view(np.uint32), od.view(np.uint32))  # same fp32 bits
    d64 = np.array([((q[i].astype(np.float64) - data[int(oi[i, 0])].astype(np.float64)) ** 2).sum()
                    if metric == 0 else -(q[i].astype(np.float64) @ data[int(oi[i, 0])].astype(np.float64))
                    for i in range(nq)])
    assert np.allclose(od[:, 0], d64, rtol=1e-4, atol=1e-5)              # within 1e-4 relative of fp64


def test_exact_edge_cases(grab, oracle):
    rng = np.random.default_rng(1)
    n, dim = 5003, 128                     # ragged: not a multiple of the scan step
    data = rng.standard_normal((n, dim)).astype(np.float32)
    data[100:110] = data[100]              # exact duplicates -> ties go to the lower id
    q = np.concatenate([data[100:101], rng.standard_normal((6, dim)).astype(np.float32)])
    ts = np.arange(n, dtype=np.uint64)
    lo = np.array([0, 0, 5000, 17, 4000, 0, 2500], dtype=np.uint64)
    hi = np.array([n, 3, 5003, 17, 4003, 1, 2600], dtype=np.uint64)   # full, tiny, tail, EMPTY, ...
    k = 16
    oi, od = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi)
    for sorted_flag in (True, False):
        f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                             hi=_t(hi.view(np.int64)), ts_sorted=sorted_flag)
        gi, gd = grab.exact_search(_t(data), _t(q), k, flt=f)
        assert np.array_equal(gi.cpu().numpy(), oi)
    assert oi[0, :10].tolist() == list(range(100, 110))
    assert (oi[3] == -1).all() and (oi[1, 3:] == -1).all()
    # unfiltered, one call-wide range, few queries -> the scan is split across CTAs and merged
    gi, _ = grab.exact_search(_t(data), _t(q[:2]), 100)
    oi2, _ = oracle.exact_search(data, q[:2], 100)
    assert np.array_equal(gi.cpu().numpy(), oi2)
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=1000, hi=3000)
    gi, _ = grab.exact_search(_t(data), _t(q), 10, flt=f)
    oi3, _ = oracle.exact_search(data, q, 10, ts=ts, lo=1000, hi=3000)
    assert np.array_equal(gi.cpu().numpy(), oi3)


def test_exact_labels_inner_product(grab, oracle):
    rng = np.random.default_rng(2)
    n, dim, nq = 30000, 768, 32
    data = clustered(n, dim, 32, 0.3, 5)
    data /= np.linalg.norm(data, axis=1, keepdims=True)
    q = data[rng.integers(0, n, nq)].copy()
    labels = rng.integers(0, 16, n).astype(np.uint8)
    masks = rng.integers(1, 1 << 16, nq).astype(np.uint32)
    oi, od = oracle.exact_search(data, q, 10, labels=labels, masks=masks, metric=1)
    f = grab.make_filter(grab.FILTER_LABELS, labels=_t(labels), masks=_t(masks.view(np.int32)))
    gi, gd = grab.exact_search(_t(data), _t(q), 10, metric=1, flt=f)
    assert np.array_equal(gi.cpu().numpy(), oi)
    assert np.array_equal(gd.cpu().numpy().view(np.uint32), od.view(np.uint32))


def test_bad_arguments_return_status_not_exit(grab):
    import torch
    data = torch.zeros((10, 6), device="cuda")         # dim not a multiple of 4
    with pytest.raises(grab.GrabError) as e:
        grab.exact_search(data, data, 2)
    assert e.value.status == 1
    data = torch.zeros((10, 8), device="cuda")
    with pytest.raises(grab.GrabError):
        grab.exact_search(data, data, 5000)            # k too large
    g = torch.zeros((10, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(grab.GrabError):
        grab.graph_search(data, g, data, 2, grab.SearchParams(hash_bitlen=30))


# ------------------------------------------------------------------ kNN + graph optimisation
def _build_small(grab, oracle, n=6000, dim=32, deg=16, nb=1, seed=21):
    data = clustered(n, dim, 20, 1.0, seed)
    offs = np.linspace(0, n, nb + 1).astype(np.uint64)
    knn_o = np.concatenate([oracle.knn_block(data[int(offs[b]):int(offs[b + 1])], 2 * deg) +
                            np.uint32(offs[b]) for b in range(nb)])
    return data, offs, knn_o


def test_knn_blocks_bit_exact(grab, oracle):
    data, offs, knn_o = _build_small(grab, oracle, nb=3)
    knn_g = _u32(grab.knn_graph_blocks(_t(data), offs, 32, mode=0))
    assert np.array_equal(knn_g, knn_o)
    # a block smaller than k: padded with 0xFFFFFFFF, never contains self
    small = np.array([0, 20, 6000], dtype=np.uint64)
    knn_s = _u32(grab.knn_graph_blocks(_t(data), small, 32, mode=0))
    assert (knn_s[:20, 19:] == 0xFFFFFFFF).all() and (knn_s[:20, :19] < 20).all()
    assert not (knn_s == np.arange(6000, dtype=np.uint32)[:, None]).any()
    # mode 1: nearest vectors OUTSIDE the own block
    cand = _u32(grab.knn_graph_blocks(_t(data), offs, 8, mode=1))
    blk = np.searchsorted(offs, np.arange(6000), side="right") - 1
    assert (np.searchsorted(offs, cand, side="right") - 1 != blk[:, None]).all()


def test_knn_constant_vector_known_answer_full_size(grab):
    # tests/test_knn_build.cu at its own size: N 10 000, dim 1024, K 10
    n, dim, k = 10000, 1024, 10
    data = (np.arange(n, dtype=np.float32) * np.float32(0.001))[:, None].repeat(dim, 1)
    knn = _u32(grab.knn_graph_blocks(_t(data), np.array([0, n], dtype=np.uint64), k))
    idx = np.arange(n)[:, None]
    assert not (knn == idx).any()
    lo = np.clip(idx - 5, 0, n - 11)
    ok = (knn >= lo) & (knn <= lo + 10)
    assert ok.mean() > 0.99


def test_prune_reverse_merge_bit_exact(grab, oracle):
    import torch
    data, offs, knn_o = _build_small(grab, oracle, nb=2)
    n, deg = data.shape[0], 16
    knn_t = _t(knn_o.view(np.int32))
    out = torch.empty((n, deg), dtype=torch.int32, device="cuda")
    det = torch.empty((n, 32), dtype=torch.uint8, device="cuda")
    L = grab.lib()
    grab.check(L.grab_optimize_prune_device(grab._p(knn_t), grab._p(out), grab.C.c_uint64(n), 32, deg,
                                            grab._p(det), None))
    po, pdet = oracle.prune(knn_o, deg, want_detour=True)
    assert np.array_equal(det.cpu().numpy(), pdet)
    assert np.array_equal(_u32(out), po)
    rev = torch.empty((n, deg), dtype=torch.int32, device="cuda")
    cnt = torch.empty(n, dtype=torch.int32, device="cuda")
    grab.check(L.grab_optimize_reverse_graph_device(grab._p(out), grab._p(rev), grab._p(cnt),
                                                    grab.C.c_uint64(n), deg, None))
    ro, co = oracle.reverse_graph(po)
    assert np.array_equal(_u32(cnt), co)
    assert np.array_equal(_u32(rev), ro)
    grab.check(L.grab_optimize_merge_graphs_device(grab._p(out), grab._p(rev), grab._p(cnt),
                                                   grab.C.c_uint64(n), deg, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(out), oracle.merge_graphs(po, ro, co))
    # rows with pads and duplicate ids take the exact (slow) path of the prune kernel
    knn_p = knn_o.copy()
    knn_p[::7, 20:] = 0xFFFFFFFF
    knn_p[::11, 5] = knn_p[::11, 2]
    out2 = torch.empty((n, deg), dtype=torch.int32, device="cuda")
    knn_pt = _t(knn_p.view(np.int32))          # keep alive: the C ABI only sees raw pointers
    grab.check(L.grab_optimize_prune_device(grab._p(knn_pt), grab._p(out2),
                                            grab.C.c_uint64(n), 32, deg, None, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(out2), oracle.prune(knn_p, deg))


def test_reverse_graph_hub(grab, oracle):
    # one node with in-degree far above the shared-memory sort size of the select kernel
    import torch
    n, deg = 3000, 8
    rng = np.random.default_rng(4)
    g = rng.integers(0, n, size=(n, deg)).astype(np.uint32)
    g[:, 3] = 7
    g[5, :] = 0xFFFFFFFF
    gt = _t(g.view(np.int32))
    rev = torch.empty((n, deg), dtype=torch.int32, device="cuda")
    cnt = torch.empty(n, dtype=torch.int32, device="cuda")
    grab.check(grab.lib().grab_optimize_reverse_graph_device(grab._p(gt), grab._p(rev), grab._p(cnt),
                                                             grab.C.c_uint64(n), deg, None))
    ro, co = oracle.reverse_graph(g)
    assert np.array_equal(_u32(cnt), co) and np.array_equal(_u32(rev), ro)


def test_remote_edges_and_injection_bit_exact(grab, oracle):
    import torch
    n, total, local, gk, nb = 4000, 16, 10, 64, 20
    rng = np.random.default_rng(8)
    bucket = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    graph = rng.integers(0, n, size=(n, total)).astype(np.uint32)
    cand = rng.integers(0, n, size=(n, gk)).astype(np.uint32)
    cand[::5, 40:] = 0xFFFFFFFF
    go, _ = oracle.remote_edges(graph, bucket, cand, local)
    gt, ct, bt = _t(graph.view(np.int32)), _t(cand.view(np.int32)), _t(bucket.view(np.int64))
    L = grab.lib()
    grab.check(L.grab_remote_edges_device(grab._p(gt), grab._p(bt), grab._p(ct), grab.C.c_uint64(n),
                                          total, local, gk, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(gt), go)
    go2 = oracle.inject_reverse_remote(go, local, 32)
    grab.check(L.grab_inject_reverse_remote_device(grab._p(gt), grab.C.c_uint64(n), total, local, 32, None))
    assert np.array_equal(_u32(gt), go2)


def test_insert_topology_bit_exact(grab, oracle):
    import torch
    L = grab.lib()
    rng = np.random.default_rng(9)
    # v1
    ne, nn, deg, sk = 3000, 200, 16, 32
    g = np.full((ne + nn, deg), 0xFFFFFFFF, dtype=np.uint32)
    g[:ne] = rng.integers(0, ne, size=(ne, deg))
    found = np.stack([rng.choice(ne // 10, size=sk, replace=False) for _ in range(nn)]).astype(np.int64)
    found[::9, -3:] = -1
    go = oracle.insert_v1(g, found, ne, sk)
    gt, ft = _t(g.view(np.int32)), _t(found)
    grab.check(L.grab_update_topology_v1(grab._p(gt), grab._p(ft), grab.C.c_uint64(ne),
                                         grab.C.c_uint64(nn), deg, sk, None))
    assert np.array_equal(_u32(gt), go)
    # time-partitioned
    total, local, kl, kg = 16, 10, 24, 24
    nbk = 30
    bucket = np.concatenate([np.repeat(np.arange(nbk, dtype=np.uint64), ne // nbk),
                             np.full(nn, nbk - 1, dtype=np.uint64)])
    g = np.full((ne + nn, total), 0xFFFFFFFF, dtype=np.uint32)
    g[:ne] = rng.integers(0, ne, size=(ne, total))
    same = np.flatnonzero(bucket[:ne] == nbk - 1)
    lk = np.stack([rng.choice(np.concatenate([same, np.arange(ne, ne + nn)]), size=kl, replace=False)
                   for _ in range(nn)]).astype(np.int64)
    gkn = np.stack([rng.choice(ne, size=kg, replace=False) for _ in range(nn)]).astype(np.int64)
    go = oracle.insert_opt(g, bucket, lk, gkn, ne, nbk - 1, local)
    gt, bt, lkt, gkt = _t(g.view(np.int32)), _t(bucket.view(np.int64)), _t(lk), _t(gkn)
    grab.check(L.grab_update_topology_opt(grab._p(gt), grab._p(bt), grab._p(lkt),
                                          grab._p(gkt), grab.C.c_uint64(ne), grab.C.c_uint64(nn),
                                          grab.C.c_uint64(nbk - 1), total, local, kl, kg, None))
    assert np.array_equal(_u32(gt), go)


def test_merge_topk_bit_exact(grab, oracle):
    rng = np.random.default_rng(10)
    nq, parts, k = 50, 8, 100
    d = np.sort(rng.random((nq, parts, k)).astype(np.float32), axis=2)
    ids = rng.integers(0, 100_000_000, size=(nq, parts, k)).astype(np.int64)
    d[:, 3, 60:] = 3.40282e38
    ids[:, 3, 60:] = -1
    d[:, :, 5] = d[:, :1, 5]                      # equal distances across parts -> id tie-break
    d = np.sort(d, axis=2)
    oi, od = oracle.merge_topk(d, ids, k)
    gi, gd = grab.merge_topk(_t(d), _t(ids), k)
    assert np.array_equal(gi.cpu().numpy(), oi)
    assert np.array_equal(gd.cpu().numpy(), od)


def test_merge_sorted_keys_bit_exact(grab, oracle):
    """grab_merge_sorted_keys (the G-way rank merge of the sharded exchange step) against the CPU merge: runs of
    different fill, equal distances across shards (id tie-break), 1..8 shards, k below / equal / above the run
    length, one query with no result at all."""
    import torch
    rng = np.random.default_rng(12)
    for parts, kp, k, nq in [(8, 10, 10, 333), (2, 16, 10, 50), (4, 100, 100, 37), (1, 10, 10, 9), (8, 5, 10, 64),
                             (3, 7, 20, 40)]:
        d = np.sort(np.round(rng.random((parts, nq, kp)) * 40).astype(np.float32) / 8, axis=2)   # many ties
        ids = rng.permutation(parts * nq * kp * 3)[: parts * nq * kp].reshape(parts, nq, kp).astype(np.int64)
        fill = rng.integers(0, kp + 1, size=(parts, nq))
        fill[:, 0] = 0                                            # query 0: every shard came back empty
        empty = np.arange(kp)[None, None, :] >= fill[:, :, None]
        f2o = lambda x: np.where(x.view(np.uint32) & 0x80000000, ~x.view(np.uint32), x.view(np.uint32) | 0x80000000)
        keys = (f2o(d).astype(np.uint64) << np.uint64(32)) | ids.astype(np.uint64)
        keys[empty] = np.uint64(0xFFFFFFFFFFFFFFFF)
        keys = np.sort(keys, axis=2)                              # runs ascending by (dist, id)
        dd = np.where(empty, np.float32(3.40282e38), d)
        ii = np.where(empty, -1, ids)
        if kp == k:       # the CPU merge takes lists of exactly k entries
            oi, od = oracle.merge_topk(np.ascontiguousarray(dd.transpose(1, 0, 2)),
                                       np.ascontiguousarray(ii.transpose(1, 0, 2)), k)
        else:             # other run lengths: the k smallest keys of the union, by definition
            flat = np.sort(keys.transpose(1, 0, 2).reshape(nq, -1), axis=1)[:, :k]
            flat = np.concatenate([flat, np.full((nq, max(0, k - flat.shape[1])), 0xFFFFFFFFFFFFFFFF, np.uint64)], axis=1)
            none = flat == np.uint64(0xFFFFFFFFFFFFFFFF)
            oi = np.where(none, -1, (flat & np.uint64(0xFFFFFFFF)).astype(np.int64))
            o32 = (flat >> np.uint64(32)).astype(np.uint32)
            od = np.where(o32 & 0x80000000, o32 & 0x7FFFFFFF, ~o32).astype(np.uint32).view(np.float32)
            od = np.where(none, np.float32(3.40282e38), od)
        gi, gd = grab.merge_sorted_keys(_t(keys.view(np.int64)), k)
        assert np.array_equal(gi.cpu().numpy(), oi), (parts, kp, k)
        assert np.array_equal(gd.cpu().numpy(), od), (parts, kp, k)


def test_search_keys_output_and_single_shard_exchange(grab, oracle):
    """grab_search_args.d_out_keys carries the same results as the id / distance outputs (global ids through
    id_scale / id_offset), and the exchange entry point with no communicator (one shard) returns them unchanged;
    two emulated stripes merged by grab_merge_sorted_keys give the exact search's ids when both stripes are searched
    exactly (the sharded result is the unsharded one)."""
    import torch
    rng = np.random.default_rng(31)
    n, dim, nq, k = 6000, 64, 64, 10
    data = rng.standard_normal((n, dim)).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    knn = oracle.knn_block(data, 32)
    g = oracle.prune(knn, 16)
    d_data, d_g, d_q = _t(data), _t(g.view(np.int32)), _t(q)
    keys = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    ids, dists = grab.graph_search(d_data, d_g, d_q, k, grab.SearchParams(64, 4, 0, 20, 11), id_scale=3, id_offset=2,
                                   out_keys=keys)
    out = (torch.empty_like(ids), torch.empty_like(dists))
    grab.check(grab.lib().grab_sharded_gather_merge(None, grab._p(keys), grab.C.c_uint64(nq), k, k, None,
                                                    grab.C.c_size_t(0), grab._p(out[0]), grab._p(out[1]), None))
    torch.cuda.synchronize()
    assert torch.equal(out[0], ids) and torch.equal(out[1], dists)
    assert ((ids % 3 == 2) | (ids < 0)).all()
    # two stripes, exact per-stripe results as keys -> merged == exact over the whole set
    want, wd = oracle.exact_search(data, q, k)
    parts = []
    for r in range(2):
        gi, gd = grab.exact_search(_t(data[r::2]), d_q, k)
        gi = gi.cpu().numpy() * 2 + r
        o = gd.cpu().numpy().view(np.uint32)
        o = np.where(o & 0x80000000, ~o, o | 0x80000000).astype(np.uint64)
        parts.append((o << np.uint64(32)) | gi.astype(np.uint64))
    mi, md = grab.merge_sorted_keys(_t(np.stack(parts).view(np.int64)), k)
    assert np.array_equal(mi.cpu().numpy(), want)
    assert np.array_equal(md.cpu().numpy(), wd)


# ------------------------------------------------------------------ filtered graph search
def _graph_fixture(oracle, n=20000, dim=64, deg=32, seed=31):
    data = clustered(n, dim, 40, 1.0, seed)
    knn = oracle.knn_block(data, 2 * deg)
    g = oracle.prune(knn, deg)
    rev, cnt = oracle.reverse_graph(g)
    return data, oracle.merge_graphs(g, rev, cnt)


@pytest.fixture(scope="module")
def small_graph(oracle):
    return _graph_fixture(oracle)


def test_graph_search_range_recall_parity(grab, oracle, small_graph):
    """Same graph, same seeds, equal itopk / width: recall against exact filtered ground
    truth within 0.5 percentage points of the reference algorithm's (CPU restatement)."""
    data, g = small_graph
    n, dim = data.shape
    rng = np.random.default_rng(32)
    nq, k = 400, 10
    q = data[rng.integers(0, n, nq)] + 0.1 * rng.standard_normal((nq, dim)).astype(np.float32)
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n - n // 2, nq).astype(np.uint64)
    hi = lo + np.uint64(n // 2)
    gt, _ = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi)
    seeds = np.stack([rng.integers(int(lo[i]), int(hi[i]), 32) for i in range(nq)]).astype(np.uint32)
    # (256, 4): the 256-entry list; (128, 12): 384 edges per iteration, 192 candidates per warp
    for itopk, width in [(64, 4), (128, 2), (256, 4), (128, 12)]:
        oi, _ = oracle.graph_search(data, g, q, k, itopk, width, 40, 13, mode=2, ts=ts, lo=lo, hi=hi, seeds=seeds)
        f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                             hi=_t(hi.view(np.int64)))
        gi, gd, st = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), k,
                                       grab.SearchParams(itopk, width, 0, 40, 13), flt=f,
                                       seeds=_t(seeds.view(np.int32)), stats=True)
        gi = gi.cpu().numpy()
        assert np.all((gi >= lo[:, None]) & (gi < hi[:, None]) | (gi < 0))      # no bound errors
        r_ref, r_gpu = oracle.recall(oi, gt), oracle.recall(gi, gt)
        assert r_gpu >= r_ref - 0.005, (r_gpu, r_ref)
        assert r_gpu > 0.85
        # returned distances are the canonical fp32 distances of the returned ids
        for i in range(0, nq, 37):
            for j in range(k):
                if gi[i, j] >= 0:
                    assert gd[i, j].item() == pytest.approx(oracle.dist(q[i], data[gi[i, j]]), rel=0, abs=0)
        assert st.distances > 0 and st.parents > 0 and st.edges >= st.distances
        assert np.all(np.diff(gd.cpu().numpy(), axis=1) >= 0)


def test_graph_search_unfiltered_and_bucket(grab, oracle, small_graph):
    data, g = small_graph
    n, dim = data.shape
    rng = np.random.default_rng(33)
    nq, k = 300, 10
    q = data[rng.integers(0, n, nq)] + 0.1 * rng.standard_normal((nq, dim)).astype(np.float32)
    gt, _ = oracle.exact_search(data, q, k)
    seeds = rng.integers(0, n, size=(nq, 32)).astype(np.uint32)
    oi, _ = oracle.graph_search(data, g, q, k, 64, 4, 40, 13, mode=0, seeds=seeds)
    gi, _ = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), k, grab.SearchParams(64, 4, 0, 40, 13),
                              seeds=_t(seeds.view(np.int32)))
    r_ref, r_gpu = oracle.recall(oi, gt), oracle.recall(gi.cpu().numpy(), gt)
    assert r_gpu >= r_ref - 0.005 and r_gpu > 0.9, (r_gpu, r_ref)
    # no seeds given: the kernel draws its own
    gi2, _ = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), k, grab.SearchParams(64, 4, 0, 40, 13))
    assert oracle.recall(gi2.cpu().numpy(), gt) > 0.9
    # bucket search: two disjoint halves, each with its own graph in the first 16 columns
    half = n // 2
    parts = []
    for b in range(2):
        kb = oracle.knn_block(data[b * half:(b + 1) * half], 32)
        pb = oracle.prune(kb, 16)
        rb, cb = oracle.reverse_graph(pb)
        parts.append(oracle.merge_graphs(pb, rb, cb) + np.uint32(b * half))
    g2 = np.concatenate([np.concatenate(parts), g[:, :16]], axis=1)   # [local 16 | anything 16]
    gt_b, _ = oracle.exact_search(data[half:], q, k)
    gt_b = gt_b + half
    seeds_b = rng.integers(half, n, size=(nq, 32)).astype(np.uint32)
    oi, _ = oracle.graph_search(data, g2, q, k, 128, 4, 40, 13, mode=1, active_deg=16, seeds=seeds_b)
    f = grab.make_filter(grab.FILTER_PREFIX, active_degree=16)
    gi, _ = grab.graph_search(_t(data), _t(g2.view(np.int32)), _t(q), k, grab.SearchParams(128, 4, 0, 40, 13),
                              flt=f, seeds=_t(seeds_b.view(np.int32)))
    gi = gi.cpu().numpy()
    assert (gi >= half).all()                                  # 0 out-of-bucket ids
    r_ref, r_gpu = oracle.recall(oi, gt_b), oracle.recall(gi, gt_b)
    assert r_gpu > 0.85 and r_gpu >= r_ref - 0.005, (r_gpu, r_ref)


def test_graph_search_labels_ip_and_sharded_ids(grab, oracle):
    rng = np.random.default_rng(35)
    n, dim, deg, nq, k = 8000, 768, 32, 100, 10
    data = clustered(n, dim, 16, 1.0, 36)
    data /= np.linalg.norm(data, axis=1, keepdims=True)
    knn = oracle.knn_block(data, 2 * deg, metric=1)
    g = oracle.prune(knn, deg)
    rev, cnt = oracle.reverse_graph(g)
    g = oracle.merge_graphs(g, rev, cnt)
    q = data[rng.integers(0, n, nq)].copy()
    labels = rng.integers(0, 4, n).astype(np.uint8)
    masks = rng.integers(1, 16, nq).astype(np.uint32)
    gt, _ = oracle.exact_search(data, q, k, labels=labels, masks=masks, metric=1)
    f = grab.make_filter(grab.FILTER_LABELS, labels=_t(labels), masks=_t(masks.view(np.int32)))
    gi, gd = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), k, grab.SearchParams(256, 4, 0, 80, 13),
                               metric=1, flt=f, id_scale=4, id_offset=3)
    gi = gi.cpu().numpy()
    assert ((gi % 4 == 3) | (gi < 0)).all()                     # striped-shard id mapping
    loc = np.where(gi >= 0, (gi - 3) // 4, -1)
    ok = loc >= 0
    assert ((masks[:, None] >> labels[np.clip(loc, 0, n - 1)]) & 1)[ok].all()
    assert oracle.recall(loc, gt) > 0.8


def test_graph_search_label_partitioned_seeds(grab, oracle):
    """Vectors grouped by label, one bucket per label: seeds drawn from the id ranges of the query's
    labels find a rare label (2 % of the data) that uniform seeds would mostly miss."""
    rng = np.random.default_rng(37)
    n, dim, total, local, nq, k = 12000, 64, 32, 24, 200, 10
    data = clustered(n, dim, 24, 1.0, 38)
    sizes = [6000, 3000, 1800, 960, 240]
    labels = np.repeat(np.arange(5, dtype=np.uint8), sizes)
    offsets = np.zeros(33, np.uint32)
    offsets[1:6] = np.cumsum(sizes)
    offsets[6:] = n
    bucket = labels.astype(np.uint64)
    graph = grab.build_time_partitioned_graph(_t(data), _t(bucket.view(np.int64)), sizes, total, local,
                                              knn_precision=grab.KNN_EXACT_SCAN)
    q = data[rng.integers(0, n, nq)].copy() + 0.01
    masks = np.full(nq, 1 << 4, np.uint32)                     # the rare label alone ...
    masks[nq // 2:] = (1 << 4) | (1 << 1)                      # ... or together with a common one
    gt, _ = oracle.exact_search(data, q, k, labels=labels, masks=masks)
    d_labels, d_masks, d_offs = _t(labels), _t(masks.view(np.int32)), _t(offsets.view(np.int32))
    f = grab.make_filter(grab.FILTER_LABELS, labels=d_labels, masks=d_masks, label_offsets=d_offs)
    gi, gd = grab.graph_search(_t(data), graph, _t(q), k, grab.SearchParams(64, 4, 0, 40, 12), flt=f)
    gi = gi.cpu().numpy()
    assert (((masks[:, None] >> labels[np.clip(gi, 0, n - 1)]) & 1) == 1)[gi >= 0].all()
    assert (gi[: nq // 2] >= offsets[4]).all() and (gi[: nq // 2] >= 0).all()
    assert oracle.recall(gi, gt) > 0.9, oracle.recall(gi, gt)


def test_graph_search_empty_range_and_global_hash(grab, oracle, small_graph):
    data, g = small_graph
    n, dim = data.shape
    q = data[:16].copy()
    ts = np.arange(n, dtype=np.uint64)
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=500, hi=500, ts_sorted=True)
    gi, gd = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), 10, grab.SearchParams(64, 4, 0, 20, 12), flt=f)
    assert (gi.cpu().numpy() == -1).all()                       # "no data in filter" -> -1
    # hash table in global memory (bitlen 14), self-drawn seeds inside a sorted-ts window
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=0, hi=n // 2, ts_sorted=True)
    gi, gd = grab.graph_search(_t(data), _t(g.view(np.int32)), _t(q), 10, grab.SearchParams(64, 4, 0, 40, 14), flt=f)
    gt, _ = oracle.exact_search(data, q, 10, ts=ts, lo=0, hi=n // 2)
    gi = gi.cpu().numpy()
    assert (gi < n // 2).all() and oracle.recall(gi, gt) > 0.8


def test_time_partitioned_build_end_to_end(grab, oracle):
    """build_time_partitioned_graph -> range search; local columns stay inside the bucket."""
    n, dim, nb, total, local = 16000, 64, 8, 32, 24
    data = clustered(n, dim, 40, 1.0, 41)
    bucket = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    graph = grab.build_time_partitioned_graph(_t(data), _t(bucket.view(np.int64)), [n // nb] * nb, total, local,
                                              knn_precision=grab.KNN_EXACT_SCAN)
    g = _u32(graph)
    blk = np.arange(n) // (n // nb)
    loc = g[:, :local]
    assert ((loc // (n // nb) == blk[:, None]) | (loc == 0xFFFFFFFF)).all()
    rem = g[:, local:]
    valid = rem != 0xFFFFFFFF
    assert valid.mean() > 0.9
    assert not (g == np.arange(n, dtype=np.uint32)[:, None]).any()
    # the local part equals the oracle pipeline bucket by bucket
    b0 = oracle.knn_block(data[:n // nb], 2 * total)
    p0 = oracle.prune(b0, total)
    r0, c0 = oracle.reverse_graph(p0)
    m0 = oracle.merge_graphs(p0, r0, c0)
    assert np.array_equal(g[:n // nb, :local], m0[:, :local])
    rng = np.random.default_rng(42)
    nq = 200
    q = data[rng.integers(0, n, nq)] + 0.1 * rng.standard_normal((nq, dim)).astype(np.float32)
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n - n // 4, nq).astype(np.uint64)
    hi = lo + np.uint64(n // 4)
    gt, _ = oracle.exact_search(data, q, 10, ts=ts, lo=lo, hi=hi)
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                         hi=_t(hi.view(np.int64)), ts_sorted=True)
    gi, _ = grab.graph_search(_t(data), graph, _t(q), 10,
                              grab.SearchParams(64, 4, 0, 40, 13), flt=f)
    assert oracle.recall(gi.cpu().numpy(), gt) > 0.9


# ------------------------------------------------------------------ tensor-core kNN (tcgen05)
def _row_recall(a, b):
    hit = sum(len(set(x[x != 0xFFFFFFFF]).intersection(y[y != 0xFFFFFFFF])) for x, y in zip(a, b))
    return hit / max(1, int((b != 0xFFFFFFFF).sum()))


@pytest.mark.parametrize("dim,metric", [(128, 0), (96, 0), (768, 1)])
def test_knn_tensor_core_matches_exact(grab, dim, metric):
    """All-pairs tile on tcgen05 + fused top-k + exact re-rank against the exact fp32 scan."""
    n, k = 20000, 64
    data = clustered(n, dim, 40, 1.0, 50 + dim)
    if metric == 1:
        data /= np.linalg.norm(data, axis=1, keepdims=True)
    offs = np.array([0, 7000, 7100, n], dtype=np.uint64)      # ragged blocks, one tiny
    d = _t(data)
    exact, exact_d = grab.knn_graph_blocks(d, offs, k, mode=0, metric=metric, want_dists=True)
    exact = _u32(exact)
    for prec, floor in [(grab.KNN_TC_SPLIT, 0.999), (grab.KNN_TC_BF16, 0.97)]:
        got, got_d = grab.knn_graph_blocks(d, offs, k, mode=0, metric=metric, want_dists=True, precision=prec)
        got = _u32(got)
        assert not (got == np.arange(n, dtype=np.uint32)[:, None]).any()          # no self loops
        blk = np.searchsorted(offs, np.arange(n), side="right") - 1
        gb = np.searchsorted(offs, np.where(got == 0xFFFFFFFF, 0, got), side="right") - 1
        assert ((gb == blk[:, None]) | (got == 0xFFFFFFFF)).all()                  # stays inside its block
        assert _row_recall(got, exact) >= floor, (prec, _row_recall(got, exact))
        gd = got_d.cpu().numpy()
        assert np.all(np.diff(gd, axis=1) >= 0)                                    # exact distances, ascending
        same = got == exact
        assert np.array_equal(gd[same], exact_d.cpu().numpy()[same])               # re-rank is the canonical fp32
    # candidates from OTHER blocks
    ex1 = _u32(grab.knn_graph_blocks(d, offs, 32, mode=1, metric=metric))
    tc1 = _u32(grab.knn_graph_blocks(d, offs, 32, mode=1, metric=metric, precision=grab.KNN_TC_SPLIT))
    assert _row_recall(tc1, ex1) >= 0.999
    blk = np.searchsorted(offs, np.arange(n), side="right") - 1
    assert (np.searchsorted(offs, tc1, side="right") - 1 != blk[:, None]).all()


def test_knn_tensor_core_integer_data_is_exact(grab, datasets):
    """Descriptor-like data (integers 0..255) is exactly representable in bf16 and the fp32
    accumulation is exact, so the tensor-core path must reproduce the exact rows bit for bit."""
    base, _ = datasets.descriptor_like(30000, 128, 100, 77)
    d = _t(base)
    offs = np.array([0, 10000, 20000, 30000], dtype=np.uint64)
    exact = _u32(grab.knn_graph_blocks(d, offs, 96, mode=0))
    tc = _u32(grab.knn_graph_blocks(d, offs, 96, mode=0, precision=grab.KNN_TC_BF16))
    assert _row_recall(tc, exact) >= 0.9999


def test_knn_constant_vector_known_answer_tensor_core(grab):
    # tests/test_knn_build.cu (N 10 000, dim 1024, K 10, vector i = constant i*0.001) through
    # the reference-shaped entry point grab_generate_knn_graph (split precision + exact re-rank)
    n, dim, k = 10000, 1024, 10
    data = (np.arange(n, dtype=np.float32) * np.float32(0.001))[:, None].repeat(dim, 1)
    d = _t(data)
    out = np.empty((n, k), dtype=np.uint32)
    grab.check(grab.lib().grab_generate_knn_graph(grab._p(d), grab.C.c_uint64(n), dim, k, grab._p(out)))
    idx = np.arange(n)[:, None]
    assert not (out == idx).any()                       # 0 self loops
    lo = np.clip(idx - 5, 0, n - 11)
    assert ((out >= lo) & (out <= lo + 10)).mean() > 0.99   # recall > 99 % (test_knn_build.cu:111)


def test_time_partitioned_build_tensor_core(grab, oracle):
    n, dim, nb, total, local = 16000, 64, 8, 32, 24
    data = clustered(n, dim, 40, 1.0, 41)
    bucket = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    g_ex = _u32(grab.build_time_partitioned_graph(_t(data), _t(bucket.view(np.int64)), [n // nb] * nb, total, local,
                                                  knn_precision=grab.KNN_EXACT_SCAN))
    g_tc = _u32(grab.build_time_partitioned_graph(_t(data), _t(bucket.view(np.int64)), [n // nb] * nb, total, local,
                                                  knn_precision=grab.KNN_TC_SPLIT))
    assert (g_ex == g_tc).mean() > 0.98


def test_time_partitioned_build_routed_search_candidates(grab, oracle):
    """Cross-bucket candidates from the routed graph search over the local edges (the linear-time
    stand-in for the all-pairs stage): remote columns leave the bucket, and range searches over several
    buckets are as good as on the all-pairs graph."""
    rng = np.random.default_rng(91)
    n, dim, nb, total, local, nq, k = 40000, 64, 10, 32, 24, 300, 10
    data = clustered(n, dim, 80, 0.6, 92)
    ts = np.arange(n, dtype=np.uint64)
    sizes = [n // nb] * nb
    bucket = (ts // np.uint64(n // nb))
    d_data, d_bucket = _t(data), _t(bucket.view(np.int64))
    q = data[rng.integers(0, n, nq)] + np.float32(0.02)
    lo = rng.integers(0, n - n // 3, nq).astype(np.uint64)
    hi = lo + np.uint64(n // 3)
    gt, _ = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi)
    f = grab.make_filter(grab.FILTER_TS_RANGE, ts=_t(ts.view(np.int64)), lo=_t(lo.view(np.int64)),
                         hi=_t(hi.view(np.int64)), ts_sorted=True)
    rec = {}
    for mode in (grab.GLOBAL_ALL_PAIRS, grab.GLOBAL_ROUTED_SEARCH):
        graph = grab.build_time_partitioned_graph(d_data, d_bucket, sizes, total, local, global_candidates=mode)
        g = _u32(graph)
        rows = np.arange(n)[:, None]
        loc, rem = g[:, :local], g[:, local:]
        assert (bucket[np.where(loc == 0xFFFFFFFF, rows, loc)] == bucket[:, None]).all()
        valid = rem != 0xFFFFFFFF
        assert valid.mean() > 0.95
        assert (bucket[np.where(valid, rem, 0)] != bucket[:, None])[valid].all()
        gi, _ = grab.graph_search(d_data, graph, _t(q), k, grab.SearchParams(64, 4, 0, 32, 12), flt=f)
        rec[mode] = oracle.recall(gi.cpu().numpy(), gt)
    assert rec[grab.GLOBAL_ROUTED_SEARCH] > 0.9
    assert rec[grab.GLOBAL_ROUTED_SEARCH] >= rec[grab.GLOBAL_ALL_PAIRS] - 0.02, rec
