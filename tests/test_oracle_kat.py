"""The CPU oracle against the reference's own known-answer tests (no GPU needed)."""
import numpy as np
import pytest


def _std_mt19937_uniform_float(seed, count, a, b):
    """Inputs of tests/test_bitonic.cu:73-79 / test_sort_impl.cu: std::mt19937(seed) through
    std::uniform_real_distribution<float>(a, b) (one 32-bit draw per value)."""
    bg = np.random.MT19937()
    bg._legacy_seeding(seed)
    raw = bg.random_raw(count).astype(np.uint32)
    canon = raw.astype(np.float32) / np.float32(4294967296.0)
    canon = np.where(canon >= 1.0, np.nextafter(np.float32(1.0), np.float32(0.0)), canon)
    return (canon * np.float32(b - a) + np.float32(a)).astype(np.float32)


@pytest.mark.parametrize("n_per_lane", [2, 4, 8])
def test_warp_sort_matches_std_sort(oracle, n_per_lane):
    # tests/test_bitonic.cu: 32*N keys U(0,100) seed 42, value = original index;
    # pass rule: output equals std::sort of the (key, value) pairs.
    total = 32 * n_per_lane
    keys = _std_mt19937_uniform_float(42, total, 0.0, 100.0)
    vals = np.arange(total, dtype=np.uint32)
    k, v = oracle.warp_sort(keys, vals)
    order = np.lexsort((vals, keys))
    assert np.array_equal(k, keys[order])
    assert np.array_equal(v, vals[order])


@pytest.mark.parametrize("cap", [64, 128, 256, 512])
def test_queue_sort_capacities(oracle, cap):
    # tests/test_sort_impl.cu:111-121: capacities 64..512, U(0,1000) seed 42, tolerance 1e-4
    keys = _std_mt19937_uniform_float(42, cap, 0.0, 1000.0)
    vals = np.arange(cap, dtype=np.uint32)
    k, v = oracle.warp_sort(keys, vals)
    assert np.allclose(k, np.sort(keys), atol=1e-4)
    assert np.array_equal(keys[v], k)


def test_warp_sort_descending(oracle):
    keys = _std_mt19937_uniform_float(7, 64, 0.0, 1.0)
    k, v = oracle.warp_sort(keys, np.arange(64, dtype=np.uint32), asc=False)
    assert np.array_equal(k, np.sort(keys)[::-1])


@pytest.mark.parametrize("bitlen,unique,dup_ratio", [(10, 500, 0.4), (8, 200, 0.0), (8, 256, 0.0)])
def test_hashmap_known_answers(oracle, bitlen, unique, dup_ratio):
    # tests/test_hashmap.cu:171-187: successes == unique keys, occupied slots == successes
    table = np.full(1 << bitlen, 0xFFFFFFFF, dtype=np.uint32)
    keys = list(range(1, unique + 1)) + list(range(1, int(unique * dup_ratio) + 1))
    res = [oracle.hash_insert(table, bitlen, k) for k in keys]
    assert sum(res) == unique
    assert res[:unique] == [1] * unique and not any(res[unique:])
    assert int((table != 0xFFFFFFFF).sum()) == unique


def test_hashmap_full_table_reports_visited(oracle):
    # hashmap.cuh:89-90: a full table answers "already there"
    table = np.full(256, 0xFFFFFFFF, dtype=np.uint32)
    for k in range(256):
        assert oracle.hash_insert(table, 8, k + 1) == 1
    assert oracle.hash_insert(table, 8, 9999) == 0


def test_knn_constant_vector_known_answer(oracle):
    # tests/test_knn_build.cu:31-38,73-111 (vector i = constant i*0.001, dim 1024, K 10):
    # ideal neighbours are i +- delta, no self loops, recall > 99 %.  N reduced from 10 000
    # so the CPU finishes in seconds.
    n, dim, k = 1500, 1024, 10
    data = (np.arange(n, dtype=np.float32) * np.float32(0.001))[:, None].repeat(dim, 1)
    knn = oracle.knn_block(data, k)
    correct = 0
    for i in range(n):
        assert i not in knn[i]
        ideal, delta = set(), 1
        while len(ideal) < k:
            if i - delta >= 0:
                ideal.add(i - delta)
            if len(ideal) >= k:
                break
            if i + delta < n:
                ideal.add(i + delta)
            delta += 1
        correct += len(ideal.intersection(int(x) for x in knn[i]))
    assert correct / (n * k) > 0.99


def test_exact_search_matches_float64(oracle):
    rng = np.random.default_rng(3)
    data = rng.standard_normal((3000, 96)).astype(np.float32)
    q = rng.standard_normal((20, 96)).astype(np.float32)
    ts = np.arange(3000, dtype=np.uint64)
    lo = rng.integers(0, 2500, size=20).astype(np.uint64)
    hi = lo + 400
    ids, dists = oracle.exact_search(data, q, 10, ts=ts, lo=lo, hi=hi)
    for i in range(20):
        sl = slice(int(lo[i]), int(hi[i]))
        d64 = ((q[i].astype(np.float64) - data[sl].astype(np.float64)) ** 2).sum(1)
        gt = np.argsort(d64, kind="stable")[:10] + int(lo[i])
        assert set(gt) == set(ids[i])
        assert np.allclose(dists[i], np.sort(d64)[:10], rtol=1e-4)
        assert np.all((ids[i] >= lo[i]) & (ids[i] < hi[i]))
    # sequential (reference) order and canonical order agree on ids here
    ids2, _ = oracle.exact_search(data, q, 10, ts=ts, lo=lo, hi=hi, canonical=False)
    assert (ids2 == ids).mean() > 0.99


def test_exact_search_ties_go_to_lower_id_and_short_results(oracle):
    data = np.zeros((50, 8), dtype=np.float32)
    data[25:] = 1.0
    q = np.zeros((1, 8), dtype=np.float32)
    ids, dists = oracle.exact_search(data, q, 5)
    assert ids[0].tolist() == [0, 1, 2, 3, 4]
    ts = np.arange(50, dtype=np.uint64)
    ids, dists = oracle.exact_search(data, q, 5, ts=ts, lo=10, hi=13)
    assert ids[0].tolist() == [10, 11, 12, -1, -1]
    ids, _ = oracle.exact_search(data, q, 5, ts=ts, lo=7, hi=7)
    assert ids[0].tolist() == [-1] * 5


def test_exact_search_labels_and_inner_product(oracle):
    rng = np.random.default_rng(5)
    data = rng.standard_normal((2000, 64)).astype(np.float32)
    data /= np.linalg.norm(data, axis=1, keepdims=True)
    q = data[:7] + 0.01
    labels = rng.integers(0, 16, size=2000).astype(np.uint8)
    masks = np.array([1 << 3 | 1 << 5] * 7, dtype=np.uint32)
    ids, dists = oracle.exact_search(data, q, 10, labels=labels, masks=masks, metric=1)
    for i in range(7):
        ok = np.isin(labels, [3, 5])
        ip = -(data[ok].astype(np.float64) @ q[i].astype(np.float64))
        gt = np.flatnonzero(ok)[np.argsort(ip, kind="stable")[:10]]
        assert set(gt) == set(ids[i])
        assert np.all(np.diff(dists[i]) >= 0)


def test_prune_known_answer(oracle):
    # cagra.cu:219-276: edge A->B at rank j counts the D ranked before it with B in nbrs(D).
    # node 0: nbrs [1,2,3]; node 1: nbrs [2,3,0]; node 2: [3,0,1]; node 3: [0,1,2]
    knn = np.array([[1, 2, 3], [2, 3, 0], [3, 0, 1], [0, 1, 2]], dtype=np.uint32)
    out, det = oracle.prune(knn, 2, want_detour=True)
    # for A=0: B=2 (rank1): D=1 has 2 -> 1.  B=3 (rank2): D=1 has 3, D=2 has 3 -> 2.
    assert det[0].tolist() == [0, 1, 2]
    assert out[0].tolist() == [1, 2]
    # stable tie rule: equal counts keep the original rank order (cagra.cu:381-385)
    knn2 = np.array([[1, 2, 3], [0, 0xFFFFFFFF, 0xFFFFFFFF], [0, 0xFFFFFFFF, 0xFFFFFFFF],
                     [0, 0xFFFFFFFF, 0xFFFFFFFF]], dtype=np.uint32)
    out2, det2 = oracle.prune(knn2, 2, want_detour=True)
    assert det2[0].tolist() == [0, 0, 0] and out2[0].tolist() == [1, 2]


def test_reverse_and_merge_known_answer(oracle):
    g = np.array([[1, 2], [2, 0], [0, 3], [0, 1]], dtype=np.uint32)
    rev, cnt = oracle.reverse_graph(g)
    # column 0 first (sources ascending), then column 1: node 0 <- 2,3 (col0) then 1 (col1)
    assert cnt.tolist() == [3, 2, 2, 1]
    assert rev[0].tolist() == [2, 3]
    assert rev[1].tolist() == [0, 3]
    assert rev[2].tolist() == [1, 0]
    assert rev[3].tolist() == [2, 0xFFFFFFFF]
    merged = oracle.merge_graphs(g, rev, cnt)
    # node 0: orig 1, rev 2, (orig 2 dup) ... -> [1, 2]; node 3: orig 0, rev 2 -> [0, 2]
    assert merged[0].tolist() == [1, 2]
    assert merged[3].tolist() == [0, 2]
    # short row keeps its pruned tail (cagra.cu:641-648)
    g2 = np.array([[1, 1], [0, 0]], dtype=np.uint32)
    rev2, cnt2 = oracle.reverse_graph(g2)
    assert oracle.merge_graphs(g2, rev2, cnt2).tolist() == [[1, 1], [0, 0]]


def test_graph_search_restatement_recall(oracle):
    # a10/a11-style thresholds on a small clustered set: bucket search > 95 % with no
    # out-of-bucket ids (tests/test_cagra_opt_search_bucket.cu:234), range search high recall
    from conftest import clustered
    n, dim, deg = 4000, 32, 16
    data = clustered(n, dim, 20, 1.0, 11)
    rng = np.random.default_rng(12)
    q = data[rng.integers(0, n, 40)] + 0.05 * rng.standard_normal((40, dim)).astype(np.float32)
    knn = oracle.knn_block(data, 2 * deg)
    g = oracle.prune(knn, deg)
    rev, cnt = oracle.reverse_graph(g)
    g = oracle.merge_graphs(g, rev, cnt)
    gt, _ = oracle.exact_search(data, q, 10)
    seeds = rng.integers(0, n, size=(40, 32)).astype(np.uint32)
    ids, d = oracle.graph_search(data, g, q, 10, 64, 4, 30, 12, mode=0, seeds=seeds)
    assert oracle.recall(ids, gt) > 0.9            # tests/test_cagra_opt.cu:216 threshold
    assert np.all(np.diff(d, axis=1) >= 0)
    ts = np.arange(n, dtype=np.uint64)
    lo, hi = 1000, 3000
    gt_r, _ = oracle.exact_search(data, q, 10, ts=ts, lo=lo, hi=hi)
    seeds_r = rng.integers(lo, hi, size=(40, 32)).astype(np.uint32)
    ids_r, _ = oracle.graph_search(data, g, q, 10, 64, 4, 30, 12, mode=2, ts=ts, lo=lo, hi=hi, seeds=seeds_r)
    assert np.all((ids_r >= lo) & (ids_r < hi))
    assert oracle.recall(ids_r, gt_r) > 0.9


def test_insert_v1_restatement(oracle):
    deg, num_existing = 4, 6
    g = np.full((8, deg), 0xFFFFFFFF, dtype=np.uint32)
    g[:6] = np.array([[1, 2, 3, 4], [0, 2, 3, 4], [0, 1, 3, 4], [0, 1, 2, 4], [0, 1, 2, 3], [0, 1, 2, 3]])
    found = np.array([[0, 1, 2, 3, 4, 5, -1, 99], [2, 2, 0, 1, 3, 4, 5, -1]], dtype=np.int64)
    out = oracle.insert_v1(g, found, num_existing, 8)
    assert out[6].tolist() == [0, 1, 2, 3]          # first deg valid old ids (insert.cu:225-254)
    assert out[7].tolist() == [2, 2, 0, 1]
    for old in range(6):                              # every old node that was found links back
        assert 6 in out[old] or 7 in out[old]
    # protected first half is rarely touched, the row keeps its width
    assert out.shape == g.shape


def test_hnsw_baseline_restatement(oracle):
    # the CPU baseline harness of tests/test_faiss_hnsw_insert.cpp in miniature: build on the first
    # half, add the second half, search with efSearch 64, recall@10 against the exact scan
    from conftest import clustered
    n, dim = 6000, 32
    data = clustered(n, dim, 20, 1.0, 91)
    h = oracle.HNSW(data, M=32, ef_construction=128)
    h.add(n // 2)
    h.add(n - n // 2)
    rng = np.random.default_rng(92)
    q = data[rng.integers(0, n, 64)] + 0.05 * rng.standard_normal((64, dim)).astype(np.float32)
    ids, d = h.search(q, 10, ef=64)
    gt, _ = oracle.exact_search(data, q, 10)
    assert oracle.recall(ids, gt) > 0.95
    assert np.all(np.diff(d, axis=1) >= 0) and (ids >= 0).all()
