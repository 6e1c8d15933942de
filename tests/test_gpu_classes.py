"""The three index classes, exercised the way the reference's own test executables do
(thresholds from those files), through the C handle API.  Needs a B200."""
import importlib
import os

import numpy as np
import pytest

from conftest import clustered

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def index_mod():
    return importlib.import_module("grab-anns_b200.index")


def _gt(grab, data, q, k, ts=None, lo=None, hi=None):
    import torch
    d, qq = torch.from_numpy(data).cuda(), torch.from_numpy(q).cuda()
    flt = None
    if ts is not None:
        flt = grab.make_filter(grab.FILTER_TS_RANGE, ts=torch.from_numpy(ts.view(np.int64)).cuda(), lo=lo, hi=hi)
    return grab.exact_search(d, qq, k, flt=flt)[0].cpu().numpy()


def test_opt_bucket_and_range_search(grab, oracle, index_mod):
    # tests/test_cagra_opt_search_bucket.cu: 4 buckets x 10 000, query_local, recall@10 > 95 %, 0 out-of-bucket ids
    nb, per, dim, k = 4, 10000, 64, 10
    data = clustered(nb * per, dim, 24, 1.0, 71)
    ts = np.repeat(np.arange(nb, dtype=np.uint64), per)
    idx = index_mod.CagraIndexOpt(dim, 32, 24)
    idx.add(data, ts)
    idx.build()
    assert idx.size() == nb * per
    g = idx.get_graph()
    blk = np.arange(nb * per) // per
    assert ((g[:, :24] // per == blk[:, None]) | (g[:, :24] == 0xFFFFFFFF)).all()   # local columns stay in the bucket
    rng = np.random.default_rng(72)
    q = data[rng.integers(0, nb * per, 320)] + 0.1 * rng.standard_normal((320, dim)).astype(np.float32)
    idx.set_query_params(128, 4, 0, 50, 13)
    for b in range(nb):
        ids, d = idx.query_local(q, k, b)
        assert ((ids >= b * per) & (ids < (b + 1) * per)).all()                      # bound errors == 0
        gt = _gt(grab, data, q, k, ts, b, b + 1)
        assert oracle.recall(ids, gt) > 0.95
        assert np.all(np.diff(d, axis=1) >= 0)
    # unfiltered query over the partitioned graph: remote edges connect the buckets
    # (tests/test_cagra_opt.cu:216, recall@10 > 90 %)
    ids, _ = idx.query(q, k)
    assert oracle.recall(ids, _gt(grab, data, q, k)) > 0.9
    # range search over buckets [1,3) (tests/test_cagra_opt_search_range.cu)
    ids, _ = idx.query_range(q, k, 1, 3)
    assert ((ids >= per) & (ids < 3 * per)).all()
    assert oracle.recall(ids, _gt(grab, data, q, k, ts, 1, 3)) > 0.95
    # empty range -> -1 / -1.0f (src/cagraIndexOpt.cu:479-485); missing bucket likewise
    ids, d = idx.query_range(q[:4], k, 9, 12)
    assert (ids == -1).all() and (d == -1.0).all()
    ids, d = idx.query_local(q[:4], k, 77)
    assert (ids == -1).all() and (d == -1.0).all()


@pytest.mark.parametrize("repair_mode", [0, 1, 2])
def test_opt_insert_then_search(grab, oracle, index_mod, tmp_path, repair_mode):
    # tests/test_cagra_opt_insert.cu: build on the first half of every bucket, insert the second
    # half; global recall > 90 %, local > 95 %, 0 bound errors (:359-360).  Both reverse-edge rules: the
    # reference's slot rule and the distance-aware repair.
    nb, per, dim, k = 4, 6000, 64, 10
    data = clustered(nb * per, dim, 24, 1.0, 73).reshape(nb, per, dim)
    half = per // 2
    idx = index_mod.CagraIndexOpt(dim, 32, 24, insert_batch=256)
    idx.set_insert_mode(routed=False, repair_mode=repair_mode)
    first = data[:, :half].reshape(-1, dim)
    idx.add(first, np.repeat(np.arange(nb, dtype=np.uint64), half))
    idx.build()
    for b in range(nb):
        idx.insert(data[b, half:], np.full(per - half, b, dtype=np.uint64))
    assert idx.size() == nb * per
    allv = np.concatenate([first] + [data[b, half:] for b in range(nb)])
    ts = np.concatenate([np.repeat(np.arange(nb, dtype=np.uint64), half)] +
                        [np.full(per - half, b, dtype=np.uint64) for b in range(nb)])
    g = idx.get_graph()
    assert not (g == np.arange(nb * per, dtype=np.uint32)[:, None]).any()             # no self loops
    assert (g[nb * half:, 0] != 0xFFFFFFFF).all()                                     # inserted rows are linked
    rng = np.random.default_rng(74)
    q = allv[rng.integers(0, nb * per, 256)] + 0.1 * rng.standard_normal((256, dim)).astype(np.float32)
    idx.set_query_params(128, 4, 0, 50, 13)
    ids, _ = idx.query(q, k)
    assert oracle.recall(ids, _gt(grab, allv, q, k)) > 0.90
    for b in (0, nb - 1):
        ids, _ = idx.query_local(q, k, b)
        assert (ts[ids] == b).all()                                                   # 0 bound errors
        assert oracle.recall(ids, _gt(grab, allv, q, k, ts, b, b + 1)) > 0.95
    # save / load round trip in the reference's "MCAG" layout
    io = importlib.import_module("grab-anns_b200.io")
    path = os.path.join(tmp_path, "opt.idx")
    idx.save(path)
    head = io.read_index_header(path)
    assert head == {"format": "CagraIndexOpt", "version": 1, "dim": dim, "graph_degree": 32, "local_degree": 24,
                    "size": nb * per}
    idx2 = index_mod.CagraIndexOpt(dim, 32, 24)
    idx2.load(path)
    idx2.set_query_params(128, 4, 0, 50, 13)
    assert np.array_equal(idx2.get_graph(), g)
    # one CTA per query is the deterministic walk (several co-operating CTAs race for nodes, so which of them
    # lists a node, and with it the tail of a result, can change from call to call)
    idx.set_small_batch_mode(1)
    idx2.set_small_batch_mode(1)
    ids2, _ = idx2.query_local(q, k, 0)
    assert np.array_equal(ids2, idx.query_local(q, k, 0)[0])


@pytest.mark.parametrize("reference_rules", [False, True])
def test_opt_streaming_insert_holds_recall(grab, oracle, index_mod, reference_rules):
    """The streaming shape of tests/test_cagra_opt_insert_auto.cu:199-204 in small: build, then batches with
    increasing timestamps, after each batch range queries over the newest 20 %.  Thresholds of
    tests/test_cagra_opt_insert.cu:359-360 (0 bound errors, recall floors); with routed inserts and the
    distance-aware repair (the class default) recall@10 must stay >= 0.95 after every batch."""
    import torch
    n0, nb, bn, dim, k = 24000, 4, 6000, 96, 10
    total = n0 + nb * bn
    data = clustered(total, dim, 40, 0.6, 81)
    ts = np.arange(total, dtype=np.uint64)
    idx = index_mod.CagraIndexOpt(dim, 32, 24, bucket_width=3000, insert_batch=2048)
    idx.set_router(128, 2, 64)
    idx.set_query_params(64, 3, 0, 8, 11)
    if reference_rules:
        idx.set_insert_mode(routed=False, repair_mode=0)
    idx.add(data[:n0], ts[:n0])
    idx.build()
    rng = np.random.default_rng(82)
    size = n0
    for b in range(nb):
        idx.insert(data[size:size + bn], ts[size:size + bn])
        size += bn
        assert idx.size() == size
        q = data[rng.integers(0, size, 400)] + 0.05 * rng.standard_normal((400, dim)).astype(np.float32)
        lo = np.full(400, size - size // 5, dtype=np.uint64)
        hi = np.full(400, size, dtype=np.uint64)
        ids, _ = idx.query_range_batch(q, k, lo, hi)
        assert (((ids >= int(lo[0])) & (ids < size)) | (ids < 0)).all()                  # 0 bound errors
        gt = _gt(grab, data[:size], q, k, ts[:size], int(lo[0]), size)
        rec = oracle.recall(ids, gt)
        assert rec > (0.90 if reference_rules else 0.95), (b, rec)
    g = idx.get_graph()
    assert not (g == np.arange(size, dtype=np.uint32)[:, None]).any()                   # no self loops
    assert (g[n0:, 0] != 0xFFFFFFFF).all()                                              # inserted rows are linked
    assert int(g[g != 0xFFFFFFFF].max()) < size


def test_opt_per_query_ranges_with_bucket_width(grab, oracle, index_mod):
    # timestamps = insertion index, buckets of 2 500 timestamps, one range per query
    n, dim, k = 20000, 64, 10
    data = clustered(n, dim, 24, 1.0, 75)
    ts = np.arange(n, dtype=np.uint64)
    idx = index_mod.CagraIndexOpt(dim, 32, 24, bucket_width=2500)
    idx.add(data, ts)
    idx.build()
    idx.set_query_params(64, 4, 0, 40, 12)
    rng = np.random.default_rng(76)
    q = data[rng.integers(0, n, 200)] + 0.1 * rng.standard_normal((200, dim)).astype(np.float32)
    lo = rng.integers(0, n - 5000, 200).astype(np.uint64)
    hi = lo + 5000
    ids, d = idx.query_range_batch(q, k, lo, hi)
    assert ((ids >= lo[:, None]) & (ids < hi[:, None])).all()
    import torch
    gt = grab.exact_search(torch.from_numpy(data).cuda(), torch.from_numpy(q).cuda(), k,
                           flt=grab.make_filter(grab.FILTER_TS_RANGE, ts=torch.from_numpy(ts.view(np.int64)).cuda(),
                                                lo=torch.from_numpy(lo.view(np.int64)).cuda(),
                                                hi=torch.from_numpy(hi.view(np.int64)).cuda()))[0].cpu().numpy()
    assert oracle.recall(ids, gt) > 0.95


def test_opt_router_on_separated_clusters_and_after_insert(grab, oracle, index_mod):
    """Well-separated clusters, short searches: with uniformly drawn seeds most queries never reach
    their cluster; the class's entry-point router (default on) starts inside it.  Inserted vectors
    join the member lists on the next query."""
    import torch
    n, extra, dim, k = 24000, 4000, 64, 10
    data = clustered(n + extra, dim, 120, 0.15, 81)
    ts = np.arange(n + extra, dtype=np.uint64)
    rng = np.random.default_rng(82)

    def recall_of(idx, upto):
        q = data[rng.integers(0, upto, 200)] + np.float32(0.01)
        lo = rng.integers(0, upto - upto // 4, 200).astype(np.uint64)
        hi = lo + np.uint64(upto // 4)
        ids, _ = idx.query_range_batch(q, k, lo, hi)
        assert (((ids >= lo[:, None]) & (ids < hi[:, None])) | (ids < 0)).all()
        f = grab.make_filter(grab.FILTER_TS_RANGE, ts=torch.from_numpy(ts[:upto].view(np.int64)).cuda(),
                             lo=torch.from_numpy(lo.view(np.int64)).cuda(), hi=torch.from_numpy(hi.view(np.int64)).cuda())
        gt = grab.exact_search(torch.from_numpy(data[:upto]).cuda(), torch.from_numpy(q).cuda(), k, flt=f)[0]
        return oracle.recall(ids, gt.cpu().numpy())

    idx = index_mod.CagraIndexOpt(dim, 32, 24, bucket_width=4000)
    idx.add(data[:n], ts[:n])
    idx.build()
    idx.set_query_params(64, 2, 0, 8, 11)
    idx.set_router(0)
    r_off = recall_of(idx, n)
    idx.set_router()                       # automatic size, the default
    r_on = recall_of(idx, n)
    assert r_on > 0.95 and r_on > r_off + 0.1, (r_off, r_on)
    idx.insert(data[n:], ts[n:])
    r_ins = recall_of(idx, n + extra)
    assert r_ins > 0.9, r_ins


def test_cagra_index_build_insert_range_save(grab, oracle, index_mod, tmp_path):
    # tests/test_cagra_insert.cu: build 50 %, insert 50 % in batches of 64, recall@10 > 90 % (:284)
    # tests/test_cagra_auto.cu: query_range at several ratios against the exact filtered ground truth
    n, dim, k = 16000, 64, 10
    data = clustered(n, dim, 16, 1.0, 77)
    ts = (np.arange(n) // 160).astype(np.uint64)                  # 100 buckets, like test_cagra_auto.cu
    idx = index_mod.CagraIndex(dim, 32)
    idx.add(data[:n // 2], ts[:n // 2])
    idx.build()
    idx.insert(data[n // 2:], ts[n // 2:])
    assert idx.size() == n
    rng = np.random.default_rng(78)
    q = data[rng.integers(0, n, 200)] + 0.1 * rng.standard_normal((200, dim)).astype(np.float32)
    idx.set_query_params(128, 4, 0, 50, 13)
    ids, d = idx.query(q, k)
    assert oracle.recall(ids, _gt(grab, data, q, k)) > 0.90
    for ratio in (0.1, 0.2, 1.0):
        end = int(100 * ratio)
        ids, _ = idx.query_range(q, k, ratio, 0, end)
        if ratio < 0.99:
            assert (ts[ids] < end).all()
        gt = _gt(grab, data, q, k, ts, 0, end)
        assert oracle.recall(ids, gt) > 0.85
    io = importlib.import_module("grab-anns_b200.io")
    path = os.path.join(tmp_path, "plain.idx")
    idx.save(path)
    assert io.read_index_header(path) == {"format": "CagraIndex", "dim": dim, "graph_degree": 32, "size": n}
    assert os.path.getsize(path) == 16 + n * dim * 4 + n * 32 * 4
    idx2 = index_mod.CagraIndex(dim, 32)
    idx2.load(path)
    idx2.set_query_params(128, 4, 0, 50, 13)
    idx.set_small_batch_mode(1)      # the deterministic one-CTA walk on both sides
    idx2.set_small_batch_mode(1)
    assert np.array_equal(idx2.query(q, k)[0], idx.query(q, k)[0])


def test_timestamp_index_routed_search(grab, oracle, index_mod):
    # tests/test_timestamp_index.cu: insert -> build_virtual_index -> routed query, recall@20 > 85 % (:263)
    nb, per, dim, topk = 5, 4000, 32, 20
    data = clustered(nb * per, dim, 10, 1.0, 79)
    ts = np.repeat(np.arange(100, 100 + nb, dtype=np.uint64), per)
    tsi = index_mod.TimeStampIndex(dim, 32)
    first = tsi.insert(data[:nb * per // 2], ts[:nb * per // 2])
    second = tsi.insert(data[nb * per // 2:], ts[nb * per // 2:])
    assert first == 0 and second == nb * per // 2 and tsi.size() == nb * per
    tsi.build_virtual_index()
    rng = np.random.default_rng(80)
    qs = data[rng.integers(0, nb * per, 40)] + 0.05 * rng.standard_normal((40, dim)).astype(np.float32)
    gt = _gt(grab, data, qs, topk)
    hit = 0
    for i, q in enumerate(qs):
        ids, d = tsi.query(q, topk, probe_buckets=5)
        hit += len(set(ids[ids >= 0].tolist()) & set(gt[i].tolist()))
    assert hit / (40 * topk) > 0.85
    ids, d = tsi.query_by_timestamp(qs[0], topk, 102)
    assert ((ids >= 2 * per) & (ids < 3 * per)).all()
    ids, d = tsi.query_by_timestamp(qs[0], topk, 999)
    assert (ids == -1).all()


def test_handles_are_bound_to_their_device(grab, oracle, index_mod):
    """A handle made with *_create_on(device) runs every call on that GPU and leaves the caller's current device
    alone; with two GPUs the index lives on the second while the first stays current."""
    import torch
    ngpu = torch.cuda.device_count()
    target = 1 if ngpu >= 2 else 0
    torch.cuda.set_device(0)
    n, dim, nb, k = 12000, 64, 4, 10
    data = clustered(n, dim, 24, 1.0, 81)
    ts = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info(0)[0]
    idx = index_mod.CagraIndexOpt(dim, 32, 24, device=target)
    idx.add(data, ts)
    idx.build()
    assert torch.cuda.current_device() == 0
    if ngpu >= 2:   # the index's memory is on the second GPU: the first one holds none of it
        assert free0 - torch.cuda.mem_get_info(0)[0] < (32 << 20)
    rng = np.random.default_rng(82)
    q = data[rng.integers(0, n, 128)] + 0.1 * rng.standard_normal((128, dim)).astype(np.float32)
    idx.set_query_params(128, 4, 0, 50, 13)
    ids, _ = idx.query_range(q, k, 1, 3)
    assert torch.cuda.current_device() == 0
    assert ((ts[ids] >= 1) & (ts[ids] < 3)).all()
    gt, _ = oracle.exact_search(data, q, k, ts=ts, lo=np.full(128, 1, np.uint64), hi=np.full(128, 3, np.uint64))
    assert oracle.recall(ids, gt) > 0.95
    with pytest.raises(Exception):
        index_mod.CagraIndexOpt(dim, 32, 24, device=ngpu + 7)   # no such GPU: a status, not a crash
