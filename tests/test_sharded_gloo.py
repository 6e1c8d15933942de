"""Host logic of the id-sharded search on two CPU ranks (gloo): striping, global-id mapping,
all_gather layout and the merge.  The per-shard search and the merge are the CPU oracle here; on
the GPU they are graph_search / exact_search and grab_merge_topk."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import torch.distributed as dist
    import oracle
    sharded = importlib.import_module("grab-anns_b200.sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)                       # same data on every rank
    n, dim, nq, k = 6001, 32, 24, 10                      # n not divisible by the world size
    data = rng.standard_normal((n, dim)).astype(np.float32)
    data[100:104] = data[100]                             # equal distances across shards -> id tie-break
    q = np.concatenate([data[100:101], rng.standard_normal((nq - 1, dim)).astype(np.float32)])
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n - 1500, nq).astype(np.uint64)
    lo[0] = 0
    hi = lo + 1500
    shard, shard_ts = sharded.stripe(data, rank, world), sharded.stripe(ts, rank, world)
    assert shard.shape[0] == len(range(rank, n, world))

    def search():
        ids, d = oracle.exact_search(shard, q, k, ts=shard_ts, lo=lo, hi=hi)
        return torch.from_numpy(sharded.local_to_global(ids, rank, world)), torch.from_numpy(d)

    def merge(d, i, kk):
        oi, od = oracle.merge_topk(d.numpy(), i.numpy(), kk)
        return torch.from_numpy(oi), torch.from_numpy(od)

    ids, d = sharded.sharded_search(search, merge, k, rank, world)
    want_ids, want_d = oracle.exact_search(data, q, k, ts=ts, lo=lo, hi=hi)
    ok = np.array_equal(ids.numpy(), want_ids) and np.array_equal(d.numpy(), want_d)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_rank_sharded_exact_search_is_bit_exact(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_striping_and_id_mapping():
    sharded = importlib.import_module("grab-anns_b200.sharded")
    gids = np.arange(23)
    seen = []
    for r in range(4):
        loc = sharded.stripe(gids, r, 4)
        back = sharded.local_to_global(np.arange(loc.size), r, 4)
        assert np.array_equal(back, loc)
        seen += back.tolist()
    assert sorted(seen) == list(range(23))
    assert sharded.local_to_global(np.array([-1, 2]), 1, 4).tolist() == [-1, 9]


# ------------------------------------------------------------------ sharded index + manifest
class _BruteIndex:
    """Stand-in for index.CagraIndexOpt on CPU ranks: exact filtered search by the oracle."""

    def __init__(self, dim):
        self.dim = dim
        self.data = np.zeros((0, dim), np.float32)
        self.ts = np.zeros(0, np.uint64)

    def add(self, v, t):
        self.data = np.concatenate([self.data, v.astype(np.float32)])
        self.ts = np.concatenate([self.ts, t.astype(np.uint64)])

    insert = add

    def build(self):
        pass

    def size(self):
        return self.data.shape[0]

    def query_range_batch(self, q, k, lo, hi):
        import oracle
        return oracle.exact_search(self.data, q, k, ts=self.ts, lo=lo, hi=hi)

    def save(self, path):
        np.savez(path + ".npz", data=self.data, ts=self.ts)
        open(path, "wb").close()

    def load(self, path):
        z = np.load(path + ".npz")
        self.data, self.ts = z["data"], z["ts"]


def _index_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch.distributed as dist
    import oracle
    sharded = importlib.import_module("grab-anns_b200.sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(9)
    n, extra, dim, nq, k = 3001, 500, 16, 16, 8
    data = rng.standard_normal((n + extra, dim)).astype(np.float32)
    ts = np.arange(n + extra, dtype=np.uint64)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    lo = rng.integers(0, n - 800, nq).astype(np.uint64)
    hi = lo + 1200
    idx = sharded.ShardedIndex(lambda: _BruteIndex(dim), rank, world)
    idx.add_and_build(data[:n], ts[:n])
    ok = True
    ids, d = idx.query_range_batch(q, k, lo, hi)
    wi, wd = oracle.exact_search(data[:n], q, k, ts=ts[:n], lo=lo, hi=hi)
    ok &= np.array_equal(ids, wi) and np.array_equal(d, wd)
    idx.insert(data[n:n + 250], ts[n:n + 250])            # an odd count: the residues shift between batches
    idx.insert(data[n + 250:], ts[n + 250:])
    ids, d = idx.query_range_batch(q, k, lo + 1500, hi + 2000)
    wi, wd = oracle.exact_search(data, q, k, ts=ts, lo=lo + 1500, hi=hi + 2000)
    ok &= np.array_equal(ids, wi) and np.array_equal(d, wd)
    shard_dir = os.path.join(out_dir, "index")
    idx.save(shard_dir, dim, 32, 24)
    again = sharded.ShardedIndex(lambda: _BruteIndex(dim), rank, world)
    m = again.load(shard_dir)
    ok &= m["total"] == n + extra and m["world"] == world
    ids2, _ = again.query_range_batch(q, k, lo + 1500, hi + 2000)
    ok &= np.array_equal(ids2, wi)
    try:
        sharded.read_manifest(shard_dir, world + 1)
        ok = False
    except ValueError:
        pass
    with open(os.path.join(out_dir, f"idx{rank}.txt"), "w") as fh:
        fh.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_rank_sharded_index_insert_save_load(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_index_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"idx{r}.txt").read_text() == "ok"


def test_host_merge_matches_oracle():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    sharded = importlib.import_module("grab-anns_b200.sharded")
    rng = np.random.default_rng(3)
    nq, parts, k = 20, 3, 6
    d = np.sort(rng.integers(0, 5, (nq, parts, k)).astype(np.float32), axis=2)      # many equal distances
    i = rng.permutation(nq * parts * k).reshape(nq, parts, k).astype(np.int64)
    i[:, 1, 4:] = -1                                                                 # short lists
    i[3] = -1
    # inside a list equal distances must come in ascending id order (the merge's precondition)
    for a in range(nq):
        for b in range(parts):
            valid = i[a, b] >= 0
            order = np.lexsort((i[a, b][valid], d[a, b][valid]))
            d[a, b][:valid.sum()], i[a, b][:valid.sum()] = d[a, b][valid][order], i[a, b][valid][order]
            d[a, b][valid.sum():], i[a, b][valid.sum():] = 3.40282e38, -1
    hi_, hd = sharded.merge_topk_host(d, i, k)
    oi, od = oracle.merge_topk(d, i, k)
    assert np.array_equal(hi_.numpy(), oi) and np.array_equal(hd.numpy(), od)


def test_manifest_validation(tmp_path):
    sharded = importlib.import_module("grab-anns_b200.sharded")
    d = str(tmp_path)
    for r in range(3):
        open(sharded.shard_file(d, r), "wb").close()
    sharded.write_manifest(d, 3, [4, 3, 3], 64, 32, 24)
    assert sharded.read_manifest(d, 3)["total"] == 10
    with pytest.raises(ValueError):
        sharded.write_manifest(d, 3, [4, 3], 64, 32, 24)
    sharded.write_manifest(d, 3, [3, 4, 3], 64, 32, 24)      # not a gid % world striping
    with pytest.raises(ValueError):
        sharded.read_manifest(d, 3)
    sharded.write_manifest(d, 3, [4, 3, 3], 64, 32, 24)
    os.remove(sharded.shard_file(d, 2))
    with pytest.raises(FileNotFoundError):
        sharded.read_manifest(d, 3)


# ------------------------------------------------------------------ step loop of the sharded benchmark
def _loop_worker(rank, world, port, out_dir):
    """Walks the step structure bench.py uses for the sharded path (sharded.run_pipelined) with a counting stub:
    a rank-dependent number of collective-free load steps first (the clock-sampling loop), then warm-up + timed
    pipelined steps with one all_gather each.  Every rank must issue the same number of collectives."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    sharded = importlib.import_module("grab-anns_b200.sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nq, kp, steps, warmup = 16, 4, 5, 3
    counts = {"search": 0, "collectives": 0}
    keys = [torch.zeros((nq, kp), dtype=torch.int64) for _ in range(2)]
    merged = [None, None]

    def search(i):
        counts["search"] += 1
        # ascending runs whose content depends on the step and the rank
        keys[i] = (torch.arange(nq * kp, dtype=torch.int64).reshape(nq, kp) * world + rank) + 1000 * counts["search"]

    def exchange(i):
        counts["collectives"] += 1
        out = [torch.empty_like(keys[i]) for _ in range(world)]
        dist.all_gather(out, keys[i])
        merged[i] = torch.sort(torch.cat(out, dim=1), dim=1)[0][:, :kp]

    for _ in range(1 + 3 * rank):        # the load loop runs a rank-dependent number of times: no collective in it
        search(0)
    counts["search"] = 0
    ms = sharded.run_pipelined(2, steps, warmup, search, exchange, sharded.HostSync(), barrier=dist.barrier)
    mine = torch.tensor([counts["collectives"], counts["search"]], dtype=torch.int64)
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    same_counts = all(torch.equal(e, every[0]) for e in every)
    last = merged[(steps + warmup - 1) % 2]
    ref = [torch.empty_like(last) for _ in range(world)]
    dist.all_gather(ref, last)
    same_result = all(torch.equal(r_, ref[0]) for r_ in ref)
    ok = same_counts and same_result and counts["collectives"] == steps + warmup and ms >= 0
    with open(os.path.join(out_dir, f"loop{rank}.txt"), "w") as fh:
        fh.write("ok" if ok else f"mismatch {counts} {same_counts} {same_result}")
    dist.destroy_process_group()


def test_two_rank_pipelined_loop_issues_equal_collectives(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_loop_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"loop{r}.txt").read_text() == "ok"
