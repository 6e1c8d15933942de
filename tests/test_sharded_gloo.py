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
