"""Id-sharded search across the GPUs of one box (no counterpart in the single-GPU reference).

Vectors are striped by global id: rank r of G holds gid with gid % G == r as local id gid // G, so
every shard sees the same filter selectivity.  Each rank builds and searches its own shard
graph; queries are the same on every rank.  The per-shard top-k carry GLOBAL ids (the search
epilogue maps local -> local*G + r), are exchanged with one all_gather over NCCL and merged by
(dist, id) on the device -- the only data-path collective.  Because the key order is total, the
merged exact result is identical to the unsharded one, bit for bit.

The two compute steps are passed in as callables so that the host logic (striping, gather layout,
merge call) is testable on CPU ranks with the gloo backend.
"""
from __future__ import annotations

import numpy as np


def stripe(array, rank: int, world: int):
    """Rows of `array` owned by `rank` (gid % world == rank), in local-id order."""
    return array[rank::world]


def local_to_global(local_ids, rank: int, world: int):
    return np.where(np.asarray(local_ids) >= 0, np.asarray(local_ids) * world + rank, -1)


def gather_and_merge(dists, ids, k: int, merge_fn, dist_mod=None, group=None):
    """dists/ids: this rank's [nq, k] result with GLOBAL ids (torch tensors).  Returns the merged
    global [nq, k] on every rank.  merge_fn(dists [nq, G, k], ids [nq, G, k], k) -> (ids, dists)."""
    import torch
    if dist_mod is None:
        import torch.distributed as dist_mod
    world = dist_mod.get_world_size(group) if dist_mod.is_initialized() else 1
    if world == 1:
        return merge_fn(dists.unsqueeze(1).contiguous(), ids.unsqueeze(1).contiguous(), k)
    nq = dists.shape[0]
    all_d = torch.empty((world, nq, k), dtype=dists.dtype, device=dists.device)
    all_i = torch.empty((world, nq, k), dtype=ids.dtype, device=ids.device)
    if dists.is_cuda:  # NCCL: one collective per buffer, straight into the gather tensor
        dist_mod.all_gather_into_tensor(all_d, dists.contiguous(), group=group)
        dist_mod.all_gather_into_tensor(all_i, ids.contiguous(), group=group)
    else:              # gloo (CPU ranks in the tests) takes a list of per-rank views
        dist_mod.all_gather(list(all_d.unbind(0)), dists.contiguous(), group=group)
        dist_mod.all_gather(list(all_i.unbind(0)), ids.contiguous(), group=group)
    # [G, nq, k] -> [nq, G, k]: one ascending run per shard and query
    return merge_fn(all_d.transpose(0, 1).contiguous(), all_i.transpose(0, 1).contiguous(), k)


class HostSync:
    """Stream / event operations of run_pipelined for hosts without streams (CPU ranks in the tests): every call
    runs in program order, so there is nothing to wait for."""

    def searched(self, i):
        pass

    def wait_exchanged(self, i):
        pass

    def on_exchange_stream(self, fn, i):
        fn(i)

    def drain(self):
        pass

    def begin(self):
        import time
        self.t0 = time.perf_counter()

    def end(self):
        import time
        return (time.perf_counter() - self.t0) * 1e3


def run_pipelined(n_sets: int, steps: int, warmup: int, search, exchange, sync, barrier=None):
    """The step loop of the sharded search.  Step i searches into buffer set i % n_sets (search(set)) and hands the
    set to the exchange stream (exchange(set): the all-gather + merge); a set is searched into again only after its
    previous exchange has finished, so with two sets the exchange of step i overlaps the search of step i+1.
    Every rank issues exactly warmup + steps exchanges, whatever its timing -- the number of collectives must not
    depend on anything a rank measures locally.  Returns milliseconds per timed step (sync.end() / steps)."""
    used = [False] * n_sets
    count = 0

    def one():
        nonlocal count
        i = count % n_sets
        count += 1
        if used[i]:
            sync.wait_exchanged(i)
        search(i)
        sync.searched(i)
        sync.on_exchange_stream(exchange, i)
        used[i] = True

    for _ in range(warmup):
        one()
    sync.drain()
    if barrier is not None:
        barrier()
    sync.begin()
    for _ in range(steps):
        one()
    sync.drain()
    ms = sync.end()
    if barrier is not None:
        barrier()
    return ms / max(steps, 1)


def sharded_search(search_fn, merge_fn, k: int, rank: int, world: int, dist_mod=None, group=None):
    """search_fn() -> (ids [nq,k] GLOBAL int64, dists [nq,k]) on this rank's shard."""
    ids, dists = search_fn()
    return gather_and_merge(dists, ids, k, merge_fn, dist_mod, group)


def merge_topk_host(dists, ids, k: int):
    """CPU merge of per-shard ascending lists [nq, G, k] by (dist, id); ids < 0 are empty.  Same
    contract as grab_merge_topk (returns (ids, dists)); used when the results live in host memory."""
    import torch
    d = dists.detach().cpu().numpy() if hasattr(dists, "detach") else np.asarray(dists)
    i = ids.detach().cpu().numpy() if hasattr(ids, "detach") else np.asarray(ids)
    nq = d.shape[0]
    d = d.reshape(nq, -1).astype(np.float32)
    i = i.reshape(nq, -1).astype(np.int64)
    empty = i < 0
    dk = np.where(empty, np.float32(np.inf), d)
    ik = np.where(empty, np.iinfo(np.int64).max, i)
    order = np.lexsort((ik, dk), axis=1)[:, :k]           # primary dist, secondary id
    out_i = np.take_along_axis(i, order, axis=1)
    out_d = np.take_along_axis(d, order, axis=1)
    gone = np.take_along_axis(empty, order, axis=1)
    out_i[gone] = -1
    out_d[gone] = np.float32(3.40282e38)
    return torch.from_numpy(out_i), torch.from_numpy(out_d)


# ---------------------------------------------------------------------------------------------
# Sharded index on disk: one index file per rank in the reference's own format plus a manifest.
# ---------------------------------------------------------------------------------------------
MANIFEST_NAME = "manifest.json"
MANIFEST_VERSION = 1


def shard_file(directory: str, rank: int) -> str:
    import os
    return os.path.join(directory, f"shard_{rank:03d}.mcag")


def write_manifest(directory: str, world: int, shard_sizes, dim: int, graph_degree: int, local_degree: int,
                   metric: int = 0, bucket_width: int = 1, fmt: str = "MCAG"):
    """Written by rank 0 after every rank saved its shard: the striping rule and what each file holds."""
    import json
    import os
    shard_sizes = [int(s) for s in shard_sizes]
    if len(shard_sizes) != world:
        raise ValueError(f"{len(shard_sizes)} shard sizes for {world} ranks")
    m = {"version": MANIFEST_VERSION, "format": fmt, "striping": "gid % world == rank, local id = gid // world",
         "world": int(world), "total": int(sum(shard_sizes)), "shard_sizes": shard_sizes, "dim": int(dim),
         "graph_degree": int(graph_degree), "local_degree": int(local_degree), "metric": int(metric),
         "bucket_width": int(bucket_width),
         "files": [os.path.basename(shard_file(directory, r)) for r in range(world)]}
    tmp = os.path.join(directory, MANIFEST_NAME + ".tmp")
    with open(tmp, "w") as fh:
        json.dump(m, fh, indent=1)
    os.replace(tmp, os.path.join(directory, MANIFEST_NAME))
    return m


def read_manifest(directory: str, world: int | None = None):
    """Loads and checks a manifest; `world` = the number of ranks that want to load it."""
    import json
    import os
    path = os.path.join(directory, MANIFEST_NAME)
    with open(path) as fh:
        m = json.load(fh)
    if m.get("version") != MANIFEST_VERSION:
        raise ValueError(f"{path}: manifest version {m.get('version')} is not {MANIFEST_VERSION}")
    if world is not None and m["world"] != world:
        raise ValueError(f"{path}: written by {m['world']} ranks, loaded by {world} (ids are striped by "
                         "gid % world, so the rank count must match)")
    if len(m["shard_sizes"]) != m["world"] or sum(m["shard_sizes"]) != m["total"]:
        raise ValueError(f"{path}: shard sizes do not add up to the total")
    sizes = m["shard_sizes"]
    want = [len(range(r, m["total"], m["world"])) for r in range(m["world"])]
    if sizes != want:
        raise ValueError(f"{path}: shard sizes {sizes} are not a gid % world striping of {m['total']} vectors")
    for f in m["files"]:
        if not os.path.exists(os.path.join(directory, f)):
            raise FileNotFoundError(os.path.join(directory, f))
    return m


class ShardedIndex:
    """One time-partitioned index per rank over the stripe gid % world == rank.

    `make_index()` returns the per-rank index (index.CagraIndexOpt in production; anything with
    add / build / insert / query_range_batch / save / load / size in the tests).  Queries are the
    same on every rank; results carry global ids and are identical on every rank.  `merge_fn` /
    `to_tensor` default to the host merge on CPU tensors (gloo); with NCCL pass
    merge_fn=grab.merge_topk and to_tensor=lambda a: torch.from_numpy(a).cuda()."""

    def __init__(self, make_index, rank: int, world: int, dist_mod=None, group=None, merge_fn=None,
                 to_tensor=None):
        import torch
        self.index = make_index()
        self.rank, self.world = rank, world
        self.dist_mod, self.group = dist_mod, group
        self.merge_fn = merge_fn or merge_topk_host
        self.to_tensor = to_tensor or (lambda a: torch.from_numpy(np.ascontiguousarray(a)))
        self.total = 0

    def add_and_build(self, vectors, timestamps):
        """vectors / timestamps: the GLOBAL arrays (the same on every rank); this rank keeps its stripe."""
        self.index.add(np.ascontiguousarray(stripe(vectors, self.rank, self.world)),
                       np.ascontiguousarray(stripe(timestamps, self.rank, self.world)))
        self.index.build()
        self.total = int(vectors.shape[0])

    def insert(self, vectors, timestamps):
        """New vectors get the global ids total, total+1, ...; each rank inserts those of its residue."""
        first = self.total
        start = (self.rank - first) % self.world          # first new row owned by this rank
        mine_v, mine_t = vectors[start::self.world], timestamps[start::self.world]
        if mine_v.shape[0]:
            self.index.insert(np.ascontiguousarray(mine_v), np.ascontiguousarray(mine_t))
        self.total += int(vectors.shape[0])

    def query_range_batch(self, queries, k: int, lo, hi):
        ids, dists = self.index.query_range_batch(queries, k, lo, hi)
        gids = local_to_global(ids, self.rank, self.world).astype(np.int64)
        out_ids, out_d = gather_and_merge(self.to_tensor(dists.astype(np.float32)), self.to_tensor(gids), k,
                                          self.merge_fn, self.dist_mod, self.group)
        return out_ids.cpu().numpy(), out_d.cpu().numpy()

    def save(self, directory: str, dim: int, graph_degree: int, local_degree: int, metric: int = 0,
             bucket_width: int = 1):
        import os
        os.makedirs(directory, exist_ok=True)
        self.index.save(shard_file(directory, self.rank))
        self._barrier()
        if self.rank == 0:
            sizes = [len(range(r, self.total, self.world)) for r in range(self.world)]
            write_manifest(directory, self.world, sizes, dim, graph_degree, local_degree, metric, bucket_width)
        self._barrier()

    def load(self, directory: str):
        m = read_manifest(directory, self.world)
        self.index.load(shard_file(directory, self.rank))
        if int(self.index.size()) != m["shard_sizes"][self.rank]:
            raise ValueError(f"shard {self.rank} holds {self.index.size()} vectors, the manifest says "
                             f"{m['shard_sizes'][self.rank]}")
        self.total = m["total"]
        return m

    def _barrier(self):
        d = self.dist_mod
        if d is None:
            import torch.distributed as d
        if d.is_initialized() and d.get_world_size(self.group) > 1:
            d.barrier(group=self.group)
