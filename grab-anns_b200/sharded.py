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


def sharded_search(search_fn, merge_fn, k: int, rank: int, world: int, dist_mod=None, group=None):
    """search_fn() -> (ids [nq,k] GLOBAL int64, dists [nq,k]) on this rank's shard."""
    ids, dists = search_fn()
    return gather_and_merge(dists, ids, k, merge_fn, dist_mod, group)
