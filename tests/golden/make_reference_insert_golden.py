"""Golden vectors from the reference's OWN insert kernels (src/index/insert.cu).

Runs on a machine with a B200 after `make -C oracle ref` built oracle/_ref/libgrab_ref.so from the
reference's sources.  Inputs are regenerated from seeds (the same code the CPU test uses); only the
kernels' outputs are stored, graphs as XOR against the seeded input graph so that untouched rows
compress to nothing.  Usage: python tests/golden/make_reference_insert_golden.py OUT.npz

What is stored, and why in stages: update_topology_gpu_v1 (insert.cu:372-440) is deterministic, its
final graph is stored whole.  update_topology_gpu_opt (:1398-1573) posts requests with atomicAdd
(:579-640), so the order inside a mailbox -- and, past its capacity, which senders survive -- is a race.
Stored are therefore (1) the fill kernel's rows and consumed candidate lists (deterministic), (2) the
request counts and each mailbox as a sorted list, (3) the apply kernel's graph when it is handed
mailboxes in ascending (new id, column) order, the order the CPU restatement and the new CUDA code fix,
and (4) the graph of the whole racy function for property checks.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

INVALID = 0xFFFFFFFF
V1_CASES = [  # (num_existing, num_new, degree, search_k, seed)
    (2000, 200, 16, 32, 301),
    (1500, 96, 64, 128, 302),     # degree > 32: the fill kernel's 64-thread block (insert.cu:386)
]
OPT_CASES = [  # (num_existing, num_new, total_degree, local_degree, k_local, k_global, buckets, seed)
    (3000, 256, 16, 10, 24, 24, 30, 311),
    (2400, 200, 32, 24, 48, 32, 60, 312),   # 60 buckets: both sides of the |bucket delta| <= 20 rule (:737)
]


def v1_inputs(case):
    ne, nn, deg, sk, seed = case
    rng = np.random.default_rng(seed)
    g = np.full((ne + nn, deg), INVALID, dtype=np.uint32)
    g[:ne] = rng.integers(0, ne, size=(ne, deg))
    hot = ne // 8                                   # few targets, many requests each
    found = rng.integers(0, hot, size=(nn, sk)).astype(np.int64)
    found[::7, -3:] = -1                            # missing results
    found[::5, 1] = ne + rng.integers(0, nn, size=found[::5].shape[0])   # a new node's id: not a valid target
    found[::3, 4] = found[::3, 2]                   # the same target twice from one source
    # a source that is already a neighbour of its target (the kernel's duplicate test, insert.cu:327-333)
    for i in range(0, nn, 11):
        t = int(found[i, 0])
        if 0 <= t < ne:
            g[t, 3] = ne + i
    return g, found


def opt_inputs(case):
    ne, nn, total, local, kl, kg, nb, seed = case
    rng = np.random.default_rng(seed)
    bucket = np.concatenate([np.sort(rng.integers(0, nb, size=ne)).astype(np.uint64),
                             np.full(nn, nb - 1, dtype=np.uint64)])
    g = np.full((ne + nn, total), INVALID, dtype=np.uint32)
    g[:ne] = rng.integers(0, ne, size=(ne, total))
    same = np.flatnonzero(bucket[:ne] == nb - 1)
    pool = np.concatenate([same, np.arange(ne, ne + nn)])          # own bucket: old members and the batch itself
    lk = np.stack([rng.choice(pool, size=kl, replace=False) for _ in range(nn)]).astype(np.int64)
    lk[::13, 2] = rng.integers(0, max(1, same[0]), size=lk[::13].shape[0])   # another bucket: rejected (:495-499)
    lk[::17, 0] = ne + np.arange(0, nn, 17)                                 # the node itself: skipped (:486)
    hot = max(8, ne // 6)
    gk = rng.integers(0, hot, size=(nn, kg)).astype(np.int64)               # hot targets: remote mailboxes overflow
    far = rng.integers(0, ne, size=(nn, kg)).astype(np.int64)
    gk = np.where(rng.random((nn, kg)) < 0.5, gk, far)
    gk[::6, 3] = -1
    gk[::4, 1] = lk[::4, 5]                                                 # already a local neighbour (:536-543)
    gk[::9, 0] = rng.choice(same, size=gk[::9].shape[0])                    # own bucket: only the back-fill takes it
    return g, bucket, lk, gk


def _sorted_lists(cnt, lst):
    """Every mailbox as an ascending list of what it holds (entries past min(count, capacity) -> 0xFFFFFFFF)."""
    cnt = np.asarray(cnt).astype(np.int64)
    lst = np.asarray(lst).view(np.uint32).copy() if lst.dtype != np.uint32 else np.array(lst, copy=True)
    cap = lst.shape[1]
    if cap == 0:
        return lst
    col = np.arange(cap)[None, :]
    lst[col >= np.minimum(cnt, cap)[:, None]] = INVALID
    return np.sort(lst, axis=1)


def main(out):
    import torch
    import oracle
    import ref_kernels
    if not ref_kernels.available():
        raise SystemExit("oracle/_ref/libgrab_ref.so is missing: run `make -C oracle ref` where the reference is")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    u32 = lambda x: x.cpu().numpy().view(np.uint32)
    res = {}
    for i, case in enumerate(V1_CASES):
        g, found = v1_inputs(case)
        ne, nn, deg, sk, _ = case
        gt = t(g.view(np.int32))
        ref_kernels.update_topology_v1(gt, t(found), ne, sk)
        res[f"v1_xor{i}"] = u32(gt) ^ g
    for i, case in enumerate(OPT_CASES):
        g, bucket, lk, gk = opt_inputs(case)
        ne, nn, total, local, kl, kg, nb, _ = case
        bt = t(bucket.view(np.int64))
        gt, lkt, gkt = t(g.view(np.int32)), t(lk), t(gk)
        ref_kernels.insert_opt_fill(gt, bt, lkt, gkt, ne, local)
        filled = u32(gt).copy()
        res[f"fill_rows{i}"] = filled[ne:]
        assert np.array_equal(filled[:ne], g[:ne])
        res[f"fill_lk{i}"] = lkt.cpu().numpy().astype(np.int32)
        res[f"fill_gk{i}"] = gkt.cpu().numpy().astype(np.int32)
        lc, ll, rc, rl = ref_kernels.insert_opt_generate(gt, bt, ne, nb - 1, local)
        res[f"gen_lcnt{i}"], res[f"gen_rcnt{i}"] = u32(lc), u32(rc)
        res[f"gen_llist{i}"] = _sorted_lists(u32(lc), u32(ll))
        res[f"gen_rlist{i}"] = _sorted_lists(u32(rc), u32(rl))
        # the apply kernel on mailboxes in ascending (new id, column) order, truncated at the capacity
        olc, oll, orc_, orl = oracle.insert_opt_mailboxes(filled, bucket, ne, nb - 1, local)
        ga = t(filled.view(np.int32))
        ref_kernels.insert_opt_apply(ga, bt, ne, local, t(olc.view(np.int32)), t(oll.view(np.int32)),
                                     t(orc_.view(np.int32)), t(orl.view(np.int32)))
        res[f"apply_xor{i}"] = u32(ga) ^ filled
        # the whole function, mailbox order as the hardware raced it
        gr, lkt, gkt = t(g.view(np.int32)), t(lk), t(gk)
        data = torch.zeros((ne + nn, 96), dtype=torch.float32, device="cuda")   # read only by the heuristic path
        ref_kernels.update_topology_opt(gr, data, bt, lkt, gkt, ne, nb - 1, local)
        res[f"racy_xor{i}"] = u32(gr) ^ filled
    np.savez_compressed(out, **res)
    print("wrote", out, os.path.getsize(out), "bytes", {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1])
