"""Golden vectors from the reference's OWN cross-bucket code (src/index/cagra_opt.cu: update_remote_edges_kernel
:209-303, kern_make_global_rev_graph :457-482, kern_inject_global_reverse_edges :487-600).

Runs on a machine with a B200 after `make -C oracle ref` built oracle/_ref/libgrab_ref.so from the reference's
sources (FAISS / RAFT / RMM names of that file's other functions are declared by oracle/faiss_shim/; those functions
are never called).  Inputs are regenerated from seeds; only the kernels' outputs are stored.
Usage: python tests/golden/make_reference_remote_golden.py OUT.npz

Stages: the selection kernel is one thread per node and deterministic -- its remote columns and the consumed
candidate lists are stored whole.  The reverse lists are claimed with atomicAdd by one thread per source, so the
order inside a list is a race: stored are the counts and every list as a sorted set (past the capacity of 32 a
subset).  The injection kernel is deterministic given the lists and is run on the CANONICAL ones (ascending source
id, then column: the order the CPU restatement and the new CUDA code fix).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

INVALID = 0xFFFFFFFF
MAX_REV = 32
CASES = [  # (n, total_degree, local_degree, candidates per node, buckets, seed)
    (3000, 16, 10, 64, 30, 501),
    (2400, 32, 24, 64, 8, 502),      # span = max(1, 8 / 5) = 1: few "nearby" buckets
    (2000, 32, 16, 96, 2, 503),      # two buckets: every other-bucket candidate is nearby, the far quota back-fills
]


def inputs(case):
    """(graph [n, total] with empty remote columns, bucket id per node (non-decreasing), candidates [n, gk])."""
    n, total, local, gk, nb, seed = case
    rng = np.random.default_rng(seed)
    bucket = np.sort(rng.integers(0, nb, size=n)).astype(np.uint64)
    bucket[-1] = nb - 1                                   # the kernel takes the bucket count from the last node
    g = np.full((n, total), INVALID, dtype=np.uint32)
    g[:, :local] = rng.integers(0, n, size=(n, local))
    hot = max(16, n // 20)                                # a few popular targets: reverse lists overflow 32
    cand = np.where(rng.random((n, gk)) < 0.3, rng.integers(0, hot, size=(n, gk)), rng.integers(0, n, size=(n, gk)))
    cand = cand.astype(np.uint32)
    cand[::7, 3] = np.arange(0, n, 7, dtype=np.uint32)    # the node itself
    cand[::5, 9] = INVALID                                # a hole
    cand[::3, 12] = cand[::3, 4]                          # the same candidate twice
    cand[::11, 1] = g[::11, 2]                            # already a local neighbour
    return g, bucket, cand


def canonical_global_rev(graph, local):
    """Reverse lists of the remote columns, ascending source id then column; counts run past the capacity."""
    n, total = graph.shape
    rev = np.full((n, MAX_REV), INVALID, dtype=np.uint32)
    cnt = np.zeros(n, dtype=np.uint32)
    for s in range(n):
        for k in range(local, total):
            d = graph[s, k]
            if d != INVALID and d < n:
                if cnt[d] < MAX_REV:
                    rev[d, cnt[d]] = s
                cnt[d] += 1
    return rev, cnt


def main(out_path):
    import torch
    import ref_kernels as ref
    out = {}
    for ci, case in enumerate(CASES):
        n, total, local, gk, nb, seed = case
        g, bucket, cand = inputs(case)
        d_g = torch.from_numpy(g.view(np.int32)).cuda()
        d_ts = torch.from_numpy(bucket.view(np.int64)).cuda()
        d_c = torch.from_numpy(cand.view(np.int32)).cuda()
        ref.update_remote_edges(d_g, d_ts, d_c, local)
        sel = d_g.cpu().numpy().view(np.uint32)
        out[f"c{ci}_remote"] = sel[:, local:].copy()
        out[f"c{ci}_consumed"] = np.packbits(d_c.cpu().numpy().view(np.uint32) == INVALID, axis=1)
        assert np.array_equal(sel[:, :local], g[:, :local])
        rev, cnt = ref.make_global_rev(d_g, local, MAX_REV)
        rev = rev.cpu().numpy().view(np.uint32)
        cnt = cnt.cpu().numpy().view(np.uint32)
        keep = np.minimum(cnt, MAX_REV)
        rev_sorted = np.full_like(rev, INVALID)
        for i in range(n):
            rev_sorted[i, :keep[i]] = np.sort(rev[i, :keep[i]])
        out[f"c{ci}_rev_sorted"], out[f"c{ci}_cnt"] = rev_sorted, cnt
        crev, ccnt = canonical_global_rev(sel, local)
        d_inj = torch.from_numpy(sel.view(np.int32).copy()).cuda()
        ref.inject_global_rev(d_inj, torch.from_numpy(crev.view(np.int32)).cuda(),
                              torch.from_numpy(ccnt.view(np.int32)).cuda(), local)
        out[f"c{ci}_injected_canonical"] = d_inj.cpu().numpy().view(np.uint32)[:, local:].copy()
        d_all = torch.from_numpy(sel.view(np.int32).copy()).cuda()
        ref.enhance_global_connectivity(d_all, local)                     # the racy whole, for property checks
        out[f"c{ci}_enhanced_raw"] = d_all.cpu().numpy().view(np.uint32)[:, local:].copy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
