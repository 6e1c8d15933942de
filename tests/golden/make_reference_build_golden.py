"""Golden vectors from the reference's OWN graph-optimisation code (src/index/cagra.cu: optimize_prune :286-401 with
kern_prune :219-276, optimize_create_reverse_graph :455-548, optimize_merge_graphs :574-650, build :665-711).

Runs on a machine with a B200 after `make -C oracle ref` built oracle/_ref/libgrab_ref.so from the reference's
sources (the FAISS names of that file's generate_knn_graph are declared by oracle/faiss_shim/; that function is
never called).  Inputs are regenerated from seeds (the same code the CPU test uses); only the reference's outputs
are stored.  Usage: python tests/golden/make_reference_build_golden.py OUT.npz

What is stored, and why in stages: optimize_prune is deterministic (detour counts, then a stable sort), its output
is stored whole.  optimize_create_reverse_graph hands out list slots with atomicAdd (kern_make_rev_graph, :418-444),
one launch per column: the sources of ONE column that point at the same node land in racing order, columns follow
each other in order.  Stored are therefore the raw lists and counts (checked group by group: every column's group
is a permutation -- past the capacity a subset -- of that column's sources) and optimize_merge_graphs, which is
deterministic, run on the CANONICAL lists (ascending source id inside a column group: the order the CPU restatement
and the new CUDA code fix).  build() = the three in a row, racy through the middle one: stored for property checks.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

INVALID = 0xFFFFFFFF
CASES = [  # (kind, n, dim, in_degree, out_degree, seed)
    ("knn", 1500, 32, 32, 16, 401),      # an exact kNN graph of clustered data
    ("knn", 1200, 64, 64, 32, 402),      # degree > 32: more than one pass of the 32-thread kernel loops
    ("random", 1000, 0, 24, 12, 403),    # random rows with repeated ids and 0xFFFFFFFF padding at the tail
]


def inputs(case):
    """The kNN graph [n, in_degree] uint32 handed to optimize_prune."""
    kind, n, dim, ind, outd, seed = case
    rng = np.random.default_rng(seed)
    if kind == "knn":
        import oracle
        from conftest import clustered
        return oracle.knn_block(clustered(n, dim, 20, 1.0, seed), ind)
    g = rng.integers(0, n, size=(n, ind)).astype(np.uint32)
    g[::5, 7] = g[::5, 2]                                    # the same neighbour twice
    g[::9, 0] = np.arange(0, n, 9, dtype=np.uint32)          # a self loop
    tail = rng.integers(0, 6, size=n)                        # up to 5 padded slots at the end of a row
    for i in range(n):
        if tail[i]:
            g[i, ind - tail[i]:] = INVALID
    return g


def canonical_reverse(graph):
    """Reverse lists in the order the restatement fixes: column by column, ascending source id inside a column;
    at most `degree` entries are kept, the count is the full number of in-edges (kern_make_rev_graph counts on)."""
    g = np.asarray(graph, dtype=np.uint32)
    n, deg = g.shape
    rev = np.full((n, deg), INVALID, dtype=np.uint32)
    cnt = np.zeros(n, dtype=np.uint32)
    for k in range(deg):
        col = g[:, k]
        for src in np.flatnonzero(col < n):          # ascending source id
            d = col[src]
            if cnt[d] < deg:
                rev[d, cnt[d]] = src
            cnt[d] += 1
    return rev, cnt


def main(out_path):
    import torch
    import ref_kernels as ref
    out = {}
    for ci, case in enumerate(CASES):
        kind, n, dim, ind, outd, seed = case
        knn = inputs(case)
        pruned = ref.optimize_prune(knn, outd)
        assert np.array_equal(ref.optimize_prune(knn, outd), pruned)          # deterministic
        rev, cnt = ref.optimize_reverse(pruned)                               # racy inside a column group
        crev, ccnt = canonical_reverse(pruned)
        merged = ref.optimize_merge(pruned, crev, ccnt)
        assert np.array_equal(ref.optimize_merge(pruned, crev, ccnt), merged)  # deterministic
        out[f"c{ci}_pruned"], out[f"c{ci}_rev_raw"], out[f"c{ci}_cnt"] = pruned, rev, cnt
        out[f"c{ci}_merged_canonical"] = merged
        if kind == "knn":
            dummy = torch.zeros((n, 4), dtype=torch.float32, device="cuda")   # build() never reads the vectors
            built = ref.build(dummy, torch.from_numpy(knn.view(np.int32)).cuda(), outd)
            out[f"c{ci}_built_raw"] = built.cpu().numpy().view(np.uint32)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
