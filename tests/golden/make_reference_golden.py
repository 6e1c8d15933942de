"""Golden vectors from the reference's OWN search kernels.

Runs on a machine with a B200 after `make -C oracle ref` built oracle/_ref/libgrab_ref.so from the
reference's sources.  Inputs are regenerated from seeds (the same code the CPU test uses); only the
kernels' outputs are stored.  Usage: python tests/golden/make_reference_golden.py OUT.npz
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

CASES = [  # (mode, itopk, width, max_iter, hash_bitlen, active_deg)
    (0, 64, 4, 40, 13, 0),    # search_kernel (plain)
    (1, 128, 4, 40, 13, 8),   # search_kernel_bucket (prefix of 8 columns)
    (2, 64, 4, 40, 13, 0),    # search_kernel_range
    (2, 64, 2, 40, 12, 0),
]
LO, HI = 1500, 4500


def inputs():
    """Seeded inputs shared by the generator and tests/test_reference_golden.py."""
    import oracle
    from conftest import clustered
    n, dim, deg, nq = 6000, 96, 16, 64   # the reference kernels exist for dims 96, 128, 256, 960, 1024, 2048 only
    data = clustered(n, dim, 6, 1.0, 161)
    knn = oracle.knn_block(data, 2 * deg)
    g = oracle.prune(knn, deg)
    rev, cnt = oracle.reverse_graph(g)
    g = oracle.merge_graphs(g, rev, cnt)
    rng = np.random.default_rng(162)
    q = data[rng.integers(0, n, nq)] + 0.1 * rng.standard_normal((nq, dim)).astype(np.float32)
    seeds_all = rng.integers(0, n, size=(nq, 32)).astype(np.uint32)
    seeds_rng = rng.integers(LO, HI, size=(nq, 32)).astype(np.uint32)
    return data, g, q, seeds_all, seeds_rng


def main(out):
    import torch
    import ref_kernels
    if not ref_kernels.available():
        raise SystemExit("oracle/_ref/libgrab_ref.so is missing: run `make -C oracle ref` where the reference is")
    data, g, q, seeds_all, seeds_rng = inputs()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_data, d_g, d_q = t(data), t(g.view(np.int32)), t(q)
    d_ts = t(np.arange(data.shape[0], dtype=np.int64))
    res = {}
    for i, (mode, itopk, width, mi, bl, adeg) in enumerate(CASES):
        seeds = seeds_rng if mode == 2 else seeds_all
        kw = dict(seeds=t(seeds.view(np.int32)))
        if mode == 2:
            kw.update(ts=d_ts, lo=LO, hi=HI)
        if mode == 1:
            kw.update(active_deg=adeg)
        ids, dists, _ = ref_kernels.search(mode, d_data, d_g, d_q, 10, itopk, width, mi, bl, **kw)
        res[f"ids{i}"] = ids.cpu().numpy().astype(np.int32)
        res[f"dists{i}"] = dists.cpu().numpy().astype(np.float32)
    np.savez_compressed(out, **res)
    print("wrote", out, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1])
