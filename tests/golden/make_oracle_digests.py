"""SHA-256 digests of the CPU oracle's outputs on seeded inputs, one per restated function.

The oracle is the checker every GPU parity test relies on; these digests make an accidental change
of its arithmetic or of a tie-break rule visible in the CPU test suite.  They were recorded after the
oracle had been pinned (the reference's known-answer tests, the golden outputs of its search kernels,
the bit-exact agreement with the CUDA path).  Usage: python tests/golden/make_oracle_digests.py OUT.json
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _h(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode() + str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


def digests():
    import oracle
    from conftest import clustered
    out = {}
    rng = np.random.default_rng(2024)
    n, dim, deg = 3000, 32, 16
    data = clustered(n, dim, 12, 0.8, 301)
    q = data[rng.integers(0, n, 40)] + np.float32(0.05) * rng.standard_normal((40, dim)).astype(np.float32)
    ts = np.arange(n, dtype=np.uint64)
    lo = rng.integers(0, n - 900, 40).astype(np.uint64)
    hi = lo + 900
    out["exact_search_range"] = _h(*oracle.exact_search(data, q, 10, ts=ts, lo=lo, hi=hi))
    labels = rng.integers(0, 8, n).astype(np.uint8)
    masks = rng.integers(1, 256, 40).astype(np.uint32)
    out["exact_search_labels_ip"] = _h(*oracle.exact_search(data, q, 10, labels=labels, masks=masks, metric=1))
    knn = oracle.knn_block(data, 2 * deg)
    out["knn_block"] = _h(knn)
    pruned, det = oracle.prune(knn, deg, want_detour=True)
    out["prune"] = _h(pruned, det)
    rev, cnt = oracle.reverse_graph(pruned)
    out["reverse_graph"] = _h(rev, cnt)
    graph = oracle.merge_graphs(pruned, rev, cnt)
    out["merge_graphs"] = _h(graph)
    nb, total, local, gk = 10, 16, 10, 64
    bucket = np.repeat(np.arange(nb, dtype=np.uint64), n // nb)
    g2 = rng.integers(0, n, size=(n, total)).astype(np.uint32)
    cand = rng.integers(0, n, size=(n, gk)).astype(np.uint32)
    cand[::5, 40:] = 0xFFFFFFFF
    g3, cand_after = oracle.remote_edges(g2, bucket, cand, local)
    out["remote_edges"] = _h(g3, cand_after)
    out["inject_reverse_remote"] = _h(oracle.inject_reverse_remote(g3, local, 32))
    seeds = rng.integers(0, n, size=(40, 32)).astype(np.uint32)
    out["graph_search_plain"] = _h(*oracle.graph_search(data, graph, q, 10, 64, 4, 30, 12, mode=0, seeds=seeds))
    out["graph_search_bucket"] = _h(*oracle.graph_search(data, graph, q, 10, 128, 4, 30, 12, mode=1, active_deg=8,
                                                         seeds=seeds))
    rs = rng.integers(500, 2000, size=(40, 32)).astype(np.uint32)
    out["graph_search_range"] = _h(*oracle.graph_search(data, graph, q, 10, 64, 4, 30, 12, mode=2, ts=ts, lo=500,
                                                        hi=2000, seeds=rs))
    ne, nn, sk = 2000, 100, 32
    gi = np.full((ne + nn, deg), 0xFFFFFFFF, dtype=np.uint32)
    gi[:ne] = rng.integers(0, ne, size=(ne, deg))
    found = np.stack([rng.choice(ne // 10, size=sk, replace=False) for _ in range(nn)]).astype(np.int64)
    found[::9, -3:] = -1
    out["insert_v1"] = _h(oracle.insert_v1(gi, found, ne, sk))
    nbk, kl, kg = 20, 24, 24
    bkt = np.concatenate([np.repeat(np.arange(nbk, dtype=np.uint64), ne // nbk), np.full(nn, nbk - 1, dtype=np.uint64)])
    go = np.full((ne + nn, total), 0xFFFFFFFF, dtype=np.uint32)
    go[:ne] = rng.integers(0, ne, size=(ne, total))
    same = np.flatnonzero(bkt[:ne] == nbk - 1)
    lk = np.stack([rng.choice(np.concatenate([same, np.arange(ne, ne + nn)]), size=kl, replace=False)
                   for _ in range(nn)]).astype(np.int64)
    gkn = np.stack([rng.choice(ne, size=kg, replace=False) for _ in range(nn)]).astype(np.int64)
    out["insert_opt"] = _h(oracle.insert_opt(go, bkt, lk, gkn, ne, nbk - 1, local))
    d = np.sort(rng.random((30, 4, 10)).astype(np.float32), axis=2)
    ids = rng.permutation(30 * 4 * 10).reshape(30, 4, 10).astype(np.int64)
    ids[:, 2, 7:] = -1
    out["merge_topk"] = _h(*oracle.merge_topk(d, ids, 10))
    cen, cnorm, offs, mem = oracle.router_build(data, 24, 0, iterations=3)
    out["router_build"] = _h(cen, cnorm, offs, mem)
    probes = oracle.nearest_centroids(q, cen, cnorm, 0, 4)
    out["nearest_centroids"] = _h(probes)
    out["route_seeds_range"] = _h(oracle.route_seeds(probes, n, offs, mem, 32, ts=ts, lo=lo, hi=hi))
    loff = np.searchsorted(np.sort(labels), np.arange(33), side="left").astype(np.uint32)
    out["route_seeds_labels"] = _h(oracle.route_seeds(probes, n, offs, mem, 32, labels=np.sort(labels), masks=masks,
                                                      label_offsets=loff))
    return out


if __name__ == "__main__":
    with open(sys.argv[1], "w") as fh:
        json.dump(digests(), fh, indent=1, sort_keys=True)
    print("wrote", sys.argv[1])
