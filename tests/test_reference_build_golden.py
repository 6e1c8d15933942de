"""The CPU restatement of prune / reverse graph / merge against outputs of the reference's OWN code
(src/index/cagra.cu compiled into oracle/_ref, run on a B200 by tests/golden/make_reference_build_golden.py; the
outputs are committed as tests/golden/reference_build.npz).  Runs without a GPU and without the reference."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_build_golden as gen  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "reference_build.npz")
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def golden():
    if not os.path.exists(GOLDEN):
        pytest.skip("tests/golden/reference_build.npz not generated yet")
    return np.load(GOLDEN)


def check_racy_reverse(pruned, rev_raw, cnt_raw):
    """The reference's lists against the canonical ones: same counts; walking a node's list, the entries of every
    column group are that column's sources in some order (the last group that still fits may be cut: a subset)."""
    n, deg = pruned.shape
    crev, ccnt = gen.canonical_reverse(pruned)
    assert np.array_equal(cnt_raw, ccnt)
    sources = [[[] for _ in range(deg)] for _ in range(n)]
    for k in range(deg):
        col = pruned[:, k]
        for src in np.flatnonzero(col < n):
            sources[col[src]][k].append(int(src))
    for d in range(n):
        pos = 0
        for k in range(deg):
            grp = sources[d][k]
            if not grp or pos >= deg:
                continue
            take = min(len(grp), deg - pos)
            got = rev_raw[d, pos:pos + take].tolist()
            if take == len(grp):
                assert sorted(got) == sorted(grp), (d, k)
            else:
                assert len(set(got)) == take and set(got) <= set(grp), (d, k)
            pos += take
        assert np.all(rev_raw[d, pos:] == INVALID)


@pytest.mark.parametrize("ci", range(len(gen.CASES)))
def test_prune_reverse_merge_against_the_reference(oracle, golden, ci):
    case = gen.CASES[ci]
    outd = case[4]
    knn = gen.inputs(case)
    pruned = golden[f"c{ci}_pruned"]
    assert np.array_equal(oracle.prune(knn, outd), pruned)                      # bit-exact
    check_racy_reverse(pruned, golden[f"c{ci}_rev_raw"], golden[f"c{ci}_cnt"])
    crev, ccnt = gen.canonical_reverse(pruned)
    orev, ocnt = oracle.reverse_graph(pruned)
    assert np.array_equal(orev, crev) and np.array_equal(ocnt, ccnt)            # the restatement IS the canonical order
    assert np.array_equal(oracle.merge_graphs(pruned, crev, ccnt), golden[f"c{ci}_merged_canonical"])  # bit-exact
    if f"c{ci}_built_raw" in golden.files:
        # the whole racy build(): the merge interleaves own and reverse entries (own first), so every row starts with
        # the row's first own neighbour, holds no node twice among its valid entries, and holds only own neighbours
        # and in-edge sources
        built = golden[f"c{ci}_built_raw"]
        n = built.shape[0]
        insrc = [set() for _ in range(n)]
        for k in range(outd):
            for src in np.flatnonzero(pruned[:, k] < n):
                insrc[pruned[src, k]].add(int(src))
        for j in range(n):
            row = built[j]
            assert row[0] == pruned[j, 0]
            valid = row[row != INVALID]
            assert len(set(valid.tolist())) == len(valid)
            assert set(valid.tolist()) <= set(pruned[j].tolist()) | insrc[j]
