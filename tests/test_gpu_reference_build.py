"""Live three-way check of prune / reverse graph / merge: the reference's OWN functions (src/index/cagra.cu compiled
into oracle/_ref/libgrab_ref.so), the CPU restatement, and the new CUDA code on the same inputs.  The stages whose
order the reference leaves to an atomics race are compared group by group (tests/test_reference_build_golden.py)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_build_golden as gen  # noqa: E402
from test_reference_build_golden import check_racy_reverse  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    import ref_kernels
    if not ref_kernels.available() or not hasattr(ref_kernels.lib(), "ref_optimize_prune"):
        pytest.skip("oracle/_ref/libgrab_ref.so lacks the graph-optimisation harness (make -C oracle ref REF=...)")
    return ref_kernels


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("ci", range(len(gen.CASES)))
def test_three_way_prune_reverse_merge(grab, oracle, ref, ci):
    import torch
    case = gen.CASES[ci]
    n, ind, outd = case[1], case[3], case[4]
    knn = gen.inputs(case)
    L, C = grab.lib(), grab.C
    # prune: reference == restatement == CUDA, bit for bit
    r_pruned = ref.optimize_prune(knn, outd)
    assert np.array_equal(oracle.prune(knn, outd), r_pruned)
    d_knn = _t(knn.view(np.int32))
    d_out = torch.empty((n, outd), dtype=torch.int32, device="cuda")
    grab.check(L.grab_optimize_prune_device(grab._p(d_knn), grab._p(d_out), C.c_uint64(n), ind, outd, None, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(d_out), r_pruned)
    # reverse graph: the reference's racy lists group by group; restatement and CUDA in the canonical order
    r_rev, r_cnt = ref.optimize_reverse(r_pruned)
    check_racy_reverse(r_pruned, r_rev, r_cnt)
    crev, ccnt = gen.canonical_reverse(r_pruned)
    d_rev = torch.empty((n, outd), dtype=torch.int32, device="cuda")
    d_cnt = torch.empty(n, dtype=torch.int32, device="cuda")
    grab.check(L.grab_optimize_reverse_graph_device(grab._p(d_out), grab._p(d_rev), grab._p(d_cnt), C.c_uint64(n),
                                                    outd, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(d_rev), crev) and np.array_equal(_u32(d_cnt), ccnt)
    # merge on the canonical lists: reference == restatement == CUDA
    r_merged = ref.optimize_merge(r_pruned, crev, ccnt)
    assert np.array_equal(oracle.merge_graphs(r_pruned, crev, ccnt), r_merged)
    grab.check(L.grab_optimize_merge_graphs_device(grab._p(d_out), grab._p(d_rev), grab._p(d_cnt), C.c_uint64(n),
                                                   outd, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(d_out), r_merged)
