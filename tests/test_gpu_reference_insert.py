"""Three-way agreement on the insert topology updates, live on the GPU: the REFERENCE's own kernels
(src/index/insert.cu compiled into oracle/_ref), the CPU restatement, and the new CUDA code behind
grab_update_topology_v1 / grab_update_topology_opt -- same seeded inputs, other seeds than the committed
golden file.  Where the reference races (mailbox order, insert.cu:579-640) its apply kernel is handed the
mailboxes in ascending (new id, column) order, the order the other two fix; the racy whole function is
checked for everything that does not depend on that order."""
import importlib.util
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

pytestmark = pytest.mark.gpu


def _mod(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref():
    import ref_kernels
    if not ref_kernels.available():
        pytest.skip("oracle/_ref/libgrab_ref.so not built (needs the reference's sources at build time)")
    return ref_kernels


@pytest.fixture(scope="module")
def gen():
    return _mod("make_reference_insert_golden", os.path.join(HERE, "golden", "make_reference_insert_golden.py"))


@pytest.fixture(scope="module")
def chk():
    return _mod("test_reference_insert_golden", os.path.join(HERE, "test_reference_insert_golden.py"))


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("case", [(2500, 300, 32, 64, 901), (1200, 128, 64, 128, 902)])
def test_v1_three_way(grab, oracle, ref, gen, case):
    ne, nn, deg, sk, _ = case
    g, found = gen.v1_inputs(case)
    want = oracle.insert_v1(g, found, ne, sk)
    gr = _t(g.view(np.int32))
    ref.update_topology_v1(gr, _t(found), ne, sk)
    assert np.array_equal(_u32(gr), want), "CPU restatement differs from the reference's update_topology_gpu_v1"
    go = _t(g.view(np.int32))
    grab.check(grab.lib().grab_update_topology_v1(grab._p(go), grab._p(_t(found)), grab.C.c_uint64(ne),
                                                  grab.C.c_uint64(nn), deg, sk, None))
    assert np.array_equal(_u32(go), want), "grab_update_topology_v1 differs from the reference's result"


@pytest.mark.parametrize("case", [(3600, 300, 32, 16, 40, 40, 50, 911), (2000, 160, 16, 12, 24, 16, 24, 912)])
def test_opt_three_way(grab, oracle, ref, gen, chk, case):
    import torch
    ne, nn, total, local, kl, kg, nb, _ = case
    target = nb - 1
    g, bucket, lk, gk = gen.opt_inputs(case)
    bt = _t(bucket.view(np.int64))
    # reference, stage by stage
    gr, lkt, gkt = _t(g.view(np.int32)), _t(lk), _t(gk)
    ref.insert_opt_fill(gr, bt, lkt, gkt, ne, local)
    filled, lk2, gk2 = oracle.insert_opt_fill(g, bucket, lk, gk, ne, local)
    assert np.array_equal(_u32(gr), filled)
    assert np.array_equal(lkt.cpu().numpy(), lk2) and np.array_equal(gkt.cpu().numpy(), gk2)
    rlc, rll, rrc, rrl = ref.insert_opt_generate(gr, bt, ne, target, local)
    lc, ll, rc, rl = oracle.insert_opt_mailboxes(filled, bucket, ne, target, local)
    loc, rem = chk.senders_of(filled, bucket, ne, target, local)
    chk.check_mailboxes(_u32(rlc), gen._sorted_lists(_u32(rlc), _u32(rll)), lc, ll, loc, local // 2)
    chk.check_mailboxes(_u32(rrc), gen._sorted_lists(_u32(rrc), _u32(rrl)), rc, rl, rem, (total - local) // 2)
    ga = _t(filled.view(np.int32))
    ref.insert_opt_apply(ga, bt, ne, local, _t(lc.view(np.int32)), _t(ll.view(np.int32)), _t(rc.view(np.int32)),
                         _t(rl.view(np.int32)))
    want = oracle.insert_opt_apply(filled, bucket, ne, local, lc, ll, rc, rl)
    assert np.array_equal(_u32(ga), want), "CPU restatement differs from the reference's apply kernel"
    # the new CUDA path: whole update in one call, mailbox order fixed
    go, lko, gko = _t(g.view(np.int32)), _t(lk), _t(gk)
    grab.check(grab.lib().grab_update_topology_opt(grab._p(go), grab._p(bt), grab._p(lko), grab._p(gko),
                                                   grab.C.c_uint64(ne), grab.C.c_uint64(nn), grab.C.c_uint64(target),
                                                   total, local, kl, kg, None))
    torch.cuda.synchronize()
    assert np.array_equal(_u32(go), want), "grab_update_topology_opt differs from the reference's kernels"
    # the reference's whole function, mailboxes in the order the hardware raced them
    gw, lkw, gkw = _t(g.view(np.int32)), _t(lk), _t(gk)
    data = torch.zeros((ne + nn, 96), dtype=torch.float32, device="cuda")
    ref.update_topology_opt(gw, data, bt, lkw, gkw, ne, target, local)
    chk.check_racy_graph(_u32(gw), filled, bucket, ne, target, local, lc, rc)
    # and the new code obeys the same order-free rules
    chk.check_racy_graph(_u32(go), filled, bucket, ne, target, local, lc, rc)


def test_find_near_nodes_against_reference(grab, oracle, ref):
    """grab_find_near_nodes against the reference's find_near_nodes (insert.cu:140-219; its base launcher
    cagra.cu:844-935 restated in the harness): same graph, exact distances ascending, overlap of the returned
    neighbour sets with the exact nearest old nodes within 0.5 points of recall."""
    import torch
    from conftest import clustered
    n, dim, deg, nn, sk = 6000, 96, 32, 256, 64
    data = clustered(n + nn, dim, 6, 1.0, 171)
    knn = oracle.knn_block(data[:n], 2 * deg)
    g = oracle.prune(knn, deg)
    rev, cnt = oracle.reverse_graph(g)
    g = oracle.merge_graphs(g, rev, cnt)
    d_data, d_g = _t(data), _t(g.view(np.int32))
    new = d_data[n:].contiguous()
    rids, rd = ref.find_near_nodes(d_data, n, new, d_g, sk, 64, 4, 40, 12)
    oi = torch.empty((nn, sk), dtype=torch.int64, device="cuda")
    od = torch.empty((nn, sk), dtype=torch.float32, device="cuda")
    p = grab.SearchParams(64, 4, 0, 40, 12)
    grab.check(grab.lib().grab_find_near_nodes(grab._p(d_data), grab.C.c_uint64(n), grab._p(new),
                                               grab.C.c_uint64(nn), grab._p(d_g), dim, deg, sk, p,
                                               grab._p(oi), grab._p(od)))
    gt, _ = oracle.exact_search(data[:n], data[n:], sk)
    rr, ro = oracle.recall(rids.cpu().numpy(), gt), oracle.recall(oi.cpu().numpy(), gt)
    assert ro >= rr - 0.005, (ro, rr)
    d = od.cpu().numpy()
    assert (np.diff(d, axis=1) >= 0).all()
