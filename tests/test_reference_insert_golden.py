"""The CPU restatement of the insert topology updates against golden outputs of the reference's own
kernels (tests/golden/reference_insert.npz, produced on a B200 by
tests/golden/make_reference_insert_golden.py from oracle/_ref = src/index/insert.cu compiled as it is).
No GPU and no reference sources are needed to run this."""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "reference_insert.npz")
INVALID = 0xFFFFFFFF

pytestmark = pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file not generated")


def gen_module():
    spec = importlib.util.spec_from_file_location("make_reference_insert_golden",
                                                  os.path.join(HERE, "golden", "make_reference_insert_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def wang_hash(s):
    """insert.cu:644-651."""
    s &= 0xFFFFFFFF
    s = ((s ^ 61) ^ (s >> 16)) & 0xFFFFFFFF
    s = (s * 9) & 0xFFFFFFFF
    s ^= s >> 4
    s = (s * 0x27d4eb2d) & 0xFFFFFFFF
    s ^= s >> 15
    return s


def touched_slots(t, n_local, n_remote, total, local, near):
    """Slots the apply kernel (insert.cu:653-765) writes for old node t that drains n_local local and n_remote
    remote requests whose senders are all `near` (|bucket delta| <= 20) or all far: the slot sequence depends on
    the node id and the request COUNT only, not on the order of the senders."""
    rng = wang_hash(t)
    out_l, out_r = [], []
    half = local // 2
    for _ in range(n_local):
        rng = wang_hash(rng)
        atk = (rng % 100) < 10
        start, ln = (0, half) if atk else (half, local - half)
        if ln > 0:
            rng = wang_hash(rng)
            out_l.append(start + rng % ln)
    rd = total - local
    for _ in range(n_remote):
        nlen = rd // 3
        start, ln = (local, nlen) if near else (local + rd // 3, rd - nlen)
        if ln > 0:
            rng = wang_hash(rng)
            out_r.append(start + rng % ln)
    return out_l, out_r


def senders_of(filled, bucket, ne, target_bucket, local):
    """Full sender sets per target, from the new rows (what insert.cu:579-640 posts)."""
    n, total = filled.shape
    loc = [[] for _ in range(n)]
    rem = [[] for _ in range(n)]
    for src in range(ne, n):
        for c, d in enumerate(filled[src]):
            if d == INVALID:
                continue
            if c < local:
                loc[d].append(src)
            elif bucket[d] != target_bucket:
                rem[d].append(src)
    return loc, rem


def check_racy_graph(racy, filled, bucket, ne, target_bucket, local, lcnt, rcnt):
    """What is race-free in the reference's whole update: new rows, untouched slots, and that every slot the
    deterministic slot sequence writes holds one of the node's senders from the right mailbox."""
    n, total = filled.shape
    lmax, rmax = local // 2, (total - local) // 2
    assert np.array_equal(racy[ne:], filled[ne:])
    loc, rem = senders_of(filled, bucket, ne, target_bucket, local)
    for t in range(ne):
        nl, nr = min(int(lcnt[t]), lmax), min(int(rcnt[t]), rmax)
        near = abs(int(bucket[t]) - int(target_bucket)) <= 20
        sl, sr = touched_slots(t, nl, nr, total, local, near)
        for s in range(total):
            if s in sl:
                assert racy[t, s] in loc[t], (t, s)
            elif s in sr:
                assert racy[t, s] in rem[t], (t, s)
            else:
                assert racy[t, s] == filled[t, s], (t, s)


def check_mailboxes(gold_cnt, gold_sorted, cnt, lst, senders, cap):
    """Counts are exact; a mailbox below its capacity holds exactly the node's senders; a full one holds `cap`
    of them (which ones is the reference's race; the restatement keeps the first in (new id, column) order)."""
    assert np.array_equal(gold_cnt, cnt)
    for t in range(len(cnt)):
        c = int(cnt[t])
        assert c == len(senders[t])
        have = gold_sorted[t][gold_sorted[t] != INVALID].tolist() if cap else []
        mine = lst[t][:min(c, cap)].tolist() if cap else []
        assert mine == senders[t][:cap]
        if c <= cap:
            assert have == sorted(senders[t])
            assert sorted(mine) == have
        else:
            assert len(have) == cap
            pool = list(senders[t])
            for h in have:          # a sub-multiset of the senders
                assert h in pool
                pool.remove(h)


def test_insert_v1_matches_reference_kernels(oracle):
    gen = gen_module()
    gold = np.load(GOLDEN)
    for i, case in enumerate(gen.V1_CASES):
        g, found = gen.v1_inputs(case)
        ne, nn, deg, sk, _ = case
        want = g ^ gold[f"v1_xor{i}"]
        got = oracle.insert_v1(g, found, ne, sk)
        assert np.array_equal(got, want), f"v1 case {i}: {(got != want).sum()} slots differ"
        assert (want[:ne] != g[:ne]).any() and (want[ne:] != INVALID).any()    # the case did something


def test_insert_opt_matches_reference_kernels(oracle):
    gen = gen_module()
    gold = np.load(GOLDEN)
    for i, case in enumerate(gen.OPT_CASES):
        g, bucket, lk, gk = gen.opt_inputs(case)
        ne, nn, total, local, kl, kg, nb, _ = case
        target = nb - 1
        # stage 1: rows of the new nodes and the consumed candidate lists
        filled, lk2, gk2 = oracle.insert_opt_fill(g, bucket, lk, gk, ne, local)
        assert np.array_equal(filled[ne:], gold[f"fill_rows{i}"])
        assert np.array_equal(filled[:ne], g[:ne])
        assert np.array_equal(lk2, gold[f"fill_lk{i}"].astype(np.int64))
        assert np.array_equal(gk2, gold[f"fill_gk{i}"].astype(np.int64))
        # stage 2: mailboxes
        lc, ll, rc, rl = oracle.insert_opt_mailboxes(filled, bucket, ne, target, local)
        loc, rem = senders_of(filled, bucket, ne, target, local)
        check_mailboxes(gold[f"gen_lcnt{i}"], gold[f"gen_llist{i}"], lc, ll, loc, local // 2)
        check_mailboxes(gold[f"gen_rcnt{i}"], gold[f"gen_rlist{i}"], rc, rl, rem, (total - local) // 2)
        assert (lc > local // 2).any() and (rc > (total - local) // 2).any()   # overflowing mailboxes are covered
        # stage 3: the apply kernel on mailboxes in ascending (new id, column) order
        want = filled ^ gold[f"apply_xor{i}"]
        got = oracle.insert_opt_apply(filled, bucket, ne, local, lc, ll, rc, rl)
        assert np.array_equal(got, want), f"opt case {i}: {(got != want).sum()} slots differ"
        assert np.array_equal(oracle.insert_opt(g, bucket, lk, gk, ne, target, local), want)
        assert (want[:ne] != filled[:ne]).any()
        # the whole reference function with its racy mailbox order: everything that does not depend on the order
        check_racy_graph(filled ^ gold[f"racy_xor{i}"], filled, bucket, ne, target, local, lc, rc)
        check_racy_graph(want, filled, bucket, ne, target, local, lc, rc)
