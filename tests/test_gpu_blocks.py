"""Device-level tests of the search building blocks (csrc/search_blocks.cuh) through the C ABI, on the
reference's own known-answer inputs: tests/test_bitonic.cu:73-156 (mt19937(42), U(0,100), warp sort ==
std::sort of the pairs), tests/test_sort_impl.cu:111-121 (U(0,1000), capacities 64..512), and the three
load cases of tests/test_hashmap.cu:171-187 (successes == unique keys, incl. the full table)."""
import numpy as np
import pytest

from test_oracle_kat import _std_mt19937_uniform_float

pytestmark = pytest.mark.gpu
MAXKEY = np.uint64(0xFFFFFFFFFFFFFFFF)


def f2ord(x):
    b = np.asarray(x, dtype=np.float32).view(np.uint32)
    return np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000)).astype(np.uint32)


def skeys(dist, ids):
    """Search-queue keys [ordered dist:32 | id:31 | expanded:1] (graph_search.cu make_skey)."""
    return (f2ord(dist).astype(np.uint64) << np.uint64(32)) | (np.asarray(ids, dtype=np.uint64) << np.uint64(1))


def sort_merge(grab, top, cand, variant=0):
    import torch
    lists, m = top.shape
    ncand = cand.shape[1]
    stride = max(ncand, 1)
    d_top = torch.from_numpy(top.view(np.int64)).cuda()
    d_cand = torch.from_numpy(np.ascontiguousarray(cand).view(np.int64)).cuda() if ncand else \
        torch.zeros((lists, 1), dtype=torch.int64, device="cuda")
    out = torch.empty_like(d_top)
    grab.check(grab.lib().grab_selftest_sort_merge(grab._p(d_top), grab._p(d_cand), grab.C.c_uint64(lists), m, ncand,
                                                   stride, variant, grab._p(out), None))
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint64)


@pytest.mark.parametrize("m,variant", [(64, 0), (128, 0), (64, 1), (256, 0), (512, 0), (64, 3), (128, 3)])
@pytest.mark.parametrize("n_per_lane", [2, 4, 8])
def test_sort_merge_reference_kat(grab, m, variant, n_per_lane):
    """test_bitonic.cu inputs: 32*N keys U(0,100), seed 42, value = index.  The merge of those candidates into an
    EMPTY list must leave the first min(m, 32*N) pairs of std::sort; into a list that already holds the first
    half, sorted, it must give the same."""
    total = 32 * n_per_lane
    keys = _std_mt19937_uniform_float(42, total, 0.0, 100.0)
    pairs = skeys(keys, np.arange(total))
    want = np.sort(pairs)[:m]
    want = np.concatenate([want, np.full(m - want.size, MAXKEY)])
    empty = np.full((1, m), MAXKEY, dtype=np.uint64)
    got = sort_merge(grab, empty, pairs[None, :], variant)
    assert np.array_equal(got[0], want)
    half = np.sort(pairs[: total // 2])[:m]
    top = np.concatenate([half, np.full(m - half.size, MAXKEY)])[None, :]
    got = sort_merge(grab, top, pairs[None, total // 2:], variant)
    assert np.array_equal(got[0], want)


@pytest.mark.parametrize("cap", [64, 128, 256, 512])
def test_queue_capacities_reference_kat(grab, cap):
    """test_sort_impl.cu:111-121: `cap` keys U(0,1000), seed 42 -> ascending, values follow their keys."""
    keys = _std_mt19937_uniform_float(42, cap, 0.0, 1000.0)
    pairs = skeys(keys, np.arange(cap))
    # the list holds the first cap/2 (sorted), the second half arrives as candidates
    top = np.concatenate([np.sort(pairs[: cap // 2]), np.full(cap - cap // 2, MAXKEY)])[None, :]
    got = sort_merge(grab, top, pairs[None, cap // 2:])[0]
    d = got >> np.uint64(32)
    assert np.all(d[1:] >= d[:-1])
    ids = ((got & np.uint64(0xFFFFFFFF)) >> np.uint64(1)).astype(np.int64)
    assert np.array_equal(np.sort(ids), np.arange(cap))
    assert np.array_equal(f2ord(keys[ids]).astype(np.uint64), d)      # values follow their keys


@pytest.mark.parametrize("m", [64, 128, 256])
def test_sort_merge_random_lists(grab, m):
    """Many lists, every candidate count from 0 to the capacity, duplicates of distances (id tie-break), flagged
    (expanded) entries in the list: result == the m smallest of the union."""
    rng = np.random.default_rng(5 + m)
    lists = 200
    for ncand in [0, 1, 2, 31, 32, 33, 63, 64, m - 1, m, min(2 * m, 192)]:
        if m <= 128 and ncand > m:
            continue      # the kernel routes more than m kept candidates of a 64/128 list through shared memory
        d_top = np.round(rng.random((lists, m)) * 50).astype(np.float32)       # many equal distances
        top = np.sort(skeys(d_top, rng.permutation(lists * m).reshape(lists, m) + 5000) |
                      (rng.random((lists, m)) < 0.3).astype(np.uint64), axis=1)
        fill = rng.integers(0, m + 1, size=lists)
        top[np.arange(m)[None, :] >= fill[:, None]] = MAXKEY                    # partially filled lists
        cand = skeys(np.round(rng.random((lists, ncand)) * 50).astype(np.float32),
                     rng.permutation(lists * max(ncand, 1)).reshape(lists, -1)[:, :ncand])
        got = sort_merge(grab, top, cand)
        want = np.sort(np.concatenate([top, cand], axis=1), axis=1)[:, :m]
        assert np.array_equal(got, want), (m, ncand)
    # more candidates than a 64/128-entry list: the shared-memory routine
    if m <= 128:
        ncand = 192
        top = np.sort(skeys(rng.random((lists, m)).astype(np.float32), np.arange(lists * m).reshape(lists, m)), axis=1)
        cand = skeys(rng.random((lists, ncand)).astype(np.float32), 100000 + np.arange(lists * ncand).reshape(lists, -1))
        got = sort_merge(grab, top, cand)
        assert np.array_equal(got, np.sort(np.concatenate([top, cand], axis=1), axis=1)[:, :m])


@pytest.mark.parametrize("m", [64, 128])
def test_split_kernel_merges_random_lists(grab, m):
    """The two merge paths of the warp-split kernel on random lists: by rank (up to 32 unsorted candidates) and two
    register-sorted runs (up to 256), lists partially filled and with expanded flags: result == the m smallest of
    the union.  Keys are distinct, as ids in a search are."""
    rng = np.random.default_rng(50 + m)
    lists = 300
    for variant, counts in [(2, [1, 2, 3, 7, 16, 31, 32]), (3, [2, 3, 17, 33, 64, 65, 128, 200, 256])]:
        for ncand in counts:
            ids = rng.permutation(lists * (m + ncand)).reshape(lists, m + ncand)
            d = np.round(rng.random((lists, m + ncand)) * 60).astype(np.float32)      # equal distances, distinct ids
            keys = skeys(d, ids)
            top = np.sort(keys[:, :m] | (rng.random((lists, m)) < 0.3).astype(np.uint64), axis=1)
            fill = rng.integers(0, m + 1, size=lists)
            top[np.arange(m)[None, :] >= fill[:, None]] = MAXKEY
            cand = keys[:, m:]
            got = sort_merge(grab, top, cand, variant)
            want = np.sort(np.concatenate([top, cand], axis=1), axis=1)[:, :m]
            assert np.array_equal(got, want), (m, variant, ncand)


def hash_run(grab, bitlen, keys, threads=64):
    import torch
    d_keys = torch.from_numpy(np.asarray(keys, dtype=np.uint32).view(np.int32)).cuda()
    table = torch.empty(1 << bitlen, dtype=torch.int32, device="cuda")
    ok = torch.empty(len(keys), dtype=torch.int32, device="cuda")
    grab.check(grab.lib().grab_selftest_hash_insert(grab._p(table), bitlen, grab._p(d_keys), len(keys), threads,
                                                    grab._p(ok), None))
    torch.cuda.synchronize()
    return ok.cpu().numpy(), table.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("bitlen,unique,dup_ratio", [(10, 500, 0.4), (8, 200, 0.0), (8, 256, 0.0)])
def test_hashmap_reference_kat(grab, oracle, bitlen, unique, dup_ratio):
    """test_hashmap.cu:171-187: low load with 40 % duplicates, high load, full table: successes == unique keys,
    occupied slots == successes, every key findable at its probe position."""
    keys = list(range(1, unique + 1)) + list(range(1, int(unique * dup_ratio) + 1))
    rng = np.random.default_rng(bitlen + unique)
    keys = np.array(keys, dtype=np.uint32)[rng.permutation(len(keys))]
    ok, table = hash_run(grab, bitlen, keys)
    assert int(ok.sum()) == unique
    for key in np.unique(keys):                      # exactly one insert of every distinct key succeeded
        assert int(ok[keys == key].sum()) == 1
    assert int((table != 0xFFFFFFFF).sum()) == unique
    assert set(table[table != 0xFFFFFFFF].tolist()) == set(range(1, unique + 1))
    # the slots agree with the reference's probe rule: every key sits between its home slot and the next hole
    mask = (1 << bitlen) - 1
    for key in range(1, unique + 1):
        idx = (key ^ (key >> bitlen)) & mask
        for _ in range(mask + 1):
            assert table[idx] != 0xFFFFFFFF
            if table[idx] == key:
                break
            idx = (idx + 1) & mask
    # one warp on the distinct keys: the same set of slots' contents as the CPU restatement's table
    ok1, table1 = hash_run(grab, bitlen, np.arange(1, unique + 1, dtype=np.uint32), threads=32)
    assert int(ok1.sum()) == unique
    ref_table = np.full(1 << bitlen, 0xFFFFFFFF, dtype=np.uint32)
    for key in range(1, unique + 1):
        oracle.hash_insert(ref_table, bitlen, key)
    assert set(table1.tolist()) == set(ref_table.tolist())


def test_hashmap_full_table_reports_visited(grab):
    """hashmap.cuh:89-90: a full table answers "already there" for a new key."""
    keys = np.concatenate([np.arange(1, 257, dtype=np.uint32), np.array([9999, 10000], dtype=np.uint32)])
    ok, table = hash_run(grab, 8, keys, threads=32)
    # 258 distinct keys, 256 slots: exactly 256 inserts succeed, the other two read "visited", nothing is lost
    assert int(ok.sum()) == 256
    assert int((table != 0xFFFFFFFF).sum()) == 256
    assert set(table.tolist()) == set(keys[ok == 1].tolist())


def test_hashmap_global_table(grab):
    """Tables above 2^13 slots live in global memory (the per-query slice of the workspace)."""
    rng = np.random.default_rng(3)
    keys = rng.integers(0, 1 << 30, size=5000).astype(np.uint32)
    ok, table = hash_run(grab, 14, np.concatenate([keys, keys[:1000]]), threads=256)
    assert int(ok.sum()) == np.unique(keys).size
    assert int((table != 0xFFFFFFFF).sum()) == np.unique(keys).size
