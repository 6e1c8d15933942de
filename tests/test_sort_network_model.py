"""Model of the register sort/merge network of the search kernel (csrc/graph_search.cu,
warp_sort_merge_regs): element e lives in register e/32 of lane e%32, strides below 32 are xor
exchanges between lanes, strides of 32 and more pair registers of one lane, the level equal to the padded
candidate count sorts ascending, candidates are folded into the list by top[M-1-i] = min(top[M-1-i], c[i])
followed by one bitonic merge level.  The model repeats that index arithmetic in numpy and compares with a
plain sort for every candidate count and both list lengths (64 and 128); the CUDA code itself is covered by
the GPU parity tests."""
import numpy as np
MAXK = np.uint64(0xFFFFFFFFFFFFFFFF)
def stage(v, R, size, stride):
    # v[r][lane]
    if stride >= 32:
        rs = stride >> 5
        for r in range(R):
            if (r & rs) == 0:
                up = ((r << 5) & size) == 0
                a, b = v[r].copy(), v[r | rs].copy()
                swap = (a > b) == up
                v[r] = np.where(swap, b, a); v[r | rs] = np.where(swap, a, b)
    else:
        lanes = np.arange(32)
        lower = (lanes & stride) == 0
        for r in range(R):
            e = lanes + (r << 5)
            up = (e & size) == 0
            other = v[r][lanes ^ stride]
            keep_min = lower == up
            mn, mx = np.minimum(v[r], other), np.maximum(v[r], other)
            v[r] = np.where(keep_min, mn, mx)
def level(v, R, LOG, size):
    for S in range(LOG - 1, -1, -1): stage(v, R, size, 1 << S)
def sort_merge(top, cand, nkeep, R):
    M = 32 * R; LOGM = {2: 6, 4: 7}[R]
    lanes = np.arange(32)
    c = [np.where(lanes + 32 * r < nkeep, np.resize(np.concatenate([cand, np.full(M, MAXK)]), M)[lanes + 32 * r], MAXK) for r in range(R)]
    t = [top[lanes + 32 * r].copy() for r in range(R)]
    padded = 32
    while padded < nkeep: padded <<= 1
    for LOG in range(1, LOGM + 1):
        SIZE = 1 << LOG
        if SIZE <= padded: level(c, R, LOG, M if SIZE == padded else SIZE)
    for r in range(R):
        partner = c[R - 1 - r][31 - lanes]
        t[r] = np.minimum(partner, t[r])
    level(t, R, LOGM, M)
    out = np.empty(M, np.uint64)
    for r in range(R): out[lanes + 32 * r] = t[r]
    return out
def test_network_sorts_and_merges_like_a_plain_sort():
    rng = np.random.default_rng(1)
    for R in (2, 4):
        M = 32 * R
        for trial in range(400):
            nq = rng.integers(0, M + 1)           # filled part of the list
            top = np.full(M, MAXK); top[:nq] = np.sort(rng.integers(0, 1 << 40, nq).astype(np.uint64))
            nkeep = int(rng.integers(1, M + 1))
            cand = rng.integers(0, 1 << 40, nkeep).astype(np.uint64)
            got = sort_merge(top, cand, nkeep, R)
            want = np.sort(np.concatenate([top, cand]))[:M]
            assert np.array_equal(got, want), (R, trial, nkeep)


def _warp_lower_bound(a, x):
    """Model of warp_lower_bound_u64 / _u32 (csrc/common.cuh): 32 probes per round at b + (l+1)*span/33."""
    n = len(a)
    b, e = 0, n
    lanes = np.arange(32, dtype=np.int64)
    rounds = 0
    while e - b > 32:
        span = e - b
        pos = b + ((lanes + 1) * span) // 33
        assert (pos > b).all() and (pos < e).all() and (np.diff(pos) >= 1).all()
        k = int((a[pos] < x).sum())
        assert ((a[pos] < x) == (lanes < k)).all()                     # a prefix of the lanes
        nb = b + (k * span) // 33 + 1 if k > 0 else b
        ne = b + ((k + 1) * span) // 33 if k < 32 else e
        b, e = nb, ne
        rounds += 1
    idx = b + lanes
    below = (idx < e) & (a[np.minimum(idx, n - 1)] < x) if n else np.zeros(32, bool)
    return b + int(below.sum()), rounds


def test_cooperative_lower_bound_model():
    rng = np.random.default_rng(2)
    for n in (0, 1, 5, 32, 33, 34, 1000, 4097, 1 << 20):
        base = np.sort(rng.integers(0, max(2, n // 3), n).astype(np.uint64))     # many duplicates
        probes = [0, 1, np.uint64(2 ** 63)] + list(rng.integers(0, max(2, n // 3) + 2, 40).astype(np.uint64))
        for x in probes:
            got, rounds = _warp_lower_bound(base, np.uint64(x))
            assert got == int(np.searchsorted(base, np.uint64(x), side="left")), (n, x)
            assert rounds <= 4                                                   # 2^20 entries: four rounds


def test_chunked_grouping_model(oracle):
    """Model of the router's grouping kernels (csrc/router.cu): per-chunk counts, a column scan over the
    chunks, offsets, then one warp per chunk walking its ids 32 at a time and ranking equal keys by lane.
    The result must be the stable grouping the oracle computes."""
    rng = np.random.default_rng(3)
    chunk = 2048
    for n, nc in ((1, 1), (31, 3), (5000, 7), (12345, 64)):
        assign = rng.integers(0, nc, n).astype(np.uint32)
        nchunks = (n + chunk - 1) // chunk
        counts = np.zeros((nchunks, nc), np.int64)
        for i, c in enumerate(assign):
            counts[i // chunk, c] += 1
        totals = counts.sum(0)
        base = np.cumsum(counts, axis=0) - counts                     # column scan, exclusive
        offsets = np.concatenate([[0], np.cumsum(totals)])
        members = np.full(n, -1, np.int64)
        for w in range(nchunks):
            row = base[w].copy()
            for i0 in range(w * chunk, min(n, (w + 1) * chunk), 32):
                ids = np.arange(i0, min(i0 + 32, n, (w + 1) * chunk))
                keys = assign[ids]
                for lane, (i, c) in enumerate(zip(ids, keys)):
                    rank = int((keys[:lane] == c).sum())              # lanes with the same key and a lower index
                    members[offsets[c] + row[c] + rank] = i
                for c in np.unique(keys):
                    row[c] += int((keys == c).sum())                  # the leader lane advances the counter
        offs, mem = oracle.group_by_centroid(assign, nc)
        assert np.array_equal(offsets.astype(np.uint32), offs) and np.array_equal(members.astype(np.uint32), mem)
