"""grab_exact_search_noalloc -- the exact filtered scan with its scratch inside the library.

It exists for callers that cannot allocate device memory at call time (a serving loop that must
not take the device-wide synchronisation of cudaMalloc/cudaFree; a process whose memory pool has
already claimed the GPU).  The test calls it through the C ABI twice in a row, with different
queries and filters, and requires the very same ids and distances as the allocating entry point:
the second call proves that leftovers of the first call in the shared scratch are never read.
This file is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _noalloc(grab, data, queries, k, flt, metric=0):
    import torch
    n, dim = data.shape
    nq = queries.shape[0]
    ids = torch.full((nq, k), -7, dtype=torch.int64, device="cuda")
    dists = torch.full((nq, k), -7.0, dtype=torch.float32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]        # device-wide figure, taken around the C call alone
    rc = grab.lib().grab_exact_search_noalloc(grab._p(data), C.c_uint64(n), C.c_uint32(dim), C.c_int(metric),
                                               C.byref(flt) if flt is not None else None, grab._p(queries),
                                               C.c_uint64(nq), C.c_uint32(k), grab._p(ids), grab._p(dists), stream)
    torch.cuda.synchronize()
    _noalloc.taken = free_before - torch.cuda.mem_get_info()[0]
    return rc, ids, dists


def test_noalloc_matches_allocating_entry_point_twice(grab):
    import torch
    rng = np.random.default_rng(123)
    n, dim = 30000, 128
    data = _t(rng.standard_normal((n, dim)).astype(np.float32))
    ts = _t(np.arange(n, dtype=np.int64))
    # call 1: few queries (the scan is split across CTAs -> partial lists in the scratch), sorted-ts windows
    q1 = _t(rng.standard_normal((40, dim)).astype(np.float32))
    lo1 = _t(rng.integers(0, n - 9000, 40).astype(np.int64))
    hi1 = lo1 + 9000
    f1 = grab.make_filter(grab.FILTER_TS_RANGE, ts=ts, lo=lo1, hi=hi1, ts_sorted=True)
    # call 2: other queries, more of them, unsorted-ts path, larger k -> different scratch layout
    q2 = _t(rng.standard_normal((300, dim)).astype(np.float32))
    lo2 = _t(rng.integers(0, n - 3000, 300).astype(np.int64))
    hi2 = lo2 + 3000
    f2 = grab.make_filter(grab.FILTER_TS_RANGE, ts=ts, lo=lo2, hi=hi2, ts_sorted=False)
    # call 3: enough queries that every query is one CTA (no partial lists), inner product, label masks
    q3 = _t(rng.standard_normal((1300, dim)).astype(np.float32))
    labels = _t(rng.integers(0, 8, n).astype(np.uint8))
    masks = _t(rng.integers(1, 256, 1300).astype(np.int32))
    f3 = grab.make_filter(grab.FILTER_LABELS, labels=labels, masks=masks)
    for call, (q, k, f, metric) in enumerate([(q1, 10, f1, 0), (q2, 50, f2, 0), (q3, 10, f3, 1)]):
        want_ids, want_d = grab.exact_search(data, q, k, metric=metric, flt=f)
        rc, got_ids, got_d = _noalloc(grab, data, q, k, f, metric)
        assert rc == 0, grab.lib().grab_last_error()
        if call > 0:
            # the call took no device memory (only the very first call on a device may: that is when the driver
            # places the library image with the scratch array, see the entry point's notes)
            assert _noalloc.taken <= 0, _noalloc.taken
        assert torch.equal(got_ids, want_ids)          # same tolerance as the exact-path tests: bit-exact
        assert torch.equal(got_d, want_d)
        assert (got_ids >= 0).all()


def test_noalloc_rejects_oversized_requests(grab):
    import torch
    n, dim = 4096, 16
    data = torch.zeros((n, dim), device="cuda")
    nq = 300000                                       # windows alone exceed the 8 MiB scratch... and so do the lists
    q = torch.zeros((nq, dim), device="cuda")
    need = grab.lib().grab_exact_search_workspace_bytes(n, nq, 10)
    assert need > (8 << 20)
    rc, _, _ = _noalloc(grab, data, q, 10, None)
    assert rc == 4                                    # GRAB_ERR_WORKSPACE
    msg = grab.lib().grab_last_error().decode()
    assert "built-in scratch" in msg and str(need) in msg
