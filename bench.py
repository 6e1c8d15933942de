#!/usr/bin/env python
"""Benchmark of the filtered-search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the timestamp-range filtered graph search over the whole query batch of
the workload (default: the 1M x 128 descriptor-like base, 10 000 queries, 10 % ranges, k 10,
degree 64).  Prints ONE JSON line (rank 0).  `value` is device-resident throughput, `e2e` the
same metric through the public call with host buffers, `roofline` the achieved algorithmic HBM
bandwidth of the search kernel, `cpu_baseline` the CPU exact filtered scan on the same box.
With N > 1 every rank holds a replica of the index and answers its own slice of queries
(no data-path collective).
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import numpy as np


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (tests / profiling)")
    ap.add_argument("--selectivity", type=float, default=0.10)
    ap.add_argument("--buckets", type=int, default=20)
    ap.add_argument("--local-degree", type=int, default=48)
    ap.add_argument("--itopk", type=int, default=64)
    ap.add_argument("--width", type=int, default=3)
    ap.add_argument("--max-iter", type=int, default=0,
                    help="0 = 5 with the entry-point router, 20 without")
    ap.add_argument("--router-centroids", type=int, default=1024,
                    help="centroids of the entry-point router that draws the seeds (0 = seeds drawn "
                         "uniformly inside the filter by the search kernel)")
    ap.add_argument("--probes", type=int, default=2, help="nearest centroids the seeds are taken from")
    ap.add_argument("--seeds", type=int, default=64, help="routed seeds per query")
    ap.add_argument("--hash-bitlen", type=int, default=11)
    ap.add_argument("--knn-precision", type=int, default=1,
                    help="0 exact scan, 1 bf16 tensor cores (exact for integer-valued data), 2 split bf16")
    ap.add_argument("--global-candidates", type=int, default=0,
                    help="cross-bucket candidates of the build: 0 auto, 1 all-pairs, 2 routed graph search")
    ap.add_argument("--cpu-sample", type=int, default=0, help="queries in the CPU sample (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true",
                    help="end-to-end steps on one stream (no overlap of the copies with the search)")
    ap.add_argument("--no-hnsw", action="store_true", help="reference arm: skip the CPU HNSW harness")
    ap.add_argument("--sharded", action="store_true",
                    help="stripe the index by id across the ranks (all_gather + device merge of the per-shard "
                         "top-k) instead of replicating it")
    return ap.parse_args()


def workload(args):
    ds = importlib.import_module("grab-anns_b200.datasets")
    w = ds.config(args.workload, args.scale)
    n = w["base"].shape[0]
    if "ts" in w:
        width = max(1, int(n * args.selectivity))
        w["lo"], w["hi"] = ds.range_queries(w["queries"].shape[0], n, width, 2003)
    else:
        # label workloads: vectors grouped by label (ids are arbitrary), one bucket per label
        order = np.argsort(w["labels"], kind="stable")
        w["base"] = np.ascontiguousarray(w["base"][order])
        w["labels"] = np.ascontiguousarray(w["labels"][order])
        w["label_offsets"] = np.searchsorted(w["labels"], np.arange(33), side="left").astype(np.uint32)
    return w


class ClockSampler:
    """nvidia-smi SM clock / throttle reasons sampled while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            p = [x.strip() for x in s.split(",")]
            if len(p) < 6:
                continue
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for nme, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons)}


def cpu_exact_qps(w, sample, threads_note=True):
    """CPU arm: exact filtered brute force (tests/test_cagra_auto.cu:57-89 restated, OpenMP over
    queries, sequential fp32 sum) on `sample` queries of the workload."""
    import oracle
    q = w["queries"][:sample]
    t0 = time.perf_counter()
    if "ts" in w:
        oracle.exact_search(w["base"], q, w["k"], ts=w["ts"], lo=w["lo"][:sample], hi=w["hi"][:sample],
                            metric=w["metric"], canonical=False)
    else:
        oracle.exact_search(w["base"], q, w["k"], labels=w["labels"], masks=w["masks"][:sample],
                            metric=w["metric"], canonical=False)
    dt = time.perf_counter() - t0
    return sample / dt, dt


def auto_cpu_sample(w, target_s=12.0):
    import oracle
    probe = min(oracle.num_threads() * 2, w["queries"].shape[0])
    qps, dt = cpu_exact_qps(w, probe)
    return int(max(probe, min(w["queries"].shape[0], qps * target_s)))


def hnsw_harness(w, base_n=50_000, add_n=50_000, batches=10, batch=32):
    """The reference's CPU baseline harness (tests/test_faiss_hnsw_insert.cpp:69-204) with its own sizes
    and parameters on the first vectors of the workload: HNSW M 32, efConstruction 128, efSearch 64; build
    on `base_n`, timed add of `add_n` -> vectors/s, `batches` x `batch` queries -> QPS and recall@10
    against the exact scan.  Unfiltered like the harness, plus a post-filtered variant for the range
    predicate (over-fetch k / selectivity).  HNSW restatement, not FAISS: parity unpinned."""
    import oracle
    n = min(base_n + add_n, w["base"].shape[0])
    base_n = n // 2
    data = np.ascontiguousarray(w["base"][:n])
    h = oracle.HNSW(data, M=32, ef_construction=128)
    t0 = time.perf_counter(); h.add(base_n); t1 = time.perf_counter()
    h.add(n - base_n); t2 = time.perf_counter()
    nq = min(batches * batch, w["queries"].shape[0])
    q = w["queries"][:nq]
    k = w["k"]
    t3 = time.perf_counter()
    for b in range(0, nq, batch):
        ids_b, _ = h.search(q[b:b + batch], k, ef=64)
        ids = ids_b if b == 0 else np.concatenate([ids, ids_b])
    t4 = time.perf_counter()
    gt, _ = oracle.exact_search(data, q, k, canonical=False)
    out = {"kind": "HNSW restatement (not FAISS), parity unpinned", "vectors": int(n), "cores": oracle.num_threads(),
           "build_s": t1 - t0, "insert_vectors_per_s": (n - base_n) / (t2 - t1),
           "qps_unfiltered": nq / (t4 - t3), "recall_at_10_unfiltered": oracle.recall(ids, gt)}
    if "ts" in w:  # range predicate by post-filtering an over-fetched result
        width = max(1, n // 10)
        rng = np.random.default_rng(7)
        lo = rng.integers(0, n - width + 1, nq).astype(np.uint64)
        hi = lo + np.uint64(width)
        fetch = min(n, 16 * k)
        t5 = time.perf_counter()
        ids_f, _ = h.search(q, fetch, ef=max(64, 2 * fetch))
        res = np.full((nq, k), -1, dtype=np.int64)
        for i in range(nq):
            keep = ids_f[i][(ids_f[i] >= lo[i]) & (ids_f[i] < hi[i])][:k]
            res[i, :keep.size] = keep
        t6 = time.perf_counter()
        gtf, _ = oracle.exact_search(data, q, k, ts=np.arange(n, dtype=np.uint64), lo=lo, hi=hi, canonical=False)
        out.update({"qps_range_10pct_postfilter": nq / (t6 - t5), "recall_at_10_range": oracle.recall(res, gtf),
                    "overfetch": int(fetch)})
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # torchrun pins OMP_NUM_THREADS to 1 for its workers; the CPU arm uses every core this process may run on
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import oracle
    w = workload(args)
    sample = args.cpu_sample or auto_cpu_sample(w, target_s=8.0)
    for _ in range(min(args.warmup, 1)):
        cpu_exact_qps(w, min(sample, oracle.num_threads()))
    times = []
    for _ in range(args.steps):
        _, dt = cpu_exact_qps(w, sample)
        times.append(dt)
    ms = 1e3 * float(np.mean(times))
    qps = sample / (ms / 1e3)
    desc = f"{sample} of {w['queries'].shape[0]} queries per step, full base of {w['base'].shape[0]} vectors"
    line = {
        "impl": "reference", "metric": "filtered QPS at recall@10>=0.95", "value": qps, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w),
        "recall_at_10": 1.0,
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": desc + "; exact filtered brute force, the reference's CPU ground-truth "
                                          "routine restated (FAISS-HNSW is not installed on this box)"},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_hnsw:
        line["hnsw_harness"] = hnsw_harness(w)
    print(json.dumps(line), flush=True)


def workload_config(args, w):
    filt = f"timestamp-range filter {args.selectivity:.0%}" if "ts" in w else "label filter (1-3 of 16 Zipf labels)"
    return {"workload": f"{args.workload}: {w['base'].shape[0]}x{w['dim']} fp32, {w['queries'].shape[0]} queries, "
                        f"{filt}, k {w['k']}, degree {w['degree']}",
            "n": int(w["base"].shape[0]), "dim": int(w["dim"]), "queries": int(w["queries"].shape[0]),
            "k": int(w["k"]), "graph_degree": int(w["degree"]), "local_degree": args.local_degree,
            "buckets": args.buckets if "ts" in w else 16, "selectivity": args.selectivity, "itopk": args.itopk,
            "search_width": args.width, "max_iterations": args.max_iter, "hash_bitlen": args.hash_bitlen,
            "router_centroids": args.router_centroids, "probes": args.probes, "routed_seeds": args.seeds,
            "l2": "inputs (dataset + graph, 768 MB at full size) exceed the 126 MB L2",
            "parallelism": ("one process per GPU, index striped by id across the ranks, queries broadcast, "
                            "all_gather + device merge of per-shard top-k") if getattr(args, "sharded", False) else
                           "one process per GPU, index replica per rank, queries partitioned"}


def main():
    args = parse()
    if args.max_iter == 0:
        args.max_iter = 5 if args.router_centroids else 20
    if args.impl == "reference":
        return run_reference(args)

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    grab = importlib.import_module("grab-anns_b200")
    grab.lib()  # raises if the CUDA extension is missing: there is no fallback

    w = workload(args)
    base, queries = w["base"], w["queries"]
    n, dim = base.shape
    k, deg = w["k"], w["degree"]
    sharded = importlib.import_module("grab-anns_b200.sharded")
    if args.sharded:
        # id-striped shard of this rank; the same queries on every rank
        base = np.ascontiguousarray(sharded.stripe(base, rank, world))
        w["ts"] = np.ascontiguousarray(sharded.stripe(w["ts"], rank, world))
        n = base.shape[0]
    # each rank answers its own, different slice of the query stream (same size on every rank)
    if world > 1 and not args.sharded:
        ds = importlib.import_module("grab-anns_b200.datasets")
        queries = np.roll(queries, rank * 997, axis=0)
        w["lo"], w["hi"] = ds.range_queries(queries.shape[0], n, max(1, int(n * args.selectivity)), 2003 + rank)
    nq = queries.shape[0]

    d_base = torch.from_numpy(base).cuda()
    by_labels = "ts" not in w
    if by_labels:
        if args.sharded:
            raise SystemExit("--sharded is implemented for the timestamp workloads")
        h_bucket = w["labels"].astype(np.uint64)               # one bucket per label
    else:
        d_ts = torch.from_numpy(w["ts"].view(np.int64)).cuda()
        n_total = n * world if args.sharded else n
        bsize = (n_total + args.buckets - 1) // args.buckets   # bucket width in timestamps
        h_bucket = w["ts"] // np.uint64(bsize)
    sizes = np.bincount(h_bucket.astype(np.int64)).tolist()    # sorted keys: buckets are id runs
    d_bucket = torch.from_numpy(h_bucket.view(np.int64)).cuda()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    graph = grab.build_time_partitioned_graph(d_base, d_bucket, sizes, deg, args.local_degree, metric=w["metric"],
                                              knn_precision=args.knn_precision,
                                              global_candidates=args.global_candidates)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    router, router_s = None, 0.0
    if args.router_centroids:
        t0 = time.perf_counter()
        router = grab.router_build(d_base, min(args.router_centroids, n), metric=w["metric"])
        torch.cuda.synchronize()
        router_s = time.perf_counter() - t0

    h_q = torch.from_numpy(queries).pin_memory()
    d_q = h_q.cuda()
    if by_labels:
        h_lo = torch.from_numpy(w["masks"].view(np.int32)).pin_memory()    # per-query label masks
        h_hi = h_lo
        d_lo = d_hi = h_lo.cuda()
        d_labels = torch.from_numpy(w["labels"]).cuda()
        d_offs = torch.from_numpy(w["label_offsets"].view(np.int32)).cuda()
        flt = grab.make_filter(grab.FILTER_LABELS, labels=d_labels, masks=d_lo, label_offsets=d_offs)
    else:
        h_lo = torch.from_numpy(w["lo"].view(np.int64)).pin_memory()
        h_hi = torch.from_numpy(w["hi"].view(np.int64)).pin_memory()
        d_lo, d_hi = h_lo.cuda(), h_hi.cuda()
        flt = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=d_lo, hi=d_hi, ts_sorted=True)
    params = grab.SearchParams(args.itopk, args.width, 0, args.max_iter, args.hash_bitlen)
    out_ids = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    h_ids = torch.empty((nq, k), dtype=torch.int64).pin_memory()
    h_d = torch.empty((nq, k), dtype=torch.float32).pin_memory()
    ws = torch.empty(grab.lib().grab_graph_search_workspace_bytes(nq, args.hash_bitlen), dtype=torch.uint8,
                     device="cuda")

    seeds = route_ws = None
    if router is not None:
        seeds = torch.empty((nq, args.seeds), dtype=torch.int32, device="cuda")
        route_ws = torch.empty(grab.lib().grab_route_seeds_workspace_bytes(nq, args.probes), dtype=torch.uint8,
                               device="cuda")

    def route():
        if router is not None:
            grab.route_seeds(router, d_q, n, flt, probes=args.probes, seeds_per_query=args.seeds, out=seeds,
                             ws=route_ws)

    id_scale, id_offset = (world, rank) if args.sharded else (1, 0)
    merge = lambda d, i, kk: grab.merge_topk(d, i, kk)
    # ground truth from the exact filtered kernel (bit-exact against the CPU oracle in tests/)
    gt_ids, gt_d = grab.exact_search(d_base, d_q, k, metric=w["metric"], flt=flt)
    route()
    ids, dd, stats = grab.graph_search(d_base, graph, d_q, k, params, metric=w["metric"], flt=flt, stats=True,
                                       seeds=seeds, out=(out_ids, out_d), ws=ws, id_scale=id_scale,
                                       id_offset=id_offset)
    if args.sharded:
        gt_ids = torch.where(gt_ids >= 0, gt_ids * world + rank, gt_ids)
        gt_ids, _ = sharded.gather_and_merge(gt_d, gt_ids, k, merge)
        ids, _ = sharded.gather_and_merge(dd, ids, k, merge)
        st = torch.tensor([stats.iterations, stats.parents, stats.edges, stats.distances, stats.seeds,
                           stats.hash_resets], device="cuda", dtype=torch.int64)
        dist.all_reduce(st) if dist is not None else None
        stats = grab.SearchStats(*st.cpu().tolist())
    gt = gt_ids.cpu().numpy()
    res = ids.cpu().numpy()
    hit = 0
    denom = 0
    for r, g in zip(res, gt):
        g = g[g >= 0]
        hit += np.intersect1d(r, g).size
        denom += g.size
    recall = hit / max(denom, 1)
    if by_labels:
        lab = w["labels"][np.clip(res, 0, n - 1)]
        in_range = bool(np.all((((w["masks"][:, None] >> lab) & 1) == 1) | (res < 0)))
    else:  # timestamps equal global ids in this workload
        in_range = bool(np.all(((res >= w["lo"][:, None].astype(np.int64)) &
                                (res < w["hi"][:, None].astype(np.int64))) | (res < 0)))
    # sorted timestamps: id-window predicate, no gather (f = 0); labels: one byte per examined edge;
    # sharded: every rank reads every query
    alg_bytes = grab.search_bytes(stats, nq * (world if args.sharded else 1), dim, deg, k, 1 if by_labels else 0)

    def search_only():
        grab.graph_search(d_base, graph, d_q, k, params, metric=w["metric"], flt=flt, seeds=seeds,
                          out=(out_ids, out_d), ws=ws, id_scale=id_scale, id_offset=id_offset)

    def step():
        route()
        search_only()
        if args.sharded:
            sharded.gather_and_merge(out_d, out_ids, k, merge)

    def e2e_step():
        d_q.copy_(h_q, non_blocking=True)
        d_lo.copy_(h_lo, non_blocking=True)
        if not by_labels:
            d_hi.copy_(h_hi, non_blocking=True)
        step()
        h_ids.copy_(out_ids, non_blocking=True)
        h_d.copy_(out_d, non_blocking=True)

    def make_pipeline():
        """End-to-end steps as a serving loop runs them: two sets of device/pinned buffers, the host->device
        copies of step i+1 and the device->host copies of step i-1 on their own streams while step i searches.
        Every step still moves its own queries, filter values and results across PCIe inside the timed region."""
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        sets = []
        for _ in range(2):
            q_ = torch.empty_like(d_q)
            lo_ = torch.empty_like(d_lo)
            hi_ = lo_ if by_labels else torch.empty_like(d_hi)
            if by_labels:
                f_ = grab.make_filter(grab.FILTER_LABELS, labels=d_labels, masks=lo_, label_offsets=d_offs)
            else:
                f_ = grab.make_filter(grab.FILTER_TS_RANGE, ts=d_ts, lo=lo_, hi=hi_, ts_sorted=True)
            sets.append(dict(q=q_, lo=lo_, hi=hi_, flt=f_, ids=torch.empty_like(out_ids), d=torch.empty_like(out_d),
                             h_ids=torch.empty((nq, k), dtype=torch.int64).pin_memory(),
                             h_d=torch.empty((nq, k), dtype=torch.float32).pin_memory(),
                             ev_in=torch.cuda.Event(), ev_done=torch.cuda.Event(), ev_out=torch.cuda.Event(),
                             used=False))
        count = [0]

        def fn():
            b = sets[count[0] % 2]
            count[0] += 1
            main = torch.cuda.current_stream()
            with torch.cuda.stream(s_in):
                if b["used"]:
                    s_in.wait_event(b["ev_done"])      # the search that read this set has finished
                b["q"].copy_(h_q, non_blocking=True)
                b["lo"].copy_(h_lo, non_blocking=True)
                if not by_labels:
                    b["hi"].copy_(h_hi, non_blocking=True)
                b["ev_in"].record(s_in)
            main.wait_event(b["ev_in"])
            if b["used"]:
                main.wait_event(b["ev_out"])           # the previous results of this set have left
            sd = None
            if router is not None:
                sd = grab.route_seeds(router, b["q"], n, b["flt"], probes=args.probes, seeds_per_query=args.seeds,
                                      out=seeds, ws=route_ws)
            grab.graph_search(d_base, graph, b["q"], k, params, metric=w["metric"], flt=b["flt"], seeds=sd,
                              out=(b["ids"], b["d"]), ws=ws)
            b["ev_done"].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(b["ev_done"])
                b["h_ids"].copy_(b["ids"], non_blocking=True)
                b["h_d"].copy_(b["d"], non_blocking=True)
                b["ev_out"].record(s_out)
            b["used"] = True

        def drain():
            main = torch.cuda.current_stream()
            for b in sets:
                if b["used"]:
                    main.wait_event(b["ev_out"])
        return fn, drain, sets

    def timed_pipeline(steps, warmup):
        fn, drain, sets = make_pipeline()
        for _ in range(warmup):
            fn()
        drain()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        drain()
        b.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        t = torch.tensor([a.elapsed_time(b)], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ref_ids = ids.cpu()
        same = all(float((s_["h_ids"] == ref_ids).float().mean()) > 0.999 for s_ in sets if s_["used"])
        return float(t.item()) / steps, same

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in evs:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    # the timed region lasts milliseconds, an nvidia-smi sample takes 100 ms: the same kernels keep the GPU
    # under load before and after the timed steps until the sampler has collected a few samples.  The loops
    # run a rank-dependent number of times, so they must not contain a collective (the sharded step does).
    def load_step():
        route()
        search_only()

    sampler = ClockSampler(local_rank)
    sampler.start()
    t_end = time.perf_counter() + 1.5
    while len(sampler.samples) < 1 and time.perf_counter() < t_end:
        load_step()
        torch.cuda.synchronize()
    ms = timed(step, args.steps, max(args.warmup, 3))
    t_end = time.perf_counter() + 1.0
    have = len(sampler.samples)
    while len(sampler.samples) < have + 3 and time.perf_counter() < t_end:
        load_step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_e2e = timed(e2e_step, args.steps, max(args.warmup, 3))
    e2e_mode = "one stream: copy in, search, copy out, per step"
    if not args.sharded and not args.no_overlap:
        ms_e2e_seq = ms_e2e
        ms_e2e, same = timed_pipeline(args.steps, max(args.warmup, 3))
        if not same:
            raise SystemExit("pipelined end-to-end steps returned different ids")
        e2e_mode = ("double-buffered: the copies of neighbouring steps overlap the search on separate streams "
                    f"(one stream, no overlap: {nq / (ms_e2e_seq / 1e3) * world:.0f} queries/s)")
    # the dominant kernel alone (the search launch with the routed seeds already written), for the roofline
    ms_search = timed(search_only, args.steps, max(args.warmup, 3)) if router is not None or args.sharded else ms

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        sample = args.cpu_sample or auto_cpu_sample(w)
        cqps, cdt = cpu_exact_qps(w, sample)
        cpu = {"value": cqps, "unit": "queries/s", "cores": oracle.num_threads(), "kind": "port",
               "sample": f"{sample} of {nq} queries over the full {n}-vector base in {cdt:.1f} s; exact filtered "
                         "brute force (recall 1.0), OpenMP over queries"}

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        if args.sharded:
            alg_bytes //= world     # counters were summed over the ranks; the roofline is one GPU's launch
        achieved = alg_bytes / (ms_search / 1e3) / 1e9
        # dram__bytes_read.sum + dram__bytes_write.sum of one search launch at the default full-size
        # configuration (ncu capture summarised in profiles/graph_search_kernel_C2.md)
        default_cfg = (args.workload == "C2" and args.scale == 1.0 and args.buckets == 20 and args.itopk == 64 and
                       args.width == 3 and args.max_iter == 5 and args.hash_bitlen == 11 and
                       args.selectivity == 0.10 and not args.sharded and args.router_centroids == 1024 and
                       args.probes == 2 and args.seeds == 64 and args.local_degree == 48 and
                       args.global_candidates in (0, 1))
        traffic = 1364566272 + 1159168 if default_cfg else None
        line = {
            "metric": "filtered QPS at recall@10>=0.95",
            "value": (1 if args.sharded else world) * nq / (ms / 1e3), "unit": "queries/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if args.sharded else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(args, w),
            "recall_at_10": recall, "results_in_range": in_range,
            "build": {"seconds": build_s, "mvec_per_s": n / build_s / 1e6, "knn_precision": args.knn_precision,
                      "global_candidates": args.global_candidates,
                      "router_seconds": router_s},
            "ms_search_kernel": ms_search, "ms_router": ms - ms_search if router is not None and not args.sharded else None,
            "e2e": {"value": (1 if args.sharded else world) * nq / (ms_e2e / 1e3), "unit": "queries/s",
                    "h2d_bytes_per_step": int(h_q.numel() * 4 + (4 if by_labels else 16) * nq),
                    "d2h_bytes_per_step": int(12 * nq * k), "mode": e2e_mode},
            # per step: nearest-centroids + seed picking (router), id windows (sorted timestamps), search,
            # and the merge after the all_gather when sharded
            "gpu_launches": ((2 if router is not None else 0) + (1 if by_labels else 2) +
                             (2 if args.sharded and world > 1 else 0)) * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "peak_source": "measured" if peaks else "fallback",
                         "algorithmic_bytes_per_launch": int(alg_bytes),
                         "counters": {"seeds": stats.seeds, "parents": stats.parents, "edges": stats.edges,
                                      "distances": stats.distances, "iterations": stats.iterations,
                                      "hash_resets": stats.hash_resets}},
            "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
