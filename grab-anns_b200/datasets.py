"""Seeded synthetic inputs with the shapes and value ranges of the benchmark configs.

They stand in for the corpora the reference's tests name (SIFT-1M, GIST, hotpotqa, wit-image),
none of which ship with it.  Generation is chunked so the 1M-vector configs stay within a few
GB of host memory.  Every generator returns float32 numpy arrays.
"""
from __future__ import annotations

import numpy as np


def _mixture(n, dim, centres, sigma, rng, chunk=1 << 18, post=None):
    out = np.empty((n, dim), dtype=np.float32)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        idx = rng.integers(0, centres.shape[0], size=e - s)
        x = centres[idx] + sigma * rng.standard_normal((e - s, dim), dtype=np.float32)
        out[s:e] = post(x) if post is not None else x
    return out


def gaussian_mixture(n, dim, n_centres, sigma, seed, centres=None):
    """Isotropic Gaussian mixture: centres ~ N(0, I), points = centre + sigma * N(0, I)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    if centres is None:
        centres = rng.standard_normal((n_centres, dim), dtype=np.float32)
    return _mixture(n, dim, centres, np.float32(sigma), rng), centres


def descriptor_like(n, dim, n_centres, seed, centres=None):
    """SIFT-like descriptors: per-dim centre ~ Gamma(1.2, 25), noise N(0, 12^2), rounded and
    clipped to [0, 255], stored as float32 (non-negative, skewed, integer valued)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    if centres is None:
        centres = rng.gamma(1.2, 25.0, size=(n_centres, dim)).astype(np.float32)
    post = lambda x: np.clip(np.rint(x), 0, 255).astype(np.float32)
    return _mixture(n, dim, centres, np.float32(12.0), rng, post=post), centres


def normalised_mixture(n, dim, n_centres, sigma, seed, centres=None, isotropic=False):
    """Embedding-like: Gaussian mixture, L2-normalised rows (inner-product metric).

    Within a cluster the noise has a 1/j variance spectrum over the dimensions (same total
    energy dim * sigma^2 as the isotropic case; participation ratio about 32 at dim 768), the
    shape trained embeddings have.  `isotropic=True` gives equal variance in every dimension:
    then all cluster mates are almost equidistant (intrinsic dimension = dim), nearest
    neighbours inside a cluster are close to random, and the recall of any graph index equals
    the fraction of the cluster it scans -- kept as a stress case."""
    rng = np.random.Generator(np.random.PCG64(seed))
    if centres is None:
        centres = rng.standard_normal((n_centres, dim), dtype=np.float32)
    if isotropic:
        sig = np.float32(sigma)
    else:
        lam = 1.0 / np.arange(1, dim + 1)
        sig = (sigma * np.sqrt(dim * lam / lam.sum())).astype(np.float32)
    post = lambda x: (x / np.linalg.norm(x, axis=1, keepdims=True)).astype(np.float32)
    return _mixture(n, dim, centres, sig, rng, post=post), centres


def zipf_labels(n, n_labels, s, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    p = 1.0 / np.arange(1, n_labels + 1) ** s
    p /= p.sum()
    return rng.choice(n_labels, size=n, p=p).astype(np.uint8)


def label_masks(nq, n_labels, seed, max_labels=3):
    rng = np.random.Generator(np.random.PCG64(seed))
    masks = np.zeros(nq, dtype=np.uint32)
    for i in range(nq):
        m = rng.integers(1, max_labels + 1)
        for lab in rng.choice(n_labels, size=m, replace=False):
            masks[i] |= np.uint32(1) << np.uint32(lab)
    return masks


def range_queries(nq, n, width, seed):
    """One timestamp range [lo, lo+width) per query, lo uniform."""
    rng = np.random.Generator(np.random.PCG64(seed))
    lo = rng.integers(0, max(1, n - width + 1), size=nq).astype(np.uint64)
    return lo, lo + np.uint64(width)


def config(name, scale=1.0, isotropic=False):
    """Workload of one benchmark config ('C1'..'C5'), optionally scaled down for tests.  C5 at scale 1 is
    100M vectors (38 GB on the host): a single process uses scale <= 0.125 (one 12.5M shard)."""
    if name == "C1":
        n, nq = int(100_000 * scale), max(8, int(1000 * scale))
        base, cen = gaussian_mixture(n, 128, 100, 0.2, 1001)
        q, _ = gaussian_mixture(nq, 128, 100, 0.2, 1002, centres=cen)
        lo, hi = range_queries(nq, n, max(1, n // 10), 1003)
        return dict(base=base, queries=q, ts=np.arange(n, dtype=np.uint64), lo=lo, hi=hi, k=10,
                    degree=32, itopk=64, metric=0, dim=128)
    if name == "C2":
        n, nq = int(1_000_000 * scale), max(8, int(10_000 * scale))
        base, cen = descriptor_like(n, 128, 1000, 2001)
        q, _ = descriptor_like(nq, 128, 1000, 2002, centres=cen)
        lo, hi = range_queries(nq, n, max(1, n // 10), 2003)
        return dict(base=base, queries=q, ts=np.arange(n, dtype=np.uint64), lo=lo, hi=hi, k=10,
                    degree=64, itopk=64, metric=0, dim=128)
    if name == "C3":
        n, nq = int(1_000_000 * scale), max(8, int(10_000 * scale))
        base, cen = normalised_mixture(n, 768, 256, 0.3, 3001, isotropic=isotropic)
        q, _ = normalised_mixture(nq, 768, 256, 0.3, 3002, centres=cen, isotropic=isotropic)
        return dict(base=base, queries=q, labels=zipf_labels(n, 16, 1.1, 3003),
                    masks=label_masks(nq, 16, 3004), k=10, degree=64, itopk=64, metric=1, dim=768)
    if name == "C4":
        n, nq = int(1_000_000 * scale), max(8, int(10_000 * scale))
        base, cen = gaussian_mixture(n, 96, 500, 0.2, 4001)
        q, _ = gaussian_mixture(nq, 96, 500, 0.2, 4002, centres=cen)
        return dict(base=base, queries=q, centres=cen, ts=np.arange(n, dtype=np.uint64), k=10,
                    degree=32, itopk=64, metric=0, dim=96)
    if name == "C5":
        n, nq = int(100_000_000 * scale), max(8, int(10_000 * min(1.0, scale * 8)))
        n_centres = max(16, int(10_000 * min(1.0, scale * 8)))
        base, cen = gaussian_mixture(n, 96, n_centres, 0.2, 5001)
        q, _ = gaussian_mixture(nq, 96, n_centres, 0.2, 5002, centres=cen)
        lo, hi = range_queries(nq, n, max(1, n // 10), 5003)
        return dict(base=base, queries=q, ts=np.arange(n, dtype=np.uint64), lo=lo, hi=hi, k=100,
                    degree=64, itopk=128, metric=0, dim=96)
    raise ValueError(name)
