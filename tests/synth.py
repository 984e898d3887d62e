"""Seeded synthetic IVF-PQ indices for the tests (numpy only, CPU).

The shapes and value distributions follow the benchmark configurations (Gaussian mixtures, one inverted
list per mixture component, list-contiguous row order with a permutation as original ids); sizes are cut
down so the CPU checkers finish in seconds.
"""
from __future__ import annotations

import numpy as np

import oracle


def mixture(n, dim, ncomp, sigma, seed, weights=None):
    """Rows in component-contiguous order. Returns (centres, data, offsets)."""
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((ncomp, dim)).astype(np.float32)
    if weights is None:
        weights = np.full(ncomp, 1.0 / ncomp)
    counts = np.floor(weights * n).astype(np.int64)
    rem = n - counts.sum()
    order = np.argsort(-(weights * n - counts), kind="stable")
    counts[order[:rem]] += 1
    offsets = np.zeros(ncomp + 1, np.int64)
    offsets[1:] = np.cumsum(counts)
    comp = np.repeat(np.arange(ncomp), counts)
    data = centres[comp] + sigma * rng.standard_normal((n, dim)).astype(np.float32)
    return centres, data.astype(np.float32), offsets


def zipf_weights(ncomp, s=1.1):
    w = 1.0 / np.arange(1, ncomp + 1) ** s
    return w / w.sum()


def train_codebook(data, M, K, seed, iters=4, sample=20000):
    """Per-subspace Lloyd k-means (CPU checker's trainer) on a sample; codebook [M][K][dsub]."""
    rng = np.random.default_rng(seed)
    n, dim = data.shape
    dsub = dim // M
    take = rng.choice(n, size=min(sample, n), replace=False)
    cb = np.empty((M, K, dsub), np.float32)
    for m in range(M):
        sub = np.ascontiguousarray(data[take, m * dsub:(m + 1) * dsub])
        init = sub[rng.choice(sub.shape[0], size=K, replace=sub.shape[0] < K)]
        cb[m], _, _ = oracle.kmeans_lloyd(sub, init, iters)
    return cb


def make_index(n, dim, nlist, M, sigma=0.25, seed=0, zipf=False, K=256, empty_lists=(), keep_vectors=True,
               residual=False):
    """residual=True: the codebook is trained on, and the codes encode, x - centroid[list(x)]."""
    w = zipf_weights(nlist) if zipf else None
    if empty_lists:
        w = np.full(nlist, 1.0) if w is None else w.copy()
        w[list(empty_lists)] = 0.0
        w = w / w.sum()
    centres, data, offsets = mixture(n, dim, nlist, sigma, seed, w)
    coded = data
    if residual:
        coded = data - centres[np.repeat(np.arange(nlist), np.diff(offsets))]
    cb = train_codebook(coded, M, K, seed + 1)
    codes = oracle.pq_encode(coded, cb)
    rng = np.random.default_rng(seed + 2)
    reordered_ids = rng.permutation(n).astype(np.int64)
    return dict(centroids=centres, offsets=offsets, reordered_ids=reordered_ids, codes=codes, codebook=cb,
                vectors=data if keep_vectors else None, dim=dim, M=M, K=K, n=n, nlist=nlist, residual=residual)


def make_queries(index, nq, sigma=0.25, seed=100, weights=None):
    rng = np.random.default_rng(seed)
    nlist, dim = index["centroids"].shape
    comp = rng.choice(nlist, size=nq, p=weights)
    return (index["centroids"][comp] + sigma * rng.standard_normal((nq, dim))).astype(np.float32)
