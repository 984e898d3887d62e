"""Generates tests/golden/*.npz by running the REFERENCE's own CPU code (oracle/_ref, compiled in place from
the reference checkout by oracle/Makefile) on small seeded inputs.  Run where the reference checkout exists:

    python tests/golden/make_golden.py            # every fixture
    python tests/golden/make_golden.py NAME ...   # only the named ones

Each fixture stores its inputs and the reference's outputs, so the tests need neither the checkout nor numpy's
random streams to stay stable.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
import synth  # noqa: E402


def ivfpq_case(name, n, dim, nlist, M, nq, nprobe, topk, n_rerank, seed, zipf=False, empty=()):
    ix = synth.make_index(n, dim, nlist, M, seed=seed, zipf=zipf, empty_lists=empty)
    q = synth.make_queries(ix, nq, seed=seed + 50)
    probes, pdist = oracle.ref_coarse(q, ix["centroids"], nprobe)
    r = oracle.ref_ivfpq_search(ix, q, probes, topk, n_rerank, fine_threads=1, rerank_threads=2)
    nr = oracle.ref_ivfpq_search(dict(ix, vectors=None), q, probes, topk, 0, fine_threads=1)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        centroids=ix["centroids"], offsets=ix["offsets"], reordered_ids=ix["reordered_ids"], codes=ix["codes"],
        codebook=ix["codebook"], vectors=ix["vectors"], queries=q,
        params=np.array([nprobe, topk, n_rerank], np.int64),
        ref_probes=probes, ref_probe_dist=pdist, ref_indices=r["indices"], ref_distances=r["distances"],
        ref_stage1=r["stage1"], ref_scanned=np.int64(r["scanned"]),
        ref_norerank_indices=nr["indices"], ref_norerank_distances=nr["distances"])
    print(name, "written", r["indices"].shape)


def ivfrespq_case(name, n, dim, nlist, M, nq, nprobe, topk, n_rerank, seed, zipf=False, empty=()):
    """Residual ADC mode: the codes encode x - centroid[list]; outputs of the reference's CPU residual path."""
    ix = synth.make_index(n, dim, nlist, M, seed=seed, zipf=zipf, empty_lists=empty, residual=True)
    q = synth.make_queries(ix, nq, seed=seed + 50)
    probes, pdist = oracle.ref_coarse(q, ix["centroids"], nprobe)
    r = oracle.ref_ivfrespq_search(ix, q, probes, topk, n_rerank, threads=2)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        centroids=ix["centroids"], offsets=ix["offsets"], reordered_ids=ix["reordered_ids"], codes=ix["codes"],
        codebook=ix["codebook"], vectors=ix["vectors"], queries=q,
        params=np.array([nprobe, topk, n_rerank], np.int64),
        ref_probes=probes, ref_probe_dist=pdist, ref_indices=r["indices"], ref_distances=r["distances"],
        ref_local=r["local"], ref_scanned=np.int64(r["scanned"]))
    print(name, "written", r["indices"].shape)


def rerank_case(name, rows, dim, batch, width, topk, seed):
    rng = np.random.default_rng(seed)
    base = rng.standard_normal((rows, dim)).astype(np.float32)
    q = rng.standard_normal((batch, dim)).astype(np.float32)
    cand = rng.integers(-3, rows + 3, size=(batch, width + 5)).astype(np.int32)  # invalid ids and duplicates
    counts = rng.integers(0, width + 1, size=batch).astype(np.int32)
    ids, dist = oracle.ref_rerank(base, q, cand, topk, candidate_count=width, counts=counts, threads=2)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), base=base, queries=q, candidates=cand, counts=counts,
                        params=np.array([width, topk], np.int64), ref_ids=ids, ref_dist=dist)
    print(name, "written")


if __name__ == "__main__":
    assert oracle.have_ref(), "build oracle/_ref first: make -C oracle ref"
    print(oracle.ref_info())
    only = set(sys.argv[1:])
    cases = [
        (ivfpq_case, dict(name="ivfpq_d32_m8", n=1500, dim=32, nlist=12, M=8, nq=24, nprobe=4, topk=10, n_rerank=40, seed=11)),
        (ivfpq_case, dict(name="ivfpq_d96_m48_zipf", n=1200, dim=96, nlist=16, M=48, nq=16, nprobe=6, topk=5, n_rerank=30,
                          seed=12, zipf=True, empty=(3,))),
        (ivfpq_case, dict(name="ivfpq_d100_m20", n=900, dim=100, nlist=8, M=20, nq=12, nprobe=8, topk=10, n_rerank=64, seed=13)),
        (rerank_case, dict(name="rerank_d96", rows=300, dim=96, batch=9, width=64, topk=10, seed=21)),
        (rerank_case, dict(name="rerank_d100", rows=200, dim=100, batch=5, width=40, topk=7, seed=22)),
        # residual mode: M = 16 and M = 8 take the reference's pairwise-tree ADC order, M = 48 the sequential one;
        # topk = 512 = candidate width returns the whole stage-1 set
        (ivfrespq_case, dict(name="ivfrespq_d64_m16", n=2400, dim=64, nlist=16, M=16, nq=12, nprobe=4, topk=512,
                             n_rerank=512, seed=31)),
        (ivfrespq_case, dict(name="ivfrespq_d32_m8", n=2500, dim=32, nlist=12, M=8, nq=16, nprobe=5, topk=10, n_rerank=600,
                             seed=32)),
        (ivfrespq_case, dict(name="ivfrespq_d96_m48_zipf", n=1500, dim=96, nlist=16, M=48, nq=16, nprobe=6, topk=20,
                             n_rerank=100, seed=33, zipf=True, empty=(5,))),
    ]
    for fn, kw in cases:
        if not only or kw["name"] in only:
            fn(**kw)
