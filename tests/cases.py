"""Known-answer input constructions shared by the CPU (oracle) and GPU (library) tests.

The formulas are those of the reference's unit tests (inputs are rebuilt from the formulas, no file is
copied): tests/unit/ivf_common/test_ivf_host_rerank.cpp:12-47, test_ivfpq_rerank_adapter.cpp:11-41,
test_plain_pq_pipeline.cu:9-26 in the ParaSelect tree.
"""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FLT_MAX = np.finfo(np.float32).max


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: z[k] for k in z.files}


def golden_index(g):
    return dict(centroids=g["centroids"], offsets=g["offsets"], reordered_ids=g["reordered_ids"], codes=g["codes"],
                codebook=g["codebook"], vectors=g["vectors"])


def host_rerank_case(dtype, dim, width):
    """Rows 263, batch 4, topk 10; candidates hold -1, out-of-range ids and duplicates; per-query counts
    0, 1, width/2, width; stride = width + 13."""
    rows, batch, topk = 263, 4, 10
    stride = width + 13
    r = np.arange(rows)[:, None]
    d = np.arange(dim)[None, :]
    base = (((r % 17) * 11 + d * 3) % 251).astype(dtype)
    queries = base[2:2 + batch].copy()
    counts = np.array([0, 1, width // 2, width], np.int32)
    cand = np.zeros((batch, stride), np.int32)
    for q in range(batch):
        for i in range(counts[q]):
            cand[q, i] = -1 if i % 19 == 0 else (rows + 2 if i % 23 == 0 else ((width - i) * 17 + q) % rows)
    exp_ids = np.full((batch, topk), -1, np.int32)
    exp_d = np.full((batch, topk), FLT_MAX, np.float32)
    for q in range(batch):
        seen, scored = set(), []
        for i in range(counts[q]):
            idx = int(cand[q, i])
            if idx < 0 or idx >= rows or idx in seen:
                continue
            seen.add(idx)
            s = np.float32(0)
            for j in range(dim):
                delta = np.float32(queries[q, j]) - np.float32(base[idx, j])
                s = np.float32(s + delta * delta)
            scored.append((s, idx))
        scored.sort()
        for k, (s, idx) in enumerate(scored[:topk]):
            exp_ids[q, k], exp_d[q, k] = idx, s
    return dict(base=base, queries=queries, cand=cand, counts=counts, width=width, topk=topk,
                exp_ids=exp_ids, exp_d=exp_d)


def adapter_case():
    """6 rows of dim 4 with row r filled by r; the query of interest is all 2s; candidates
    {3,2,2,1,-1,999,4,5}: expected rows {2,1,3}, distances {0,4,4}."""
    dim = 4
    base = np.repeat(np.arange(6, dtype=np.float32)[:, None], dim, axis=1)
    queries = np.zeros((2, dim), np.float32)
    queries[0] = 2
    cand = np.array([[3, 2, 2, 1, -1, 999, 4, 5], [0, 1, 2, 3, 4, 5, 0, 0]], np.int32)
    counts = np.array([8, 0], np.int32)
    return dict(base=base, queries=queries, cand=cand, counts=counts, topk=3,
                exp_ids=np.array([[2, 1, 3], [-1, -1, -1]], np.int32),
                exp_d=np.array([[0, 4, 4], [FLT_MAX] * 3], np.float32))


def plain_pq_pipeline_case(m, dim, rerank=512, empty_first=False):
    """Codes reproduce the base exactly (codebook[m][c][d] = c, code = (37 r + 11 j + r/256) % 256), four equal
    lists, queries are base rows 47 q % rows, nprobe = nlist: the search must equal exhaustive exact top-10."""
    nlist, nq, topk = 4, 19, 10
    rows = max(1024, rerank * 2)
    dsub = dim // m
    r = np.arange(rows)[:, None]
    j = np.arange(m)[None, :]
    codes = ((r * 37 + j * 11 + r // 256) % 256).astype(np.uint8)
    base = np.repeat(codes.astype(np.float32), dsub, axis=1)
    book = np.broadcast_to(np.arange(256, dtype=np.float32)[None, :, None], (m, 256, dsub)).copy()
    offsets = np.array([0, rows // 4, rows // 2, rows * 3 // 4, rows], np.int64)
    if empty_first:
        offsets[1] = 0
    queries = base[(np.arange(nq) * 47) % rows].copy()
    centroids = np.zeros((nlist, dim), np.float32)
    ids = np.arange(rows, dtype=np.int64)
    d2 = ((queries[:, None, :].astype(np.float64) - base[None, :, :].astype(np.float64)) ** 2).sum(-1)
    order = np.lexsort((np.broadcast_to(np.arange(rows), d2.shape), d2), axis=1)[:, :topk]
    exp_d = np.take_along_axis(d2, order, axis=1).astype(np.float32)  # integers: exact in fp32
    index = dict(centroids=centroids, offsets=offsets, reordered_ids=ids, codes=codes, codebook=book, vectors=base)
    return dict(index=index, queries=queries, nprobe=nlist, topk=topk, n_rerank=rerank,
                exp_ids=order.astype(np.int64), exp_d=exp_d)


def residual_pq_pipeline_case(m, dim, rerank=512):
    """The plain construction above moved into residual mode: list l has the integer centroid (3 l - 4, repeated), the
    codes reproduce base - centroid[list] exactly, so ADC = exact distance and the search must equal exhaustive top-10."""
    c = plain_pq_pipeline_case(m, dim, rerank)
    ix = c["index"]
    nlist = ix["centroids"].shape[0]
    cen = np.repeat((3.0 * np.arange(nlist, dtype=np.float32) - 4.0)[:, None], dim, axis=1)
    lists = np.repeat(np.arange(nlist), np.diff(ix["offsets"]))
    base = ix["vectors"] + cen[lists]
    rows, nq, topk = base.shape[0], c["queries"].shape[0], c["topk"]
    queries = base[(np.arange(nq) * 47) % rows].copy()
    d2 = ((queries[:, None, :].astype(np.float64) - base[None, :, :].astype(np.float64)) ** 2).sum(-1)
    order = np.lexsort((np.broadcast_to(np.arange(rows), d2.shape), d2), axis=1)[:, :topk]
    exp_d = np.take_along_axis(d2, order, axis=1).astype(np.float32)
    index = dict(ix, centroids=cen, vectors=base)
    return dict(index=index, queries=queries, nprobe=nlist, topk=topk, n_rerank=rerank,
                exp_ids=order.astype(np.int64), exp_d=exp_d)


def stage1_sets_match(got_rows, want_rows, want_dist_of):
    """Candidate sets must be equal except for members tied (equal ADC distance) at the boundary.
    want_dist_of(q, row) -> the checker's ADC distance."""
    for q in range(got_rows.shape[0]):
        a = set(int(x) for x in got_rows[q] if x >= 0)
        b = set(int(x) for x in want_rows[q] if x >= 0)
        if a == b:
            continue
        if len(a) != len(b):
            return False
        da = sorted(want_dist_of(q, r) for r in a - b)
        db = sorted(want_dist_of(q, r) for r in b - a)
        if da != db:
            return False
    return True
