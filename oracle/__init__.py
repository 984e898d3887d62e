"""TEST INFRASTRUCTURE: ctypes loaders for the CPU checkers.

`lib()` is the plain-C restatement (oracle/psb_oracle.c, parity pinned against the reference's
own CPU code).  `ref()` is that reference CPU code itself, compiled in place by oracle/Makefile
into oracle/_ref/ (present only where it was built).  Only tests, the smoke entry and the
bench's CPU legs may import this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "libpsb_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libpsb_ref.so")
REF_TRAIN_SO = os.path.join(_HERE, "_ref", "libpsb_ref_train.so")
REF_ROWCORR_SO = os.path.join(_HERE, "_ref", "libpsb_ref_rowcorr.so")
REF_CACHE_SO = os.path.join(_HERE, "_ref", "libpsb_ref_cache.so")
REF_KMEANS_INIT_SO = os.path.join(_HERE, "_ref", "libpsb_ref_kmeans_init.so")
_lib = None
_ref = None
_ref_train = None
_ref_rowcorr = None

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")


def build(ref_too: bool = True) -> None:
    """Compile the restatement and, when the reference checkout is present, oracle/_ref."""
    targets = ["oracle"] + (["ref"] if ref_too else [])
    subprocess.run(["make", "-s", "-C", _HERE] + targets, check=True)


def _ptr(a, ctype=None):
    if a is None:
        return None
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(ref_too=False)
        _lib = C.CDLL(ORACLE_SO)
        _lib.psbo_l2_exact.restype = C.c_float
        _lib.psbo_recall.restype = C.c_double
    return _lib


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref():
    global _ref
    if _ref is None:
        _ref = C.CDLL(REF_SO)
        _ref.psbref_last_error.restype = C.c_char_p
        _ref.psbref_fp32_isa.restype = C.c_char_p
    return _ref


def have_ref_train() -> bool:
    return os.path.exists(REF_TRAIN_SO)


def ref_train():
    """The reference's IVF-Flat search, CPU Lloyd k-means and CPU PQ trainer / encoder (oracle/ref_train_harness.cu)."""
    global _ref_train
    if _ref_train is None:
        _ref_train = C.CDLL(REF_TRAIN_SO)
    return _ref_train


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------- restatement wrappers
def l2_exact(q, v):
    q = _c(q, np.float32); v = _c(v, np.float32)
    return float(lib().psbo_l2_exact(_ptr(q), _ptr(v), C.c_int(q.size)))


def coarse(queries, centroids, nprobe):
    queries = _c(queries, np.float32); centroids = _c(centroids, np.float32)
    nq, dim = queries.shape
    ids = np.empty((nq, nprobe), np.int64); dist = np.empty((nq, nprobe), np.float32)
    rc = lib().psbo_coarse(_ptr(queries), nq, _ptr(centroids), centroids.shape[0], dim, nprobe, _ptr(ids), _ptr(dist))
    if rc:
        raise ValueError("oracle coarse: invalid arguments")
    return ids, dist


def pq_lut(queries, codebook):
    queries = _c(queries, np.float32); codebook = _c(codebook, np.float32)
    nq, dim = queries.shape
    M, K, _ = codebook.shape
    luts = np.empty((nq, M, K), np.float32)
    rc = lib().psbo_pq_lut_batch(_ptr(queries), nq, dim, _ptr(codebook), M, K, _ptr(luts))
    if rc:
        raise ValueError("oracle lut: invalid arguments")
    return luts


def pq_lut_u8(lut, residual=False):
    lut = _c(lut, np.float32)
    M, K = lut.shape
    q8 = np.empty((M, K), np.uint8); scales = np.empty(M, np.float32)
    lo = C.c_float(); inf = C.c_float()
    lib().psbo_pq_lut_u8(_ptr(lut), M, K, int(residual), _ptr(q8), _ptr(scales), C.byref(lo), C.byref(inf))
    return q8, scales, lo.value, inf.value


def pq_scan(queries, probes, offsets, codes, codebook, stage1_k):
    queries = _c(queries, np.float32); probes = _c(probes, np.int64); offsets = _c(offsets, np.int64)
    codes = _c(codes, np.uint8); codebook = _c(codebook, np.float32)
    nq, dim = queries.shape
    M, K, _ = codebook.shape
    rows = np.empty((nq, stage1_k), np.int32); dist = np.empty((nq, stage1_k), np.float32)
    cnt = np.empty(nq, np.int32); scanned = C.c_longlong()
    rc = lib().psbo_pq_scan(_ptr(queries), nq, dim, _ptr(probes), probes.shape[1], _ptr(offsets), offsets.size - 1,
                            _ptr(codes), _ptr(codebook), M, K, stage1_k, _ptr(rows), _ptr(dist), _ptr(cnt),
                            C.byref(scanned))
    if rc:
        raise ValueError("oracle scan: invalid arguments")
    return rows, dist, cnt, scanned.value


def rerank(base, queries, candidates, topk, candidate_count=None, counts=None):
    """base/queries fp32 or uint8 (matching); candidates int32 [batch][stride]."""
    u8 = base.dtype == np.uint8
    base = _c(base, np.uint8 if u8 else np.float32); queries = _c(queries, np.uint8 if u8 else np.float32)
    candidates = _c(candidates, np.int32)
    batch, stride = candidates.shape
    cc = stride if candidate_count is None else candidate_count
    ids = np.empty((batch, topk), np.int32); dist = np.empty((batch, topk), np.float32)
    cnts = None if counts is None else _c(counts, np.int32)
    rc = lib().psbo_rerank(None if u8 else _ptr(base), _ptr(base) if u8 else None, C.c_int64(base.shape[0]),
                           base.shape[1], None if u8 else _ptr(queries), _ptr(queries) if u8 else None,
                           _ptr(candidates), batch, cc, stride, topk, _ptr(cnts), _ptr(ids), _ptr(dist))
    if rc:
        raise ValueError("oracle rerank: invalid arguments")
    return ids, dist


def map_ids(local, reordered_ids):
    local = _c(local, np.int32); reordered_ids = _c(reordered_ids, np.int64)
    out = np.empty(local.shape, np.int64)
    lib().psbo_map_ids(_ptr(local), C.c_int64(local.size), _ptr(reordered_ids), _ptr(out))
    return out


def ivfpq_search(index, queries, nprobe, topk, n_rerank):
    """index: dict(centroids, offsets, reordered_ids, codes, codebook[M,K,dsub], vectors or None)."""
    queries = _c(queries, np.float32)
    nq, dim = queries.shape
    cen = _c(index["centroids"], np.float32); off = _c(index["offsets"], np.int64)
    rid = _c(index["reordered_ids"], np.int64); codes = _c(index["codes"], np.uint8)
    cb = _c(index["codebook"], np.float32)
    vec = index.get("vectors")
    vec = None if vec is None else _c(vec, np.float32)
    M, K, _ = cb.shape
    n = codes.shape[0]
    rr = vec is not None and n_rerank > topk
    s1 = min(n_rerank, n) if rr else topk
    out_i = np.empty((nq, topk), np.int64); out_d = np.empty((nq, topk), np.float32)
    out_c = np.empty((nq, nprobe), np.int64); out_s = np.empty((nq, s1), np.int32)
    scanned = C.c_longlong()
    rc = lib().psbo_ivfpq_search(_ptr(cen), cen.shape[0], dim, _ptr(off), _ptr(rid), C.c_int64(n), _ptr(codes),
                                 _ptr(cb), M, K, _ptr(vec), _ptr(queries), nq, nprobe, topk, n_rerank,
                                 _ptr(out_i), _ptr(out_d), _ptr(out_c), _ptr(out_s), C.byref(scanned))
    if rc:
        raise ValueError("oracle ivfpq_search: invalid arguments")
    return dict(indices=out_i, distances=out_d, coarse=out_c, stage1=out_s, scanned=scanned.value)


def rotate_rows(rows, matrix):
    """rows @ matrix.T with the in-order fp32 fma chain (matrix row-major [out][in])."""
    rows = _c(rows, np.float32); matrix = _c(matrix, np.float32)
    out = np.empty_like(rows)
    if lib().psbo_rotate_rows(_ptr(rows), _ptr(matrix), C.c_int64(rows.shape[0]), rows.shape[1], _ptr(out)):
        raise ValueError("oracle rotate_rows: invalid arguments")
    return out


def ivfpq_search_opq(index, queries, nprobe, topk, n_rerank, opq_matrix):
    """The plain pipeline on an OPQ index: coarse and exact re-ranking on the caller's queries, PQ tables and code scan on the
    rotated ones (src/search/ivfpq/ivfpq_index.cu:205-217, stage/ivfpq_fine_cpu_lut.cpp:29-31)."""
    queries = _c(queries, np.float32)
    vec = index.get("vectors")
    n = index["codes"].shape[0]
    rr = vec is not None and n_rerank > topk
    s1 = min(n_rerank, n) if rr else topk
    probes, _ = coarse(queries, index["centroids"], nprobe)
    rows, dist, cnt, scanned = pq_scan(rotate_rows(queries, opq_matrix), probes, index["offsets"], index["codes"], index["codebook"], s1)
    if rr:
        local, d = rerank(vec, queries, rows, topk, counts=cnt)
    else:
        local, d = rows[:, :topk].astype(np.int64), dist[:, :topk]
    return dict(indices=map_ids(local, index["reordered_ids"]), distances=d, coarse=probes, stage1=rows, scanned=scanned)


def pq_scan_residual(queries, probes, centroids, offsets, codes, codebook, stage1_k, want_luts=False):
    """Stage 1 of the residual mode; returns rows, dist, count, scanned (and the tables [nq][nprobe][M*K])."""
    queries = _c(queries, np.float32); probes = _c(probes, np.int64); offsets = _c(offsets, np.int64)
    centroids = _c(centroids, np.float32); codes = _c(codes, np.uint8); codebook = _c(codebook, np.float32)
    nq, dim = queries.shape
    M, K, _ = codebook.shape
    rows = np.empty((nq, stage1_k), np.int32); dist = np.empty((nq, stage1_k), np.float32)
    cnt = np.empty(nq, np.int32); scanned = C.c_longlong()
    luts = np.zeros((nq, probes.shape[1], M * K), np.float32) if want_luts else None
    rc = lib().psbo_pq_scan_residual(_ptr(queries), nq, dim, _ptr(probes), probes.shape[1], _ptr(centroids),
                                     _ptr(offsets), offsets.size - 1, _ptr(codes), _ptr(codebook), M, K, stage1_k,
                                     _ptr(rows), _ptr(dist), _ptr(cnt), _ptr(luts), C.byref(scanned))
    if rc:
        raise ValueError("oracle residual scan: invalid arguments")
    return (rows, dist, cnt, scanned.value, luts) if want_luts else (rows, dist, cnt, scanned.value)


def residual_stage1_width(topk, n_rerank):
    return int(lib().psbo_residual_stage1_width(topk, n_rerank))


def ivfrespq_search(index, queries, nprobe, topk, n_rerank):
    """Residual ADC mode (codes encode x - centroid[list]); index as for ivfpq_search, vectors required."""
    queries = _c(queries, np.float32)
    nq, dim = queries.shape
    cen = _c(index["centroids"], np.float32); off = _c(index["offsets"], np.int64)
    rid = _c(index["reordered_ids"], np.int64); codes = _c(index["codes"], np.uint8)
    cb = _c(index["codebook"], np.float32); vec = _c(index["vectors"], np.float32)
    M, K, _ = cb.shape
    n = codes.shape[0]
    s1 = residual_stage1_width(topk, n_rerank)
    out_i = np.empty((nq, topk), np.int64); out_d = np.empty((nq, topk), np.float32)
    out_c = np.empty((nq, nprobe), np.int64); out_s = np.empty((nq, s1), np.int32); out_n = np.empty(nq, np.int32)
    scanned = C.c_longlong()
    rc = lib().psbo_ivfrespq_search(_ptr(cen), cen.shape[0], dim, _ptr(off), _ptr(rid), C.c_int64(n), _ptr(codes),
                                    _ptr(cb), M, K, _ptr(vec), _ptr(queries), nq, nprobe, topk, n_rerank,
                                    _ptr(out_i), _ptr(out_d), _ptr(out_c), _ptr(out_s), _ptr(out_n), C.byref(scanned))
    if rc:
        raise ValueError("oracle ivfrespq_search: invalid arguments")
    return dict(indices=out_i, distances=out_d, coarse=out_c, stage1=out_s, stage1_count=out_n, scanned=scanned.value)


def ivfflat_search(centroids, offsets, reordered_ids, base, queries, nprobe, topk):
    queries = _c(queries, np.float32); centroids = _c(centroids, np.float32); base = _c(base, np.float32)
    offsets = _c(offsets, np.int64)
    rid = None if reordered_ids is None else _c(reordered_ids, np.int64)
    nq, dim = queries.shape
    out_i = np.empty((nq, topk), np.int64); out_d = np.empty((nq, topk), np.float32)
    rc = lib().psbo_ivfflat_search(_ptr(centroids), centroids.shape[0], dim, _ptr(offsets), _ptr(rid), _ptr(base),
                                   _ptr(queries), nq, nprobe, topk, _ptr(out_i), _ptr(out_d))
    if rc:
        raise ValueError("oracle ivfflat_search: invalid arguments")
    return out_i, out_d


def kmeans_lloyd(data, init_centroids, iters):
    data = _c(data, np.float32); cen = np.array(init_centroids, dtype=np.float32, order="C", copy=True)
    n, dim = data.shape
    assign = np.empty(n, np.int32); obj = np.empty(iters + 1, np.float64)
    lib().psbo_kmeans_lloyd(_ptr(data), C.c_int64(n), dim, _ptr(cen), cen.shape[0], iters, _ptr(assign), _ptr(obj))
    return cen, assign, obj


def kmeans_assign(data, centroids):
    data = _c(data, np.float32); centroids = _c(centroids, np.float32)
    n, dim = data.shape
    assign = np.empty(n, np.int32); dist = np.empty(n, np.float32)
    lib().psbo_kmeans_assign(_ptr(data), C.c_int64(n), dim, _ptr(centroids), centroids.shape[0], _ptr(assign), _ptr(dist))
    return assign, dist


def pq_encode(data, codebook):
    data = _c(data, np.float32); codebook = _c(codebook, np.float32)
    n, dim = data.shape
    M, K, _ = codebook.shape
    codes = np.empty((n, M), np.uint8)
    rc = lib().psbo_pq_encode(_ptr(data), C.c_int64(n), dim, _ptr(codebook), M, K, _ptr(codes))
    if rc:
        raise ValueError("oracle pq_encode: invalid arguments")
    return codes


def recall(got, truth):
    got = _c(got, np.int64); truth = _c(truth, np.int64)
    return float(lib().psbo_recall(_ptr(got), _ptr(truth), got.shape[0], got.shape[1]))


# ---------------------------------------------------------------- reference (oracle/_ref) wrappers
def ref_info():
    r = ref()
    return dict(isa=r.psbref_fp32_isa().decode(), physical_cores=int(r.psbref_physical_cores()))


def ref_coarse(queries, centroids, nprobe, threads=0):
    queries = _c(queries, np.float32); centroids = _c(centroids, np.float32)
    nq, dim = queries.shape
    ids = np.empty((nq, nprobe), np.int64); dist = np.empty((nq, nprobe), np.float32)
    rc = ref().psbref_coarse(_ptr(queries), nq, _ptr(centroids), centroids.shape[0], dim, nprobe, _ptr(ids), _ptr(dist), threads)
    if rc:
        raise ValueError(ref().psbref_last_error().decode())
    return ids, dist


def ref_ivfpq_search(index, queries, probes, topk, n_rerank, fine_threads=1, rerank_threads=0):
    queries = _c(queries, np.float32); probes = _c(probes, np.int64)
    nq, dim = queries.shape
    nprobe = probes.shape[1]
    cen = _c(index["centroids"], np.float32); off = _c(index["offsets"], np.int64)
    rid = _c(index["reordered_ids"], np.int64); codes = _c(index["codes"], np.uint8)
    cb = _c(index["codebook"], np.float32)
    vec = index.get("vectors")
    vec = None if vec is None else _c(vec, np.float32)
    M, K, _ = cb.shape
    n = codes.shape[0]
    rr = vec is not None and n_rerank > topk
    s1 = min(n_rerank, n) if rr else topk
    out_i = np.empty((nq, topk), np.int64); out_d = np.empty((nq, topk), np.float32)
    out_s = np.empty((nq, s1), np.int32)
    times = np.zeros(3, np.float64); scanned = C.c_longlong()
    rc = ref().psbref_ivfpq_search(_ptr(cen), cen.shape[0], dim, _ptr(off), _ptr(rid), C.c_int64(n), _ptr(codes),
                                   _ptr(cb), M, K, _ptr(vec), _ptr(queries), nq, _ptr(probes), nprobe, topk, n_rerank,
                                   fine_threads, rerank_threads, _ptr(out_i), _ptr(out_d), _ptr(out_s),
                                   _ptr(times), C.byref(scanned))
    if rc:
        raise RuntimeError(ref().psbref_last_error().decode())
    return dict(indices=out_i, distances=out_d, stage1=out_s, times_ms=times, scanned=scanned.value)


def ref_ivfrespq_search(index, queries, probes, topk, n_rerank, threads=1):
    queries = _c(queries, np.float32); probes = _c(probes, np.int64)
    nq, dim = queries.shape
    nprobe = probes.shape[1]
    cen = _c(index["centroids"], np.float32); off = _c(index["offsets"], np.int64)
    rid = _c(index["reordered_ids"], np.int64); codes = _c(index["codes"], np.uint8)
    cb = _c(index["codebook"], np.float32); vec = _c(index["vectors"], np.float32)
    M, K, _ = cb.shape
    n = codes.shape[0]
    out_l = np.empty((nq, topk), np.int32); out_i = np.empty((nq, topk), np.int64)
    out_d = np.full((nq, topk), np.finfo(np.float32).max, np.float32)
    times = np.zeros(3, np.float64); scanned = C.c_longlong()
    rc = ref().psbref_ivfrespq_search(_ptr(cen), cen.shape[0], dim, _ptr(off), _ptr(rid), C.c_int64(n), _ptr(codes),
                                      _ptr(cb), M, K, _ptr(vec), _ptr(queries), nq, _ptr(probes), nprobe, topk,
                                      n_rerank, threads, _ptr(out_l), _ptr(out_i), _ptr(out_d), _ptr(times),
                                      C.byref(scanned))
    if rc:
        raise RuntimeError(ref().psbref_last_error().decode())
    return dict(indices=out_i, distances=out_d, local=out_l, times_ms=times, scanned=scanned.value)


def ref_rerank(base, queries, candidates, topk, candidate_count=None, counts=None, threads=1, prefetch=4):
    u8 = base.dtype == np.uint8
    base = _c(base, np.uint8 if u8 else np.float32); queries = _c(queries, np.uint8 if u8 else np.float32)
    candidates = _c(candidates, np.int32)
    batch, stride = candidates.shape
    cc = stride if candidate_count is None else candidate_count
    ids = np.empty((batch, topk), np.int32); dist = np.empty((batch, topk), np.float32)
    cnts = None if counts is None else _c(counts, np.int32)
    rc = ref().psbref_rerank_host(None if u8 else _ptr(base), _ptr(base) if u8 else None, C.c_int64(base.shape[0]),
                                  base.shape[1], None if u8 else _ptr(queries), _ptr(queries) if u8 else None,
                                  _ptr(candidates), batch, cc, stride, topk, _ptr(cnts), threads, prefetch,
                                  _ptr(ids), _ptr(dist))
    if rc == 1:
        raise ValueError(ref().psbref_last_error().decode())
    if rc:
        raise RuntimeError(ref().psbref_last_error().decode())
    return ids, dist


# ---------------------------------------------------------------- reference wrappers: IVF-Flat, k-means, PQ training
def ref_cpu_ivf_search(centroids, offsets, reordered_ids, base, queries, nprobe, topk):
    """cpu_ivf_search (src/cpu/search/cpu_search.h:226-332): ids, distances, coarse ids, coarse distances."""
    queries = _c(queries, np.float32); centroids = _c(centroids, np.float32); base = _c(base, np.float32)
    offsets = _c(offsets, np.int64)
    rid = None if reordered_ids is None else _c(reordered_ids, np.int64)
    nq, dim = queries.shape
    out_i = np.empty((nq, topk), np.int64); out_d = np.empty((nq, topk), np.float32)
    c_i = np.empty((nq, nprobe), np.int64); c_d = np.empty((nq, nprobe), np.float32)
    ref_train().psbref_cpu_ivf_search(_ptr(queries), nq, dim, _ptr(base), _ptr(centroids), centroids.shape[0], _ptr(offsets),
                                      _ptr(rid), nprobe, topk, _ptr(out_i), _ptr(out_d), _ptr(c_i), _ptr(c_d))
    return out_i, out_d, c_i, c_d


def ref_kmeans_lloyd(data, init_centroids, iters):
    """cpu_kmeans_lloyd (src/cpu/clustering/cpu_kmeans.h:27-143): centroids after `iters` iterations, the assignment made in
    the last iteration (against the centroids it started from) and that iteration's objective."""
    data = _c(data, np.float32); cen = np.array(init_centroids, dtype=np.float32, order="C", copy=True)
    n, dim = data.shape
    assign = np.empty(n, np.int32); obj = C.c_float()
    ref_train().psbref_cpu_kmeans_lloyd(_ptr(data), n, dim, cen.shape[0], iters, _ptr(cen), _ptr(assign), C.byref(obj))
    return cen, assign, float(obj.value)


def ref_pq_train_encode(data, M, K):
    """PQQuantizerCPU::train + ::encode (src/quantization/pq/pq_quantizer_cpu.cpp:26-68): codebook [M][K][dsub], codes [n][M]."""
    data = _c(data, np.float32)
    n, dim = data.shape
    cb = np.empty((M, K, dim // M), np.float32); codes = np.empty((n, M), np.uint8)
    rc = ref_train().psbref_pq_train_encode(_ptr(data), n, dim, M, K, _ptr(cb), _ptr(codes))
    if rc:
        raise ValueError("reference PQ training refused the shape")
    return cb, codes


def ref_pq_init_rows(n, K, seed):
    rows = np.empty(K, np.int32)
    ref_train().psbref_pq_init_rows(n, K, C.c_uint(seed), _ptr(rows))
    return rows


def ref_pq_kmeans_subspace(sub, K, iters, seed):
    sub = _c(sub, np.float32)
    n, dsub = sub.shape
    out = np.empty((K, dsub), np.float32)
    ref_train().psbref_pq_kmeans_subspace(_ptr(sub), n, dsub, K, iters, C.c_uint(seed), _ptr(out))
    return out


# ---------------------------------------------------------------- the reference's row-correction code (oracle/ref_rowcorr_harness.cpp)
def have_ref_rowcorr() -> bool:
    return os.path.exists(REF_ROWCORR_SO)


def ref_rowcorr():
    global _ref_rowcorr
    if _ref_rowcorr is None:
        _ref_rowcorr = C.CDLL(REF_ROWCORR_SO)
        _ref_rowcorr.ref_rc_value.restype = C.c_float
        _ref_rowcorr.ref_rc_pq_value.restype = C.c_float
        _ref_rowcorr.ref_rc_decode.restype = C.c_float
    return _ref_rowcorr


def ref_rc_build_pq(entry_dir, centroids, offsets, codes, codebook):
    """Runs the reference's builder into entry_dir; returns (payload bytes, fp32 audit values)."""
    cen = _c(centroids, np.float32); off = _c(offsets, np.int64); codes = _c(codes, np.uint8); cb = _c(codebook, np.float32)
    m, k, dsub = cb.shape
    rc = ref_rowcorr().ref_rc_build_pq(entry_dir.encode(), C.c_int64(codes.shape[0]), cen.shape[1], cen.shape[0], m, k,
                                       _ptr(cen), _ptr(off), _ptr(codes), _ptr(cb))
    if rc != 0:
        raise RuntimeError(f"reference row-correction builder failed ({rc})")
    payload = open(os.path.join(entry_dir, "row_correction.u16a"), "rb").read()
    audit = np.fromfile(os.path.join(entry_dir, "row_correction.f32"), np.float32, offset=8)
    return payload, audit


def ref_rc_pq_value(centroid, codebook, code):
    cb = _c(codebook, np.float32); cen = _c(centroid, np.float32); code = _c(code, np.uint8)
    return float(ref_rowcorr().ref_rc_pq_value(_ptr(cen), _ptr(cb), _ptr(code), cb.shape[0], cb.shape[1], cb.shape[2]))


def ref_rc_for_pq(centroids, codebook):
    cen = _c(centroids, np.float32); cb = _c(codebook, np.float32)
    sc = C.c_float(); off = C.c_float()
    if ref_rowcorr().ref_rc_for_pq(_ptr(cen), cen.shape[0], _ptr(cb), cb.shape[0], cb.shape[1], cb.shape[2], C.byref(sc), C.byref(off)) != 0:
        raise ValueError("reference quantiser refused the model")
    return sc.value, off.value


def ref_rc_encode(scale, offset, v):
    out = C.c_uint16()
    if ref_rowcorr().ref_rc_encode(C.c_float(scale), C.c_float(offset), C.c_float(v), C.byref(out)) != 0:
        raise ValueError("reference quantiser refused the value")
    return out.value


def ref_rc_decode(scale, offset, code):
    return float(ref_rowcorr().ref_rc_decode(C.c_float(scale), C.c_float(offset), C.c_uint16(code)))


# ---------------------------------------------------------------- the reference's cache classes (oracle/ref_cache_harness.cpp)
_ref_cache = None


def have_ref_cache() -> bool:
    return os.path.exists(REF_CACHE_SO)


def ref_cache():
    global _ref_cache
    if _ref_cache is None:
        _ref_cache = C.CDLL(REF_CACHE_SO)
    return _ref_cache


def ref_cluster_save(root, dataset, centroids, reordered, offsets, recipe_json):
    cen = _c(centroids, np.float32); ids = _c(reordered, np.int64); off = _c(offsets, np.int64)
    counts = np.diff(off).astype(np.int32)
    rc = ref_cache().ref_cluster_save(root.encode(), dataset.encode(), ids.size, cen.shape[0], cen.shape[1], recipe_json.encode(),
                                      _ptr(cen), _ptr(ids), _ptr(counts), _ptr(off))
    if rc:
        raise RuntimeError("reference ClusterCache::save failed")


def ref_cluster_load(root, dataset, n, nlist, dim, recipe_json, layout_id=""):
    """None on a miss, else dict(entry, layout_id, centroids, reordered_ids, counts, offsets)."""
    cen = np.empty((nlist, dim), np.float32); ids = np.empty(n, np.int64)
    counts = np.empty(nlist, np.int32); off = np.empty(nlist + 1, np.int64)
    entry = C.create_string_buffer(4096); layout = C.create_string_buffer(4096)
    rc = ref_cache().ref_cluster_load(root.encode(), dataset.encode(), n, nlist, dim, recipe_json.encode(), layout_id.encode(),
                                      _ptr(cen), _ptr(ids), _ptr(counts), _ptr(off), entry, layout, 4096)
    if rc == 2:
        return None
    if rc:
        raise RuntimeError("reference ClusterCache::try_load failed")
    return dict(entry=entry.value.decode(), layout_id=layout.value.decode(), centroids=cen, reordered_ids=ids, counts=counts, offsets=off)


def ref_pq_save(root, dataset, n, dim, nlist, layout_id, codebook, codes, iters, residual, train_rows=0):
    cb = _c(codebook, np.float32); cd = _c(codes, np.uint8)
    rc = ref_cache().ref_pq_save(root.encode(), dataset.encode(), n, dim, nlist, layout_id.encode(), cb.shape[0], cb.shape[1], iters,
                                 int(residual), train_rows, _ptr(cb), _ptr(cd))
    if rc:
        raise RuntimeError("reference ResidualPQCache::save failed")


def ref_pq_load(root, dataset, n, dim, nlist, layout_id, m, k, iters, residual, train_rows=0):
    cb = np.empty((m, k, dim // m), np.float32); cd = np.empty((n, m), np.uint8)
    entry = C.create_string_buffer(4096)
    rc = ref_cache().ref_pq_load(root.encode(), dataset.encode(), n, dim, nlist, layout_id.encode(), m, k, iters, int(residual), train_rows,
                                 _ptr(cb), _ptr(cd), entry, 4096)
    if rc == 2:
        return None
    if rc:
        raise RuntimeError("reference ResidualPQCache::try_load failed")
    return dict(entry=entry.value.decode(), codebook=cb, codes=cd)


def ref_storage_id(manifest_json):
    out = C.create_string_buffer(256)
    if ref_cache().ref_storage_id(manifest_json.encode(), out, 256):
        raise RuntimeError("reference storage_id failed")
    return out.value.decode()


def ref_manifest_matches(actual_json, expected_json):
    return int(ref_cache().ref_manifest_matches(actual_json.encode(), expected_json.encode()))


def ref_opq_save(cache_dir, dataset, n, train_n, rotation, m, k, opq_iters, pq_iters, seed):
    """The reference's save_opq_rotation_cache under its own key; returns the key."""
    rot = _c(rotation, np.float32)
    key = C.create_string_buffer(1024)
    if ref_train().psbref_opq_save(cache_dir.encode(), dataset.encode(), n, train_n, rot.shape[0], m, k, opq_iters, pq_iters, C.c_uint(seed),
                                   _ptr(rot), key, 1024):
        raise RuntimeError("reference save_opq_rotation_cache failed")
    return key.value.decode()


def ref_opq_load(cache_dir, key, dim):
    rot = np.empty((dim, dim), np.float32)
    return rot if ref_train().psbref_opq_load(cache_dir.encode(), key.encode(), dim, _ptr(rot)) == 0 else None


# ---------------------------------------------------------------- the reference's k-means initialisation (oracle/ref_kmeans_init_harness.cu)
_ref_kmeans_init = None


def have_ref_kmeans_init() -> bool:
    if not os.path.exists(REF_KMEANS_INIT_SO):
        return False
    try:   # needs the CUDA toolkit's cuBLAS at load time (the Lloyd part of the same translation unit links it)
        _load_kmeans_init()
        return True
    except OSError:
        return False


def _load_kmeans_init():
    global _ref_kmeans_init
    if _ref_kmeans_init is None:
        _ref_kmeans_init = C.CDLL(REF_KMEANS_INIT_SO)
    return _ref_kmeans_init


def ref_kmeans_init(data, k, seed, policy=0):
    """init_centroids_by_sampling of the reference on host data; policy 0 auto, 1 random rows, 2 k-means++."""
    x = _c(data, np.float32)
    out = np.empty((k, x.shape[1]), np.float32)
    _load_kmeans_init().psbref_kmeans_init(x.shape[0], x.shape[1], k, seed, policy, _ptr(x), _ptr(out))
    return out


# ---- TurboQuant 1-bit residual codec (restatement: partly pinned, see oracle/psb_oracle.c) ----------------------
REF_SIGN_SO = os.path.join(_HERE, "_ref", "libpsb_ref_sign.so")
_ref_sign = None


def _sign_lib():
    L = lib()
    for name in ("psbo_sign_scale_l2", "psbo_sign_binary_l2", "psbo_sign_score_mse", "psbo_sign_score_binary"):
        getattr(L, name).restype = C.c_float
    return L


def sign_padded_dim(dim):
    return lib().psbo_sign_padded_dim(int(dim))


def sign_scale(padded):
    """1/sqrt(padded) rounded to fp32 (the kernels take rsqrtf on the device; tests pass the device's value instead)."""
    return float(np.float32(1.0) / np.sqrt(np.float32(padded)))


def sign_pack(values):
    v = _c(values, np.float32).reshape(-1)
    out = np.zeros((v.size + 31) // 32, np.uint32)
    lib().psbo_sign_pack(_ptr(v), v.size, _ptr(out))
    return out


def sign_hamming(a, b, dim):
    a = _c(a, np.uint32); b = _c(b, np.uint32)
    return lib().psbo_sign_hamming(_ptr(a), _ptr(b), int(dim))


def sign_scale_l2(query, code, scale):
    q = _c(query, np.float32).reshape(-1); c = _c(code, np.uint32)
    return float(_sign_lib().psbo_sign_scale_l2(_ptr(q), _ptr(c), q.size, C.c_float(scale)))


def sign_binary_l2(qcode, code, dim, qn, dn):
    a = _c(qcode, np.uint32); b = _c(code, np.uint32)
    return float(_sign_lib().psbo_sign_binary_l2(_ptr(a), _ptr(b), int(dim), C.c_float(qn), C.c_float(dn)))


def sign_rotate(rows, padded, seed=17, scale=None):
    """Rotated rows, sign words, sqrt and sum of squares of each row."""
    x = _c(rows, np.float32)
    n, dim = x.shape
    scale = sign_scale(padded) if scale is None else scale
    rot = np.empty((n, padded), np.float32); codes = np.empty((n, padded // 32), np.uint32)
    norms = np.empty(n, np.float32); nsq = np.empty(n, np.float32)
    if lib().psbo_sign_rotate(_ptr(x), C.c_int64(n), dim, int(padded), C.c_uint32(seed), C.c_float(scale),
                              _ptr(rot), _ptr(codes), _ptr(norms), _ptr(nsq)):
        raise ValueError("oracle sign_rotate: invalid arguments")
    return rot, codes, norms, nsq


def sign_encode_database(rows, centroids, offsets, padded, seed=17, scale=None, row_offset=0, total_rows=None,
                         codes=None, scales=None):
    """Sign words and L1 scales of the list-contiguous rows [row_offset, row_offset + len(rows)), u8 or fp32."""
    x = np.ascontiguousarray(rows)
    if x.dtype != np.uint8:
        x = _c(x, np.float32)
    cen = _c(centroids, np.float32); off = _c(offsets, np.int64)
    n, dim = x.shape
    total = int(off[-1]) if total_rows is None else total_rows
    scale = sign_scale(padded) if scale is None else scale
    if codes is None:
        codes = np.zeros((total, padded // 32), np.uint32); scales = np.zeros(total, np.float32)
    if lib().psbo_sign_encode_database(_ptr(x), x.dtype.itemsize, C.c_int64(n), _ptr(cen), _ptr(off), cen.shape[0], dim,
                                       int(padded), C.c_uint32(seed), C.c_float(scale), C.c_int64(row_offset),
                                       _ptr(codes), _ptr(scales)):
        raise ValueError("oracle sign_encode_database: invalid arguments")
    return codes, scales


def sign_encode_queries(queries, centroids, probes, padded, seed=17, scale=None):
    """Per (query, probe): rotated residual state, its sum of squares, its sign words, its norm."""
    q = _c(queries, np.float32); cen = _c(centroids, np.float32); pr = _c(probes, np.int32)
    nq, nprobe = pr.shape
    scale = sign_scale(padded) if scale is None else scale
    states = np.empty((nq * nprobe, padded), np.float32); nsq = np.empty(nq * nprobe, np.float32)
    sc = np.empty((nq * nprobe, padded // 32), np.uint32); norms = np.empty(nq * nprobe, np.float32)
    if lib().psbo_sign_encode_queries(_ptr(q), _ptr(cen), _ptr(pr), nq, nprobe, cen.shape[0], q.shape[1], int(padded),
                                      C.c_uint32(seed), C.c_float(scale), _ptr(states), _ptr(nsq), _ptr(sc), _ptr(norms)):
        raise ValueError("oracle sign_encode_queries: invalid arguments")
    return states, nsq, sc, norms


def sign_candidates(mode, codes, row_params, offsets, probes, candidate_count, states=None, norm_sq=None,
                    state_codes=None, norms=None):
    """The candidate_count rows of the probed lists with the smallest (score, row); mode 0 float states, 1 sign-coded."""
    codes = _c(codes, np.uint32); rp = _c(row_params, np.float32); off = _c(offsets, np.int64); pr = _c(probes, np.int32)
    nq, nprobe = pr.shape
    padded = codes.shape[1] * 32
    st = None if states is None else _c(states, np.float32)
    ns = None if norm_sq is None else _c(norm_sq, np.float32)
    sc = None if state_codes is None else _c(state_codes, np.uint32)
    nm = None if norms is None else _c(norms, np.float32)
    rows = np.empty((nq, candidate_count), np.int32); dist = np.empty((nq, candidate_count), np.float32)
    if lib().psbo_sign_candidates(int(mode), _ptr(st), _ptr(ns), _ptr(sc), _ptr(nm), _ptr(codes), _ptr(rp), _ptr(off),
                                  off.size - 1, _ptr(pr), nq, nprobe, padded, int(candidate_count), _ptr(rows), _ptr(dist)):
        raise ValueError("oracle sign_candidates: invalid arguments")
    return rows, dist


def have_ref_sign() -> bool:
    return os.path.exists(REF_SIGN_SO)


def ref_sign():
    global _ref_sign
    if _ref_sign is None:
        _ref_sign = C.CDLL(REF_SIGN_SO)
        for name in ("ref_sign_scale_l2", "ref_sign_binary_l2", "ref_sign_mse"):
            getattr(_ref_sign, name).restype = C.c_float
    return _ref_sign


def ref_sign_pack(values):
    v = _c(values, np.float32).reshape(-1)
    out = np.zeros(ref_sign().ref_sign_words(v.size), np.uint32)
    ref_sign().ref_sign_pack(_ptr(v), v.size, _ptr(out))
    return out


def ref_sign_hamming(a, b, dim):
    a = _c(a, np.uint32); b = _c(b, np.uint32)
    return ref_sign().ref_sign_hamming(_ptr(a), _ptr(b), int(dim))


def ref_sign_scale_l2(query, code, scale):
    q = _c(query, np.float32).reshape(-1); c = _c(code, np.uint32)
    return float(ref_sign().ref_sign_scale_l2(_ptr(q), _ptr(c), q.size, C.c_float(scale)))


def ref_sign_binary_l2(qcode, code, dim, qn, dn):
    a = _c(qcode, np.uint32); b = _c(code, np.uint32)
    return float(ref_sign().ref_sign_binary_l2(_ptr(a), _ptr(b), int(dim), C.c_float(qn), C.c_float(dn)))


def ref_sign_cache_publish(root, dataset, staged, n, dim, nlist, seed, layout_id, codes, scales):
    """TurboQuantCache::publish_staged of the reference over payload files written by the harness into `staged`."""
    cd = _c(codes, np.uint32); sc = _c(scales, np.float32)
    if ref_cache().ref_sign_cache_publish(root.encode(), dataset.encode(), staged.encode(), n, dim, nlist, seed, layout_id.encode(),
                                          _ptr(cd), _ptr(sc)):
        raise RuntimeError("reference TurboQuantCache::publish_staged failed")


def ref_sign_cache_map(root, dataset, n, dim, nlist, seed, layout_id):
    """TurboQuantCache::try_map of the reference: None on a miss."""
    cd = np.empty((n, dim // 32), np.uint32); sc = np.empty(n, np.float32)
    entry = C.create_string_buffer(4096)
    rc = ref_cache().ref_sign_cache_map(root.encode(), dataset.encode(), n, dim, nlist, seed, layout_id.encode(), _ptr(cd), _ptr(sc),
                                        entry, 4096)
    if rc == 2:
        return None
    if rc:
        raise RuntimeError("reference TurboQuantCache::try_map failed")
    return dict(entry=entry.value.decode(), codes=cd, scales=sc)
