"""ctypes binding of libpsb.so (the C ABI declared in include/psb.h) with numpy / torch conveniences.

The names follow the reference's view API (IVFCoarseIndexView, IVFListLayoutView, IVFPQCodeStorageView,
IVFQueryBatchView, IVFSearchParams, IVFSearchOutputView: src/search/ivf_common/ivf_search_types.h:41-75 in
the ParaSelect tree).  There is no CPU path here: every compute call goes to the CUDA library and raises
PsbError if the library or a usable sm_100 device is missing.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpsb.so")

PSB_OK = 0
STATUS_NAMES = {0: "PSB_OK", 1: "PSB_INVALID_ARGUMENT", 2: "PSB_UNSUPPORTED_SHAPE", 3: "PSB_CUDA_ERROR",
                4: "PSB_OUT_OF_MEMORY", 5: "PSB_NO_DEVICE", 6: "PSB_INTERNAL", 7: "PSB_TIMEOUT"}
EXACT_HOST_MAPPED, EXACT_HOST_STAGED, EXACT_RESIDENT, EXACT_HOST_CACHED, EXACT_HOST_HYBRID = 0, 1, 2, 3, 4


class PsbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(status, status), message))
        self.status = status


class InvalidArgument(PsbError, ValueError):
    """PSB_INVALID_ARGUMENT: where the reference throws std::invalid_argument."""


class CoarseIndexView(C.Structure):
    _fields_ = [("centroids", C.c_void_p), ("nlist", C.c_int), ("dim", C.c_int)]


class ListLayoutView(C.Structure):
    _fields_ = [("offsets", C.c_void_p), ("reordered_ids", C.c_void_p), ("nlist", C.c_int), ("n_vectors", C.c_int64)]


class PQCodeStorageView(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("code_storage", C.c_void_p), ("codebook", C.c_void_p),
                ("subvectors", C.c_int), ("codebook_size", C.c_int)]


class HostStorageView(C.Structure):
    _fields_ = [("fp32", C.c_void_p), ("u8", C.c_void_p), ("count", C.c_int64), ("dim", C.c_int),
                ("source_rows", C.c_void_p)]


class QueryBatchView(C.Structure):
    _fields_ = [("fp32", C.c_void_p), ("u8", C.c_void_p), ("count", C.c_int), ("dim", C.c_int), ("fp16", C.c_void_p)]


class SearchParams(C.Structure):
    _fields_ = [("nprobe", C.c_int), ("topk", C.c_int), ("batch_size", C.c_int), ("distance", C.c_int),
                ("fp16_coarse", C.c_ubyte)]


class SearchOutputView(C.Structure):
    _fields_ = [("indices", C.c_void_p), ("distances", C.c_void_p), ("coarse_ids", C.c_void_p)]


class IndexView(C.Structure):
    _fields_ = [("coarse", CoarseIndexView), ("lists", ListLayoutView), ("pq", PQCodeStorageView),
                ("exact", HostStorageView)]


class Options(C.Structure):
    _fields_ = [("device", C.c_int), ("n_rerank", C.c_int), ("exact_mode", C.c_int), ("max_batch", C.c_int),
                ("list_begin", C.c_int), ("list_end", C.c_int), ("stream", C.c_void_p), ("list_global_begin", C.c_void_p),
                ("coarse_mode", C.c_int),
                ("time_kernels", C.c_int), ("serial_pipeline", C.c_int), ("scan_mode", C.c_int), ("adc_mode", C.c_int), ("reserve_sms", C.c_int),
                ("seed_sigma", C.c_float), ("pipeline_parts", C.c_int), ("even_cuts", C.c_int), ("gather_ctas", C.c_int),
                ("tc_min_visitors", C.c_int), ("test_wait_limit", C.c_int), ("test_skip_mma", C.c_int), ("zero_copy_pct", C.c_int),
                ("row_correction_fp32", C.c_void_p), ("row_correction_u16", C.c_void_p), ("rc_scale", C.c_float), ("rc_offset", C.c_float),
                ("opq_matrix", C.c_void_p), ("host_threads", C.c_int)]


class Stats(C.Structure):
    _fields_ = [("total_ms", C.c_double), ("coarse_search_ms", C.c_double), ("pq_lut_build_ms", C.c_double),
                ("pq_adc_scan_ms", C.c_double), ("pq_rerank_ms", C.c_double), ("pq_map_ids_ms", C.c_double),
                ("h2d_ms", C.c_double), ("d2h_ms", C.c_double), ("pq_scanned_codes", C.c_longlong),
                ("pq_adc_lookups", C.c_longlong), ("threshold_candidates", C.c_longlong),
                ("fallback_queries", C.c_longlong), ("h2d_bytes", C.c_longlong), ("d2h_bytes", C.c_longlong),
                ("kernel_launches", C.c_longlong), ("scan_kernel_ms", C.c_double), ("scan_kernel_launches", C.c_longlong),
                ("coarse_gemm_ms", C.c_double), ("coarse_gemm_launches", C.c_longlong),
                ("batches", C.c_int), ("coarse_fallback_queries", C.c_int), ("prefilter_survivors", C.c_longlong),
                ("tc_wait_item_cycles", C.c_longlong), ("tc_wait_rows_cycles", C.c_longlong), ("tc_wait_acc_cycles", C.c_longlong),
                ("tc_tiles", C.c_longlong), ("staged_gather_ms", C.c_double), ("staged_gather_bytes", C.c_longlong),
                ("reserved", C.c_int * 4)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


EXPORTS = [
    "psb_last_error", "psb_device_count", "psb_version", "psb_session_create", "psb_session_destroy",
    "psb_session_search", "psb_session_search_device", "psb_session_sync", "psb_session_set_stream", "psb_stage_coarse", "psb_stage_build_lut", "psb_stage_build_lut_residual", "psb_stage_quantize_lut_u8", "psb_stage_scan", "psb_stage_scan_queries",
    "psb_stage_rerank", "psb_stage_rerank_partial", "psb_stage_select_topk", "psb_stage_map_ids", "psb_stage_merge", "psb_session_counters", "psb_rerank_host",
    "psb_flat_session_create", "psb_flat_session_search", "psb_flat_session_search_device", "psb_flat_session_destroy",
    "psb_row_correction_compute", "psb_row_correction_quantize_u16", "psb_row_correction_write_u16", "psb_row_correction_read_u16",
    "psb_row_correction_model_u16", "psb_row_correction_encode_u16",
    "psb_sizeof", "psb_kmeans_assign_bounded", "psb_group_create", "psb_group_set", "psb_group_search_device", "psb_group_searched_again", "psb_group_destroy",
    "psb_sign_padded_dim", "psb_sign_rotation_scale", "psb_sign_rotate", "psb_sign_encode_database", "psb_sign_encode_queries", "psb_sign_search_candidates",
    "psb_kmeans_init", "psb_rotate_rows", "psb_stage_rotate_queries", "psb_scan_sample_words", "psb_stage_scan_sample", "psb_stage_scan_shared",
    "psb_ivf_layout_from_assignment", "psb_reorder_rows", "psb_coarse_host", "psb_coarse_search_static", "psb_knn_exact", "psb_kmeans_train", "psb_kmeans_assign", "psb_kmeans_accumulate", "psb_kmeans_update", "psb_residual_rows", "psb_pq_train", "psb_pq_encode", "psb_gen_mixture_rows", "psb_gen_normal",
]

_lib = None


def lib():
    """The loaded CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PsbError(-1, "libpsb.so is not built: run `python -m paraselect_b200.build`")
        _lib = C.CDLL(LIB_PATH)
        _lib.psb_last_error.restype = C.c_char_p
        _lib.psb_version.restype = C.c_char_p
    return _lib


def load(path):
    """Use another build of the library (e.g. build.build_nvtx_variant()'s) instead of libpsb.so; call before anything else."""
    global _lib
    _lib = C.CDLL(path)
    _lib.psb_last_error.restype = C.c_char_p
    _lib.psb_version.restype = C.c_char_p
    return _lib


def _check(status):
    if status != PSB_OK:
        msg = lib().psb_last_error().decode()
        raise (InvalidArgument if status == 1 else PsbError)(status, msg)


def device_count() -> int:
    return int(lib().psb_device_count())


def _np(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def _p(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return int(a.data_ptr())  # torch tensor


class Session:
    """Prepare once, search many (IVFResPQSession / IVFPQIndex of the reference).

    index: dict with centroids [nlist,dim] f32, offsets [nlist+1] i64, reordered_ids [n] i64, codes [n,M] u8,
    codebook [M,K,dsub] f32 and optionally vectors [n,dim] f32 (or u8) for the exact rerank.  The arrays are
    borrowed: they must stay alive (and, in mapped mode, unmoved) for the session's lifetime.
    """

    def __init__(self, index, n_rerank=0, device=0, exact_mode=EXACT_HOST_MAPPED, max_batch=0, list_begin=0,
                 list_end=0, stream=None, coarse_mode=0, time_kernels=False, list_global_begin=None, scan_mode=0, serial_pipeline=False, residual=False, reserve_sms=0,
                 seed_sigma=0.0, pipeline_parts=0, even_cuts=False, gather_ctas=0, tc_min_visitors=0, test_wait_limit=0, test_skip_mma=0,
                 row_correction=None, rc_scale=0.0, rc_offset=0.0, opq_matrix=None, zero_copy_pct=0, host_threads=0):
        self._keep = []
        cen = _np(index["centroids"], np.float32)
        off = _np(index["offsets"], np.int64)
        rid = _np(index["reordered_ids"], np.int64)
        codes = _np(index["codes"], np.uint8)
        cb = _np(index["codebook"], np.float32)
        vec = index.get("vectors")
        self._keep += [cen, off, rid, codes, cb]
        iv = IndexView()
        iv.coarse = CoarseIndexView(_p(cen), cen.shape[0], cen.shape[1])
        n = int(codes.shape[0])
        iv.lists = ListLayoutView(_p(off), _p(rid), int(index.get("nlist", cen.shape[0])), n)
        iv.pq = PQCodeStorageView(_p(codes), None, _p(cb), cb.shape[0], cb.shape[1])
        if vec is not None:
            if exact_mode == EXACT_RESIDENT:
                fp32 = vec.dtype != __import__("torch").uint8
                ptr = int(vec.data_ptr())
                rows, d = int(vec.shape[0]), int(vec.shape[1])
            else:
                fp32 = vec.dtype != np.uint8
                vec = _np(vec, np.float32 if fp32 else np.uint8)
                ptr, rows, d = _p(vec), int(vec.shape[0]), int(vec.shape[1])
            self._keep.append(vec)
            iv.exact = HostStorageView(ptr if fp32 else None, None if fp32 else ptr, rows, d, None)
        self.dim, self.nlist, self.M, self.K, self.n = cen.shape[1], cen.shape[0], cb.shape[0], cb.shape[1], n
        self.n_rerank = n_rerank
        self.residual = bool(residual)
        self.device = device
        gb = _np(list_global_begin, np.int64)
        self._keep.append(gb)
        opt = Options(list_global_begin=_p(gb), device=device, n_rerank=n_rerank, exact_mode=exact_mode, max_batch=max_batch,
                      list_begin=list_begin, list_end=list_end, stream=stream, coarse_mode=coarse_mode,
                      time_kernels=int(time_kernels), scan_mode=scan_mode, serial_pipeline=int(serial_pipeline), adc_mode=int(bool(residual)), reserve_sms=reserve_sms,
                      seed_sigma=float(seed_sigma), pipeline_parts=int(pipeline_parts), even_cuts=int(even_cuts),
                      gather_ctas=int(gather_ctas), tc_min_visitors=int(tc_min_visitors), test_wait_limit=int(test_wait_limit),
                      test_skip_mma=int(test_skip_mma), zero_copy_pct=int(zero_copy_pct), host_threads=int(host_threads))
        if opq_matrix is not None:  # OPQ index: rotation [dim][dim], row-major [out][in]
            rot = _np(opq_matrix, np.float32)
            if rot.shape != (iv.coarse.dim, iv.coarse.dim):
                raise InvalidArgument(1, "opq_matrix must be [dim, dim]")
            self._keep.append(rot)
            opt.opq_matrix = _p(rot)
        if row_correction is not None:  # residual mode: the index's per-row correction, fp32 or affine u16 (kept alive with the session)
            rc = np.ascontiguousarray(row_correction)
            self._keep.append(rc)
            if rc.dtype == np.uint16:
                opt.row_correction_u16, opt.rc_scale, opt.rc_offset = _p(rc), float(rc_scale), float(rc_offset)
            else:
                rc = _np(rc, np.float32); self._keep.append(rc)
                opt.row_correction_fp32 = _p(rc)
        self._h = C.c_void_p()
        _check(lib().psb_session_create(C.byref(iv), C.byref(opt), C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().psb_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- whole search, host arrays in and out -----------------------------------------------------
    def search(self, queries, nprobe, topk, batch_size=10000, queries_u8=None, want_coarse=False, out=None):
        q = _np(queries, np.float32)
        if q.ndim != 2:
            raise InvalidArgument(1, "queries must be [count, dim]")
        nq = q.shape[0]
        qu8 = _np(queries_u8, np.uint8)
        if out is None:
            ids = np.empty((nq, max(topk, 0)), np.int64)
            dist = np.empty((nq, max(topk, 0)), np.float32)
        else:
            ids, dist = out
        coarse = np.empty((nq, max(nprobe, 0)), np.int32) if want_coarse else None
        qv = QueryBatchView(_p(q), _p(qu8), nq, q.shape[1], None)
        pr = SearchParams(nprobe, topk, batch_size, 0, 0)
        ov = SearchOutputView(_p(ids), _p(dist), _p(coarse))
        st = Stats()
        _check(lib().psb_session_search(self._h, C.byref(qv), C.byref(pr), C.byref(ov), C.byref(st)))
        res = dict(indices=ids, distances=dist, stats=st.as_dict())
        if want_coarse:
            res["coarse"] = coarse
        return res

    def search_raw(self, q_ptr, nq, nprobe, topk, batch_size, ids_ptr, dist_ptr, stats=None):
        """Same call with raw host pointers (pinned buffers in the bench)."""
        qv = QueryBatchView(q_ptr, None, nq, self.dim, None)
        pr = SearchParams(nprobe, topk, batch_size, 0, 0)
        ov = SearchOutputView(ids_ptr, dist_ptr, None)
        _check(lib().psb_session_search(self._h, C.byref(qv), C.byref(pr), C.byref(ov),
                                        C.byref(stats) if stats is not None else None))

    def search_device(self, d_queries, nq, nprobe, topk, d_ids, d_dist, d_coarse=None, d_queries_u8=None):
        """Whole search with device tensors in and out, asynchronous on the session's stream."""
        pr = SearchParams(nprobe, topk, nq, 0, 0)
        _check(lib().psb_session_search_device(self._h, C.c_void_p(_p(d_queries)),
                                               C.c_void_p(_p(d_queries_u8)) if d_queries_u8 is not None else None, nq,
                                               C.byref(pr), C.c_void_p(_p(d_ids)), C.c_void_p(_p(d_dist)),
                                               C.c_void_p(_p(d_coarse)) if d_coarse is not None else None))

    # ---- stage level, device pointers (torch tensors or ints) ---------------------------------------
    def stage_coarse(self, d_queries, nq, nprobe, d_ids, d_dist=None):
        _check(lib().psb_stage_coarse(self._h, C.c_void_p(_p(d_queries)), nq, nprobe, C.c_void_p(_p(d_ids)),
                                      C.c_void_p(_p(d_dist)) if d_dist is not None else None))

    def set_stream(self, stream=None, background=False):
        """Redirects the stage calls to `stream` (a cudaStream_t value; None = the session's own stream)."""
        _check(lib().psb_session_set_stream(self._h, _stream_ptr(stream), int(background)))

    def scan_sample_words(self, stage1_k):
        return int(lib().psb_scan_sample_words(self._h, stage1_k))

    def stage_scan_sample(self, d_queries, d_lut, nq, d_probes, nprobe, stage1_k, d_samples):
        _check(lib().psb_stage_scan_sample(self._h, C.c_void_p(_p(d_queries)), C.c_void_p(_p(d_lut)), nq, C.c_void_p(_p(d_probes)), nprobe,
                                           stage1_k, C.c_void_p(_p(d_samples))))

    def stage_scan_shared(self, d_queries, d_lut, nq, d_probes, nprobe, stage1_k, d_all_samples, shards, d_rows, d_dist, d_count,
                          d_cutoff=None, d_rows_scanned=None):
        _check(lib().psb_stage_scan_shared(self._h, C.c_void_p(_p(d_queries)), C.c_void_p(_p(d_lut)), nq, C.c_void_p(_p(d_probes)), nprobe,
                                           stage1_k, C.c_void_p(_p(d_all_samples)), shards, C.c_void_p(_p(d_rows)), C.c_void_p(_p(d_dist)),
                                           C.c_void_p(_p(d_count)), C.c_void_p(_p(d_cutoff)), C.c_void_p(_p(d_rows_scanned))))

    def stage_rotate_queries(self, d_queries, nq, d_rotated):
        _check(lib().psb_stage_rotate_queries(self._h, C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_rotated))))

    def stage_build_lut(self, d_queries, nq, d_lut):
        _check(lib().psb_stage_build_lut(self._h, C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_lut))))

    def stage_build_lut_residual(self, d_queries, nq, d_probes, nprobe, d_lut):
        _check(lib().psb_stage_build_lut_residual(self._h, C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_probes)), nprobe,
                                                  C.c_void_p(_p(d_lut))))

    def stage_quantize_lut_u8(self, d_lut, tables, d_q8, d_scales, d_lo_sum, d_inflation):
        _check(lib().psb_stage_quantize_lut_u8(self._h, C.c_void_p(_p(d_lut)), C.c_int64(tables), C.c_void_p(_p(d_q8)),
                                               C.c_void_p(_p(d_scales)), C.c_void_p(_p(d_lo_sum)), C.c_void_p(_p(d_inflation))))

    def stage_scan(self, d_lut, nq, d_probes, nprobe, stage1_k, d_rows, d_dist=None, d_count=None):
        _check(lib().psb_stage_scan(self._h, C.c_void_p(_p(d_lut)), nq, C.c_void_p(_p(d_probes)), nprobe, stage1_k,
                                    C.c_void_p(_p(d_rows)), C.c_void_p(_p(d_dist)) if d_dist is not None else None,
                                    C.c_void_p(_p(d_count)) if d_count is not None else None))

    def stage_scan_queries(self, d_queries, d_lut, nq, d_probes, nprobe, stage1_k, d_rows, d_dist=None, d_count=None):
        _check(lib().psb_stage_scan_queries(self._h, C.c_void_p(_p(d_queries)), C.c_void_p(_p(d_lut)), nq, C.c_void_p(_p(d_probes)),
                                            nprobe, stage1_k, C.c_void_p(_p(d_rows)),
                                            C.c_void_p(_p(d_dist)) if d_dist is not None else None,
                                            C.c_void_p(_p(d_count)) if d_count is not None else None))

    def stage_rerank(self, d_queries, nq, d_cand, count, stride, d_counts, topk, d_out_rows, d_out_dist):
        _check(lib().psb_stage_rerank(self._h, C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_cand)), count, stride,
                                      C.c_void_p(_p(d_counts)) if d_counts is not None else None, topk,
                                      C.c_void_p(_p(d_out_rows)), C.c_void_p(_p(d_out_dist))))

    def stage_rerank_partial(self, d_queries, nq, d_cand, count, stride, d_counts, d_dist):
        _check(lib().psb_stage_rerank_partial(self._h, C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_cand)), count, stride,
                                              C.c_void_p(_p(d_counts)) if d_counts is not None else None,
                                              C.c_void_p(_p(d_dist))))

    def stage_select_topk(self, d_dist, d_cand, nq, count, stride, d_counts, topk, d_out_rows, d_out_dist):
        _check(lib().psb_stage_select_topk(self._h, C.c_void_p(_p(d_dist)), C.c_void_p(_p(d_cand)), nq, count, stride,
                                           C.c_void_p(_p(d_counts)) if d_counts is not None else None, topk,
                                           C.c_void_p(_p(d_out_rows)), C.c_void_p(_p(d_out_dist))))

    def stage_map_ids(self, d_rows, n, d_indices):
        _check(lib().psb_stage_map_ids(self._h, C.c_void_p(_p(d_rows)), C.c_int64(n), C.c_void_p(_p(d_indices))))

    def stage_merge(self, d_rows, d_dist, parts, nq, k, d_out_rows, d_out_dist):
        _check(lib().psb_stage_merge(self._h, C.c_void_p(_p(d_rows)), C.c_void_p(_p(d_dist)), parts, nq, k,
                                     C.c_void_p(_p(d_out_rows)), C.c_void_p(_p(d_out_dist))))

    def sync(self):
        _check(lib().psb_session_sync(self._h))

    def counters(self, reset=False):
        st = Stats()
        _check(lib().psb_session_counters(self._h, C.byref(st), int(reset)))
        return st.as_dict()


class FlatIndexView(C.Structure):
    _fields_ = [("coarse", CoarseIndexView), ("lists", ListLayoutView), ("rowmajor_fp32", C.c_void_p)]


class FlatSession:
    """IVF-Flat with device-resident rows (ivfflat_search of the reference, src/search/ivfflat/ivfflat_search.cuh:41-51).

    index: dict with centroids [nlist,dim] f32, offsets [nlist+1] i64, reordered_ids [n] i64, vectors [n,dim] f32 (list-contiguous).
    """

    def __init__(self, index, device=0, max_batch=0, stream=None, coarse_mode=0, time_kernels=False):
        cen = _np(index["centroids"], np.float32)
        off = _np(index["offsets"], np.int64)
        rid = _np(index["reordered_ids"], np.int64)
        vec = _np(index["vectors"], np.float32)
        self._keep = [cen, off, rid, vec]
        fv = FlatIndexView()
        fv.coarse = CoarseIndexView(_p(cen), cen.shape[0], cen.shape[1])
        fv.lists = ListLayoutView(_p(off), _p(rid), cen.shape[0], int(vec.shape[0]))
        fv.rowmajor_fp32 = _p(vec)
        self.dim, self.nlist = cen.shape[1], cen.shape[0]
        opt = Options(device=device, max_batch=max_batch, stream=stream, coarse_mode=coarse_mode, time_kernels=int(time_kernels))
        self._h = C.c_void_p()
        _check(lib().psb_flat_session_create(C.byref(fv), C.byref(opt), C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().psb_flat_session_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def search(self, queries, nprobe, topk, batch_size=10000, want_coarse=False):
        q = _np(queries, np.float32)
        nq = q.shape[0]
        ids = np.empty((nq, max(topk, 0)), np.int64)
        dist = np.empty((nq, max(topk, 0)), np.float32)
        coarse = np.empty((nq, max(nprobe, 0)), np.int32) if want_coarse else None
        qv = QueryBatchView(_p(q), None, nq, q.shape[1], None)
        pr = SearchParams(nprobe, topk, batch_size, 0, 0)
        ov = SearchOutputView(_p(ids), _p(dist), _p(coarse))
        st = Stats()
        _check(lib().psb_flat_session_search(self._h, C.byref(qv), C.byref(pr), C.byref(ov), C.byref(st)))
        res = dict(indices=ids, distances=dist, stats=st.as_dict())
        if want_coarse:
            res["coarse"] = coarse
        return res

    def search_raw(self, q_ptr, nq, nprobe, topk, batch_size, ids_ptr, dist_ptr, stats=None):
        qv = QueryBatchView(q_ptr, None, nq, self.dim, None)
        pr = SearchParams(nprobe, topk, batch_size, 0, 0)
        ov = SearchOutputView(ids_ptr, dist_ptr, None)
        _check(lib().psb_flat_session_search(self._h, C.byref(qv), C.byref(pr), C.byref(ov),
                                             C.byref(stats) if stats is not None else None))

    def counters(self, reset=False):
        st = Stats()
        _check(lib().psb_session_counters(self._h, C.byref(st), int(reset)))
        return st.as_dict()

    def search_device(self, d_queries, nq, nprobe, topk, d_ids, d_dist):
        pr = SearchParams(nprobe, topk, nq, 0, 0)
        _check(lib().psb_flat_session_search_device(self._h, C.c_void_p(_p(d_queries)), nq, C.byref(pr), C.c_void_p(_p(d_ids)),
                                                    C.c_void_p(_p(d_dist))))


# ---- one-shot operators on host arrays ---------------------------------------------------------------
def rerank_host(base, queries, candidates, topk, candidate_count=None, counts=None, device=0):
    """ivf_rerank_host of the reference (src/search/ivf_common/ivf_host_rerank.h:7-27) on the GPU."""
    u8 = base.dtype == np.uint8
    base = _np(base, np.uint8 if u8 else np.float32)
    queries = _np(queries, np.uint8 if u8 else np.float32)
    cand = _np(candidates, np.int32)
    batch, stride = cand.shape
    cc = stride if candidate_count is None else candidate_count
    ids = np.empty((batch, max(topk, 0)), np.int32)
    dist = np.empty((batch, max(topk, 0)), np.float32)
    cnt = _np(counts, np.int32)
    st = HostStorageView(None if u8 else _p(base), _p(base) if u8 else None, base.shape[0], base.shape[1], None)
    _check(lib().psb_rerank_host(C.byref(st), C.c_void_p(_p(queries)) if u8 else None,
                                 None if u8 else C.c_void_p(_p(queries)), C.c_void_p(_p(cand)), batch, cc, stride, topk,
                                 C.c_void_p(_p(ids)), C.c_void_p(_p(dist)), C.c_void_p(_p(cnt)) if cnt is not None else None,
                                 device))
    return ids, dist


def coarse_host(queries, centroids, nprobe, coarse_mode=0, device=0):
    q = _np(queries, np.float32)
    c = _np(centroids, np.float32)
    ids = np.empty((q.shape[0], max(nprobe, 0)), np.int64)
    dist = np.empty((q.shape[0], max(nprobe, 0)), np.float32)
    _check(lib().psb_coarse_host(C.c_void_p(_p(q)), q.shape[0], C.c_void_p(_p(c)), c.shape[0], c.shape[1], nprobe,
                                 coarse_mode, C.c_void_p(_p(ids)), C.c_void_p(_p(dist)), device))
    return ids, dist


def coarse_search_static(d_queries, nq, d_centroids, nlist, dim, nprobe, d_ids, d_dist=None, stream=None):
    """Coarse stage on device tensors that allocates nothing: its scratch is a fixed array inside the library
    (nq * nlist <= 4,194,304).  For callers that may not allocate device memory when they search."""
    _check(lib().psb_coarse_search_static(C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_centroids)), nlist, dim, nprobe,
                                          C.c_void_p(_p(d_ids)), C.c_void_p(_p(d_dist)) if d_dist is not None else None,
                                          C.c_void_p(stream) if stream else None))


def ivf_layout_from_assignment(assign, nlist):
    """(offsets [nlist+1], reordered_ids [n]): rows ordered by (list, original id)."""
    a = _np(assign, np.int32)
    off = np.empty(nlist + 1, np.int64); rid = np.empty(a.shape[0], np.int64)
    _check(lib().psb_ivf_layout_from_assignment(C.c_void_p(_p(a)), C.c_int64(a.shape[0]), nlist, C.c_void_p(_p(off)), C.c_void_p(_p(rid))))
    return off, rid


def reorder_rows(src, reordered_ids):
    """dst[local] = src[reordered_ids[local]] (any row type)."""
    src = np.ascontiguousarray(src)
    rid = _np(reordered_ids, np.int64)
    dst = np.empty_like(src)
    _check(lib().psb_reorder_rows(C.c_void_p(_p(src)), C.c_int64(src.shape[0]), C.c_size_t(src.strides[0]), C.c_void_p(_p(rid)),
                                  C.c_void_p(_p(dst))))
    return dst


class Group:
    """One rank of a sharded search driven by the library itself (psb_group_*): `session` holds this rank's shard, the two
    communicators are ncclComm_t handles (integers) created by the caller with the NCCL library at `nccl_library`."""

    def __init__(self, session, nccl_comm, nccl_comm_samples, max_batch, nprobe, topk, nccl_library=None, parts=4, shared_cutoff=True):
        self._h = C.c_void_p()
        self.session = session
        _check(lib().psb_group_create(session._h, C.c_void_p(nccl_comm), C.c_void_p(nccl_comm_samples) if nccl_comm_samples else None,
                                      nccl_library.encode() if nccl_library else None, max_batch, nprobe, topk, C.byref(self._h)))
        _check(lib().psb_group_set(self._h, parts, int(shared_cutoff)))

    def search_device(self, d_queries, nq, nprobe, topk, d_ids, d_dist):
        p = SearchParams(nprobe=nprobe, topk=topk, batch_size=nq, distance=0, fp16_coarse=0)
        _check(lib().psb_group_search_device(self._h, C.c_void_p(_p(d_queries)), nq, C.byref(p), C.c_void_p(_p(d_ids)), C.c_void_p(_p(d_dist))))

    def searched_again(self):
        lib().psb_group_searched_again.restype = C.c_longlong
        return int(lib().psb_group_searched_again(self._h))

    def close(self):
        if self._h:
            lib().psb_group_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class RowCorrectionHeader(C.Structure):
    _fields_ = [("magic", C.c_char * 8), ("version", C.c_uint32), ("header_bytes", C.c_uint32), ("count", C.c_uint64),
                ("scale", C.c_float), ("offset", C.c_float)]


def row_correction_compute(centroids, offsets, codes, codebook):
    """value[row] = |recon|^2 + 2 <centroid[list], recon> (fp64 accumulation, rounded once), host side."""
    cen = _np(centroids, np.float32); off = _np(offsets, np.int64); codes = _np(codes, np.uint8); cb = _np(codebook, np.float32)
    out = np.empty(codes.shape[0], np.float32)
    _check(lib().psb_row_correction_compute(C.c_void_p(_p(cen)), C.c_void_p(_p(off)), cen.shape[0], cen.shape[1], C.c_void_p(_p(codes)),
                                            C.c_void_p(_p(cb)), cb.shape[0], cb.shape[1], C.c_void_p(_p(out))))
    return out


def row_correction_quantize_u16(values):
    v = _np(values, np.float32)
    hdr = RowCorrectionHeader(); u = np.empty(v.shape[0], np.uint16)
    _check(lib().psb_row_correction_quantize_u16(C.c_void_p(_p(v)), C.c_int64(v.shape[0]), C.byref(hdr), C.c_void_p(_p(u))))
    return hdr, u


def row_correction_model_u16(centroids, codebook):
    """(scale, offset) of the fixed-model u16 form: valid for every code combination of (centroids, codebook [m][k][dsub])."""
    cen = _np(centroids, np.float32); cb = _np(codebook, np.float32)
    sc = C.c_float(); off = C.c_float()
    _check(lib().psb_row_correction_model_u16(C.c_void_p(_p(cen)), cen.shape[0], C.c_void_p(_p(cb)), cb.shape[0], cb.shape[1], cb.shape[2],
                                              C.byref(sc), C.byref(off)))
    return sc.value, off.value


def row_correction_encode_u16(values, scale, offset):
    v = _np(values, np.float32); u = np.empty(v.shape[0], np.uint16)
    _check(lib().psb_row_correction_encode_u16(C.c_void_p(_p(v)), C.c_int64(v.shape[0]), C.c_float(scale), C.c_float(offset), C.c_void_p(_p(u))))
    return u


def row_correction_write_u16(path, header, u16):
    u = _np(u16, np.uint16)
    _check(lib().psb_row_correction_write_u16(path.encode(), C.byref(header), C.c_void_p(_p(u))))


def row_correction_read_u16(path):
    hdr = RowCorrectionHeader()
    _check(lib().psb_row_correction_read_u16(path.encode(), C.byref(hdr), None, C.c_int64(0)))
    u = np.empty(int(hdr.count), np.uint16)
    _check(lib().psb_row_correction_read_u16(path.encode(), C.byref(hdr), C.c_void_p(_p(u)), C.c_int64(u.shape[0])))
    return hdr, u


def rotate_rows(d_in, d_matrix, n, dim, d_out, device=0, stream=None):
    """d_out[r] = matrix @ d_in[r] on the device (matrix row-major [out][in])."""
    _check(lib().psb_rotate_rows(C.c_void_p(_p(d_in)), C.c_void_p(_p(d_matrix)), C.c_int64(n), dim, C.c_void_p(_p(d_out)), device,
                                 _stream_ptr(stream)))


# ---- TurboQuant 1-bit residual codec --------------------------------------------------------------------
SIGN_ROTATION_SEED = 17
SIGN_FLOAT_STATES, SIGN_CODED_STATES = 0, 1   # TurboQuant1BitScoreMode::MseFloatQuery / BinaryQuery
SIGN_MAX_CANDIDATES = 8192


def _vp(a):
    return C.c_void_p(_p(a)) if a is not None else None


def sign_padded_dim(dim):
    return lib().psb_sign_padded_dim(int(dim))


def sign_rotation_scale(padded_dim, device=0, stream=None):
    """rsqrtf(padded_dim) as the device computes it."""
    out = C.c_float(0)
    _check(lib().psb_sign_rotation_scale(int(padded_dim), C.byref(out), device, _stream_ptr(stream)))
    return out.value


def sign_rotate(d_rows, n, dim, padded_dim, d_rotated=None, d_codes=None, d_norms=None, d_norm_sq=None,
                seed=SIGN_ROTATION_SEED, device=0, stream=None):
    _check(lib().psb_sign_rotate(_vp(d_rows), C.c_int64(n), dim, padded_dim, C.c_uint32(seed), _vp(d_rotated), _vp(d_codes),
                                 _vp(d_norms), _vp(d_norm_sq), device, _stream_ptr(stream)))


def sign_encode_database(d_rows, elem_bytes, n, d_centroids, d_offsets, nlist, dim, padded_dim, d_codes, d_scales,
                         row_offset=0, seed=SIGN_ROTATION_SEED, device=0, stream=None):
    _check(lib().psb_sign_encode_database(_vp(d_rows), elem_bytes, C.c_int64(n), _vp(d_centroids), _vp(d_offsets), nlist, dim,
                                          padded_dim, C.c_uint32(seed), C.c_int64(row_offset), _vp(d_codes), _vp(d_scales),
                                          device, _stream_ptr(stream)))


def sign_encode_queries(d_queries, d_centroids, d_probes, nq, nprobe, nlist, dim, padded_dim, d_states=None, d_norm_sq=None,
                        d_state_codes=None, d_norms=None, seed=SIGN_ROTATION_SEED, device=0, stream=None):
    _check(lib().psb_sign_encode_queries(_vp(d_queries), _vp(d_centroids), _vp(d_probes), nq, nprobe, nlist, dim, padded_dim,
                                         C.c_uint32(seed), _vp(d_states), _vp(d_norm_sq), _vp(d_state_codes), _vp(d_norms),
                                         device, _stream_ptr(stream)))


def sign_search_candidates(mode, d_codes, d_row_params, d_offsets, nlist, d_probes, nq, nprobe, padded_dim, candidate_count,
                           d_rows_out, d_dist_out=None, d_states=None, d_norm_sq=None, d_state_codes=None, d_norms=None,
                           device=0, stream=None):
    _check(lib().psb_sign_search_candidates(int(mode), _vp(d_states), _vp(d_norm_sq), _vp(d_state_codes), _vp(d_norms),
                                            _vp(d_codes), _vp(d_row_params), _vp(d_offsets), nlist, _vp(d_probes), nq, nprobe,
                                            padded_dim, candidate_count, _vp(d_rows_out), _vp(d_dist_out), device,
                                            _stream_ptr(stream)))


class SignIndex:
    """The reference's IVFResTurboQuant index and search workspace in one object
    (src/search/ivf_res_turboquant/ivf_res_turboquant_search.cuh:25-112): build_u8 / build_cached_u32 put sign codes, scales,
    centroids and list offsets on the device; search_candidates takes host queries and probe ids and returns candidate rows."""

    ENCODE_CHUNK_ROWS = 1 << 20   # the host corpus goes through the device in bounded chunks, as in residual_encoding.cu:24

    def __init__(self, device=0):
        import torch
        self._t = torch
        self.device = device
        self.dev = torch.device("cuda", device)
        self.n_vectors = self.n_clusters = self.dim = self.padded_dim = 0
        self.rotation_seed = SIGN_ROTATION_SEED
        self.codes = self.scales = self.centroids = self.offsets = None

    @property
    def bytes_per_vector(self):
        return self.padded_dim // 32 * 4 + 4

    def _place(self, centroids, offsets, n_vectors, dim):
        t = self._t
        centroids = np.ascontiguousarray(centroids, np.float32)
        offsets = np.ascontiguousarray(offsets, np.int64)
        padded = sign_padded_dim(dim)
        if n_vectors <= 0 or centroids.ndim != 2 or centroids.shape[1] != dim or offsets.size != centroids.shape[0] + 1 or padded < 0:
            raise InvalidArgument(1, "IVFResTurboQuant index build received invalid input")
        self.n_vectors, self.n_clusters, self.dim, self.padded_dim = int(n_vectors), centroids.shape[0], int(dim), padded
        self.centroids = t.from_numpy(centroids).to(self.dev)
        self.offsets = t.from_numpy(offsets).to(self.dev)
        self.host_offsets = offsets
        self.codes = t.empty((self.n_vectors, padded // 32), dtype=t.int32, device=self.dev)
        self.scales = t.empty(self.n_vectors, dtype=t.float32, device=self.dev)

    def build_u8(self, host_vectors, host_centroids, host_cluster_offsets, rotation_seed=SIGN_ROTATION_SEED):
        t = self._t
        rows = np.ascontiguousarray(host_vectors)
        if rows.dtype != np.uint8 and rows.dtype != np.float32:
            raise InvalidArgument(1, "rows must be uint8 or float32")
        self._place(host_centroids, host_cluster_offsets, rows.shape[0], rows.shape[1])
        self.rotation_seed = int(rotation_seed)
        for start in range(0, self.n_vectors, self.ENCODE_CHUNK_ROWS):
            chunk = t.from_numpy(rows[start:start + self.ENCODE_CHUNK_ROWS]).to(self.dev)
            sign_encode_database(chunk, rows.dtype.itemsize, chunk.shape[0], self.centroids, self.offsets, self.n_clusters,
                                 self.dim, self.padded_dim, self.codes, self.scales, row_offset=start, seed=self.rotation_seed,
                                 device=self.device)
            t.cuda.synchronize(self.dev)
        return self

    def build_cached_u32(self, host_codes, host_scales, host_centroids, host_cluster_offsets):
        t = self._t
        codes = np.ascontiguousarray(host_codes, np.uint32)
        scales = np.ascontiguousarray(host_scales, np.float32)
        dim = np.asarray(host_centroids).shape[1]
        if dim % 32 != 0 or codes.ndim != 2 or codes.shape[0] != scales.shape[0]:
            raise InvalidArgument(1, "IVFResTurboQuant cached build received invalid input")
        self._place(host_centroids, host_cluster_offsets, codes.shape[0], dim)
        if codes.shape[1] != self.padded_dim // 32:
            raise InvalidArgument(1, "IVFResTurboQuant cached build received invalid input")
        self.rotation_seed = SIGN_ROTATION_SEED
        self.codes.copy_(t.from_numpy(codes.view(np.int32)))
        self.scales.copy_(t.from_numpy(scales))
        return self

    def search_candidates(self, host_queries, host_probe_ids, candidate_count=512, score_mode=SIGN_FLOAT_STATES,
                          want_distances=False):
        """host_queries [nq][dim] fp32, host_probe_ids [nq][nprobe] (ids outside the index are skipped); candidate rows
        [nq][candidate_count] int32 in ascending (score, row) order, -1 where fewer rows were scanned."""
        t = self._t
        if self.n_vectors <= 0:
            raise InvalidArgument(1, "IVFResTurboQuant search received invalid input")
        q = np.ascontiguousarray(host_queries, np.float32)
        probes = np.ascontiguousarray(host_probe_ids)
        if q.ndim != 2 or q.shape[1] != self.dim or probes.ndim != 2 or probes.shape[0] != q.shape[0] or q.shape[0] <= 0 \
                or probes.shape[1] <= 0 or candidate_count <= 0:
            raise InvalidArgument(1, "IVFResTurboQuant search received invalid input")
        nq, nprobe = probes.shape
        bad = (probes < 0) | (probes >= self.n_clusters)
        d_probes = t.from_numpy(np.where(bad, -1, probes).astype(np.int32)).to(self.dev)
        d_q = t.from_numpy(q).to(self.dev)
        words = self.padded_dim // 32
        st = nsq = sc = nm = None
        if score_mode == SIGN_FLOAT_STATES:
            st = t.empty((nq * nprobe, self.padded_dim), dtype=t.float32, device=self.dev)
            nsq = t.empty(nq * nprobe, dtype=t.float32, device=self.dev)
        else:
            sc = t.empty((nq * nprobe, words), dtype=t.int32, device=self.dev)
            nm = t.empty(nq * nprobe, dtype=t.float32, device=self.dev)
        sign_encode_queries(d_q, self.centroids, d_probes, nq, nprobe, self.n_clusters, self.dim, self.padded_dim, d_states=st,
                            d_norm_sq=nsq, d_state_codes=sc, d_norms=nm, seed=self.rotation_seed, device=self.device)
        rows = t.empty((nq, candidate_count), dtype=t.int32, device=self.dev)
        dist = t.empty((nq, candidate_count), dtype=t.float32, device=self.dev) if want_distances else None
        sign_search_candidates(score_mode, self.codes, self.scales, self.offsets, self.n_clusters, d_probes, nq, nprobe,
                               self.padded_dim, candidate_count, rows, dist, d_states=st, d_norm_sq=nsq, d_state_codes=sc,
                               d_norms=nm, device=self.device)
        t.cuda.synchronize(self.dev)
        return (rows.cpu().numpy(), dist.cpu().numpy()) if want_distances else rows.cpu().numpy()

    def search(self, host_queries, host_vectors, nprobe, topk, n_rerank=512, reordered_ids=None, queries_u8=None,
               score_mode=SIGN_FLOAT_STATES):
        """The whole search with the sign codes as the first stage: coarse top-nprobe lists (exact fp32), the n_rerank rows with
        the smallest sign-code scores, exact re-ranking of those from the host rows (`host_vectors`, list-contiguous, fp32 or
        u8 - u8 rows are compared with `queries_u8`, as ivf_rerank_host does), ids through `reordered_ids` when given.
        Returns (ids [nq][topk] int64, distances [nq][topk]); -1 / FLT_MAX where fewer rows were scanned."""
        q = np.ascontiguousarray(host_queries, np.float32)
        base = np.ascontiguousarray(host_vectors)
        if base.shape[0] != self.n_vectors or base.shape[1] != self.dim or n_rerank < topk or topk <= 0:
            raise InvalidArgument(1, "IVFResTurboQuant search received invalid input")
        if base.dtype == np.uint8 and queries_u8 is None:
            raise InvalidArgument(1, "u8 rows are re-ranked against u8 queries")
        probes, _ = coarse_host(q, self.centroids.cpu().numpy(), nprobe, device=self.device)
        cand = self.search_candidates(q, probes, n_rerank, score_mode=score_mode)
        rows, dist = rerank_host(base, queries_u8 if base.dtype == np.uint8 else q, cand, topk, device=self.device)
        ids = rows.astype(np.int64)
        if reordered_ids is not None:
            rid = np.ascontiguousarray(reordered_ids, np.int64)
            ids = np.where(ids >= 0, rid[np.maximum(ids, 0)], -1)
        return ids, dist


def knn_exact(d_queries, nq, d_base, n, dim, k, d_rows, d_dist, device=0, stream=None):
    _check(lib().psb_knn_exact(C.c_void_p(_p(d_queries)), nq, C.c_void_p(_p(d_base)), C.c_int64(n), dim, k,
                               C.c_void_p(_p(d_rows)), C.c_void_p(_p(d_dist)), device, C.c_void_p(stream) if stream else None))


# ---- training / encoding / generators on device tensors -------------------------------------------------
def _stream_ptr(stream):
    return C.c_void_p(stream) if stream else None


def kmeans_train(d_data, n, dim, d_centroids, k, iters, d_assign=None, device=0, stream=None):
    obj = np.zeros(iters + 1, np.float64)
    _check(lib().psb_kmeans_train(C.c_void_p(_p(d_data)), C.c_int64(n), dim, C.c_void_p(_p(d_centroids)), k, iters,
                                  C.c_void_p(_p(d_assign)) if d_assign is not None else None, C.c_void_p(_p(obj)),
                                  device, _stream_ptr(stream)))
    return obj


def kmeans_assign(d_data, n, dim, d_centroids, k, d_assign, d_best, device=0, stream=None, have_previous=False):
    """have_previous: d_assign holds the previous iteration's assignment on entry (one filter pass instead of two)."""
    _check(lib().psb_kmeans_assign_bounded(C.c_void_p(_p(d_data)), C.c_int64(n), dim, C.c_void_p(_p(d_centroids)), k,
                                           C.c_void_p(_p(d_assign)), C.c_void_p(_p(d_best)), int(bool(have_previous)), device,
                                           _stream_ptr(stream)))


def kmeans_accumulate(d_data, n, dim, d_assign, d_best, k, d_sums, d_counts, d_objective, device=0, stream=None):
    _check(lib().psb_kmeans_accumulate(C.c_void_p(_p(d_data)), C.c_int64(n), dim, C.c_void_p(_p(d_assign)),
                                       C.c_void_p(_p(d_best)), k, C.c_void_p(_p(d_sums)), C.c_void_p(_p(d_counts)),
                                       C.c_void_p(_p(d_objective)), device, _stream_ptr(stream)))


def kmeans_update(d_sums, d_counts, k, dim, d_centroids, device=0, stream=None):
    _check(lib().psb_kmeans_update(C.c_void_p(_p(d_sums)), C.c_void_p(_p(d_counts)), k, dim, C.c_void_p(_p(d_centroids)),
                                   device, _stream_ptr(stream)))


def residual_rows(d_data, n, dim, d_centroids, d_assign, d_out, device=0, stream=None):
    _check(lib().psb_residual_rows(C.c_void_p(_p(d_data)), C.c_int64(n), dim, C.c_void_p(_p(d_centroids)),
                                   C.c_void_p(_p(d_assign)), C.c_void_p(_p(d_out)), device, _stream_ptr(stream)))


def kmeans_init(data, k, seed, policy=0):
    """Initial centroids the reference's way (host data); returns (centroids [k][dim], rows picked [k])."""
    x = _np(data, np.float32)
    cen = np.empty((k, x.shape[1]), np.float32); rows = np.empty(k, np.int64)
    _check(lib().psb_kmeans_init(C.c_void_p(_p(x)), C.c_int64(x.shape[0]), x.shape[1], k, seed, policy, C.c_void_p(_p(cen)), C.c_void_p(_p(rows))))
    return cen, rows


def pq_train(d_data, n, dim, M, K, iters, seed, d_codebook, device=0, stream=None):
    _check(lib().psb_pq_train(C.c_void_p(_p(d_data)), C.c_int64(n), dim, M, K, iters, C.c_uint64(seed),
                              C.c_void_p(_p(d_codebook)), device, _stream_ptr(stream)))


def pq_encode(d_data, n, dim, d_codebook, M, K, d_codes, device=0, stream=None):
    _check(lib().psb_pq_encode(C.c_void_p(_p(d_data)), C.c_int64(n), dim, C.c_void_p(_p(d_codebook)), M, K,
                               C.c_void_p(_p(d_codes)), device, _stream_ptr(stream)))


def gen_mixture_rows(d_centres, d_offsets, ncomp, dim, sigma, seed, row_begin, n, d_out, device=0, stream=None):
    _check(lib().psb_gen_mixture_rows(C.c_void_p(_p(d_centres)), C.c_void_p(_p(d_offsets)), ncomp, dim, C.c_float(sigma),
                                      C.c_uint64(seed), C.c_int64(row_begin), C.c_int64(n), C.c_void_p(_p(d_out)), device,
                                      _stream_ptr(stream)))


def gen_normal(seed, first, n, scale, d_out, device=0, stream=None):
    _check(lib().psb_gen_normal(C.c_uint64(seed), C.c_int64(first), C.c_int64(n), C.c_float(scale), C.c_void_p(_p(d_out)),
                                device, _stream_ptr(stream)))
