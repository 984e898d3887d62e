"""GPU parity tests of the tensor-core pre-filter scan (tcgen05 GEMM of visiting queries against code rows decoded on the
fly, survivors re-scored exactly): through the C ABI, bit-exact against the CPU checker, and with the same admitted-row
and fallback counters as the fp32 SIMT scan - the filter may only let extra pairs through, never drop a true candidate."""
import numpy as np
import pytest

import cases
import oracle
import synth

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def dev(a):
    return _torch().from_numpy(np.ascontiguousarray(a)).cuda()


def run_scan(psb, ix, q, probes, stage1_k, scan_mode, residual=False, **kw):
    torch = _torch()
    nq, nprobe = probes.shape
    index = ix if residual else dict(ix, vectors=None)
    with psb.Session(index, residual=residual, scan_mode=scan_mode, **kw) as s:
        dq = dev(q)
        dp = dev(probes.astype(np.int32))
        if residual:
            lut = torch.zeros((nq, nprobe, s.M * s.K), dtype=torch.float32, device="cuda")
            s.stage_build_lut_residual(dq, nq, dp, nprobe, lut)
        else:
            lut = torch.empty((nq, s.M, s.K), dtype=torch.float32, device="cuda")
            s.stage_build_lut(dq, nq, lut)
        rows = torch.empty((nq, stage1_k), dtype=torch.int32, device="cuda")
        dist = torch.empty((nq, stage1_k), dtype=torch.float32, device="cuda")
        cnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
        s.stage_scan_queries(dq, lut, nq, dp, nprobe, stage1_k, rows, dist, cnt)
        s.sync()
        return rows.cpu().numpy(), dist.cpu().numpy(), cnt.cpu().numpy(), s.counters()


def check_against_fp32_scan(psb, ix, q, probes, stage1_k, residual=False, **kw):
    """Tensor-core scan == checker, and its counters == the fp32 SIMT scan's (same cutoffs, so the same admitted rows)."""
    rows, dist, cnt, c_tc = run_scan(psb, ix, q, probes, stage1_k, 3, residual, **kw)
    if residual:
        orow, odist, ocnt, scanned = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"],
                                                             stage1_k)[:4]
    else:
        orow, odist, ocnt, scanned = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], stage1_k)
    assert np.array_equal(cnt, ocnt)
    assert np.array_equal(rows, orow)
    assert np.array_equal(dist, odist)
    _, _, _, c_ref = run_scan(psb, ix, q, probes, stage1_k, 1, residual, **kw)
    assert c_tc["pq_scanned_codes"] == scanned == c_ref["pq_scanned_codes"]
    assert c_tc["fallback_queries"] == c_ref["fallback_queries"]
    assert c_tc["threshold_candidates"] == c_ref["threshold_candidates"]
    assert c_tc["prefilter_survivors"] >= c_tc["threshold_candidates"]
    return c_tc


@pytest.mark.parametrize("M,dim", [(48, 96), (32, 128), (16, 128), (8, 32), (16, 32), (64, 128), (32, 64), (12, 48)])
def test_tc_scan_matches_checker(psb, M, dim):
    # dsub 2, 4 and 8; operand tiles of 256 and 128 rows; M a multiple of 16 and not
    ix = synth.make_index(9000, dim, 12, M, seed=M + dim, zipf=True)
    q = synth.make_queries(ix, 150, seed=M + 1, weights=synth.zipf_weights(12))
    probes, _ = oracle.coarse(q, ix["centroids"], 5)
    check_against_fp32_scan(psb, ix, q, probes, 60)


@pytest.mark.parametrize("stage1_k,n,nprobe", [(10, 40000, 8), (100, 60000, 12), (1000, 120000, 16), (2048, 90000, 16)])
def test_tc_scan_with_threshold_admission(psb, stage1_k, n, nprobe):
    ix = synth.make_index(n, 32, 16, 8, seed=stage1_k, zipf=True)
    q = synth.make_queries(ix, 40, seed=7, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], nprobe)
    c = check_against_fp32_scan(psb, ix, q, probes, stage1_k)
    assert c["threshold_candidates"] < c["pq_scanned_codes"]          # the cutoff pruned
    assert c["prefilter_survivors"] < 2 * c["threshold_candidates"]   # and the bf16 filter is tight


def test_tc_scan_many_visitors_and_long_lists(psb):
    # one list above the 16,384-row chunk size, several hundred visitors per list: many visitor tiles and row chunks
    ix = synth.make_index(70000, 96, 6, 48, seed=11, zipf=True)
    q = synth.make_queries(ix, 700, seed=12, weights=synth.zipf_weights(6))
    probes, _ = oracle.coarse(q, ix["centroids"], 3)
    c = check_against_fp32_scan(psb, ix, q, probes, 200)
    assert c["prefilter_survivors"] < 2 * c["threshold_candidates"]


def test_tc_scan_edge_cases(psb):
    ix = synth.make_index(3000, 32, 8, 8, seed=5, empty_lists=(2, 5))
    q = synth.make_queries(ix, 5, seed=9)
    probes = np.array([[2, 5, -1, 99], [0, 2, 1, 5], [3, -5, 4, 8], [5, 2, 5, 2], [6, 1, 0, 3]], np.int64)
    keep = [0, 1, 2, 4]  # duplicate probes (row 3) would visit a list twice on both sides
    rows, dist, cnt, _ = run_scan(psb, ix, q[keep], probes[keep], 64, 3)
    orow, odist, ocnt, _ = oracle.pq_scan(q[keep], probes[keep], ix["offsets"], ix["codes"], ix["codebook"], 64)
    assert np.array_equal(cnt, ocnt) and np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert cnt[0] == 0 and np.all(rows[0] == -1) and np.all(dist[0] == cases.FLT_MAX)


def test_tc_scan_pool_overflow_goes_to_the_exact_fallback(psb):
    ix = synth.make_index(50000, 32, 4, 8, seed=1)
    ix["codes"][:] = ix["codes"][0]   # every distance ties with the cutoff -> pools overflow
    q = synth.make_queries(ix, 5, seed=2)
    probes = np.tile(np.arange(4), (5, 1)).astype(np.int64)
    rows, dist, cnt, c = run_scan(psb, ix, q, probes, 100, 3)
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 100)
    assert c["fallback_queries"] == 5
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist) and np.array_equal(cnt, ocnt)


@pytest.mark.parametrize("M,dim,stage1_k,n", [(8, 32, 512, 60000), (16, 64, 600, 40000), (48, 96, 1000, 90000)])
def test_tc_scan_residual_mode(psb, M, dim, stage1_k, n):
    # M = 8 and 16 re-score in the pairwise-tree order, M = 48 sequentially
    ix = synth.make_index(n, dim, 16, M, seed=stage1_k, zipf=True, residual=True)
    q = synth.make_queries(ix, 60, seed=7, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], 10)
    check_against_fp32_scan(psb, ix, q, probes, stage1_k, residual=True)


def test_tc_scan_residual_mode_without_tables(psb):
    """Residual mode with no per-(query, probe) table at all (d_lut = NULL): the scan works on q - centroid, the cutoff, the
    re-scoring selection and the fallback compute table entries from the query, the centroid and the codebook."""
    torch = _torch()
    ix = synth.make_index(90000, 96, 16, 48, seed=51, zipf=True, residual=True)
    q = synth.make_queries(ix, 60, seed=7, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], 10)
    orow, odist, ocnt, _ = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"], 700)[:4]
    with psb.Session(ix, residual=True, scan_mode=3) as s:
        dq, dp = dev(q), dev(probes.astype(np.int32))
        rows = torch.empty((60, 700), dtype=torch.int32, device="cuda")
        dist = torch.empty((60, 700), dtype=torch.float32, device="cuda")
        cnt = torch.empty((60,), dtype=torch.int32, device="cuda")
        s.stage_scan_queries(dq, None, 60, dp, 10, 700, rows, dist, cnt)
        s.sync()
        assert np.array_equal(cnt.cpu().numpy(), ocnt)
        assert np.array_equal(rows.cpu().numpy(), orow) and np.array_equal(dist.cpu().numpy(), odist)
    # every distance ties -> pools overflow -> the exact fallback builds its tables on the fly too
    ix2 = synth.make_index(50000, 32, 4, 8, seed=1, residual=True)
    ix2["codes"][:] = ix2["codes"][0]
    q2 = synth.make_queries(ix2, 5, seed=2)
    p2 = np.tile(np.arange(4), (5, 1)).astype(np.int64)
    o2 = oracle.pq_scan_residual(q2, p2, ix2["centroids"], ix2["offsets"], ix2["codes"], ix2["codebook"], 512)[:3]
    with psb.Session(ix2, residual=True, scan_mode=3) as s:
        rows = torch.empty((5, 512), dtype=torch.int32, device="cuda")
        dist = torch.empty((5, 512), dtype=torch.float32, device="cuda")
        cnt = torch.empty((5,), dtype=torch.int32, device="cuda")
        s.stage_scan_queries(dev(q2), None, 5, dev(p2.astype(np.int32)), 4, 512, rows, dist, cnt)
        s.sync()
        assert s.counters()["fallback_queries"] == 5
        assert np.array_equal(rows.cpu().numpy(), o2[0]) and np.array_equal(dist.cpu().numpy(), o2[1])
    # plain mode cannot go without its tables
    with psb.Session(dict(synth.make_index(3000, 32, 8, 8, seed=5), vectors=None), scan_mode=3) as s:
        with pytest.raises(psb.InvalidArgument):
            s.stage_scan_queries(dev(q2), None, 5, dev(p2.astype(np.int32)), 4, 16, rows, dist, cnt)


@pytest.mark.parametrize("form", ["fp32", "u16", "u16_model"])
def test_tc_scan_residual_with_the_callers_row_correction(psb, form):
    """The per-row correction handed in by the caller (fp32, the affine u16 payload, or u16 on the fixed-model range) places
    the cutoff; the selected rows and distances stay the exact ones and no query needs the fallback."""
    torch = _torch()
    ix = synth.make_index(90000, 96, 16, 48, seed=61, zipf=True, residual=True)
    q = synth.make_queries(ix, 60, seed=8, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], 10)
    orow, odist, ocnt, _ = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"], 700)[:4]
    v = psb.row_correction_compute(ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"])
    kw = dict(row_correction=v)
    if form == "u16":
        hdr, u = psb.row_correction_quantize_u16(v)
        kw = dict(row_correction=u, rc_scale=hdr.scale, rc_offset=hdr.offset)
    elif form == "u16_model":
        sc, off = psb.row_correction_model_u16(ix["centroids"], ix["codebook"])
        kw = dict(row_correction=psb.row_correction_encode_u16(v, sc, off), rc_scale=sc, rc_offset=off)
    with psb.Session(ix, residual=True, scan_mode=3, **kw) as s:
        rows = torch.empty((60, 700), dtype=torch.int32, device="cuda")
        dist = torch.empty((60, 700), dtype=torch.float32, device="cuda")
        cnt = torch.empty((60,), dtype=torch.int32, device="cuda")
        s.stage_scan_queries(dev(q), None, 60, dev(probes.astype(np.int32)), 10, 700, rows, dist, cnt)
        s.sync()
        assert s.counters()["fallback_queries"] == 0
        assert np.array_equal(cnt.cpu().numpy(), ocnt)
        assert np.array_equal(rows.cpu().numpy(), orow) and np.array_equal(dist.cpu().numpy(), odist)
    with pytest.raises(psb.InvalidArgument):
        psb.Session(ix, residual=True, scan_mode=3, row_correction=np.zeros(90000, np.uint16), rc_scale=0.0)


def test_tc_scan_split_by_visitor_count(psb):
    """tc_min_visitors = 20: lists with fewer visitors stay with the SIMT scan, the others go to the tensor-core kernel;
    the pools then hold exact keys and unscored survivors side by side."""
    ix = synth.make_index(60000, 96, 24, 48, seed=21, zipf=True)
    q = synth.make_queries(ix, 200, seed=22, weights=synth.zipf_weights(24))
    probes, _ = oracle.coarse(q, ix["centroids"], 6)
    visitors = np.bincount(probes.ravel(), minlength=24)
    assert (visitors >= 20).any() and ((visitors > 0) & (visitors < 20)).any()
    rows, dist, cnt, c = run_scan(psb, ix, q, probes, 300, 0, tc_min_visitors=20)
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 300)
    assert np.array_equal(cnt, ocnt) and np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert c["prefilter_survivors"] > 0


def test_tc_scan_refuses_unsupported_shapes(psb):
    ix = synth.make_index(3000, 100, 8, 20, seed=3)   # dsub 5
    q = synth.make_queries(ix, 8, seed=4)
    probes, _ = oracle.coarse(q, ix["centroids"], 4)
    with pytest.raises(psb.PsbError) as e:
        run_scan(psb, ix, q, probes, 20, 3)
    assert e.value.status == 2
    rows, dist, cnt, _ = run_scan(psb, ix, q, probes, 20, 0)   # auto: the SIMT scan takes it
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 20)
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist)


@pytest.mark.parametrize("residual", [False, True])
def test_search_with_tc_scan_matches_checker(psb, residual):
    ix = synth.make_index(80000, 96, 64, 48, seed=31, zipf=True, residual=residual)
    q = synth.make_queries(ix, 500, seed=32, weights=synth.zipf_weights(64))
    search = oracle.ivfrespq_search if residual else oracle.ivfpq_search
    want = search(ix, q[:150], 12, 10, 200)
    with psb.Session(ix, n_rerank=200, residual=residual, scan_mode=3) as s:
        got = s.search(q, 12, 10, batch_size=500)
    assert np.array_equal(got["indices"][:150], want["indices"])
    assert np.array_equal(got["distances"][:150], want["distances"])
    assert got["stats"]["prefilter_survivors"] > 0
    with psb.Session(ix, n_rerank=200, residual=residual, scan_mode=1) as s:
        ref = s.search(q, 12, 10, batch_size=500)
    assert np.array_equal(got["indices"], ref["indices"]) and np.array_equal(got["distances"], ref["distances"])


def test_tc_scan_bounded_wait_gives_up_cleanly(psb):
    """The time-out path: with the issuing warp told to skip its tcgen05.mma (nothing is left in flight) every role that
    waits for a result runs into the shortened poll limit, the kernel frees its tensor memory and returns, and the call
    reports PSB_TIMEOUT.  The device stays usable: the next session's scan gives the right answer."""
    ix = synth.make_index(9000, 96, 12, 48, seed=41, zipf=True)
    q = synth.make_queries(ix, 64, seed=42)
    probes, _ = oracle.coarse(q, ix["centroids"], 4)
    with pytest.raises(psb.PsbError) as e:
        run_scan(psb, ix, q, probes, 50, 3, test_skip_mma=1, test_wait_limit=4096)
    assert e.value.status == 7
    rows, dist, cnt, _ = run_scan(psb, ix, q, probes, 50, 3)
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 50)
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist) and np.array_equal(cnt, ocnt)
