"""GPU parity tests of the residual ADC mode (codes encode row - centroid[list]): tables per (query, probe), scan,
selection and the whole search, through the C ABI, bit-exact against the CPU checker and the reference's golden outputs."""
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


def run_residual_scan(psb, ix, q, probes, stage1_k, **kw):
    torch = _torch()
    nq, nprobe = probes.shape
    with psb.Session(ix, residual=True, **kw) as s:
        dq = dev(q)
        dp = dev(probes.astype(np.int32))
        lut = torch.zeros((nq, nprobe, s.M * s.K), dtype=torch.float32, device="cuda")
        s.stage_build_lut_residual(dq, nq, dp, nprobe, lut)
        rows = torch.empty((nq, stage1_k), dtype=torch.int32, device="cuda")
        dist = torch.empty((nq, stage1_k), dtype=torch.float32, device="cuda")
        cnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
        s.stage_scan(lut, nq, dp, nprobe, stage1_k, rows, dist, cnt)
        s.sync()
        counters = s.counters()
        return lut.cpu().numpy(), rows.cpu().numpy(), dist.cpu().numpy(), cnt.cpu().numpy(), counters


@pytest.mark.parametrize("scan_mode", [0, 1])
@pytest.mark.parametrize("M,dim", [(8, 32), (16, 64), (20, 100), (32, 128), (48, 96), (12, 48)])
def test_residual_tables_and_scan_match_checker(psb, M, dim, scan_mode):
    # M = 8 and 16 take the pairwise-tree ADC order, the others the sequential one; M = 12 runs the generic kernel
    ix = synth.make_index(6000, dim, 24, M, seed=M + 3, zipf=(M % 16 == 0), residual=True)
    q = synth.make_queries(ix, 33, seed=M + 1)
    probes, _ = oracle.coarse(q, ix["centroids"], 6)
    lut, rows, dist, cnt, _ = run_residual_scan(psb, ix, q, probes, 50, scan_mode=scan_mode)
    orow, odist, ocnt, _, oluts = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"],
                                                          ix["codebook"], 50, want_luts=True)
    assert np.array_equal(lut, oluts)
    assert np.array_equal(cnt, ocnt)
    assert np.array_equal(rows, orow)
    assert np.array_equal(dist, odist)


@pytest.mark.parametrize("M,stage1_k,n,nprobe", [(8, 512, 60000, 12), (16, 1000, 120000, 16), (48, 2048, 90000, 16)])
def test_residual_scan_with_threshold_admission(psb, M, stage1_k, n, nprobe):
    ix = synth.make_index(n, 96 if M == 48 else 32, 16, M, seed=stage1_k, zipf=True, residual=True)
    q = synth.make_queries(ix, 40, seed=7, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], nprobe)
    _, rows, dist, cnt, counters = run_residual_scan(psb, ix, q, probes, stage1_k)
    orow, odist, ocnt, scanned = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"],
                                                         ix["codebook"], stage1_k)
    assert counters["pq_scanned_codes"] == scanned
    assert np.array_equal(cnt, ocnt)
    assert np.array_equal(rows, orow)
    assert np.array_equal(dist, odist)
    assert counters["threshold_candidates"] < scanned  # the cutoff pruned


def test_residual_scan_edge_cases_and_fallback(psb):
    ix = synth.make_index(3000, 32, 8, 8, seed=5, empty_lists=(2, 5), residual=True)
    q = synth.make_queries(ix, 5, seed=9)
    probes = np.array([[2, 5, -1, 99], [0, 2, 1, 5], [3, -5, 4, 8], [5, 2, 6, 7], [6, 1, 0, 3]], np.int64)
    _, rows, dist, cnt, _ = run_residual_scan(psb, ix, q, probes, 64)
    orow, odist, ocnt, _ = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"], 64)
    assert np.array_equal(cnt, ocnt) and np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert cnt[0] == 0 and np.all(rows[0] == -1) and np.all(dist[0] == cases.FLT_MAX)
    # one code for every row: each list's distances tie with the cutoff, pools overflow, the exact fallback answers
    big = synth.make_index(50000, 32, 4, 8, seed=1, residual=True)
    big["codes"][:] = big["codes"][0]
    q = synth.make_queries(big, 5, seed=2)
    probes = np.tile(np.arange(4), (5, 1)).astype(np.int64)
    _, rows, dist, cnt, counters = run_residual_scan(psb, big, q, probes, 100)
    orow, odist, ocnt, _ = oracle.pq_scan_residual(q, probes, big["centroids"], big["offsets"], big["codes"], big["codebook"], 100)
    assert counters["fallback_queries"] >= 1
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist) and np.array_equal(cnt, ocnt)


@pytest.mark.parametrize("name", ["ivfrespq_d64_m16", "ivfrespq_d32_m8", "ivfrespq_d96_m48_zipf"])
@pytest.mark.parametrize("scan_mode", [0, 1])
def test_residual_search_matches_reference_golden(psb, name, scan_mode):
    g = cases.load_golden(name)
    nprobe, topk, n_rerank = (int(x) for x in g["params"])
    with psb.Session(cases.golden_index(g), n_rerank=n_rerank, residual=True, scan_mode=scan_mode) as s:
        r = s.search(g["queries"], nprobe, topk, want_coarse=True)
    assert np.array_equal(r["coarse"], g["ref_probes"])
    assert np.array_equal(r["indices"], g["ref_indices"])
    assert np.array_equal(r["distances"], g["ref_distances"])
    assert r["stats"]["pq_scanned_codes"] == int(g["ref_scanned"])


@pytest.mark.parametrize("m,dim,rerank", [(16, 96, 512), (8, 32, 512), (20, 100, 2048)])
def test_residual_pq_pipeline_equals_exhaustive(psb, m, dim, rerank):
    c = cases.residual_pq_pipeline_case(m, dim, rerank)
    with psb.Session(c["index"], n_rerank=c["n_rerank"], residual=True) as s:
        r = s.search(c["queries"], c["nprobe"], c["topk"])
    assert np.array_equal(r["indices"], c["exp_ids"])
    assert np.array_equal(r["distances"], c["exp_d"])


@pytest.mark.parametrize("n,dim,nlist,M,nprobe,topk,n_rerank,zipf", [
    (50000, 128, 64, 32, 8, 10, 100, False),     # residual-trained PQ configuration, cut down
    (80000, 96, 128, 48, 16, 100, 1000, True),
    (20000, 64, 32, 16, 32, 10, 0, False),       # n_rerank below the floor: candidate width 512
])
def test_residual_search_matches_checker(psb, n, dim, nlist, M, nprobe, topk, n_rerank, zipf):
    ix = synth.make_index(n, dim, nlist, M, seed=n % 97, zipf=zipf, residual=True)
    w = synth.zipf_weights(nlist) if zipf else None
    q = synth.make_queries(ix, 64, seed=17, weights=w)
    o = oracle.ivfrespq_search(ix, q, nprobe, topk, n_rerank)
    with psb.Session(ix, n_rerank=n_rerank, residual=True) as s:
        r = s.search(q, nprobe, topk, batch_size=50, want_coarse=True)
    assert np.array_equal(r["coarse"], o["coarse"])
    assert np.array_equal(r["indices"], o["indices"])
    assert np.array_equal(r["distances"], o["distances"])
    assert r["stats"]["pq_scanned_codes"] == o["scanned"]


def test_residual_overlapped_pipeline_and_device_entry(psb):
    """2600 queries run as sub-batches whose rerank overlaps the next scan; same results as the serial pipeline."""
    torch = _torch()
    ix = synth.make_index(60000, 64, 64, 16, seed=61, zipf=True, residual=True)
    q = synth.make_queries(ix, 2600, seed=62, weights=synth.zipf_weights(64))
    res = {}
    for serial in (False, True):
        with psb.Session(ix, n_rerank=120, serial_pipeline=serial, residual=True) as s:
            res[serial] = s.search(q, 8, 10, batch_size=2600, want_coarse=True)
    for k in ("indices", "distances", "coarse"):
        assert np.array_equal(res[False][k], res[True][k])
    want = oracle.ivfrespq_search(ix, q[:200], 8, 10, 120)
    assert np.array_equal(res[False]["indices"][:200], want["indices"])
    assert np.array_equal(res[False]["distances"][:200], want["distances"])
    with psb.Session(ix, n_rerank=120, max_batch=2600, residual=True) as s:
        ids = torch.empty((2600, 10), dtype=torch.int64, device="cuda")
        dd = torch.empty((2600, 10), dtype=torch.float32, device="cuda")
        s.search_device(dev(q), 2600, 8, 10, ids, dd)
        s.sync()
        assert np.array_equal(ids.cpu().numpy(), res[True]["indices"])
        assert np.array_equal(dd.cpu().numpy(), res[True]["distances"])


def test_residual_mode_needs_exact_rows(psb):
    ix = synth.make_index(2000, 32, 8, 8, seed=4, residual=True)
    with pytest.raises(psb.InvalidArgument):
        psb.Session(dict(ix, vectors=None), residual=True)
