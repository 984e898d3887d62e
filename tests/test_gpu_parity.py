"""GPU parity tests: every stage of the CUDA path, called through the C ABI, against the CPU checker on
the same seeded inputs - bit-exact ids, rows and distances."""
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
    torch = _torch()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ---------------------------------------------------------------------------------------------- coarse
@pytest.mark.parametrize("nq,nlist,dim,nprobe", [(37, 300, 96, 8), (5, 64, 100, 17), (130, 1000, 128, 64),
                                                  (3, 7, 8, 7), (64, 4096, 96, 1), (9, 5000, 32, 513)])
def test_coarse_matches_checker(psb, nq, nlist, dim, nprobe):
    rng = np.random.default_rng(nq * 7 + nlist)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    c = rng.standard_normal((nlist, dim)).astype(np.float32)
    ids, dist = psb.coarse_host(q, c, nprobe)
    oi, od = oracle.coarse(q, c, nprobe)
    assert np.array_equal(ids, oi)
    assert np.array_equal(dist, od)


def test_coarse_integer_grid_with_ties(psb):
    # integer-valued inputs: many exactly equal distances; ties resolve by list id
    rng = np.random.default_rng(3)
    q = rng.integers(-3, 4, (40, 16)).astype(np.float32)
    c = rng.integers(-3, 4, (500, 16)).astype(np.float32)
    ids, dist = psb.coarse_host(q, c, 65)
    oi, od = oracle.coarse(q, c, 65)
    assert np.array_equal(ids, oi) and np.array_equal(dist, od)
    zeros = np.zeros((4, 16), np.float32)
    ids, dist = psb.coarse_host(q[:2], zeros, 4)
    assert np.array_equal(ids, np.tile(np.arange(4), (2, 1)))


def test_coarse_rejects_bad_nprobe(psb):
    with pytest.raises(psb.InvalidArgument):
        psb.coarse_host(np.zeros((1, 8), np.float32), np.zeros((4, 8), np.float32), 5)


# ---------------------------------------------------------------------------------------------- LUT + scan
def run_stage_scan(psb, ix, q, probes, stage1_k, **kw):
    torch = _torch()
    nq = q.shape[0]
    with psb.Session(dict(ix, vectors=None), **kw) as s:
        dq = dev(q)
        lut = torch.empty((nq, s.M, s.K), dtype=torch.float32, device="cuda")
        s.stage_build_lut(dq, nq, lut)
        dp = dev(probes.astype(np.int32))
        rows = torch.empty((nq, stage1_k), dtype=torch.int32, device="cuda")
        dist = torch.empty((nq, stage1_k), dtype=torch.float32, device="cuda")
        cnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
        s.stage_scan(lut, nq, dp, probes.shape[1], stage1_k, rows, dist, cnt)
        s.sync()
        counters = s.counters()
        return lut.cpu().numpy(), rows.cpu().numpy(), dist.cpu().numpy(), cnt.cpu().numpy(), counters


@pytest.mark.parametrize("M,dim", [(8, 32), (16, 96), (20, 100), (32, 128), (48, 96), (64, 128), (12, 48)])
def test_lut_and_scan_match_checker(psb, M, dim):
    ix = synth.make_index(6000, dim, 24, M, seed=M, zipf=(M % 16 == 0))
    q = synth.make_queries(ix, 33, seed=M + 1)
    probes, _ = oracle.coarse(q, ix["centroids"], 6)
    lut, rows, dist, cnt, _ = run_stage_scan(psb, ix, q, probes, 50)
    assert np.array_equal(lut, oracle.pq_lut(q, ix["codebook"]))
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 50)
    assert np.array_equal(cnt, ocnt)
    assert np.array_equal(rows, orow)
    assert np.array_equal(dist, odist)


@pytest.mark.parametrize("stage1_k,n,nprobe", [(10, 40000, 8), (100, 60000, 12), (1000, 120000, 16), (2048, 90000, 16)])
def test_scan_with_threshold_admission(psb, stage1_k, n, nprobe):
    # enough rows per query that the sampled cutoff, the pools and the selection are all exercised
    ix = synth.make_index(n, 32, 16, 8, seed=stage1_k, zipf=True)
    q = synth.make_queries(ix, 40, seed=7, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], nprobe)
    _, rows, dist, cnt, counters = run_stage_scan(psb, ix, q, probes, stage1_k)
    orow, odist, ocnt, scanned = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], stage1_k)
    assert counters["pq_scanned_codes"] == scanned
    assert np.array_equal(cnt, ocnt)
    assert np.array_equal(rows, orow)
    assert np.array_equal(dist, odist)
    assert counters["threshold_candidates"] < scanned  # the cutoff pruned


def test_scan_edge_cases(psb):
    ix = synth.make_index(3000, 32, 8, 8, seed=5, empty_lists=(2, 5))
    q = synth.make_queries(ix, 6, seed=9)
    probes = np.array([[2, 5, -1, 99], [0, 2, 1, 5], [7, 7, 7, 7], [3, -5, 4, 8], [5, 2, 5, 2], [6, 1, 0, 3]], np.int64)
    # duplicate probes (row 2) would visit a list twice on both sides; keep them out of the comparison
    keep = [0, 1, 3, 4, 5]
    _, rows, dist, cnt, _ = run_stage_scan(psb, ix, q[keep], probes[keep], 64)
    orow, odist, ocnt, _ = oracle.pq_scan(q[keep], probes[keep], ix["offsets"], ix["codes"], ix["codebook"], 64)
    assert np.array_equal(cnt, ocnt) and np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert cnt[0] == 0 and np.all(rows[0] == -1) and np.all(dist[0] == cases.FLT_MAX)


def test_scan_exact_fallback_on_pool_overflow(psb):
    # every row has the same code -> every distance ties with the cutoff -> pools overflow -> exact fallback
    ix = synth.make_index(50000, 32, 4, 8, seed=1)
    ix["codes"][:] = ix["codes"][0]
    q = synth.make_queries(ix, 5, seed=2)
    probes = np.tile(np.arange(4), (5, 1)).astype(np.int64)
    _, rows, dist, cnt, counters = run_stage_scan(psb, ix, q, probes, 100)
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 100)
    assert counters["fallback_queries"] == 5
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist) and np.array_equal(cnt, ocnt)


def test_scan_shard_ranges_partition_the_work(psb):
    ix = synth.make_index(30000, 32, 16, 8, seed=8, zipf=True)
    q = synth.make_queries(ix, 20, seed=3)
    probes, _ = oracle.coarse(q, ix["centroids"], 8)
    full = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 100)
    parts_r, parts_d = [], []
    for lb, le in ((0, 5), (5, 11), (11, 16)):
        _, rows, dist, cnt, _ = run_stage_scan(psb, ix, q, probes, 100, list_begin=lb, list_end=le)
        masked = np.where((probes >= lb) & (probes < le), probes, -1)
        orow, odist, ocnt, _ = oracle.pq_scan(q, masked, ix["offsets"], ix["codes"], ix["codebook"], 100)
        assert np.array_equal(rows, orow) and np.array_equal(dist, odist)
        parts_r.append(rows); parts_d.append(dist)
    torch = _torch()
    with psb.Session(dict(ix, vectors=None)) as s:
        out_r = torch.empty((20, 100), dtype=torch.int32, device="cuda")
        out_d = torch.empty((20, 100), dtype=torch.float32, device="cuda")
        s.stage_merge(dev(np.stack(parts_r)), dev(np.stack(parts_d)), 3, 20, 100, out_r, out_d)
        s.sync()
    assert np.array_equal(out_r.cpu().numpy(), full[0])
    assert np.array_equal(out_d.cpu().numpy(), full[1])


# ---------------------------------------------------------------------------------------------- rerank
@pytest.mark.parametrize("dtype", [np.uint8, np.float32])
@pytest.mark.parametrize("dim", [100, 128])
@pytest.mark.parametrize("width", [128, 256, 512, 1024, 2048])
def test_host_rerank_known_answer(psb, dtype, dim, width):
    c = cases.host_rerank_case(dtype, dim, width)
    ids, dist = psb.rerank_host(c["base"], c["queries"], c["cand"], c["topk"], candidate_count=width, counts=c["counts"])
    assert np.array_equal(ids, c["exp_ids"])
    assert np.array_equal(dist, c["exp_d"])
    with pytest.raises(psb.InvalidArgument):
        psb.rerank_host(c["base"], c["queries"], c["cand"], c["topk"], candidate_count=width,
                        counts=np.array([0, width + 1, 0, 0], np.int32))


def test_rerank_adapter_known_answer(psb):
    c = cases.adapter_case()
    ids, dist = psb.rerank_host(c["base"], c["queries"], c["cand"], c["topk"], counts=c["counts"])
    assert np.array_equal(ids, c["exp_ids"])
    assert np.array_equal(dist, c["exp_d"])


@pytest.mark.parametrize("name", ["rerank_d96", "rerank_d100"])
def test_rerank_matches_reference_golden(psb, name):
    g = cases.load_golden(name)
    width, topk = (int(x) for x in g["params"])
    ids, dist = psb.rerank_host(g["base"], g["queries"], g["candidates"], topk, candidate_count=width, counts=g["counts"])
    assert np.array_equal(ids, g["ref_ids"])
    assert np.array_equal(dist, g["ref_dist"])  # bit-exact with the reference's AVX-512 kernel order


@pytest.mark.parametrize("dim", [8, 24, 96, 100, 128, 200])
def test_rerank_random_matches_checker(psb, dim):
    rng = np.random.default_rng(dim)
    base = rng.standard_normal((500, dim)).astype(np.float32)
    q = rng.standard_normal((11, dim)).astype(np.float32)
    cand = rng.integers(-2, 503, (11, 300)).astype(np.int32)
    ids, dist = psb.rerank_host(base, q, cand, 25)
    oi, od = oracle.rerank(base, q, cand, 25)
    assert np.array_equal(ids, oi) and np.array_equal(dist, od)


# ---------------------------------------------------------------------------------------------- whole search
@pytest.mark.parametrize("name", ["ivfpq_d32_m8", "ivfpq_d96_m48_zipf", "ivfpq_d100_m20"])
@pytest.mark.parametrize("mode", [0, 1, 4])
def test_search_matches_reference_golden(psb, name, mode):
    g = cases.load_golden(name)
    nprobe, topk, n_rerank = (int(x) for x in g["params"])
    ix = cases.golden_index(g)
    with psb.Session(ix, n_rerank=n_rerank, exact_mode=mode) as s:
        r = s.search(g["queries"], nprobe, topk, batch_size=7, want_coarse=True)  # tail batch on purpose
    assert np.array_equal(r["coarse"], g["ref_probes"])
    assert np.array_equal(r["indices"], g["ref_indices"])
    assert np.array_equal(r["distances"], g["ref_distances"])
    with psb.Session(dict(ix, vectors=None)) as s:
        r = s.search(g["queries"], nprobe, topk)
    assert np.array_equal(r["distances"], g["ref_norerank_distances"])


@pytest.mark.parametrize("m,dim,rerank,empty", [(16, 96, 512, False), (16, 96, 512, True), (20, 100, 2048, False),
                                                 (16, 128, 2048, False)])
def test_plain_pq_pipeline_equals_exhaustive(psb, m, dim, rerank, empty):
    c = cases.plain_pq_pipeline_case(m, dim, rerank, empty)
    with psb.Session(c["index"], n_rerank=c["n_rerank"]) as s:
        r = s.search(c["queries"], c["nprobe"], c["topk"], batch_size=8)
    assert np.array_equal(r["indices"], c["exp_ids"])
    assert np.array_equal(r["distances"], c["exp_d"])


@pytest.mark.parametrize("n,dim,nlist,M,nprobe,topk,n_rerank,zipf", [
    (50000, 128, 64, 32, 8, 10, 100, False),    # IVF-PQ 1M configuration, cut down
    (80000, 96, 128, 48, 16, 100, 1000, True),  # IVF-PQ 100M sharded configuration, cut down
    (20000, 64, 32, 16, 32, 10, 0, False),      # no rerank: ADC distances out
])
def test_search_matches_checker(psb, n, dim, nlist, M, nprobe, topk, n_rerank, zipf):
    ix = synth.make_index(n, dim, nlist, M, seed=n % 97, zipf=zipf)
    w = synth.zipf_weights(nlist) if zipf else None
    q = synth.make_queries(ix, 64, seed=17, weights=w)
    o = oracle.ivfpq_search(ix if n_rerank else dict(ix, vectors=None), q, nprobe, topk, n_rerank)
    with psb.Session(ix if n_rerank else dict(ix, vectors=None), n_rerank=n_rerank) as s:
        r = s.search(q, nprobe, topk, batch_size=50, want_coarse=True)
    assert np.array_equal(r["coarse"], o["coarse"])
    assert np.array_equal(r["indices"], o["indices"])
    assert np.array_equal(r["distances"], o["distances"])
    assert r["stats"]["pq_scanned_codes"] == o["scanned"]
    assert r["stats"]["kernel_launches"] > 0


def test_search_argument_errors(psb):
    ix = synth.make_index(2000, 32, 8, 8, seed=4)
    q = synth.make_queries(ix, 4)
    with psb.Session(ix, n_rerank=50) as s:
        for bad in (dict(nprobe=0, topk=5), dict(nprobe=9, topk=5), dict(nprobe=4, topk=0)):
            with pytest.raises(psb.InvalidArgument):
                s.search(q, **bad)
        with pytest.raises(psb.InvalidArgument):
            s.search(q[:, :16], 4, 5)
        empty = s.search(q[:0], 4, 5)
        assert empty["indices"].shape == (0, 5)


# ---------------------------------------------------------------------------------------------- training
def test_pq_encode_matches_checker(psb):
    torch = _torch()
    for M, dim in ((8, 32), (48, 96), (20, 100)):
        ix = synth.make_index(3000, dim, 8, M, seed=M + 40)
        codes = torch.empty((3000, M), dtype=torch.uint8, device="cuda")
        psb.pq_encode(dev(ix["vectors"]), 3000, dim, dev(ix["codebook"]), M, 256, codes)
        torch.cuda.synchronize()
        assert np.array_equal(codes.cpu().numpy(), oracle.pq_encode(ix["vectors"], ix["codebook"]))


def test_kmeans_matches_checker_objective(psb):
    torch = _torch()
    centres, data, _ = synth.mixture(20000, 32, 40, 0.3, seed=6)
    init = data[:64].copy()
    ocen, oassign, oobj = oracle.kmeans_lloyd(data, init, 5)
    dcen = dev(init)
    dassign = torch.empty((20000,), dtype=torch.int32, device="cuda")
    obj = psb.kmeans_train(dev(data), 20000, 32, dcen, 64, 5, dassign)
    # same criterion as the reference's own k-means test: relative objective error and centroid RMSE
    assert np.allclose(obj, oobj, rtol=1e-5)
    assert np.sqrt(np.mean((dcen.cpu().numpy() - ocen) ** 2)) < 1e-5
    assert np.mean(dassign.cpu().numpy() == oassign) > 0.9999
    assert np.all(np.diff(obj) <= 1e-6 * obj[0])


def test_pq_train_reduces_quantisation_error(psb):
    torch = _torch()
    _, data, _ = synth.mixture(30000, 32, 16, 0.5, seed=9)
    cb = torch.empty((8, 256, 4), dtype=torch.float32, device="cuda")
    d = dev(data)
    errs = []
    for iters in (0, 8):
        psb.pq_train(d, 30000, 32, 8, 256, iters, 1234, cb)
        codes = oracle.pq_encode(data, cb.cpu().numpy())
        rec = cb.cpu().numpy()[np.arange(8)[None, :], codes].reshape(30000, 32)
        errs.append(float(((rec - data) ** 2).sum(1).mean()))
    assert errs[1] < 0.8 * errs[0]


def test_pq_train_iterations_are_lloyd_iterations(psb):
    """Three training iterations from the initial codewords equal three Lloyd iterations on the host (nearest codeword by
    exact distance, mean of the members, a codeword without members kept): the trainer's assignment uses |c|^2 - 2 x.c, so
    a row within rounding of two codewords may go either way - nearly all entries agree closely, all agree loosely."""
    torch = _torch()
    _, data, _ = synth.mixture(20000, 32, 16, 0.5, seed=21)
    d = dev(data)
    cb0 = torch.empty((8, 256, 4), dtype=torch.float32, device="cuda")
    cb3 = torch.empty((8, 256, 4), dtype=torch.float32, device="cuda")
    psb.pq_train(d, 20000, 32, 8, 256, 0, 77, cb0)
    psb.pq_train(d, 20000, 32, 8, 256, 3, 77, cb3)
    want = cb0.cpu().numpy().astype(np.float64)
    x = data.reshape(20000, 8, 4).astype(np.float64)
    for _ in range(3):
        for sub in range(8):
            d2 = ((x[:, sub, None, :] - want[sub][None]) ** 2).sum(2)
            a = d2.argmin(1)
            for c in np.unique(a):
                want[sub, c] = x[a == c, sub].mean(0)
    got = cb3.cpu().numpy().astype(np.float64)
    close = np.isclose(got, want, rtol=1e-4, atol=1e-4)
    assert close.mean() > 0.995
    assert np.allclose(got, want, rtol=0.05, atol=0.05)


def test_generators_are_deterministic_and_gaussian(psb):
    torch = _torch()
    a = torch.empty((1 << 20,), dtype=torch.float32, device="cuda")
    b = torch.empty((1 << 20,), dtype=torch.float32, device="cuda")
    psb.gen_normal(77, 0, 1 << 20, 1.0, a)
    psb.gen_normal(77, 1 << 19, 1 << 19, 1.0, b)
    torch.cuda.synchronize()
    assert torch.equal(a[1 << 19:], b[: 1 << 19])  # counter-based: independent of the launch shape
    assert abs(float(a.mean())) < 5e-3 and abs(float(a.std()) - 1.0) < 5e-3
    assert abs(float((a ** 4).mean()) - 3.0) < 0.05


# ---------------------------------------------------------------------------------------------- striped shards
def test_striped_shards_reproduce_the_whole_index_search(psb):
    """Three striped shard sessions on one GPU, combined the way the ranks of a multi-GPU run combine them
    (candidate merge, elementwise-min of partial rerank scores, max of partial ids)."""
    torch = _torch()
    from fake_engine import stripe_index
    ix = synth.make_index(40000, 64, 24, 16, seed=55, zipf=True)
    q = synth.make_queries(ix, 32, seed=56, weights=synth.zipf_weights(24))
    nq, nprobe, topk, width, world = 32, 6, 10, 200, 3
    want = oracle.ivfpq_search(ix, q, nprobe, topk, width)
    dq = dev(q)
    sessions = []
    for r in range(world):
        local, gb = stripe_index(ix, r, world)
        sessions.append(psb.Session(local, n_rerank=width, list_global_begin=gb))
    rows = torch.empty((world, nq, width), dtype=torch.int32, device="cuda")
    dist = torch.empty((world, nq, width), dtype=torch.float32, device="cuda")
    for r, s in enumerate(sessions):
        probes = torch.empty((nq, nprobe), dtype=torch.int32, device="cuda")
        lut = torch.empty((nq, s.M, s.K), dtype=torch.float32, device="cuda")
        cnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
        s.stage_coarse(dq, nq, nprobe, probes)
        s.stage_build_lut(dq, nq, lut)
        s.stage_scan(lut, nq, probes, nprobe, width, rows[r], dist[r], cnt)
        s.sync()
    m_rows = torch.empty((nq, width), dtype=torch.int32, device="cuda")
    m_dist = torch.empty((nq, width), dtype=torch.float32, device="cuda")
    sessions[0].stage_merge(rows, dist, world, nq, width, m_rows, m_dist)
    sessions[0].sync()
    assert np.array_equal(m_rows.cpu().numpy(), want["stage1"])
    part = torch.empty((world, nq, width), dtype=torch.float32, device="cuda")
    for r, s in enumerate(sessions):
        s.stage_rerank_partial(dq, nq, m_rows, width, width, None, part[r])
        s.sync()
    finite = torch.isfinite(part).sum(0)
    assert int(finite.max()) == 1 and int(finite.min()) == 1  # every candidate row is held by exactly one shard
    comb = part.min(0).values.contiguous()
    o_rows = torch.empty((nq, topk), dtype=torch.int32, device="cuda")
    o_dist = torch.empty((nq, topk), dtype=torch.float32, device="cuda")
    sessions[1].stage_select_topk(comb, m_rows, nq, width, width, None, topk, o_rows, o_dist)
    ids = torch.empty((world, nq, topk), dtype=torch.int64, device="cuda")
    for r, s in enumerate(sessions):
        s.stage_map_ids(o_rows, nq * topk, ids[r])
        s.sync()
    sessions[1].sync()
    assert np.array_equal(ids.max(0).values.cpu().numpy(), want["indices"])
    assert np.array_equal(o_dist.cpu().numpy(), want["distances"])
    for s in sessions:
        s.close()


# ---------------------------------------------------------------------------------------------- scan variants
@pytest.mark.parametrize("M,dim,zipf", [(48, 96, True), (32, 128, False), (20, 100, True), (16, 64, False), (8, 32, True)])
def test_half_prefilter_scan_equals_fp32_scan(psb, M, dim, zipf):
    """The fp16 pre-filter scan (8 visitors per item, exact fp32 re-scoring of the pairs that pass) must admit
    exactly the rows the fp32 scan admits and return the same candidates."""
    nlist = 20
    ix = synth.make_index(120000, dim, nlist, M, seed=M + 7, zipf=zipf)
    q = synth.make_queries(ix, 48, seed=M + 8, weights=synth.zipf_weights(nlist) if zipf else None)
    probes, _ = oracle.coarse(q, ix["centroids"], 10)
    out = {}
    for mode in (0, 1):
        _, rows, dist, cnt, counters = run_stage_scan(psb, ix, q, probes, 300, scan_mode=mode)
        out[mode] = (rows, dist, cnt, counters)
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    assert np.array_equal(out[0][2], out[1][2])
    assert out[0][3]["threshold_candidates"] == out[1][3]["threshold_candidates"]
    assert out[0][3]["fallback_queries"] == out[1][3]["fallback_queries"]
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 300)
    assert np.array_equal(out[0][0], orow) and np.array_equal(out[0][1], odist)


def test_half_prefilter_scan_extreme_table_values(psb):
    """Tables with tiny, huge and zero entries: the power-of-two scaling keeps fp16 sums finite and the lower bound valid."""
    rng = np.random.default_rng(0)
    for scale in (1e-4, 1.0, 3e3):
        ix = synth.make_index(60000, 32, 8, 8, seed=3)
        ix["codebook"] = (ix["codebook"] * scale).astype(np.float32)
        ix["codebook"][:, :8, :] = 0.0  # exact zeros among the codewords
        q = (synth.make_queries(ix, 16, seed=4) * scale).astype(np.float32)
        probes = np.tile(np.arange(8), (16, 1)).astype(np.int64)
        _, rows, dist, cnt, _ = run_stage_scan(psb, ix, q, probes, 200)
        orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 200)
        assert np.array_equal(rows, orow) and np.array_equal(dist, odist)


# ---------------------------------------------------------------------------------------------- overlapped pipeline
def test_overlapped_pipeline_equals_serial_pipeline(psb):
    """Batches of >= 2048 queries run as sub-batches whose rerank overlaps the next scan on a second stream; results
    must equal the serial pipeline's and the checker's."""
    torch = _torch()
    ix = synth.make_index(60000, 64, 64, 16, seed=61, zipf=True)
    q = synth.make_queries(ix, 2600, seed=62, weights=synth.zipf_weights(64))
    res = {}
    for serial in (False, True):
        with psb.Session(ix, n_rerank=120, serial_pipeline=serial) as s:
            res[serial] = s.search(q, 8, 10, batch_size=2600, want_coarse=True)
    for k in ("indices", "distances", "coarse"):
        assert np.array_equal(res[False][k], res[True][k])
    want = oracle.ivfpq_search(ix, q[:200], 8, 10, 120)
    assert np.array_equal(res[False]["indices"][:200], want["indices"])
    assert np.array_equal(res[False]["distances"][:200], want["distances"])
    # device-resident entry point
    with psb.Session(ix, n_rerank=120, max_batch=2600) as s:
        ids = torch.empty((2600, 10), dtype=torch.int64, device="cuda")
        dd = torch.empty((2600, 10), dtype=torch.float32, device="cuda")
        s.search_device(dev(q), 2600, 8, 10, ids, dd)
        s.sync()
        assert np.array_equal(ids.cpu().numpy(), res[True]["indices"])
        assert np.array_equal(dd.cpu().numpy(), res[True]["distances"])


@pytest.mark.parametrize("residual", [False, True])
def test_short_tail_batch_after_an_overlapped_batch(psb, residual):
    """batch_size 2600 with 2600 + 1500 queries: the full batch runs as four overlapped sub-batches of 650, the tail batch
    (below the overlap limit of 2048) runs in one piece of 1500 - larger than any sub-batch before it.  The workspaces
    must follow; results equal the serial pipeline's and the checker's."""
    ix = synth.make_index(60000, 64, 64, 16, seed=161, zipf=True, residual=residual)
    q = synth.make_queries(ix, 4100, seed=162, weights=synth.zipf_weights(64))
    res = {}
    for serial in (False, True):
        with psb.Session(ix, n_rerank=120, serial_pipeline=serial, residual=residual) as s:
            res[serial] = s.search(q, 8, 10, batch_size=2600)
    for k in ("indices", "distances"):
        assert np.array_equal(res[False][k], res[True][k])
    search = oracle.ivfrespq_search if residual else oracle.ivfpq_search
    for lo in (0, 2600, 3900):  # first batch, start of the tail batch, its end
        want = search(ix, q[lo:lo + 200], 8, 10, 120)
        assert np.array_equal(res[False]["indices"][lo:lo + 200], want["indices"])
        assert np.array_equal(res[False]["distances"][lo:lo + 200], want["distances"])


def test_knn_exact_short_last_tile(psb):
    """A base whose last tile would hold fewer than k rows: those rows must still be candidates."""
    torch = _torch()
    rng = np.random.default_rng(5)
    n, dim, k, nq = 4096 * 3 + 7, 16, 10, 65536   # 65,536 queries -> tiles of 4,096 base rows; the last 7 rows are a short tail
    base = rng.standard_normal((n, dim)).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    q[:3] = base[[n - 1, n - 3, 17]] + 1e-3   # two of the checked queries sit on rows of the short tail
    rows = torch.empty((nq, k), dtype=torch.int32, device="cuda")
    dist = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    psb.knn_exact(dev(q), nq, dev(base), n, dim, k, rows, dist)
    torch.cuda.synchronize()
    d2 = ((q[:3, None, :].astype(np.float64) - base[None, :, :]) ** 2).sum(-1)
    want = np.argsort(d2, axis=1, kind="stable")[:, :k]
    assert np.array_equal(rows[:3].cpu().numpy(), want)


def test_sharded_step_with_second_stream_equals_search(psb):
    """The sharded step on one rank, cut into sub-batches whose exchange half (rerank, id map) runs on a second stream
    through psb_session_set_stream while the next sub-batch scans: same results as the session's own search."""
    torch = _torch()
    from paraselect_b200.multi import SessionEngine, ShardedSearch
    ix = synth.make_index(60000, 64, 64, 16, seed=71, zipf=True)
    q = synth.make_queries(ix, 700, seed=72, weights=synth.zipf_weights(64))
    with psb.Session(ix, n_rerank=120) as s:
        want = s.search(q, 8, 10, batch_size=700)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with psb.Session(ix, n_rerank=120, max_batch=700, stream=stream.cuda_stream) as s:
            search = ShardedSearch(SessionEngine(s, torch), None, 1, 700, 64, 16, 256, 8, 10, 120, torch, rerank=True, parts=3)
            dq = dev(q)
            for parts in (1, 3, 3):
                ids, dd = search.step(dq, parts=parts)
                torch.cuda.synchronize()
                assert np.array_equal(ids.cpu().numpy(), want["indices"])
                assert np.array_equal(dd.cpu().numpy(), want["distances"])


def test_staged_transport_overlapped_by_a_host_worker_equals_mapped(psb):
    """Host-staged rerank transport: batches of >= 2048 queries hand each sub-batch's candidates to a host worker thread that
    gathers rows into pinned rings while the next sub-batch scans; results must equal the mapped transport's."""
    ix = synth.make_index(60000, 64, 64, 16, seed=81, zipf=True)
    q = synth.make_queries(ix, 2600, seed=82, weights=synth.zipf_weights(64))
    res = {}
    for name, kw in (("mapped", dict()), ("staged", dict(exact_mode=psb.EXACT_HOST_STAGED)),
                     ("staged_serial", dict(exact_mode=psb.EXACT_HOST_STAGED, serial_pipeline=True)),
                     ("hybrid", dict(exact_mode=psb.EXACT_HOST_HYBRID)),
                     ("hybrid_70", dict(exact_mode=psb.EXACT_HOST_HYBRID, zero_copy_pct=70)),
                     ("hybrid_serial", dict(exact_mode=psb.EXACT_HOST_HYBRID, serial_pipeline=True))):
        with psb.Session(ix, n_rerank=120, **kw) as s:
            res[name] = s.search(q, 8, 10, batch_size=2600)
            again = s.search(q, 8, 10, batch_size=2600)  # buffers are reused across batches
            assert np.array_equal(again["indices"], res[name]["indices"])
    for name in ("staged", "staged_serial", "hybrid", "hybrid_70", "hybrid_serial"):
        assert np.array_equal(res[name]["indices"], res["mapped"]["indices"])
        assert np.array_equal(res[name]["distances"], res["mapped"]["distances"])


@pytest.mark.skipif(not oracle.have_ref_kmeans_init(), reason="reference k-means initialisation not compiled here")
@pytest.mark.parametrize("n", [20000, 90000])   # n * 256 below and above the reference's k-means++ budget of 2e7
def test_pq_train_starts_from_the_references_initial_codewords(psb, n):
    """iters = 0 returns the initial codebook: subspace s = the rows the reference's initialisation picks with seed + s * 104729
    on the sub-vectors of that subspace (src/quantization/pq/pq_trainer.cu:62)."""
    torch = _torch()
    rng = np.random.default_rng(n)
    data = rng.standard_normal((n, 16)).astype(np.float32)
    cb = torch.empty((4, 256, 4), dtype=torch.float32, device="cuda")
    psb.pq_train(dev(data), n, 16, 4, 256, 0, 1234, cb)
    got = cb.cpu().numpy()
    for s in range(4):
        want = oracle.ref_kmeans_init(data[:, 4 * s:4 * s + 4], 256, 1234 + s * 104729, 0)
        assert np.array_equal(got[s], want), s


def test_residual_rows_feed_residual_training(psb):
    """psb_residual_rows (in place) = row - centroid[assign]; PQ trained on and encoding the residuals gives an index the
    residual search accepts (codes equal the checker's encoding of the same residuals)."""
    torch = _torch()
    centres, data, offsets = synth.mixture(12000, 32, 24, 0.3, seed=33)
    lists = np.repeat(np.arange(24), np.diff(offsets)).astype(np.int32)
    x = dev(data)
    psb.residual_rows(x, 12000, 32, dev(centres), dev(lists), x)
    want = (data - centres[lists]).astype(np.float32)
    assert np.array_equal(x.cpu().numpy(), want)
    cb = torch.empty((8, 256, 4), dtype=torch.float32, device="cuda")
    psb.pq_train(x, 12000, 32, 8, 256, 4, 5, cb)
    codes = torch.empty((12000, 8), dtype=torch.uint8, device="cuda")
    psb.pq_encode(x, 12000, 32, cb, 8, 256, codes)
    torch.cuda.synchronize()
    assert np.array_equal(codes.cpu().numpy(), oracle.pq_encode(want, cb.cpu().numpy()))


@pytest.mark.parametrize("M,dim,residual", [(8, 32, False), (48, 96, False), (20, 100, True)])
def test_u8_table_quantiser_matches_checker(psb, M, dim, residual):
    """psb_stage_quantize_lut_u8 against the checker's restatement of the reference's u8 table quantiser: codes, scales,
    lo_sum and inflation bit for bit."""
    torch = _torch()
    ix = synth.make_index(3000, dim, 8, M, seed=50 + M, residual=residual)
    q = synth.make_queries(ix, 7, seed=4)
    with psb.Session(ix, residual=residual) as s:
        lut = torch.empty((7, M, 256), dtype=torch.float32, device="cuda")
        s.stage_build_lut(dev(q), 7, lut)
        q8 = torch.empty((7, M, 256), dtype=torch.uint8, device="cuda")
        scales = torch.empty((7, M), dtype=torch.float32, device="cuda")
        lo = torch.empty((7,), dtype=torch.float32, device="cuda")
        infl = torch.empty((7,), dtype=torch.float32, device="cuda")
        s.stage_quantize_lut_u8(lut, 7, q8, scales, lo, infl)
        s.sync()
    luts = lut.cpu().numpy()
    for i in range(7):
        oq8, osc, olo, oinf = oracle.pq_lut_u8(luts[i], residual=residual)
        assert np.array_equal(q8[i].cpu().numpy(), oq8.reshape(M, 256))
        assert np.array_equal(scales[i].cpu().numpy(), osc)
        assert lo[i].item() == olo and infl[i].item() == oinf


def test_device_cached_exact_rows_equal_host_rows(psb):
    """PSB_EXACT_HOST_CACHED: the session's own device copy of the caller's host rows gives the same results."""
    ix = synth.make_index(30000, 64, 32, 16, seed=91, zipf=True)
    q = synth.make_queries(ix, 2300, seed=92, weights=synth.zipf_weights(32))
    with psb.Session(ix, n_rerank=100) as s:
        want = s.search(q, 8, 10, batch_size=2300)
    with psb.Session(ix, n_rerank=100, exact_mode=psb.EXACT_HOST_CACHED) as s:
        got = s.search(q, 8, 10, batch_size=2300)
    assert np.array_equal(got["indices"], want["indices"])
    assert np.array_equal(got["distances"], want["distances"])
