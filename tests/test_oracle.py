"""CPU tests: the plain-C restatement (oracle/psb_oracle.c) against the reference's golden outputs, the
reference's own known-answer tests, and - where oracle/_ref is built - the reference's code itself."""
import numpy as np
import pytest

import cases
import oracle
import synth

GOLDEN_IVFPQ = ["ivfpq_d32_m8", "ivfpq_d96_m48_zipf", "ivfpq_d100_m20"]


@pytest.mark.parametrize("name", GOLDEN_IVFPQ)
def test_restatement_matches_reference_golden(name):
    g = cases.load_golden(name)
    nprobe, topk, n_rerank = (int(x) for x in g["params"])
    ix = cases.golden_index(g)
    o = oracle.ivfpq_search(ix, g["queries"], nprobe, topk, n_rerank)
    assert np.array_equal(o["coarse"], g["ref_probes"])
    assert np.array_equal(o["indices"], g["ref_indices"])
    assert np.array_equal(o["distances"], g["ref_distances"])  # bit-exact
    assert o["scanned"] == int(g["ref_scanned"])
    luts = oracle.pq_lut(g["queries"], g["codebook"])

    def adc(q, row):
        return _adc(luts[q], g["codes"][row])
    assert cases.stage1_sets_match(o["stage1"], g["ref_stage1"], adc)
    nr = oracle.ivfpq_search(dict(ix, vectors=None), g["queries"], nprobe, topk, 0)
    assert np.array_equal(nr["distances"], g["ref_norerank_distances"])  # ADC distances, bit-exact
    same = nr["indices"] == g["ref_norerank_indices"]
    # ids may differ only inside groups of equal ADC distance
    assert np.array_equal(np.sort(nr["distances"][~same]), np.sort(g["ref_norerank_distances"][~same]))


def _adc(lut, code):
    d = np.float32(0)
    for m in range(lut.shape[0]):
        d = np.float32(d + lut[m, code[m]])
    return float(d)


@pytest.mark.parametrize("name", ["rerank_d96", "rerank_d100"])
def test_rerank_matches_reference_golden(name):
    g = cases.load_golden(name)
    width, topk = (int(x) for x in g["params"])
    ids, dist = oracle.rerank(g["base"], g["queries"], g["candidates"], topk, candidate_count=width, counts=g["counts"])
    assert np.array_equal(ids, g["ref_ids"])
    assert np.array_equal(dist, g["ref_dist"])


@pytest.mark.parametrize("dtype", [np.uint8, np.float32])
@pytest.mark.parametrize("dim", [100, 128])
@pytest.mark.parametrize("width", [128, 512, 2048])
def test_host_rerank_known_answer(dtype, dim, width):
    c = cases.host_rerank_case(dtype, dim, width)
    ids, dist = oracle.rerank(c["base"], c["queries"], c["cand"], c["topk"], candidate_count=width, counts=c["counts"])
    assert np.array_equal(ids, c["exp_ids"])
    assert np.array_equal(dist, c["exp_d"])  # integer-valued data: every summation order is exact
    with pytest.raises(ValueError):
        oracle.rerank(c["base"], c["queries"], c["cand"], c["topk"], candidate_count=width,
                      counts=np.array([0, width + 1, 0, 0], np.int32))


def test_rerank_adapter_known_answer():
    c = cases.adapter_case()
    ids, dist = oracle.rerank(c["base"], c["queries"], c["cand"], c["topk"], counts=c["counts"])
    assert np.array_equal(ids, c["exp_ids"])
    assert np.array_equal(dist, c["exp_d"])


@pytest.mark.parametrize("m,dim,rerank,empty", [(16, 96, 512, False), (16, 96, 512, True), (20, 100, 2048, False),
                                                 (16, 128, 512, False)])
def test_plain_pq_pipeline_equals_exhaustive(m, dim, rerank, empty):
    c = cases.plain_pq_pipeline_case(m, dim, rerank, empty)
    o = oracle.ivfpq_search(c["index"], c["queries"], c["nprobe"], c["topk"], c["n_rerank"])
    assert np.array_equal(o["indices"], c["exp_ids"])
    assert np.array_equal(o["distances"], c["exp_d"])


GOLDEN_RESIDUAL = ["ivfrespq_d64_m16", "ivfrespq_d32_m8", "ivfrespq_d96_m48_zipf"]


@pytest.mark.parametrize("name", GOLDEN_RESIDUAL)
def test_residual_restatement_matches_reference_golden(name):
    """Residual ADC mode against outputs of the reference's cpu_fine_kernel_pq_resid_cpu_lut_timed; the m16 fixture asks
    for topk = candidate width, so its output is the whole stage-1 set."""
    g = cases.load_golden(name)
    nprobe, topk, n_rerank = (int(x) for x in g["params"])
    o = oracle.ivfrespq_search(cases.golden_index(g), g["queries"], nprobe, topk, n_rerank)
    assert np.array_equal(o["coarse"], g["ref_probes"])
    assert np.array_equal(o["indices"], g["ref_indices"])
    assert np.array_equal(o["distances"], g["ref_distances"])  # bit-exact
    assert o["scanned"] == int(g["ref_scanned"])
    assert o["stage1"].shape[1] == max(n_rerank, topk, 512)


@pytest.mark.parametrize("m,dim,rerank", [(16, 96, 512), (8, 32, 512), (20, 100, 2048)])
def test_residual_pq_pipeline_equals_exhaustive(m, dim, rerank):
    c = cases.residual_pq_pipeline_case(m, dim, rerank)
    o = oracle.ivfrespq_search(c["index"], c["queries"], c["nprobe"], c["topk"], c["n_rerank"])
    assert np.array_equal(o["indices"], c["exp_ids"])
    assert np.array_equal(o["distances"], c["exp_d"])


def test_residual_tables_and_tree_order():
    """Tables are built on q - centroid; M = 16 / 8 with K = 256 sum as a balanced pairwise tree, other shapes in order."""
    for M, dim in ((16, 64), (8, 32), (12, 48)):
        ix = synth.make_index(3000, dim, 12, M, seed=40 + M, residual=True)
        q = synth.make_queries(ix, 9, seed=3)
        probes, _ = oracle.coarse(q, ix["centroids"], 3)
        rows, dist, cnt, scanned, luts = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"],
                                                                 ix["codebook"], 20, want_luts=True)
        for qi in range(q.shape[0]):
            for p in range(3):
                want = oracle.pq_lut((q[qi] - ix["centroids"][probes[qi, p]])[None, :], ix["codebook"])[0]
                assert np.array_equal(luts[qi, p].reshape(want.shape), want)
        lists = np.repeat(np.arange(12), np.diff(ix["offsets"]))
        for qi in range(q.shape[0]):
            for i in range(int(cnt[qi])):
                row = rows[qi, i]
                p = int(np.nonzero(probes[qi] == lists[row])[0][0])
                t = luts[qi, p].reshape(M, 256)[np.arange(M), ix["codes"][row]].astype(np.float32)
                if M in (8, 16):
                    while t.size > 1:
                        t = (t[0::2] + t[1::2]).astype(np.float32)
                    want = t[0]
                else:
                    want = np.float32(0)
                    for v in t:
                        want = np.float32(want + v)
                assert dist[qi, i] == want


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref (reference compiled in place) not built")
@pytest.mark.parametrize("seed,dim,M,nlist,zipf,topk,nr", [(41, 64, 16, 24, True, 10, 100), (42, 32, 8, 16, False, 512, 512),
                                                           (43, 96, 48, 16, True, 100, 1000), (44, 48, 12, 8, False, 600, 0)])
def test_residual_restatement_vs_reference_live(seed, dim, M, nlist, zipf, topk, nr):
    ix = synth.make_index(4000, dim, nlist, M, seed=seed, zipf=zipf, residual=True)
    q = synth.make_queries(ix, 30, seed=seed + 1)
    o = oracle.ivfrespq_search(ix, q, 5, topk, nr)
    r = oracle.ref_ivfrespq_search(ix, q, o["coarse"], topk, nr, threads=3)
    assert np.array_equal(r["indices"], o["indices"])
    assert np.array_equal(r["distances"], o["distances"])
    assert r["scanned"] == o["scanned"]


def test_u8_lut_identities():
    rng = np.random.default_rng(5)
    for M, dsub in ((16, 8), (20, 5)):
        cb = rng.standard_normal((M, 256, dsub)).astype(np.float32)
        q = rng.standard_normal((1, M * dsub)).astype(np.float32)
        lut = oracle.pq_lut(q, cb)[0]
        ref = ((q.reshape(M, 1, dsub) - cb) ** 2).sum(-1)
        assert np.allclose(lut, ref, rtol=1e-5, atol=1e-5)
        q8, scales, lo_sum, infl = oracle.pq_lut_u8(lut)
        lo = lut.min(axis=1)
        assert np.all(np.abs(lo[:, None] + scales[:, None] * q8 - lut) <= 0.5001 * scales[:, None])
        assert np.isclose(lo_sum, lo.sum(), rtol=1e-6)
        assert np.isclose(infl, 0.5 * scales.sum(), rtol=1e-6)
        _, _, _, infl_r = oracle.pq_lut_u8(lut, residual=True)
        assert np.isclose(infl_r, scales.sum(), rtol=1e-6)


def test_ivfflat_config1_shape_small():
    """IVF-Flat CPU configuration (cut down): exact search over probed lists equals brute force when nprobe = nlist."""
    centres, data, offsets = synth.mixture(3000, 32, 16, 0.3, seed=0)
    rng = np.random.default_rng(1)
    q = (centres[rng.integers(0, 16, 20)] + 0.3 * rng.standard_normal((20, 32))).astype(np.float32)
    ids, dist = oracle.ivfflat_search(centres, offsets, None, data, q, 16, 10)
    d2 = ((q[:, None, :].astype(np.float64) - data[None].astype(np.float64)) ** 2).sum(-1)
    assert np.array_equal(ids, np.argsort(d2, axis=1, kind="stable")[:, :10])
    assert np.allclose(dist, np.sort(d2, axis=1)[:, :10], rtol=1e-5)


def test_edge_cases():
    ix = synth.make_index(400, 16, 4, 4, seed=2, empty_lists=(1,))
    q = synth.make_queries(ix, 3)
    # fewer rows than topk in the probed lists: padding -1 / FLT_MAX
    small = dict(ix)
    o = oracle.ivfpq_search(small, q, 4, 10, 500)  # n_rerank > n_vectors -> stage1_k = n_vectors
    assert o["stage1"].shape[1] == 400
    rows, dist, cnt, _ = oracle.pq_scan(q, np.array([[1, -1, 99]] * 3, np.int64), ix["offsets"], ix["codes"],
                                        ix["codebook"], 5)
    assert np.all(rows == -1) and np.all(cnt == 0) and np.all(dist == cases.FLT_MAX)
    with pytest.raises(ValueError):
        oracle.coarse(q, ix["centroids"], 5)  # nprobe > nlist


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref (reference compiled in place) not built")
@pytest.mark.parametrize("seed,dim,M,nlist,zipf", [(31, 96, 48, 24, True), (32, 128, 32, 16, False), (33, 100, 20, 8, False)])
def test_restatement_vs_reference_live(seed, dim, M, nlist, zipf):
    ix = synth.make_index(3000, dim, nlist, M, seed=seed, zipf=zipf)
    q = synth.make_queries(ix, 30, seed=seed + 1)
    o = oracle.ivfpq_search(ix, q, 5, 10, 50)
    pr, pd = oracle.ref_coarse(q, ix["centroids"], 5)
    assert np.array_equal(pr, o["coarse"])
    r = oracle.ref_ivfpq_search(ix, q, pr, 10, 50, fine_threads=2, rerank_threads=2)
    assert np.array_equal(r["indices"], o["indices"])
    if oracle.ref_info()["isa"] == "avx512":
        assert np.array_equal(r["distances"], o["distances"])
    else:
        assert np.allclose(r["distances"], o["distances"], rtol=1e-5)
    assert r["scanned"] == o["scanned"]


# ---------------------------------------------------------------------------------------------- IVF-Flat, k-means, PQ training
# The restatement against more of the reference's own CPU code (oracle/ref_train_harness.cu): live where that library was built.
needs_ref_train = pytest.mark.skipif(not oracle.have_ref_train(), reason="oracle/_ref/libpsb_ref_train.so is not built here")


@needs_ref_train
def test_ivfflat_and_coarse_match_the_reference_cpu_search():
    # cpu_ivf_search (src/cpu/search/cpu_search.h:226-332); its partial_sort / nth_element leave the order of equal distances
    # open, so ids are compared where distances are distinct (all of them, for real-valued data) and as sets inside ties
    ix = synth.make_index(20000, 128, 64, 8, seed=9)
    q = synth.make_queries(ix, 50, seed=10)
    want_i, want_d, want_ci, want_cd = oracle.ref_cpu_ivf_search(ix["centroids"], ix["offsets"], ix["reordered_ids"], ix["vectors"], q, 8, 10)
    got_i, got_d = oracle.ivfflat_search(ix["centroids"], ix["offsets"], ix["reordered_ids"], ix["vectors"], q, 8, 10)
    assert np.array_equal(got_d, want_d)  # bit-exact distances
    assert np.array_equal(got_i, want_i)
    ci, cd = oracle.coarse(q, ix["centroids"], 8)
    assert np.array_equal(cd, want_cd) and np.array_equal(ci, want_ci)
    # integer grid: many exactly equal distances - the multiset of distances and, per distance, the id sets must agree
    rng = np.random.default_rng(1)
    base = rng.integers(-2, 3, (3000, 16)).astype(np.float32)
    cen = rng.integers(-2, 3, (16, 16)).astype(np.float32)
    cen[1] = cen[0] + 1  # keep centroids distinct enough that coarse ties stay rare
    off = np.linspace(0, 3000, 17).astype(np.int64)
    qq = rng.integers(-2, 3, (20, 16)).astype(np.float32)
    wi, wd, _, _ = oracle.ref_cpu_ivf_search(cen, off, None, base, qq, 16, 25)
    gi, gd = oracle.ivfflat_search(cen, off, None, base, qq, 16, 25)
    assert np.array_equal(gd, wd)
    for a, b, d in zip(gi, wi, gd):
        inner = d < d[-1]  # below the boundary distance the sets are fully determined
        assert set(a[inner].tolist()) == set(b[inner].tolist())


@needs_ref_train
def test_kmeans_assignment_and_update_match_the_reference_cpu_kmeans():
    # cpu_kmeans_lloyd (src/cpu/clustering/cpu_kmeans.h:27-143): strict <, lowest index wins; empty clusters keep their centroid
    _, data, _ = synth.mixture(6000, 24, 30, 0.3, seed=21)
    init = data[:40].copy()
    init[7] = 1e3  # a centroid no row is assigned to
    cen1, assign0, obj0 = oracle.ref_kmeans_lloyd(data, init, 1)
    a, d = oracle.kmeans_assign(data, init)
    assert np.array_equal(a, assign0)                            # assignment: bit-exact
    assert abs(float(d.astype(np.float64).sum()) - obj0) <= 1e-5 * obj0
    mine, _, _ = oracle.kmeans_lloyd(data, init, 1)
    assert np.array_equal(mine[7], init[7])                      # the empty cluster kept its centroid on both sides
    assert np.array_equal(cen1[7], init[7])
    # the reference accumulates the sums in fp32 per thread; the restatement's means agree to fp32 accumulation error
    assert np.allclose(mine, cen1, rtol=2e-5, atol=2e-6)
    cen5, assign4, obj4 = oracle.ref_kmeans_lloyd(data, init, 5)
    mine5, _, objs = oracle.kmeans_lloyd(data, init, 5)
    assert np.allclose(mine5, cen5, rtol=1e-3, atol=1e-4) and abs(objs[4] - obj4) <= 1e-4 * obj4


@needs_ref_train
def test_pq_encode_and_training_match_the_reference_cpu_quantiser():
    # PQQuantizerCPU (src/quantization/pq/pq_quantizer_cpu.cpp:26-68) on top of pq_kmeans_subspace (pq_kmeans.cpp:12-74)
    _, data, _ = synth.mixture(3000, 32, 20, 0.3, seed=31)
    cb, codes = oracle.ref_pq_train_encode(data, 8, 64)
    assert np.array_equal(oracle.pq_encode(data, cb), codes)     # encoding: nearest codeword, ties to the lowest code - bit-exact
    # training: pq_kmeans_subspace draws its initial codewords with std::mt19937(42 + m) (with replacement) and runs Lloyd
    # iterations accumulating in fp32 row by row.  One iteration from the same initial rows gives the same codewords as the
    # restatement for every codeword that got rows; a codeword WITHOUT rows is zeroed by this CPU trainer, while the
    # reference's GPU trainer (src/clustering/kmeans/kmeans_utils.cu:267-284) - the one the library follows - keeps it.
    for m in (0, 5):
        sub = np.ascontiguousarray(data[:, m * 4:(m + 1) * 4])
        rows = oracle.ref_pq_init_rows(sub.shape[0], 64, 42 + m)
        init = sub[rows]
        ref1 = oracle.ref_pq_kmeans_subspace(sub, 64, 1, 42 + m)
        mine, assign, _ = oracle.kmeans_lloyd(sub, init, 1)
        a0, _ = oracle.kmeans_assign(sub, init)
        used = np.bincount(a0, minlength=64) > 0
        assert np.allclose(mine[used], ref1[used], rtol=2e-5, atol=2e-6)
        assert np.all(ref1[~used] == 0) and np.array_equal(mine[~used], init[~used])
        assert np.array_equal(oracle.ref_pq_kmeans_subspace(sub, 64, 25, 42 + m), cb[m])  # train() == 25 iterations of it


def test_opq_pipeline_restatement_reduces_to_the_plain_one():
    """Identity rotation: the composed OPQ pipeline is the plain pipeline; a true rotation changes only the PQ side."""
    ix = synth.make_index(6000, 32, 12, 8, seed=91)
    q = synth.make_queries(ix, 40, seed=92)
    eye = np.eye(32, dtype=np.float32)
    a = oracle.ivfpq_search(ix, q, 4, 5, 50)
    b = oracle.ivfpq_search_opq(ix, q, 4, 5, 50, eye)
    assert np.array_equal(a["indices"], b["indices"]) and np.array_equal(a["distances"], b["distances"])
    a = oracle.ivfpq_search(dict(ix, vectors=None), q, 4, 5, 0)
    b = oracle.ivfpq_search_opq(dict(ix, vectors=None), q, 4, 5, 0, eye)
    assert np.array_equal(a["indices"], b["indices"]) and np.array_equal(a["distances"], b["distances"])
    # orientation: matrix is [out][in]
    rot = np.zeros((32, 32), np.float32); rot[0, 1] = 2.0
    y = oracle.rotate_rows(q, rot)
    assert np.array_equal(y[:, 0], 2.0 * q[:, 1]) and not y[:, 1:].any()


@pytest.mark.skipif(not oracle.have_ref_kmeans_init(), reason="reference k-means initialisation not compiled here")
@pytest.mark.parametrize("n,dim,k,seed,policy", [(500, 8, 16, 123, 0), (3000, 4, 256, 42, 0), (3000, 4, 256, 42 + 104729, 0),
                                                  (100000, 2, 256, 7, 0), (100000, 2, 256, 7, 2), (900, 16, 64, 5, 1),
                                                  (40, 6, 64, 9, 0), (40, 6, 64, 9, 1)])
def test_kmeans_init_equals_the_reference(n, dim, k, seed, policy):
    """psb_kmeans_init (a host function of the library, no GPU) against the reference's init_centroids_by_sampling: the same
    rows, draw for draw - k-means++ below n * k = 2e7, partial Fisher-Yates above, forced either way, and k > n."""
    from paraselect_b200 import api
    rng = np.random.default_rng(n + k)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    x[::7] = x[0]   # duplicate rows: zero distances in the k-means++ weights
    want = oracle.ref_kmeans_init(x, k, seed, policy)
    got, rows = api.kmeans_init(x, k, seed, policy)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(x[rows], got)
