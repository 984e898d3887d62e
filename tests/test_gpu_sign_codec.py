"""TurboQuant 1-bit codec on the GPU against the CPU checker, bit for bit: rotation, sign words and scales of database rows
(at once and in chunks: tests/unit/turboquant/test_turboquant_1bit_encode.cu:78-145 of the reference), query states, and the
candidate search in both score modes (exact candidate_count smallest (score, row) keys in order, as
tests/unit/turboquant/test_turboquant_1bit_scan.cu:23-80 asserts against a sorted host list).  The checker takes the
rotation's scale from the device (rsqrtf is a device function)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

FLT_MAX = np.finfo(np.float32).max


def dev(a):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def host_u32(t):
    return t.cpu().numpy().view(np.uint32)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("padded", [32, 64, 128, 256])
def test_rotation_scale(psb, padded):
    s = psb.sign_rotation_scale(padded)
    assert abs(s * s * padded - 1.0) < 1e-6


@pytest.mark.parametrize("n,dim,padded", [(3, 70, 128), (1, 8, 32), (257, 64, 64), (1000, 128, 128), (33, 200, 256), (40, 256, 256), (9, 1, 32)])
def test_rotate_bit_exact(psb, n, dim, padded):
    import torch
    rng = np.random.default_rng(n * 7 + dim)
    x = (rng.standard_normal((n, dim)) * 3).astype(np.float32)
    x[0, : dim // 2] = 0.0
    rot = torch.empty((n, padded), dtype=torch.float32, device="cuda")
    codes = torch.empty((n, padded // 32), dtype=torch.int32, device="cuda")
    norms = torch.empty(n, dtype=torch.float32, device="cuda")
    nsq = torch.empty(n, dtype=torch.float32, device="cuda")
    psb.sign_rotate(dev(x), n, dim, padded, rot, codes, norms, nsq, seed=17)
    torch.cuda.synchronize()
    w_rot, w_codes, w_norms, w_nsq = oracle.sign_rotate(x, padded, seed=17, scale=psb.sign_rotation_scale(padded))
    assert np.array_equal(host_u32(rot), bits(w_rot))
    assert np.array_equal(host_u32(codes), w_codes)
    assert np.array_equal(host_u32(norms), bits(w_norms)) and np.array_equal(host_u32(nsq), bits(w_nsq))
    # outputs are optional one by one
    only = torch.empty((n, padded // 32), dtype=torch.int32, device="cuda")
    psb.sign_rotate(dev(x), n, dim, padded, d_codes=only, seed=17)
    assert np.array_equal(host_u32(only), w_codes)
    other = torch.empty_like(only)
    psb.sign_rotate(dev(x), n, dim, padded, d_codes=other, seed=18)
    assert n < 3 or not np.array_equal(host_u32(other), w_codes)


def test_rotate_refuses_bad_shapes(psb):
    import torch
    x = torch.zeros((2, 40), device="cuda")
    out = torch.empty((2, 64), device="cuda")
    with pytest.raises(psb.InvalidArgument):
        psb.sign_rotate(x, 2, 40, 32, out)        # dim above padded_dim
    with pytest.raises(psb.InvalidArgument):
        psb.sign_rotate(x, 2, 40, 48, out)        # not a supported power of two
    with pytest.raises(psb.InvalidArgument):
        psb.sign_rotate(x, 2, 40, 64)             # no output
    assert psb.sign_padded_dim(300) == -1 and psb.sign_padded_dim(129) == 256


def make_lists(rng, nlist, lo, hi, empties=()):
    sizes = rng.integers(lo, hi, nlist)
    for e in empties:
        sizes[e] = 0
    return np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)


@pytest.mark.parametrize("dim,padded,u8", [(8, 32, True), (128, 128, True), (96, 128, False), (200, 256, False)])
def test_database_encoding_bit_exact_at_once_and_in_chunks(psb, dim, padded, u8):
    import torch
    rng = np.random.default_rng(dim + padded)
    nlist = 9
    off = make_lists(rng, nlist, 1, 400, empties=(0, 4, 8))
    n = int(off[-1])
    cen = rng.uniform(0, 120, (nlist, dim)).astype(np.float32)
    rows = rng.integers(0, 256, (n, dim)).astype(np.uint8) if u8 else rng.uniform(0, 200, (n, dim)).astype(np.float32)
    scale = psb.sign_rotation_scale(padded)
    w_codes, w_scales = oracle.sign_encode_database(rows, cen, off, padded, scale=scale)
    d_cen, d_off = dev(cen), dev(off)
    codes = torch.zeros((n, padded // 32), dtype=torch.int32, device="cuda")
    scales = torch.zeros(n, dtype=torch.float32, device="cuda")
    psb.sign_encode_database(dev(rows), rows.dtype.itemsize, n, d_cen, d_off, nlist, dim, padded, codes, scales)
    torch.cuda.synchronize()
    assert np.array_equal(host_u32(codes), w_codes) and np.array_equal(host_u32(scales), bits(w_scales))
    c2 = torch.zeros_like(codes); s2 = torch.zeros_like(scales)
    cuts = [0, 3, 4, n // 2, n]
    for a, b in zip(cuts[:-1], cuts[1:]):
        if b > a:
            psb.sign_encode_database(dev(rows[a:b]), rows.dtype.itemsize, b - a, d_cen, d_off, nlist, dim, padded, c2, s2, row_offset=a)
    torch.cuda.synchronize()
    assert torch.equal(c2, codes) and torch.equal(s2, scales)


def test_query_states_bit_exact(psb):
    import torch
    rng = np.random.default_rng(11)
    nlist, dim, padded, nq, nprobe = 20, 100, 128, 37, 5
    cen = rng.standard_normal((nlist, dim)).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    probes = rng.integers(0, nlist, (nq, nprobe)).astype(np.int32)
    probes[3, 1] = -1; probes[5, 0] = nlist
    st = torch.empty((nq * nprobe, padded), dtype=torch.float32, device="cuda")
    nsq = torch.empty(nq * nprobe, dtype=torch.float32, device="cuda")
    sc = torch.empty((nq * nprobe, padded // 32), dtype=torch.int32, device="cuda")
    nm = torch.empty(nq * nprobe, dtype=torch.float32, device="cuda")
    psb.sign_encode_queries(dev(q), dev(cen), dev(probes), nq, nprobe, nlist, dim, padded, st, nsq, sc, nm)
    torch.cuda.synchronize()
    w = oracle.sign_encode_queries(q, cen, probes, padded, scale=psb.sign_rotation_scale(padded))
    assert np.array_equal(host_u32(st), bits(w[0])) and np.array_equal(host_u32(nsq), bits(w[1]))
    assert np.array_equal(host_u32(sc), w[2]) and np.array_equal(host_u32(nm), bits(w[3]))


def make_sign_index(seed, nlist, dim, padded, lo, hi, empties=(), u8=False):
    rng = np.random.default_rng(seed)
    off = make_lists(rng, nlist, lo, hi, empties)
    n = int(off[-1])
    cen = (rng.standard_normal((nlist, dim)) * 4 + 60).astype(np.float32)
    lists = np.repeat(np.arange(nlist), np.diff(off))
    rows = cen[lists] + rng.standard_normal((n, dim)).astype(np.float32) * np.float32(6.0)
    rows = np.clip(np.rint(rows), 0, 255).astype(np.uint8) if u8 else rows.astype(np.float32)
    return dict(rows=rows, centroids=cen, offsets=off, nlist=nlist, dim=dim, padded=padded, n=n, rng=rng)


def run_candidates(psb, ix, q, probes, k, mode, scale):
    import torch
    nq, nprobe = probes.shape
    padded = ix["padded"]
    codes, scales = oracle.sign_encode_database(ix["rows"], ix["centroids"], ix["offsets"], padded, scale=scale)
    states, nsq, sc, norms = oracle.sign_encode_queries(q, ix["centroids"], probes, padded, scale=scale)
    rows = torch.empty((nq, k), dtype=torch.int32, device="cuda")
    dist = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    if mode == 0:
        psb.sign_search_candidates(0, dev(codes), dev(scales), dev(ix["offsets"]), ix["nlist"], dev(probes), nq, nprobe, padded, k,
                                   rows, dist, d_states=dev(states), d_norm_sq=dev(nsq))
        want = oracle.sign_candidates(0, codes, scales, ix["offsets"], probes, k, states=states, norm_sq=nsq)
    else:
        psb.sign_search_candidates(1, dev(codes), dev(scales), dev(ix["offsets"]), ix["nlist"], dev(probes), nq, nprobe, padded, k,
                                   rows, dist, d_state_codes=dev(sc), d_norms=dev(norms))
        want = oracle.sign_candidates(1, codes, scales, ix["offsets"], probes, k, state_codes=sc, norms=norms)
    torch.cuda.synchronize()
    return rows.cpu().numpy(), dist.cpu().numpy(), want


# nq below twice the SM count splits each query's probes over several CTAs and merges; above it one CTA does a query.
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("nq,nprobe,k,dim,padded", [(5, 6, 10, 70, 128), (3, 8, 512, 128, 128), (320, 4, 64, 128, 128),
                                                   (7, 3, 2048, 64, 64), (2, 5, 100, 200, 256), (400, 2, 7, 20, 32),
                                                   (2, 24, 8192, 128, 128)])
def test_candidates_equal_checker(psb, mode, nq, nprobe, k, dim, padded):
    ix = make_sign_index(nq * 31 + k, 24, dim, padded, 1, 900, empties=(2, 23))
    rng = ix["rng"]
    q = (rng.standard_normal((nq, dim)) * 5 + 60).astype(np.float32)
    probes = np.stack([rng.permutation(ix["nlist"])[:nprobe] for _ in range(nq)]).astype(np.int32)
    if nprobe > 1:
        probes[0, 0] = -1
        probes[nq - 1, 1] = 2   # an empty list
    rows, dist, (w_rows, w_dist) = run_candidates(psb, ix, q, probes, k, mode, psb.sign_rotation_scale(padded))
    assert np.array_equal(rows, w_rows)
    assert np.array_equal(bits(dist), bits(w_dist))
    assert np.all(rows[0][rows[0] >= 0] < ix["n"])


def test_candidates_pad_when_few_rows_and_break_ties_by_row(psb):
    import torch
    padded, n = 128, 3000
    rng = np.random.default_rng(3)
    codes = np.tile(rng.integers(0, 2 ** 32, (1, 4), dtype=np.uint64).astype(np.uint32), (n, 1))   # every row the same code
    scales = np.full(n, 0.75, np.float32)
    off = np.array([0, 5, 5, n], np.int64)
    states = rng.standard_normal((4, padded)).astype(np.float32)   # 2 queries x 2 probes
    nsq = (states ** 2).sum(1).astype(np.float32)
    probes = np.array([[0, 1], [2, 0]], np.int32)
    k = 600
    rows = torch.empty((2, k), dtype=torch.int32, device="cuda")
    dist = torch.empty((2, k), dtype=torch.float32, device="cuda")
    psb.sign_search_candidates(0, dev(codes), dev(scales), dev(off), 3, dev(probes), 2, 2, padded, k, rows, dist,
                               d_states=dev(states), d_norm_sq=dev(nsq))
    torch.cuda.synchronize()
    w_rows, w_dist = oracle.sign_candidates(0, codes, scales, off, probes, k, states=states, norm_sq=nsq)
    got = rows.cpu().numpy()
    assert np.array_equal(got, w_rows) and np.array_equal(bits(dist.cpu().numpy()), bits(w_dist))
    assert got[0, :5].tolist() == [0, 1, 2, 3, 4] and np.all(got[0, 5:] == -1)
    assert np.all(dist.cpu().numpy()[0, 5:] == FLT_MAX)
    # within one (query, probe) all scores are equal: rows come in ascending order
    one_probe = got[1][(got[1] >= 5)]
    assert np.all(np.diff(one_probe) > 0)


def test_candidates_refuse_bad_requests(psb):
    import torch
    z = torch.zeros(64, dtype=torch.int32, device="cuda")
    f = torch.zeros(64, dtype=torch.float32, device="cuda")
    off = dev(np.array([0, 1], np.int64))
    with pytest.raises(psb.InvalidArgument):
        psb.sign_search_candidates(0, z, f, off, 1, z, 1, 1, 32, psb.SIGN_MAX_CANDIDATES + 1, z, f, d_states=f, d_norm_sq=f)
    with pytest.raises(psb.InvalidArgument):
        psb.sign_search_candidates(0, z, f, off, 1, z, 1, 1, 32, 4, z, f, d_state_codes=z, d_norms=f)   # float states missing
    with pytest.raises(psb.InvalidArgument):
        psb.sign_search_candidates(2, z, f, off, 1, z, 1, 1, 32, 4, z, f, d_states=f, d_norm_sq=f)
    with pytest.raises(psb.InvalidArgument):
        psb.sign_search_candidates(0, z, f, off, 1, z, 1, 1, 48, 4, z, f, d_states=f, d_norm_sq=f)


@pytest.mark.parametrize("u8", [True, False])
def test_index_object_end_to_end(psb, u8):
    ix = make_sign_index(77, 40, 128, 128, 50, 700, empties=(7,), u8=u8)
    rng = ix["rng"]
    nq, nprobe, k = 64, 8, 512
    q = (rng.standard_normal((nq, 128)) * 5 + 60).astype(np.float32)
    # probes: the nearest centroids, int64 ids as the reference's callers pass them, one of them out of range
    d2 = ((q[:, None, :] - ix["centroids"][None]) ** 2).sum(2)
    probes = np.argsort(d2, axis=1)[:, :nprobe].astype(np.int64)
    probes[4, 7] = 1 << 40
    index = psb.SignIndex().build_u8(ix["rows"], ix["centroids"], ix["offsets"])
    chunked = psb.SignIndex()
    chunked.ENCODE_CHUNK_ROWS = 1000
    chunked.build_u8(ix["rows"], ix["centroids"], ix["offsets"])
    assert index.bytes_per_vector == 20
    scale = psb.sign_rotation_scale(128)
    codes, scales = oracle.sign_encode_database(ix["rows"], ix["centroids"], ix["offsets"], 128, scale=scale)
    assert np.array_equal(host_u32(index.codes), codes) and np.array_equal(host_u32(chunked.codes), codes)
    assert np.array_equal(host_u32(index.scales), bits(scales)) and np.array_equal(host_u32(chunked.scales), bits(scales))
    p32 = np.where((probes < 0) | (probes >= 40), -1, probes).astype(np.int32)
    states, nsq, sc, norms = oracle.sign_encode_queries(q, ix["centroids"], p32, 128, scale=scale)
    got, dist = index.search_candidates(q, probes, k, want_distances=True)
    w_rows, w_dist = oracle.sign_candidates(0, codes, scales, ix["offsets"], p32, k, states=states, norm_sq=nsq)
    assert np.array_equal(got, w_rows) and np.array_equal(bits(dist), bits(w_dist))
    got_b = index.search_candidates(q, probes, k, score_mode=psb.SIGN_CODED_STATES)
    w_b, _ = oracle.sign_candidates(1, codes, scales, ix["offsets"], p32, k, state_codes=sc, norms=norms)
    assert np.array_equal(got_b, w_b)
    cached = psb.SignIndex().build_cached_u32(codes, scales, ix["centroids"], ix["offsets"])
    assert np.array_equal(cached.search_candidates(q, probes, k), w_rows)
    # the sign codes carry the neighbourhood: the exact nearest scanned row is among the candidates for most queries
    rows_f = ix["rows"].astype(np.float32)
    hits = 0
    for qi in range(nq):
        scanned = np.concatenate([np.arange(ix["offsets"][l], ix["offsets"][l + 1]) for l in p32[qi] if l >= 0])
        best = scanned[np.argmin(((rows_f[scanned] - q[qi]) ** 2).sum(1))]
        hits += int(best in got[qi])
    assert hits >= nq * 0.8
    with pytest.raises(psb.InvalidArgument):
        index.search_candidates(q[:, :64], probes, k)


def test_full_size_lists_properties(psb):
    """2 M rows in 256 lists, 512 candidates from 32 probes: too many scores for the checker on every query, so the first
    queries are compared with it and all of them through what holds at any size: ascending keys, rows from probed lists only,
    no row twice, and the same rows whether one CTA or several take a query."""
    import torch
    rng = np.random.default_rng(2024)
    nlist, padded, n = 256, 128, 2_000_000
    sizes = rng.multinomial(n, rng.dirichlet(np.full(nlist, 2.0)))
    off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    codes = rng.integers(0, 2 ** 32, (n, 4), dtype=np.uint64).astype(np.uint32)
    scales = rng.uniform(0.2, 1.5, n).astype(np.float32)
    nq, nprobe, k = 600, 32, 512
    states = rng.standard_normal((nq * nprobe, padded)).astype(np.float32)
    nsq = (states.astype(np.float64) ** 2).sum(1).astype(np.float32)
    probes = np.stack([rng.permutation(nlist)[:nprobe] for _ in range(nq)]).astype(np.int32)
    d_codes, d_scales, d_off, d_states, d_nsq = dev(codes), dev(scales), dev(off), dev(states), dev(nsq)
    rows = torch.empty((nq, k), dtype=torch.int32, device="cuda")
    dist = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    psb.sign_search_candidates(0, d_codes, d_scales, d_off, nlist, dev(probes), nq, nprobe, padded, k, rows, dist,
                               d_states=d_states, d_norm_sq=d_nsq)
    torch.cuda.synchronize()
    got, gd = rows.cpu().numpy(), dist.cpu().numpy()
    assert np.all(got >= 0)
    assert np.all((np.diff(gd, axis=1) > 0) | ((np.diff(gd, axis=1) == 0) & (np.diff(got, axis=1) > 0)))
    lists_of = np.searchsorted(off, got.reshape(-1), side="right").reshape(nq, k) - 1
    for qi in range(nq):
        assert np.isin(lists_of[qi], probes[qi]).all()
        assert np.unique(got[qi]).size == k
    few = 4   # split path: the same queries alone
    r2 = torch.empty((few, k), dtype=torch.int32, device="cuda")
    d2 = torch.empty((few, k), dtype=torch.float32, device="cuda")
    psb.sign_search_candidates(0, d_codes, d_scales, d_off, nlist, dev(probes[:few]), few, nprobe, padded, k, r2, d2,
                               d_states=dev(states[: few * nprobe]), d_norm_sq=dev(nsq[: few * nprobe]))
    torch.cuda.synchronize()
    assert np.array_equal(r2.cpu().numpy(), got[:few]) and np.array_equal(bits(d2.cpu().numpy()), bits(gd[:few]))
    w_rows, w_dist = oracle.sign_candidates(0, codes, scales, off, probes[:few], k, states=states[: few * nprobe], norm_sq=nsq[: few * nprobe])
    assert np.array_equal(got[:few], w_rows) and np.array_equal(bits(gd[:few]), bits(w_dist))


def test_whole_search_with_sign_codes_as_first_stage(psb):
    """coarse lists -> sign-code candidates -> exact re-ranking -> ids, against the same chain of CPU checkers."""
    ix = make_sign_index(91, 64, 128, 128, 100, 600)
    rng = ix["rng"]
    nq, nprobe, topk, width = 50, 8, 10, 256
    pick = rng.integers(0, ix["n"], nq)
    q = (ix["rows"][pick] + rng.standard_normal((nq, 128)).astype(np.float32)).astype(np.float32)
    rid = rng.permutation(ix["n"]).astype(np.int64)
    index = psb.SignIndex().build_u8(ix["rows"], ix["centroids"], ix["offsets"])
    ids, dist = index.search(q, ix["rows"], nprobe, topk, n_rerank=width, reordered_ids=rid)
    scale = psb.sign_rotation_scale(128)
    probes = oracle.coarse(q, ix["centroids"], nprobe)[0].astype(np.int32)
    codes, scales = oracle.sign_encode_database(ix["rows"], ix["centroids"], ix["offsets"], 128, scale=scale)
    states, nsq, _, _ = oracle.sign_encode_queries(q, ix["centroids"], probes, 128, scale=scale)
    cand, _ = oracle.sign_candidates(0, codes, scales, ix["offsets"], probes, width, states=states, norm_sq=nsq)
    w_rows, w_dist = oracle.rerank(ix["rows"], q, cand, topk)
    w_ids = np.where(w_rows >= 0, rid[np.maximum(w_rows, 0)], -1)
    assert np.array_equal(ids, w_ids) and np.array_equal(bits(dist), bits(w_dist))
    # the query's own source row is found (it sits in a probed list and its residual signs match the query's)
    assert np.mean(ids[:, 0] == rid[pick]) >= 0.9
    with pytest.raises(psb.InvalidArgument):
        index.search(q, ix["rows"], nprobe, topk, n_rerank=5)
