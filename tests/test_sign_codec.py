"""CPU checks of the TurboQuant 1-bit codec's checker: the restatement against the host functions of the reference
(compiled in place: bit layout, Hamming count, unfused distance formulas), the known answers of the reference's format test
(tests/unit/turboquant/test_turboquant_1bit_format.cpp:15-47), and the properties its encode and scan tests assert
(tests/unit/turboquant/test_turboquant_1bit_encode.cu:57-76,78-145, test_turboquant_1bit_scan.cu:49-80)."""
import numpy as np
import pytest

import oracle

needs_ref = pytest.mark.skipif(not oracle.have_ref_sign(), reason="the reference's sign codec header is not compiled here")


def bits_set(indices, n):
    v = np.full(n, -1.0, np.float32)
    v[list(indices)] = 1.0
    return v


def test_format_known_answers():
    a = bits_set([0, 1, 31, 32, 63, 69], 70)
    b = bits_set([0, 2, 31, 33, 63, 68], 70)
    pa, pb = oracle.sign_pack(a), oracle.sign_pack(b)
    assert pa.tolist() == [(1 << 0) | (1 << 1) | (1 << 31), (1 << 0) | (1 << 31), 1 << 5]
    assert oracle.sign_hamming(pa, pb, 70) == 6
    dot = 2.0 * 3.0 * (70.0 - 2.0 * 6.0) / 70.0
    assert abs(oracle.sign_binary_l2(pa, pb, 70, 2.0, 3.0) - (4.0 + 9.0 - 2.0 * dot)) <= 1e-5
    # sign reconstruction with one magnitude: sum (other - (+-c))^2
    c = 0.25
    want = float(np.sum((b - np.where(a > 0, c, -c)) ** 2))
    assert abs(oracle.sign_scale_l2(b, pa, c) - want) <= 1e-4


@needs_ref
@pytest.mark.parametrize("dim", [1, 31, 32, 33, 70, 128, 200, 256])
def test_restatement_equals_reference_header(dim):
    rng = np.random.default_rng(dim)
    for trial in range(20):
        v = rng.standard_normal(dim).astype(np.float32)
        w = rng.standard_normal(dim).astype(np.float32) * np.float32(3.0)
        if trial == 0:
            v[: dim // 2] = 0.0   # zero counts as positive
            v[-1] = -0.0
        a, c = oracle.sign_pack(v), oracle.sign_pack(w)
        assert np.array_equal(a, oracle.ref_sign_pack(v))
        assert oracle.sign_hamming(a, c, dim) == oracle.ref_sign_hamming(a, c, dim)
        s = float(np.float32(rng.uniform(0.01, 2.0)))
        assert np.float32(oracle.sign_scale_l2(w, a, s)).view(np.uint32) == np.float32(oracle.ref_sign_scale_l2(w, a, s)).view(np.uint32)
        qn, dn = float(np.float32(rng.uniform(0.1, 9))), float(np.float32(rng.uniform(0.1, 9)))
        assert np.float32(oracle.sign_binary_l2(a, c, dim, qn, dn)).view(np.uint32) == \
            np.float32(oracle.ref_sign_binary_l2(a, c, dim, qn, dn)).view(np.uint32)


def test_padded_dim():
    assert [oracle.sign_padded_dim(d) for d in (1, 32, 33, 64, 70, 128, 129, 256)] == [32, 32, 64, 64, 128, 128, 256, 256]
    assert oracle.sign_padded_dim(257) == -1 and oracle.sign_padded_dim(0) == -1


@pytest.mark.parametrize("dim,padded", [(70, 128), (8, 32), (64, 64), (128, 128), (200, 256)])
def test_rotation_keeps_norms_and_codes_follow_signs(dim, padded):
    rows = np.array([[((r + 3) * (d + 5)) % 23 - 11 for d in range(dim)] for r in range(3)], np.float32) / np.float32(7.0)
    rot, codes, norms, nsq = oracle.sign_rotate(rows, padded)
    want = (rows.astype(np.float64) ** 2).sum(1)
    assert np.all(np.abs(nsq - want) < 1e-3)
    assert np.all(np.abs((rot.astype(np.float64) ** 2).sum(1) - want) < 1e-3)
    assert np.all(np.abs(norms.astype(np.float64) ** 2 - want) < 1e-3)
    bit = (codes[:, np.arange(padded) // 32] >> (np.arange(padded) % 32).astype(np.uint32)) & 1
    assert np.array_equal(bit.astype(bool), rot >= 0)


def test_rotation_is_sign_flip_then_hadamard():
    padded = 64
    eye = np.eye(padded, dtype=np.float32)
    rot, _, _, _ = oracle.sign_rotate(eye, padded, seed=17)
    # rows of the rotation matrix: +-1/8 everywhere, orthonormal
    assert np.allclose(np.abs(rot), 1.0 / 8.0)
    assert np.allclose(rot @ rot.T, np.eye(padded), atol=1e-6)
    other, _, _, _ = oracle.sign_rotate(eye, padded, seed=18)
    assert not np.array_equal(rot, other)


def test_rotation_equals_flip_times_sylvester_hadamard_matrix():
    """An independent statement of the rotation: y = H (D x) / sqrt(P), H the Sylvester (natural order) Hadamard matrix, D the
    diagonal of seeded signs (mix(seed ^ d) odd -> -1).  The butterflies compute exactly this, up to fp32 rounding."""
    from scipy.linalg import hadamard

    def mix(v):
        v &= 0xFFFFFFFF
        v ^= v >> 16; v = (v * 0x7feb352d) & 0xFFFFFFFF
        v ^= v >> 15; v = (v * 0x846ca68b) & 0xFFFFFFFF
        return v ^ (v >> 16)

    rng = np.random.default_rng(12)
    for dim, padded, seed in ((70, 128, 17), (32, 32, 5), (200, 256, 99)):
        x = rng.standard_normal((6, dim)).astype(np.float32)
        rot, _, _, _ = oracle.sign_rotate(x, padded, seed=seed)
        xp = np.zeros((6, padded)); xp[:, :dim] = x
        signs = np.array([-1.0 if mix(seed ^ d) & 1 else 1.0 for d in range(padded)])
        want = (xp * signs) @ hadamard(padded).astype(np.float64) / np.sqrt(padded)
        assert np.allclose(rot, want, rtol=1e-5, atol=1e-5)


def small_database():
    rng = np.random.default_rng(5)
    sizes = [4, 0, 5, 1, 0, 7]
    off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    dim = 8
    rows = rng.integers(0, 90, (int(off[-1]), dim)).astype(np.uint8)
    cen = rng.uniform(0, 40, (len(sizes), dim)).astype(np.float32)
    return rows, cen, off


def test_chunked_database_encoding_equals_one_shot():
    rows, cen, off = small_database()
    codes, scales = oracle.sign_encode_database(rows, cen, off, 32)
    c2 = np.zeros_like(codes); s2 = np.zeros_like(scales)
    for start, count in ((0, 3), (3, 1), (4, 9), (13, 4)):
        oracle.sign_encode_database(rows[start:start + count], cen, off, 32, row_offset=start, codes=c2, scales=s2)
    assert np.array_equal(codes, c2) and np.array_equal(scales.view(np.uint32), s2.view(np.uint32))
    # the scale is the mean magnitude of the rotated residual of the row's own list
    lists = np.repeat(np.arange(len(off) - 1), np.diff(off))
    resid = rows.astype(np.float32) - cen[lists]
    rot, rc, _, _ = oracle.sign_rotate(resid, 32)
    assert np.array_equal(rc, codes)
    assert np.allclose(scales, np.abs(rot).mean(1), rtol=1e-6)
    # fp32 rows with the same values give the same bits
    cf, sf = oracle.sign_encode_database(rows.astype(np.float32), cen, off, 32)
    assert np.array_equal(cf, codes) and np.array_equal(sf.view(np.uint32), scales.view(np.uint32))


def test_query_states():
    rows, cen, off = small_database()
    rng = np.random.default_rng(6)
    q = rng.uniform(0, 60, (3, 8)).astype(np.float32)
    probes = np.array([[0, 2], [5, -1], [3, 9]], np.int32)
    states, nsq, sc, norms = oracle.sign_encode_queries(q, cen, probes, 32)
    for st, (qi, list_) in enumerate([(0, 0), (0, 2), (1, 5), (1, -1), (2, 3), (2, 9)]):
        if list_ < 0 or list_ >= cen.shape[0]:
            assert not states[st].any() and nsq[st] == 0
            continue
        r = (q[qi] - cen[list_])[None]
        rot, codes, nm, ns = oracle.sign_rotate(r, 32)
        assert np.array_equal(rot[0].view(np.uint32), states[st].view(np.uint32))
        assert np.array_equal(codes[0], sc[st]) and ns[0] == nsq[st] and nm[0] == norms[st]


@pytest.mark.parametrize("mode", [0, 1])
def test_candidates_are_the_smallest_scores_in_order(mode):
    rng = np.random.default_rng(7 + mode)
    nlist, dim, padded = 12, 70, 128
    sizes = rng.integers(0, 60, nlist); sizes[3] = 0
    off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    n = int(off[-1])
    cen = rng.standard_normal((nlist, dim)).astype(np.float32)
    lists = np.repeat(np.arange(nlist), sizes)
    rows = (cen[lists] + rng.standard_normal((n, dim)).astype(np.float32) * np.float32(0.5)).astype(np.float32)
    codes, scales = oracle.sign_encode_database(rows, cen, off, padded)
    q = rng.standard_normal((5, dim)).astype(np.float32)
    probes = np.stack([rng.permutation(nlist)[:4] for _ in range(5)]).astype(np.int32)
    probes[1, 2] = -1
    states, nsq, sc, norms = oracle.sign_encode_queries(q, cen, probes, padded)
    k = 16
    if mode == 0:
        got, dist = oracle.sign_candidates(0, codes, scales, off, probes, k, states=states, norm_sq=nsq)
    else:
        got, dist = oracle.sign_candidates(1, codes, scales, off, probes, k, state_codes=sc, norms=norms)
    for qi in range(5):
        pairs = []
        for p in range(4):
            list_ = probes[qi, p]
            if list_ < 0:
                continue
            st = qi * 4 + p
            for r in range(off[list_], off[list_ + 1]):
                if mode == 0:   # the host formula of the reference, to rounding
                    s = oracle.sign_scale_l2(states[st], codes[r], float(scales[r]))
                else:
                    s = oracle.sign_binary_l2(sc[st], codes[r], padded, float(norms[st]), float(scales[r]))
                pairs.append((s, r))
        pairs.sort()
        m = min(k, len(pairs))
        assert np.all(np.diff(dist[qi, :m]) >= 0)
        assert np.allclose(dist[qi, :m], [p[0] for p in pairs[:m]], rtol=1e-4, atol=1e-3)
        # ids agree wherever the scores are not within rounding of a neighbour's
        want = [p[1] for p in pairs[:m]]
        gaps = np.diff([p[0] for p in pairs[:m + 1]]) if len(pairs) > 1 else np.array([])
        for i in range(m):
            near = (i > 0 and gaps[i - 1] < 1e-3) or (i < len(gaps) and gaps[i] < 1e-3)
            if not near:
                assert got[qi, i] == want[i]
        assert np.all(got[qi, m:] == -1) and np.all(dist[qi, m:] == np.finfo(np.float32).max)
    # residual reconstruction tracks the true distance: better than chance ranking of the true neighbour
    if mode == 0:
        hits = 0
        for qi in range(5):
            scanned = np.concatenate([np.arange(off[l], off[l + 1]) for l in probes[qi] if l >= 0])
            true_best = scanned[np.argmin(((rows[scanned] - q[qi]) ** 2).sum(1))]
            hits += int(true_best in got[qi])
        assert hits >= 3


def test_ties_break_by_row():
    padded = 32
    codes = np.tile(np.array([[0x12345678]], np.uint32), (10, 1))
    scales = np.full(10, 0.5, np.float32)
    off = np.array([0, 10], np.int64)
    state = np.linspace(-1, 1, padded, dtype=np.float32)[None]
    nsq = np.array([float((state ** 2).sum())], np.float32)
    got, dist = oracle.sign_candidates(0, codes, scales, off, np.array([[0]], np.int32), 4, states=state, norm_sq=nsq)
    assert got.tolist() == [[0, 1, 2, 3]] and len(set(dist[0].tolist())) == 1
