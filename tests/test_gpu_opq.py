"""OPQ index on the GPU path: the rotation kernel against the CPU checker (bit for bit: one in-order fp32 fma chain per
element on both sides) and the whole search with the PQ side on rotated queries."""
import numpy as np
import pytest

import oracle
import synth

pytestmark = pytest.mark.gpu


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def random_rotation(dim, seed):
    rng = np.random.default_rng(seed)
    qm, _ = np.linalg.qr(rng.standard_normal((dim, dim)))
    return qm.astype(np.float32)


@pytest.mark.parametrize("n,dim", [(1, 4), (37, 96), (1000, 128), (70, 33), (5, 1)])
def test_rotate_rows_bit_exact(psb, n, dim):
    import torch
    rng = np.random.default_rng(n * 131 + dim)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    rot = rng.standard_normal((dim, dim)).astype(np.float32)   # any matrix: orientation errors would show
    out = torch.empty((n, dim), dtype=torch.float32, device="cuda")
    psb.rotate_rows(dev(x), dev(rot), n, dim, out)
    torch.cuda.synchronize()
    want = oracle.rotate_rows(x, rot)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.allclose(want, x.astype(np.float64) @ rot.astype(np.float64).T, rtol=1e-4, atol=1e-4)


def test_rotate_rows_orientation_known_answers(psb):
    import torch
    # a permutation (swap 0<->1, 2<->3) and a non-symmetric plane rotation: y = R x, R stored [out][in]
    x = np.array([[1, 2, 3, 4], [-1, 0.5, 2, 8]], np.float32)
    perm = np.array([[0, 1, 0, 0], [1, 0, 0, 0], [0, 0, 0, 1], [0, 0, 1, 0]], np.float32)
    rot = np.array([[.6, -.8, 0, 0], [.8, .6, 0, 0], [0, 0, 0, -1], [0, 0, 1, 0]], np.float32)
    out = torch.empty((2, 4), dtype=torch.float32, device="cuda")
    psb.rotate_rows(dev(x), dev(perm), 2, 4, out)
    assert np.array_equal(out.cpu().numpy(), x[:, [1, 0, 3, 2]])
    psb.rotate_rows(dev(x), dev(rot), 2, 4, out)
    want = np.stack([[.6 * a - .8 * b, .8 * a + .6 * b, -d, c] for a, b, c, d in x.astype(np.float64)])
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-6, atol=2e-6)
    with pytest.raises(psb.InvalidArgument):
        psb.rotate_rows(out, dev(rot), 2, 4, out)   # in place is refused


def make_opq_index(n, dim, nlist, M, seed):
    """An index whose PQ side lives in the rotated space: codebook trained on R x, codes = encode(R x); coarse lists and the
    exact rows stay in the caller's space."""
    ix = synth.make_index(n, dim, nlist, M, seed=seed, zipf=True)
    rot = random_rotation(dim, seed + 1)
    xr = oracle.rotate_rows(ix["vectors"], rot)
    K = ix["codebook"].shape[1]
    dsub = dim // M
    rng = np.random.default_rng(seed + 2)
    pick = rng.choice(n, K, replace=False)
    cb = np.stack([xr[pick, j * dsub:(j + 1) * dsub] for j in range(M)]).astype(np.float32)
    ix["codebook"] = cb
    ix["codes"] = oracle.pq_encode(xr, cb)
    return ix, rot


@pytest.mark.parametrize("scan_mode", [1, 3])
@pytest.mark.parametrize("rerank", [True, False])
def test_search_on_an_opq_index(psb, scan_mode, rerank):
    ix, rot = make_opq_index(60000, 96, 48, 48, seed=71)
    q = synth.make_queries(ix, 300, seed=72, weights=synth.zipf_weights(48))
    n_rerank = 200 if rerank else 0
    want = oracle.ivfpq_search_opq(ix, q[:120], 10, 10, n_rerank, rot)
    index = ix if rerank else dict(ix, vectors=None)
    with psb.Session(index, n_rerank=n_rerank, scan_mode=scan_mode, opq_matrix=rot) as s:
        got = s.search(q, 10, 10, batch_size=300)
    assert np.array_equal(got["indices"][:120], want["indices"])
    assert np.array_equal(got["distances"][:120], want["distances"])
    # without the rotation the PQ side reads the wrong space: recall of the ADC order collapses (sanity of the test itself)
    if not rerank:
        with psb.Session(index, n_rerank=0, scan_mode=scan_mode) as s:
            plain = s.search(q, 10, 10, batch_size=300)
        assert not np.array_equal(plain["indices"][:120], want["indices"])


def test_stage_rotate_queries_and_refusals(psb):
    import torch
    ix, rot = make_opq_index(8000, 32, 8, 8, seed=81)
    q = synth.make_queries(ix, 20, seed=82)
    with psb.Session(dict(ix, vectors=None), opq_matrix=rot) as s:
        out = torch.empty((20, 32), dtype=torch.float32, device="cuda")
        s.stage_rotate_queries(dev(q), 20, out)
        s.sync()
        assert np.array_equal(out.cpu().numpy(), oracle.rotate_rows(q, rot))
    with psb.Session(dict(ix, vectors=None)) as s:
        with pytest.raises(psb.InvalidArgument):
            s.stage_rotate_queries(dev(q), 20, out)
    with pytest.raises(psb.InvalidArgument):
        psb.Session(synth.make_index(8000, 32, 8, 8, seed=83, residual=True), residual=True, opq_matrix=rot)
    with pytest.raises(psb.InvalidArgument):
        psb.Session(dict(ix, vectors=None), opq_matrix=rot[:16])
