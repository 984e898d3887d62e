"""GPU parity tests of the IVF-Flat path (coarse + exact fine scan over device-resident rows) through the C ABI, bit-exact
against the CPU checker, which is itself pinned against the reference's cpu_ivf_search (tests/test_oracle.py)."""
import numpy as np
import pytest

import cases
import oracle
import synth

pytestmark = pytest.mark.gpu


def flat_index(n, dim, nlist, seed, zipf=False, empty_lists=()):
    ix = synth.make_index(n, dim, nlist, 8 if dim % 8 == 0 else 4, seed=seed, zipf=zipf, empty_lists=empty_lists)
    return dict(centroids=ix["centroids"], offsets=ix["offsets"], reordered_ids=ix["reordered_ids"], vectors=ix["vectors"]), ix


@pytest.mark.parametrize("n,dim,nlist,nq,nprobe,topk", [(20000, 128, 64, 70, 8, 10), (5000, 96, 16, 33, 16, 100),
                                                          (3000, 100, 8, 9, 3, 1), (40000, 32, 256, 300, 16, 10)])
def test_flat_search_matches_checker(psb, n, dim, nlist, nq, nprobe, topk):
    fx, ix = flat_index(n, dim, nlist, seed=n + dim, zipf=(nlist == 64))
    q = synth.make_queries(ix, nq, seed=5)
    want_i, want_d = oracle.ivfflat_search(fx["centroids"], fx["offsets"], fx["reordered_ids"], fx["vectors"], q, nprobe, topk)
    with psb.FlatSession(fx) as s:
        got = s.search(q, nprobe, topk, batch_size=64, want_coarse=True)   # several batches, a ragged last one
    assert np.array_equal(got["indices"], want_i)
    assert np.array_equal(got["distances"], want_d)
    assert np.array_equal(got["coarse"], oracle.coarse(q, fx["centroids"], nprobe)[0])
    scanned = sum(int(fx["offsets"][l + 1] - fx["offsets"][l]) for row in got["coarse"] for l in row)
    assert got["stats"]["pq_scanned_codes"] == scanned


def test_flat_search_edge_cases(psb):
    fx, ix = flat_index(600, 32, 8, seed=3, empty_lists=(2, 5))
    q = synth.make_queries(ix, 7, seed=4)
    # more results asked for than rows probed: padded with -1 / FLT_MAX
    want_i, want_d = oracle.ivfflat_search(fx["centroids"], fx["offsets"], fx["reordered_ids"], fx["vectors"], q, 2, 400)
    with psb.FlatSession(fx) as s:
        got = s.search(q, 2, 400)
        assert np.array_equal(got["indices"], want_i) and np.array_equal(got["distances"], want_d)
        assert (got["indices"] == -1).any() and got["distances"].max() == cases.FLT_MAX
        # integer-valued rows: many exactly equal distances, ties resolve by row
        rng = np.random.default_rng(1)
        fx2 = dict(fx, vectors=rng.integers(-2, 3, fx["vectors"].shape).astype(np.float32))
    with psb.FlatSession(fx2) as s:
        qq = rng.integers(-2, 3, (12, 32)).astype(np.float32)
        got = s.search(qq, 8, 50)
        wi, wd = oracle.ivfflat_search(fx2["centroids"], fx2["offsets"], fx2["reordered_ids"], fx2["vectors"], qq, 8, 50)
        assert np.array_equal(got["indices"], wi) and np.array_equal(got["distances"], wd)
        with pytest.raises(psb.InvalidArgument):
            s.search(qq, 9, 5)       # nprobe > nlist
        with pytest.raises(psb.InvalidArgument):
            s.search(qq[:, :16], 2, 5)  # wrong dim
    with pytest.raises(psb.InvalidArgument):
        psb.FlatSession(dict(fx, offsets=fx["offsets"][::-1].copy()))


def test_flat_device_entry_point(psb):
    import torch
    fx, ix = flat_index(9000, 64, 32, seed=8)
    q = synth.make_queries(ix, 40, seed=9)
    wi, wd = oracle.ivfflat_search(fx["centroids"], fx["offsets"], fx["reordered_ids"], fx["vectors"], q, 6, 20)
    with psb.FlatSession(fx, max_batch=64) as s:
        ids = torch.empty((40, 20), dtype=torch.int64, device="cuda")
        dd = torch.empty((40, 20), dtype=torch.float32, device="cuda")
        s.search_device(torch.from_numpy(q).cuda(), 40, 6, 20, ids, dd)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy(), wi) and np.array_equal(dd.cpu().numpy(), wd)
