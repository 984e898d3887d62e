"""Sharded scan with cutoffs placed on all shards' rows (psb_stage_scan_sample / psb_stage_scan_shared): the shards of an
index run as sessions of one GPU, one after the other; their candidates merged must be the unsharded scan's, while every
shard admits far fewer rows than it would looking for stage1_k rows of its own."""
import numpy as np
import pytest

import oracle
import synth
from fake_engine import stripe_index

pytestmark = pytest.mark.gpu


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_shards(psb, ix, q, probes, width, world, scan_mode, residual=False):
    import torch
    nq, nprobe = probes.shape
    sessions, gbs = [], []
    for r in range(world):
        local, gb = stripe_index(ix, r, world, min_slice=2048)
        sessions.append(psb.Session(local if residual else dict(local, vectors=None), residual=residual, scan_mode=scan_mode,
                                    list_global_begin=gb))
        gbs.append(gb)
    try:
        dq, dp = dev(q), dev(probes.astype(np.int32))
        words = sessions[0].scan_sample_words(width)
        every = torch.zeros((world, nq, words), dtype=torch.int32, device="cuda")
        luts = []
        for r, s in enumerate(sessions):
            lut = None
            if not residual:
                lut = torch.empty((nq, s.M, s.K), dtype=torch.float32, device="cuda")
                s.stage_build_lut(dq, nq, lut)
            luts.append(lut)
        # each shard's scan workspace is its own, so all shards may sample first and scan afterwards
        for r, s in enumerate(sessions):
            s.stage_scan_sample(dq, luts[r], nq, dp, nprobe, width, every[r])
            s.sync()
        out = []
        for r, s in enumerate(sessions):
            rows = torch.empty((nq, width), dtype=torch.int32, device="cuda")
            dist = torch.empty((nq, width), dtype=torch.float32, device="cuda")
            cnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
            cut = torch.empty((nq,), dtype=torch.float32, device="cuda")
            nscan = torch.empty((nq,), dtype=torch.int64, device="cuda")
            s.stage_scan_shared(dq, luts[r], nq, dp, nprobe, width, every, world, rows, dist, cnt, cut, nscan)
            s.sync()
            out.append(dict(rows=rows.cpu().numpy(), dist=dist.cpu().numpy(), cnt=cnt.cpu().numpy(), cut=cut.cpu().numpy(),
                            nscan=nscan.cpu().numpy(), counters=s.counters()))
        return out
    finally:
        for s in sessions:
            s.close()


def merged(out, width):
    nq = out[0]["rows"].shape[0]
    rows = np.full((nq, width), -1, np.int32)
    dist = np.full((nq, width), np.finfo(np.float32).max, np.float32)
    for q in range(nq):
        r = np.concatenate([o["rows"][q][:o["cnt"][q]] for o in out])
        d = np.concatenate([o["dist"][q][:o["cnt"][q]] for o in out])
        order = np.lexsort((r, d))[:width]
        rows[q, :order.size] = r[order]
        dist[q, :order.size] = d[order]
    return rows, dist


@pytest.mark.parametrize("scan_mode", [1, 3])
@pytest.mark.parametrize("world", [2, 4])
def test_shared_cutoff_shards_merge_to_the_unsharded_scan(psb, scan_mode, world):
    width = 600
    ix = synth.make_index(160000, 96, 24, 48, seed=91, zipf=True)
    q = synth.make_queries(ix, 48, seed=92, weights=synth.zipf_weights(24))
    probes, _ = oracle.coarse(q, ix["centroids"], 10)
    orow, odist, ocnt, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], width)
    out = run_shards(psb, ix, q, probes, width, world, scan_mode)
    rows, dist = merged(out, width)
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist)
    # every shard saw the same cutoffs and row totals, and the cutoffs did their work: the shards together return far fewer
    # candidates than world x width, and no query needed the exact fallback
    for o in out[1:]:
        assert np.array_equal(o["cut"], out[0]["cut"]) and np.array_equal(o["nscan"], out[0]["nscan"])
    assert np.isfinite(out[0]["cut"]).all()
    # (about 4 x width rows lie below a cutoff with this margin, so the saving shows from four shards on)
    total = sum(int(o["cnt"].sum()) for o in out)
    if world >= 4:
        assert total < 0.9 * world * width * q.shape[0]
        assert all(int(o["cnt"].min()) < width for o in out)
    assert all(o["counters"]["fallback_queries"] == 0 for o in out)
    assert np.array_equal(out[0]["nscan"], np.array([sum(int(ix["offsets"][l + 1] - ix["offsets"][l]) for l in p) for p in probes]))


def test_shared_cutoff_small_shards(psb):
    """Few rows per query (fewer than a shard's pool holds): the shards still record their samples, complete ones, and the
    merged result is the unsharded one whatever the cutoffs come out as."""
    ix = synth.make_index(6000, 32, 12, 8, seed=77, zipf=True)
    q = synth.make_queries(ix, 16, seed=78)
    probes, _ = oracle.coarse(q, ix["centroids"], 5)
    orow, odist, _, _ = oracle.pq_scan(q, probes, ix["offsets"], ix["codes"], ix["codebook"], 40)
    out = run_shards(psb, ix, q, probes, 40, 2, 1)
    rows, dist = merged(out, 40)
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert all(o["counters"]["fallback_queries"] == 0 for o in out)


def test_shared_cutoff_residual_mode(psb):
    width = 700
    ix = synth.make_index(120000, 96, 16, 48, seed=95, zipf=True, residual=True)
    q = synth.make_queries(ix, 40, seed=96, weights=synth.zipf_weights(16))
    probes, _ = oracle.coarse(q, ix["centroids"], 8)
    orow, odist = oracle.pq_scan_residual(q, probes, ix["centroids"], ix["offsets"], ix["codes"], ix["codebook"], width)[:2]
    out = run_shards(psb, ix, q, probes, width, 2, 3, residual=True)
    rows, dist = merged(out, width)
    assert np.array_equal(rows, orow) and np.array_equal(dist, odist)
    assert np.isfinite(out[0]["cut"]).all()
