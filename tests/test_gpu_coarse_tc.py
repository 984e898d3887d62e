"""GPU parity tests of the tensor-core coarse stage (bf16 tcgen05 filter + exact fp32 refinement): its output must
be bit-identical to the CPU checker's exact coarse search, ids and distances."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def check(psb, q, c, nprobe):
    ids, dist = psb.coarse_host(q, c, nprobe, coarse_mode=2)
    oi, od = oracle.coarse(q, c, nprobe)
    assert np.array_equal(ids, oi)
    assert np.array_equal(dist, od)


@pytest.mark.parametrize("nq,nlist,dim,nprobe", [(300, 4096, 96, 64), (130, 1024, 128, 32), (200, 2148, 100, 16),
                                                  (1000, 8192, 64, 128), (64, 5000, 128, 8), (257, 3000, 32, 1)])
def test_tc_coarse_matches_checker_gaussian(psb, nq, nlist, dim, nprobe):
    rng = np.random.default_rng(nq + nlist)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    c = rng.standard_normal((nlist, dim)).astype(np.float32)
    check(psb, q, c, nprobe)


def test_tc_coarse_unit_norm_inputs(psb):
    # the "coarse stage only" configuration cut down: N(0,1) scaled to unit mean norm, d = 96, top-64
    rng = np.random.default_rng(2)
    q = rng.standard_normal((2000, 96)).astype(np.float32)
    c = rng.standard_normal((16384, 96)).astype(np.float32)
    q /= np.linalg.norm(q, axis=1).mean()
    c /= np.linalg.norm(c, axis=1).mean()
    check(psb, q, c, 64)


def test_tc_coarse_far_from_origin(psb):
    # data far from the origin: centring on the mean centroid keeps the bf16 error bound tight
    rng = np.random.default_rng(3)
    q = (rng.standard_normal((256, 64)) + 40.0).astype(np.float32)
    c = (rng.standard_normal((2048, 64)) + 40.0).astype(np.float32)
    check(psb, q, c, 32)


def test_tc_coarse_integer_grid_with_ties(psb):
    rng = np.random.default_rng(4)
    q = rng.integers(-3, 4, (200, 32)).astype(np.float32)
    c = rng.integers(-3, 4, (4096, 32)).astype(np.float32)
    check(psb, q, c, 65)


def test_tc_coarse_candidate_overflow_falls_back_to_exact_rows(psb):
    # every centroid identical: every approximate distance ties, the candidate lists overflow, and the per-query
    # exact kernel must return ids 0..nprobe-1
    q = np.random.default_rng(5).standard_normal((128, 64)).astype(np.float32)
    c = np.tile(np.random.default_rng(6).standard_normal((1, 64)).astype(np.float32), (4096, 1))
    check(psb, q, c, 40)


def test_tc_coarse_mode_rejects_unsupported_shapes(psb):
    q = np.zeros((8, 16), np.float32)
    c = np.zeros((64, 16), np.float32)
    with pytest.raises(psb.PsbError) as e:
        psb.coarse_host(q, c, 4, coarse_mode=2)
    assert e.value.status == 2


def test_tc_filter_does_the_work_not_the_fallback(psb):
    """On ordinary data the tensor-core filter must hand (almost) no query to the exact per-query kernel, and the
    session must give the same probes with the filter on and off."""
    import torch
    import synth
    ix = synth.make_index(30000, 96, 2048, 48, seed=9)
    q = synth.make_queries(ix, 500, seed=10)
    dq = torch.from_numpy(q).cuda()
    out = {}
    for mode in (1, 2):
        with psb.Session(dict(ix, vectors=None), coarse_mode=mode) as s:
            ids = torch.empty((500, 64), dtype=torch.int32, device="cuda")
            dist = torch.empty((500, 64), dtype=torch.float32, device="cuda")
            s.stage_coarse(dq, 500, 64, ids, dist)
            s.sync()
            out[mode] = (ids.cpu().numpy(), dist.cpu().numpy(), s.counters()["coarse_fallback_queries"])
    assert np.array_equal(out[1][0], out[2][0]) and np.array_equal(out[1][1], out[2][1])
    assert out[2][2] == 0
    oi, od = oracle.coarse(q, ix["centroids"], 64)
    assert np.array_equal(out[2][0], oi) and np.array_equal(out[2][1], od)


def test_kmeans_assignment_on_the_tensor_core_filter(psb):
    """k = 1024 centroids takes the tensor-core filter with exact refinement for the assignment step (the coarse stage
    with nprobe 1); assignments, objective and centroids must equal the exact SIMT path's, i.e. the checker's."""
    import torch
    import synth
    _, data, _ = synth.mixture(30000, 64, 300, 0.3, seed=16)
    rng = np.random.default_rng(5)
    init = data[rng.choice(30000, size=1024, replace=False)].copy()
    ocen, oassign, oobj = oracle.kmeans_lloyd(data, init, 3)
    dcen = torch.from_numpy(init).cuda()
    dassign = torch.empty((30000,), dtype=torch.int32, device="cuda")
    obj = psb.kmeans_train(torch.from_numpy(data).cuda(), 30000, 64, dcen, 1024, 3, dassign)
    assert np.allclose(obj, oobj, rtol=1e-5)
    assert np.sqrt(np.mean((dcen.cpu().numpy() - ocen) ** 2)) < 1e-5
    assert np.mean(dassign.cpu().numpy() == oassign) > 0.9999
    # final assignment against the final centroids, exactly
    fa, fd = oracle.kmeans_assign(data, dcen.cpu().numpy())
    assert np.array_equal(dassign.cpu().numpy(), fa)


def test_three_call_lloyd_iteration_equals_kmeans_train(psb):
    """psb_kmeans_assign / accumulate / update, as the data-parallel trainer calls them, against psb_kmeans_train."""
    import torch
    import synth
    from paraselect_b200.multi import TrainEngine, sharded_kmeans
    _, data, _ = synth.mixture(30000, 64, 300, 0.3, seed=26)
    rng = np.random.default_rng(7)
    init = data[rng.choice(30000, size=1024, replace=False)].copy()
    x = torch.from_numpy(data).cuda()
    cen_a = torch.from_numpy(init).cuda()
    assign_a = torch.empty((30000,), dtype=torch.int32, device="cuda")
    obj_a = psb.kmeans_train(x, 30000, 64, cen_a, 1024, 3, assign_a)
    cen_b = torch.from_numpy(init).cuda()
    obj_b, assign_b = sharded_kmeans(TrainEngine(psb, torch), None, 1, x, 30000, 64, cen_b, 1024, 3, torch)
    torch.cuda.synchronize()
    assert np.allclose(obj_a, obj_b, rtol=1e-9)
    assert np.allclose(cen_a.cpu().numpy(), cen_b.cpu().numpy(), rtol=1e-6, atol=1e-7)
    assert np.mean(assign_a.cpu().numpy() == assign_b.cpu().numpy()) > 0.9999


def test_coarse_tc_bounded_wait_gives_up_cleanly(psb):
    """The time-out path of the coarse kernel: its producer lane told to issue no load at all (nothing is left in flight), the
    MMA lane and the epilogue warps run into the shortened poll limit, the kernel frees its tensor memory and returns, and the
    call reports PSB_TIMEOUT.  The device stays usable: the next session's coarse stage gives the right answer."""
    import torch
    import synth
    ix = synth.make_index(30000, 64, 2048, 8, seed=71)
    q = synth.make_queries(ix, 300, seed=72)
    out = torch.empty((300, 16), dtype=torch.int32, device="cuda")
    with psb.Session(dict(ix, vectors=None), coarse_mode=2, test_skip_mma=2, test_wait_limit=4096) as s:
        s.stage_coarse(torch.from_numpy(q).cuda(), 300, 16, out)
        with pytest.raises(psb.PsbError) as e:
            s.sync()
        assert e.value.status == 7
    with psb.Session(dict(ix, vectors=None), coarse_mode=2) as s:
        s.stage_coarse(torch.from_numpy(q).cuda(), 300, 16, out)
        s.sync()
        want, _ = oracle.coarse(q, ix["centroids"], 16)
        assert np.array_equal(out.cpu().numpy(), want)
