"""The allocation-free coarse entry point (psb_coarse_search_static), called through the C ABI.

Some callers cannot allocate device memory at search time (a fixed budget granted at start-up, a host that
forbids cudaMalloc after initialisation).  For them the library carries the coarse stage's distance tile as a
fixed 16 MiB device array.  This test checks that the entry point returns exactly what the allocating coarse
stage returns, on two calls in a row (the second call reuses the array with the first call's leftovers in it),
and that it refuses shapes beyond the array's size.  It lives in a file that pytest collects last.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_coarse_matches_allocating_coarse_twice(psb):
    import torch
    rng = np.random.default_rng(123)
    for nq, nlist, dim, nprobe in ((300, 4096, 96, 64), (57, 1000, 128, 17)):  # second call: smaller, reuses the array
        q = rng.standard_normal((nq, dim)).astype(np.float32)
        c = rng.standard_normal((nlist, dim)).astype(np.float32)
        want_ids, want_dist = psb.coarse_host(q, c, nprobe)          # existing entry point (allocates)
        dq, dc = torch.from_numpy(q).cuda(), torch.from_numpy(c).cuda()
        ids = torch.full((nq, nprobe), -7, dtype=torch.int32, device="cuda")
        dist = torch.full((nq, nprobe), -7.0, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        psb.coarse_search_static(dq, nq, dc, nlist, dim, nprobe, ids, dist)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy().astype(np.int64), want_ids)   # bit-exact, like the other parity tests
        assert np.array_equal(dist.cpu().numpy(), want_dist)


def test_static_coarse_rejects_shapes_beyond_its_scratch(psb):
    import torch
    dq = torch.zeros((4097, 8), dtype=torch.float32, device="cuda")
    dc = torch.zeros((1024, 8), dtype=torch.float32, device="cuda")
    ids = torch.zeros((4097, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(psb.PsbError) as e:
        psb.coarse_search_static(dq, 4097, dc, 1024, 8, 4, ids)   # 4097 * 1024 > 4,194,304
    assert e.value.status == 2 and "4,194,304" in str(e.value)
    with pytest.raises(psb.InvalidArgument):
        psb.coarse_search_static(dq, 4, dc, 1024, 8, 2000, ids)   # nprobe > nlist
