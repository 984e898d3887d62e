"""Worker of tests/test_multi_cpu.py: one gloo rank of the sharded search with the CPU checker as engine."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
import synth  # noqa: E402
from fake_engine import CpuCheckerEngine, stripe_index  # noqa: E402
from paraselect_b200.multi import ShardedSearch  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ix = synth.make_index(6000, 32, 12, 8, seed=77, zipf=True)
    q = synth.make_queries(ix, 16, seed=78, weights=synth.zipf_weights(12))
    nprobe, topk, width = 5, 7, 40
    local, gb = stripe_index(ix, rank, world)
    eng = CpuCheckerEngine(local, gb)
    s = ShardedSearch(eng, dist, world, q.shape[0], 32, 8, 256, nprobe, topk, width, torch, rerank=True)
    ids, dd = s.step(torch.from_numpy(q))
    want = oracle.ivfpq_search(ix, q, nprobe, topk, width)
    ok = np.array_equal(ids.numpy(), want["indices"]) and np.array_equal(dd.numpy(), want["distances"])
    # a batch size the ranks do not divide evenly: the last query slice of the exchange is padded
    q5 = q[:5]
    s5 = ShardedSearch(eng, dist, world, 5, 32, 8, 256, nprobe, topk, width, torch, rerank=True)
    ids5, dd5 = s5.step(torch.from_numpy(q5))
    ok = ok and np.array_equal(ids5.numpy(), want["indices"][:5]) and np.array_equal(dd5.numpy(), want["distances"][:5])
    # without the rerank the merged ADC candidates are the result
    sn = ShardedSearch(eng, dist, world, q.shape[0], 32, 8, 256, nprobe, topk, width, torch, rerank=False)
    idn, ddn = sn.step(torch.from_numpy(q))
    wantn = oracle.ivfpq_search(dict(ix, vectors=None), q, nprobe, topk, 0)
    ok = ok and np.array_equal(idn.numpy(), wantn["indices"]) and np.array_equal(ddn.numpy(), wantn["distances"])
    # the same batch cut into three sub-batches (16 = 6 + 6 + 4): each runs its own exchange
    ids3, dd3 = s.step(torch.from_numpy(q), parts=3)
    ok = ok and np.array_equal(ids3.numpy(), want["indices"]) and np.array_equal(dd3.numpy(), want["distances"])
    # cutoffs placed on all shards' rows: a larger index, so that the sampled cutoffs are finite and the shards come back with
    # fewer than `width` rows each; the result must not change
    big = synth.make_index(40000, 32, 12, 8, seed=79, zipf=True)
    qb = synth.make_queries(big, 12, seed=80, weights=synth.zipf_weights(12))
    wantb = oracle.ivfpq_search(big, qb, 6, 7, 40)
    lb, gbb = stripe_index(big, rank, world)
    engb = CpuCheckerEngine(lb, gbb, shared_sigma=2.0)
    sb = ShardedSearch(engb, dist, world, 12, 32, 8, 256, 6, 7, 40, torch, rerank=True)
    idb, ddb = sb.step(torch.from_numpy(qb), parts=2)
    if world > 1:
        ok = ok and engb.shared_calls == 2 and sb.redone == 0 and bool(torch.isfinite(sb.cut).all())
    ok = ok and np.array_equal(idb.numpy(), wantb["indices"]) and np.array_equal(ddb.numpy(), wantb["distances"])
    # ... and a cutoff placed too low is noticed after the merge: the batch runs again with per-shard cutoffs
    engl = CpuCheckerEngine(lb, gbb, shared_sigma=2.0, cut_scale=0.5)
    sl = ShardedSearch(engl, dist, world, 12, 32, 8, 256, 6, 7, 40, torch, rerank=True)
    idl, ddl = sl.step(torch.from_numpy(qb))
    if world > 1:
        ok = ok and sl.redone == 1
    ok = ok and np.array_equal(idl.numpy(), wantb["indices"]) and np.array_equal(ddl.numpy(), wantb["distances"])
    # switched off, the exchange is the plain one
    sp = ShardedSearch(engb, dist, world, 12, 32, 8, 256, 6, 7, 40, torch, rerank=True, shared_cutoff=False)
    idp, ddp = sp.step(torch.from_numpy(qb))
    ok = ok and np.array_equal(idp.numpy(), wantb["indices"]) and np.array_equal(ddp.numpy(), wantb["distances"])
    # data-parallel k-means: rows split between the ranks, sums and counts all-reduced every iteration
    from fake_engine import CpuTrainEngine
    from paraselect_b200.multi import sharded_kmeans
    _, data, _ = synth.mixture(4000, 16, 20, 0.3, seed=91)
    init = data[:50].copy()
    want_cen, want_assign, want_obj = oracle.kmeans_lloyd(data, init, 4)
    lo, hi = 4000 * rank // world, 4000 * (rank + 1) // world
    cen = torch.from_numpy(init.copy())
    hist, assign = sharded_kmeans(CpuTrainEngine(), dist, world, torch.from_numpy(data[lo:hi].copy()), hi - lo, 16, cen, 50, 4, torch)
    ok = ok and np.allclose(hist, want_obj, rtol=1e-6) and np.allclose(cen.numpy(), want_cen, rtol=1e-6, atol=1e-7)
    ok = ok and np.array_equal(assign.numpy(), want_assign[lo:hi])
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_OK" if int(flag.item()) == 1 else "MULTI_MISMATCH")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
