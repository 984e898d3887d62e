"""Worker of tests/test_gpu_group.py: one rank (= one GPU) of a sharded search driven through the C ABI's psb_group_*.
torch.distributed (gloo) only carries the NCCL unique ids between the ranks; the two NCCL communicators are created here with
the NCCL library itself, through ctypes, the way a C or C++ caller of the group would create them."""
import ctypes as C
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
from fake_engine import stripe_index  # noqa: E402
from paraselect_b200 import api  # noqa: E402


def nccl_library():
    """The NCCL copy torch already loaded into this process (so that one copy serves both)."""
    torch.cuda.nccl.version()
    for line in open("/proc/self/maps"):
        if "libnccl.so" in line:
            return line.split()[-1]
    return "libnccl.so.2"


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def make_comm(nccl, rank, world):
    uid = UniqueId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(C.byref(uid)) == 0
    t = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).clone()
    dist.broadcast(t, 0)
    C.memmove(C.byref(uid), bytes(t.numpy().tobytes()), 128)
    comm = C.c_void_p()
    rc = nccl.ncclCommInitRank(C.byref(comm), world, uid, rank)
    assert rc == 0, rc
    return comm


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(rank)
    path = nccl_library()
    nccl = C.CDLL(path)
    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
    comm_a, comm_b = make_comm(nccl, rank, world), make_comm(nccl, rank, world)
    ok = True
    for residual, n_rerank in ((False, 400), (True, 400), (False, 0)):
        ix = synth.make_index(120000, 96, 32, 48, seed=101, zipf=True, residual=residual)
        q = synth.make_queries(ix, 2500, seed=102, weights=synth.zipf_weights(32))
        nprobe, topk = 8, 10
        search = oracle.ivfrespq_search if residual else oracle.ivfpq_search
        want = search(ix if n_rerank else dict(ix, vectors=None), q[:200], nprobe, topk, n_rerank)
        local, gb = stripe_index(ix, rank, world, min_slice=1024)
        if not n_rerank:
            local = dict(local, vectors=None)
        dq = torch.from_numpy(q).cuda()
        ids = torch.empty((2500, topk), dtype=torch.int64, device="cuda")
        dd = torch.empty((2500, topk), dtype=torch.float32, device="cuda")
        with api.Session(local, n_rerank=n_rerank, device=rank, max_batch=2500, residual=residual, list_global_begin=gb,
                         reserve_sms=16) as sess:
            for shared in (True, False):
                with api.Group(sess, comm_a.value, comm_b.value, 2500, nprobe, topk, nccl_library=path, shared_cutoff=shared) as grp:
                    for _ in range(2):   # buffers are reused from batch to batch
                        grp.search_device(dq, 2500, nprobe, topk, ids, dd)
                        sess.sync()
                        ok = ok and np.array_equal(ids.cpu().numpy()[:200], want["indices"])
                        ok = ok and np.array_equal(dd.cpu().numpy()[:200], want["distances"])
                    ok = ok and grp.searched_again() == 0
                    # a short batch runs in one piece
                    grp.search_device(dq, 300, nprobe, topk, ids, dd)
                    sess.sync()
                    ok = ok and np.array_equal(ids.cpu().numpy()[:200], want["indices"])
        if not ok:
            print("rank %d: mismatch in case residual=%s n_rerank=%d" % (rank, residual, n_rerank), flush=True)
            break
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    nccl.ncclCommDestroy(comm_a)
    nccl.ncclCommDestroy(comm_b)
    dist.destroy_process_group()
    if rank == 0:
        print("GROUP_OK" if int(flag.item()) == 1 else "GROUP_MISMATCH")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
