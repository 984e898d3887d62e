"""Multi-GPU search: inverted lists striped across ranks, one exchange of candidates per batch.

Every rank holds, for every inverted list, one contiguous slice of the list's rows (codes, exact rows and ids of
that slice), plus replicated centroids and codebook.  Slicing every list - instead of giving each rank whole
lists - keeps ranks balanced when list sizes are skewed (a Zipf head list would otherwise pin one rank).

Per batch (`ShardedSearch.step`):
  1. every rank: coarse (all queries, replicated centroids) -> LUT -> ADC scan of its slices -> local
     top-stage1_k candidates, as index-wide row numbers with ADC distances
  2. all-to-all of the candidate lists: rank g receives every rank's lists for ITS slice of the queries only and merges
     them to the index-wide top-stage1_k of that slice (1/world of the bytes and of the merge work of an all-gather);
     an all-gather of the merged rows (4 bytes per candidate) gives every rank the whole candidate table
  3. every rank scores exactly the candidates whose rows it holds (+inf elsewhere); all-reduce(min)
  4. top-k by (distance,row) on the combined scores; ids come from the rank holding each row; all-reduce(max)
The results are those of a single-GPU search of the whole index, bit for bit.

The collective calls go through `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).  The compute goes
through an *engine*: `SessionEngine` drives the CUDA library; the CPU tests substitute their own engine to check
this orchestration without a GPU.
"""
from __future__ import annotations

import numpy as np


def stripe_layout(offsets, rank, world, min_slice=4096):
    """Rows of every list held by `rank`: returns (global_begin [nlist], local_offsets [nlist+1]).

    A list with at least world * min_slice rows is cut into `world` contiguous slices at floor(len * g / world), one per
    rank, so that a few huge lists cannot pin one rank.  A shorter list goes whole to rank (list % world): slicing it
    would leave every rank with the same number of (tiny) work items and nothing to gain.  The other ranks hold an
    empty range of it."""
    offsets = np.asarray(offsets, np.int64)
    nlist = offsets.size - 1
    length = offsets[1:] - offsets[:-1]
    big = length >= world * min_slice
    mine = (np.arange(nlist) % world) == rank
    lo = np.where(big, offsets[:-1] + (length * rank) // world, offsets[:-1])
    hi = np.where(big, offsets[:-1] + (length * (rank + 1)) // world, np.where(mine, offsets[1:], offsets[:-1]))
    local = np.zeros(offsets.size, np.int64)
    local[1:] = np.cumsum(hi - lo)
    return lo, local


def owned_mask_rows(global_begin, local_offsets, r0, r1):
    """Boolean mask over global rows [r0, r1): True where the row belongs to the stripe."""
    rows = np.arange(r0, r1, dtype=np.int64)
    l = np.searchsorted(global_begin, rows, side="right") - 1
    ok = l >= 0
    lc = np.clip(l, 0, None)
    ok &= rows < global_begin[lc] + (local_offsets[lc + 1] - local_offsets[lc])
    return ok


def raw_nccl_comms(dist, torch, count=2):
    """NCCL communicators for api.Group (psb_group_*) in a process that already runs torch.distributed: created with the NCCL
    copy torch loaded, the unique ids carried by a broadcast of the default process group.  Returns (library path, [handles],
    destroy function).  A C or C++ caller creates its communicators with ncclCommInitRank directly."""
    import ctypes as C

    torch.cuda.nccl.version()   # makes sure the library is loaded
    path = "libnccl.so.2"
    for line in open("/proc/self/maps"):
        if "libnccl.so" in line:
            path = line.split()[-1]
            break
    nccl = C.CDLL(path)

    class UniqueId(C.Structure):
        _fields_ = [("internal", C.c_char * 128)]

    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
    rank, world = dist.get_rank(), dist.get_world_size()
    on_gpu = dist.get_backend() == "nccl"
    comms = []
    for _ in range(count):
        uid = UniqueId()
        if rank == 0 and nccl.ncclGetUniqueId(C.byref(uid)) != 0:
            raise RuntimeError("ncclGetUniqueId failed")
        t = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).clone()
        if on_gpu:
            t = t.cuda()
        dist.broadcast(t, 0)
        C.memmove(C.byref(uid), t.cpu().numpy().tobytes(), 128)
        comm = C.c_void_p()
        rc = nccl.ncclCommInitRank(C.byref(comm), world, uid, rank)
        if rc != 0:
            raise RuntimeError("ncclCommInitRank failed (%d)" % rc)
        comms.append(comm.value)

    def destroy():
        for c in comms:
            nccl.ncclCommDestroy(C.c_void_p(c))

    return path, comms, destroy


class SessionEngine:
    """The CUDA library as the compute engine of ShardedSearch (device tensors are torch CUDA tensors)."""

    def __init__(self, session, torch):
        self.s = session
        self.torch = torch
        # residual sessions run without tables: the tensor-core scan works on q - centroid and the selection re-scores from
        # the codebook (the session refuses the call where the shape does not allow that)
        self.residual = bool(getattr(session, "residual", False))

    streams = True  # stage calls can be redirected to a second CUDA stream

    def set_stream(self, stream, background):
        self.s.set_stream(stream, background)

    def empty(self, shape, dtype):
        return self.torch.empty(shape, dtype=dtype, device="cuda")

    def coarse(self, dq, nq, nprobe, out):
        self.s.stage_coarse(dq, nq, nprobe, out)

    def lut(self, dq, nq, out):
        if not self.residual:
            self.s.stage_build_lut(dq, nq, out)

    def scan(self, dq, lut, nq, probes, nprobe, width, rows, dist, count):
        # with the queries at hand the scan can take the tensor-core pre-filter
        self.s.stage_scan_queries(dq, None if self.residual else lut, nq, probes, nprobe, width, rows, dist, count)

    shared_cutoff = True  # the scan can place its cutoffs on the rows of all shards (scan_sample / scan_shared)

    def sample_words(self, width):
        return self.s.scan_sample_words(width)

    def scan_sample(self, dq, lut, nq, probes, nprobe, width, samples):
        self.s.stage_scan_sample(dq, None if self.residual else lut, nq, probes, nprobe, width, samples)

    def scan_shared(self, dq, lut, nq, probes, nprobe, width, all_samples, shards, rows, dist, count, cutoff, rows_scanned):
        self.s.stage_scan_shared(dq, None if self.residual else lut, nq, probes, nprobe, width, all_samples, shards, rows, dist, count,
                                 cutoff, rows_scanned)

    def merge(self, rows, dist, parts, nq, width, out_rows, out_dist):
        self.s.stage_merge(rows, dist, parts, nq, width, out_rows, out_dist)

    def rerank_partial(self, dq, nq, cand, width, out_dist):
        self.s.stage_rerank_partial(dq, nq, cand, width, width, None, out_dist)

    def select_topk(self, dist, cand, nq, width, topk, out_rows, out_dist):
        self.s.stage_select_topk(dist, cand, nq, width, width, None, topk, out_rows, out_dist)

    def map_ids(self, rows, n, out):
        self.s.stage_map_ids(rows, n, out)


class ShardedSearch:
    def __init__(self, engine, dist, world, nq, dim, M, K, nprobe, topk, width, torch, rerank=True, parts=1, shared_cutoff=True):
        self.e, self.dist, self.world, self.torch = engine, dist, world, torch
        self.spans = None
        # Cutoffs placed on all shards' rows: every rank then admits about 1 / world of what an unsharded scan admits instead of
        # looking for `width` rows of its own.  The merged candidates are checked after every exchange; a batch in which a
        # cutoff turned out too low (practically never) is searched again with per-shard cutoffs (self.redone counts them).
        self.shared = bool(shared_cutoff) and world > 1 and getattr(engine, "shared_cutoff", False)
        self.rank = dist.get_rank() if world > 1 else 0
        self.redone = 0
        # The sample records travel on a communicator of their own.  On the default one their all-gather would queue behind
        # the exchange half of the previous sub-batch (a process group runs its collectives one after the other), and the scan
        # that waits for the records would lose its overlap with that exchange.  Every rank issues the collectives of both
        # groups in the same order, and nothing a collective waits for depends on the other group.
        self.front_group = dist.new_group(ranks=list(range(world))) if self.shared else None
        self.parts, self.aux = parts, None
        self.nq, self.nprobe, self.topk, self.width, self.rerank = nq, nprobe, topk, width, rerank
        t = torch
        self.probes = engine.empty((nq, nprobe), t.int32)
        self.lut = engine.empty((nq, M, K), t.float32)
        self.l_rows = engine.empty((nq, width), t.int32)
        self.l_dist = engine.empty((nq, width), t.float32)
        self.l_cnt = engine.empty((nq,), t.int32)
        # exchange buffers, sized for the whole batch in one piece; a query slice is ceil(nq / world) queries (the last is padded)
        ms = (nq + world - 1) // world
        self.s_key = engine.empty((world * ms, width), t.int64)   # send: packed (distance bits << 32 | row), all my local lists
        self.r_key = engine.empty((world, ms, width), t.int64)    # receive: every rank's lists for my slice
        self.g_rows = engine.empty((world, ms, width), t.int32)
        self.g_dist = engine.empty((world, ms, width), t.float32)
        self.mg_rows = engine.empty((ms, width), t.int32)         # merged candidates of my slice
        self.mg_dist = engine.empty((ms, width), t.float32)
        self.m_rows = engine.empty((world * ms, width), t.int32)  # merged candidates of every slice (all-gather)
        self.p_dist = engine.empty((nq, width), t.float32)
        self.o_rows = engine.empty((nq, topk), t.int32)
        self.o_dist = engine.empty((nq, topk), t.float32)
        self.o_ids = engine.empty((nq, topk), t.int64)
        if self.shared:
            self.words = engine.sample_words(width)
            self.smp = engine.empty((nq, self.words), t.int32)            # this shard's sample records
            self.smp_all = engine.empty((world, nq, self.words), t.int32)  # every shard's
            self.cut = engine.empty((nq,), t.float32)
            self.n_scan = engine.empty((nq,), t.int64)
            self.low = engine.empty((1,), t.int32)                         # != 0: some query of the batch came back short
        self.marks = None

    def _mark(self, name):
        if self.marks is not None:
            ev = self.torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def stage_times(self):
        """Milliseconds between the marks of the last profiled step (after a device synchronisation)."""
        m = self.marks or []
        return {m[i + 1][0]: round(m[i][1].elapsed_time(m[i + 1][1]), 3) for i in range(len(m) - 1)}

    def _front(self, dq, q0, m):
        """Local half of queries [q0, q0 + m): tables and ADC scan of this rank's slices -> local candidates."""
        e = self.e
        sl = slice(q0, q0 + m)
        e.lut(dq[sl], m, self.lut[:m])
        if self.use_shared:
            w, words = self.world, self.words
            mine = self.smp.view(-1)[:m * words].view(m, words)
            every = self.smp_all.view(-1)[:w * m * words].view(w, m, words)
            e.scan_sample(dq[sl], self.lut[:m], m, self.probes[sl], self.nprobe, self.width, mine)
            self.dist.all_gather_into_tensor(every.view(w * m, words), mine, group=self.front_group)
            e.scan_shared(dq[sl], self.lut[:m], m, self.probes[sl], self.nprobe, self.width, every, w, self.l_rows[sl], self.l_dist[sl],
                          self.l_cnt[sl], self.cut[sl], self.n_scan[sl])
        else:
            e.scan(dq[sl], self.lut[:m], m, self.probes[sl], self.nprobe, self.width, self.l_rows[sl], self.l_dist[sl], self.l_cnt[sl])
        self._mark("lut+scan")

    def _back(self, dq, q0, m):
        """Exchange half of queries [q0, q0 + m): candidate all-to-all and sliced merge, partial exact scoring, combination."""
        e, d, w, width = self.e, self.dist, self.world, self.width
        sl = slice(q0, q0 + m)
        m_rows = self.l_rows[sl]
        if w > 1:
            t = self.torch
            ms = (m + w - 1) // w                      # queries per slice of this sub-batch (the last slice may be padded)
            s_key = self.s_key.view(-1)[:w * ms * width].view(w * ms, width)
            r_key = self.r_key.view(-1)[:w * ms * width].view(w, ms, width)
            g_rows = self.g_rows.view(-1)[:w * ms * width].view(w, ms, width)
            g_dist = self.g_dist.view(-1)[:w * ms * width].view(w, ms, width)
            mg_rows = self.mg_rows.view(-1)[:ms * width].view(ms, width)
            mg_dist = self.mg_dist.view(-1)[:ms * width].view(ms, width)
            all_rows = self.m_rows.view(-1)[:w * ms * width].view(w * ms, width)
            # one word per candidate: distance bits << 32 | row; padding queries carry (FLT_MAX, -1)
            t.bitwise_or(self.l_dist[sl].view(t.int32).to(t.int64) << 32, self.l_rows[sl].to(t.int64) & 0xFFFFFFFF, out=s_key[:m])
            if w * ms > m:
                s_key[m:].fill_((0x7F7FFFFF << 32) | 0xFFFFFFFF)
            d.all_to_all_single(r_key.view(w * ms, width), s_key)   # slice g of my lists -> rank g; I receive my slice from everyone
            halves = r_key.view(t.int32).view(w, ms, width, 2)       # little-endian: [..., 0] = row, [..., 1] = distance bits
            g_rows.copy_(halves[..., 0])                             # reinterpreted, not value-converted: -1 stays -1
            g_dist.view(t.int32).copy_(halves[..., 1])
            self._mark("all_to_all")
            e.merge(g_rows, g_dist, w, ms, width, mg_rows, mg_dist)
            if self.use_shared:   # my slice: a finite cutoff must have left min(width, rows scanned) candidates among all shards
                a = min(q0 + self.rank * ms, q0 + m)
                b = min(a + ms, q0 + m)
                if b > a:
                    have = (mg_rows[:b - a] >= 0).sum(dim=1)
                    need = self.n_scan[a:b].clamp(max=width)
                    short = ((have < need) & t.isfinite(self.cut[a:b])).any()
                    self.low.add_(short.to(t.int32))
            self._mark("merge")
            d.all_gather_into_tensor(all_rows, mg_rows)              # 4 bytes per candidate: the whole sub-batch's candidate table
            self._mark("all_gather")
            m_rows = all_rows[:m]
        if self.rerank:
            e.rerank_partial(dq[sl], m, m_rows, width, self.p_dist[sl])
            self._mark("rerank_partial")
            if w > 1:
                d.all_reduce(self.p_dist[sl], op=d.ReduceOp.MIN)
                self._mark("all_reduce_min")
            e.select_topk(self.p_dist[sl], m_rows, m, width, self.topk, self.o_rows[sl], self.o_dist[sl])
            self._mark("select_topk")
        else:
            if w > 1:  # no rerank: the merged ADC distances of my slice go round with the rows
                all_dist = self.g_dist.view(-1)[:w * ms * width].view(w * ms, width)
                d.all_gather_into_tensor(all_dist, mg_dist.clone())
                self.o_rows[sl].copy_(m_rows[:, :self.topk])
                self.o_dist[sl].copy_(all_dist[:m, :self.topk])
            else:
                self.o_rows[sl].copy_(m_rows[:, :self.topk])
                self.o_dist[sl].copy_(self.l_dist[sl][:, :self.topk])
        # ids of the rows this rank holds, -1 elsewhere; step() combines them with ONE all-reduce(max) for the whole batch
        e.map_ids(self.o_rows[sl], m * self.topk, self.o_ids[sl])
        self._mark("map_ids")

    def _combine_ids(self):
        if self.world > 1:
            self.dist.all_reduce(self.o_ids, op=self.dist.ReduceOp.MAX)
        self._mark("all_reduce_max")

    def _span(self, name, fn):
        """Runs fn between two events of the current stream when a timeline is being recorded (step(trace=True))."""
        if self.spans is None:
            return fn()
        a, b = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        self.spans.append((name, a, b))
        return out

    def timeline(self):
        """(name, start ms, end ms) of the halves of the last step(trace=True), relative to its first event."""
        sp = self.spans or []
        if not sp:
            return []
        t0 = sp[0][1]
        return [(n, round(t0.elapsed_time(a), 3), round(t0.elapsed_time(b), 3)) for n, a, b in sp]

    def step(self, dq, profile=False, parts=None, shared=None, trace=False):
        self.spans = [] if trace else None
        """One batch.  parts > 1 cuts the batch into sub-batches; on an engine with streams the exchange half of
        sub-batch i (collectives, PCIe rerank) then runs on a second stream beside the scan of sub-batch i + 1.
        profile=True runs the batch serially in one piece and records per-stage times."""
        self.use_shared = self.shared if shared is None else (bool(shared) and self.shared)
        if self.use_shared:
            self.low.zero_()
        out = self._step(dq, profile, parts)
        if self.use_shared:   # one word for the whole batch: did any rank see a query come back short?
            self.dist.all_reduce(self.low, op=self.dist.ReduceOp.MAX)
            if int(self.low.item()) != 0:
                self.redone += 1
                return self.step(dq, profile, parts, shared=False)
        return out

    def _step(self, dq, profile, parts):
        e, nq = self.e, self.nq
        parts = 1 if profile else (self.parts if parts is None else parts)
        parts = max(1, min(parts, nq))
        self.marks = [] if profile else None
        self._mark("start")
        e.coarse(dq, nq, self.nprobe, self.probes)
        self._mark("coarse")
        sb = (nq + parts - 1) // parts
        cuts = list(range(0, nq, sb)) + [nq]
        streams = parts > 1 and getattr(e, "streams", False)
        if streams and parts == 4 and nq >= 4096:
            # the exchange half (PCIe rerank) is the longer one: a small first sub-batch lets it start early
            cuts = [0, int(0.10 * nq), int(0.40 * nq), int(0.70 * nq), nq]
        if not streams:
            for q0, q1 in zip(cuts[:-1], cuts[1:]):
                self._front(dq, q0, q1 - q0)
                self._back(dq, q0, q1 - q0)
            self._combine_ids()
            return self.o_ids, self.o_dist
        t = self.torch
        main = t.cuda.current_stream()
        if self.aux is None:
            self.aux = t.cuda.Stream(priority=0)
        aux = self.aux
        aux.wait_stream(main)  # the second stream starts after everything already queued
        # The front half of sub-batch i + 1 is queued BEFORE the back half of sub-batch i: a back half may keep this thread busy
        # (the host's share of a hybrid rerank transport), and the GPU must not run dry meanwhile.
        spans = list(zip(cuts[:-1], cuts[1:]))
        done = []
        for i in range(len(spans) + 1):
            if i < len(spans):
                q0, q1 = spans[i]
                self._span("front %d" % q0, lambda: self._front(dq, q0, q1 - q0))
                ev = t.cuda.Event()
                ev.record(main)
                done.append(ev)
            if i >= 1:
                p0, p1 = spans[i - 1]
                aux.wait_event(done[i - 1])
                e.set_stream(aux.cuda_stream, True)
                try:
                    with t.cuda.stream(aux):
                        self._span("back %d" % p0, lambda: self._back(dq, p0, p1 - p0))
                finally:
                    e.set_stream(None, False)
        main.wait_stream(aux)
        self._combine_ids()
        return self.o_ids, self.o_dist

    # The engine and torch.distributed are driven from torch's current stream (the bench creates the session on it, and
    # the pipelined step redirects both to the second stream together), so stream order serialises kernels and collectives.


# ---------------------------------------------------------------------------------------------------------------
# Data-parallel k-means: rows sharded across ranks, one all-reduce of the per-centroid sums and counts per iteration
# (the reference's multi-GPU trainers reduce on the host instead: src/clustering/kmeans/kmeans_multigpu_train.cu:49-139).

class TrainEngine:
    """The CUDA library's three-call Lloyd iteration on torch CUDA tensors (calls run on torch's current stream)."""

    bounded_assign = True   # assign() can take the previous assignment as a bound

    def __init__(self, api, torch, device=0):
        self.api, self.torch, self.device = api, torch, device

    def _st(self):
        return self.torch.cuda.current_stream().cuda_stream

    def empty(self, shape, dtype):
        return self.torch.empty(shape, dtype=dtype, device="cuda")

    def assign(self, x, n, dim, cen, k, assign, best, have_previous=False):
        self.api.kmeans_assign(x, n, dim, cen, k, assign, best, device=self.device, stream=self._st(), have_previous=have_previous)

    def accumulate(self, x, n, dim, assign, best, k, sums, counts, obj):
        self.api.kmeans_accumulate(x, n, dim, assign, best, k, sums, counts, obj, device=self.device, stream=self._st())

    def update(self, sums, counts, k, dim, cen):
        self.api.kmeans_update(sums, counts, k, dim, cen, device=self.device, stream=self._st())


def sharded_kmeans(engine, dist, world, x, n, dim, cen, k, iters, torch):
    """Lloyd k-means over row shards.  x [n][dim]: this rank's rows; cen [k][dim]: the same initial centroids on every
    rank, updated in place (identically on every rank).  Returns (objective per iteration [iters + 1], assignment of the
    local rows against the final centroids)."""
    assign = engine.empty((n,), torch.int32)
    best = engine.empty((n,), torch.float32)
    sums = engine.empty((k, dim), torch.float64)
    counts = engine.empty((k,), torch.int32)
    obj = engine.empty((1,), torch.float64)
    history = []
    for it in range(iters + 1):
        if it > 0 and getattr(engine, "bounded_assign", False):
            engine.assign(x, n, dim, cen, k, assign, best, have_previous=True)   # the assignment of the iteration before bounds this one
        else:
            engine.assign(x, n, dim, cen, k, assign, best)
        engine.accumulate(x, n, dim, assign, best, k, sums, counts, obj)
        if world > 1:
            dist.all_reduce(sums)
            dist.all_reduce(counts)
            dist.all_reduce(obj)
        history.append(float(obj.item()))
        if it < iters:
            engine.update(sums, counts, k, dim, cen)
    return history, assign
