"""TEST INFRASTRUCTURE: a CPU stand-in for the CUDA engine of paraselect_b200.multi.ShardedSearch, built on the
CPU checker.  It lets the multi-rank orchestration (striping, candidate exchange, partial rerank, id ownership)
run as gloo ranks without a GPU.  Tensors are torch CPU tensors."""
import numpy as np
import torch

import oracle

INF = np.float32(np.inf)
FLT_MAX = np.finfo(np.float32).max


SEED_TAIL = 4  # words after the keys of a sample record: stride, key count, rows scanned (low, high)


def _pool_capacity(stage1_k):
    c = 1024
    while c < 16 * stage1_k and c < 16384:
        c <<= 1
    return c


def _export_count(mu, sigma):
    c = mu
    for _ in range(6):
        c = mu + sigma * np.sqrt(c) + 2.0
    return int(np.ceil(c)) + 8


def _record_keys(stage1_k, sigma=6.0):
    return (_export_count(stage1_k / 16.0 + 16.0, sigma) + 31) // 32 * 32


def _f2key(d):
    """Order-preserving uint32 image of non-negative fp32 distances."""
    return (np.asarray(d, np.float32).view(np.uint32) | np.uint32(0x80000000)).astype(np.uint32)


def _key2f(k):
    return (np.asarray(k, np.uint32) & np.uint32(0x7FFFFFFF)).view(np.float32)


def pick_shared_cutoff(records, keys, stage1_k, sigma):
    """The cutoff of one query from every shard's record [shards][keys + SEED_TAIL]: the rule of the library's k_pick_cutoff."""
    ents = []
    smax = 0
    for rec in records:
        stride, have = int(rec[keys]), int(rec[keys + 1])
        if have:
            smax = max(smax, stride)
        for j in range(have):
            ents.append((int(rec[j]), stride))
    ents.sort()
    A = B = 0.0
    for key, stride in ents:
        A += stride; B += stride * stride
        if A - sigma * np.sqrt(B) - 2.0 * smax >= stage1_k:
            return float(_key2f(np.uint32(key)))
    return float("inf")


class CpuCheckerEngine:
    def __init__(self, index, global_begin, shared_sigma=6.0, cut_scale=1.0):
        self.ix = index                      # local (striped) index: offsets are local
        self.gb = np.asarray(global_begin, np.int64)
        self.loff = np.asarray(index["offsets"], np.int64)
        self.q = None
        self.shared_sigma = shared_sigma     # margin of the shared cutoff (the library uses 6)
        self.cut_scale = cut_scale           # < 1 puts every shared cutoff too low: exercises the caller's second pass
        self.shared_calls = 0

    shared_cutoff = True

    def sample_words(self, width):
        return _record_keys(width) + SEED_TAIL

    def scan_sample(self, dq, lut, nq, probes, nprobe, width, samples):
        """Per query the smallest sample keys of this shard (every stride-th row of each probed list), as the library's
        sampling kernel records them."""
        keys = _record_keys(width)
        lut = oracle.pq_lut(self.q_sub, self.ix["codebook"])
        M = lut.shape[1]
        codes = self.ix["codes"]
        out = np.full((nq, keys + SEED_TAIL), 0xFFFFFFFF, np.uint32)
        pr = probes.numpy().astype(np.int64)
        for q in range(nq):
            lists = [l for l in pr[q] if 0 <= l < self.loff.size - 1]
            N = int(sum(self.loff[l + 1] - self.loff[l] for l in lists))
            out[q, keys:] = (0, 0, N & 0xFFFFFFFF, N >> 32)
            if N <= 0:
                continue
            stride = min(max(width // 16, 16), 64)
            rows = np.concatenate([np.arange(self.loff[l], self.loff[l + 1], stride) for l in lists])
            ns = rows.size
            mu = width * ns / N
            r = _export_count(mu, self.shared_sigma)
            d = np.zeros(ns, np.float32)
            for m in range(M):
                d += lut[q, m][codes[rows, m]]
            k = np.sort(_f2key(d))[:r]
            n_out = min(r, keys, k.size)
            out[q, :n_out] = k[:n_out]
            out[q, keys] = stride
            out[q, keys + 1] = n_out
        samples.copy_(torch.from_numpy(out.view(np.int32)))

    def scan_shared(self, dq, lut, nq, probes, nprobe, width, all_samples, shards, rows, dist, count, cutoff, rows_scanned):
        self.shared_calls += 1
        keys = _record_keys(width)
        rec = all_samples.numpy().view(np.uint32)
        cut = np.array([pick_shared_cutoff(rec[:, q], keys, width, self.shared_sigma) for q in range(nq)], np.float32)
        cut = np.where(np.isfinite(cut), cut * np.float32(self.cut_scale), cut).astype(np.float32)
        self.scan(dq, lut, nq, probes, nprobe, width, rows, dist, count)
        r, d = rows.numpy(), dist.numpy()
        drop = d > cut[:, None]
        r[drop] = -1
        d[drop] = FLT_MAX
        count.copy_(torch.from_numpy((r >= 0).sum(1).astype(np.int32)))
        cutoff.copy_(torch.from_numpy(cut))
        n_all = (rec[:, :, keys + 2].astype(np.int64) | (rec[:, :, keys + 3].astype(np.int64) << 32)).sum(0)
        rows_scanned.copy_(torch.from_numpy(n_all))

    def empty(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype)

    def _local(self, rows):
        rows = np.asarray(rows, np.int64)
        l = np.searchsorted(self.gb, rows, side="right") - 1
        lc = np.clip(l, 0, None)
        loc = self.loff[lc] + (rows - self.gb[lc])
        ok = (rows >= 0) & (l >= 0) & (loc < self.loff[lc + 1])
        return np.where(ok, loc, -1)

    def coarse(self, dq, nq, nprobe, out):
        self.q = dq.numpy()
        ids, _ = oracle.coarse(self.q, self.ix["centroids"], nprobe)
        out.copy_(torch.from_numpy(ids.astype(np.int32)))

    def lut(self, dq, nq, out):
        self.q_sub = dq.numpy()  # the scan below belongs to the same (sub-)batch of queries
        out.copy_(torch.from_numpy(oracle.pq_lut(self.q_sub, self.ix["codebook"])))

    def scan(self, dq, lut, nq, probes, nprobe, width, rows, dist, count):
        r, d, c, _ = oracle.pq_scan(self.q_sub, probes.numpy().astype(np.int64), self.loff, self.ix["codes"],
                                    self.ix["codebook"], width)
        # local rows -> index-wide rows; the checker orders ties by local row, which is monotone in the global row
        lists = np.searchsorted(self.loff, np.clip(r, 0, None), side="right") - 1
        g = np.where(r >= 0, r + (self.gb[lists] - self.loff[lists]), -1)
        rows.copy_(torch.from_numpy(g.astype(np.int32)))
        dist.copy_(torch.from_numpy(d))
        count.copy_(torch.from_numpy(c))

    def merge(self, rows, dist, parts, nq, width, out_rows, out_dist):
        r = rows.numpy().transpose(1, 0, 2).reshape(nq, parts * width)
        d = dist.numpy().transpose(1, 0, 2).reshape(nq, parts * width)
        o_r = np.full((nq, width), -1, np.int32)
        o_d = np.full((nq, width), FLT_MAX, np.float32)
        for q in range(nq):
            ok = r[q] >= 0
            order = np.lexsort((r[q][ok], d[q][ok]))[:width]
            o_r[q, :order.size] = r[q][ok][order]
            o_d[q, :order.size] = d[q][ok][order]
        out_rows.copy_(torch.from_numpy(o_r))
        out_dist.copy_(torch.from_numpy(o_d))

    def rerank_partial(self, dq, nq, cand, width, out_dist):
        q = dq.numpy()
        c = cand.numpy()
        loc = self._local(c)
        out = np.full((nq, width), INF, np.float32)
        for i in range(nq):
            for j in range(width):
                if loc[i, j] >= 0:
                    out[i, j] = oracle.l2_exact(q[i], self.ix["vectors"][loc[i, j]])
        out_dist.copy_(torch.from_numpy(out))

    def select_topk(self, dist, cand, nq, width, topk, out_rows, out_dist):
        d, c = dist.numpy(), cand.numpy()
        o_r = np.full((nq, topk), -1, np.int32)
        o_d = np.full((nq, topk), FLT_MAX, np.float32)
        for q in range(nq):
            ok = (c[q] >= 0) & np.isfinite(d[q])
            pairs = sorted(set(zip(d[q][ok].tolist(), c[q][ok].tolist())))[:topk]
            for k, (dd, rr) in enumerate(pairs):
                o_r[q, k], o_d[q, k] = rr, np.float32(dd)
        out_rows.copy_(torch.from_numpy(o_r))
        out_dist.copy_(torch.from_numpy(o_d))

    def map_ids(self, rows, n, out):
        loc = self._local(rows.numpy().reshape(-1))
        ids = np.where(loc >= 0, self.ix["reordered_ids"][np.clip(loc, 0, None)], -1)
        out.copy_(torch.from_numpy(ids.reshape(out.shape).astype(np.int64)))


def stripe_index(ix, rank, world, min_slice=64):
    """Local (striped) view of a whole synthetic index for `rank` (small min_slice: the test lists are small)."""
    from paraselect_b200.multi import stripe_layout
    gb, loff = stripe_layout(ix["offsets"], rank, world, min_slice=min_slice)
    keep = np.concatenate([np.arange(gb[l], gb[l] + (loff[l + 1] - loff[l])) for l in range(gb.size)]).astype(np.int64)
    local = dict(ix)
    local.update(offsets=loff, reordered_ids=ix["reordered_ids"][keep], codes=ix["codes"][keep],
                 vectors=None if ix.get("vectors") is None else ix["vectors"][keep])
    return local, gb


class CpuTrainEngine:
    """CPU stand-in for paraselect_b200.multi.TrainEngine (the three-call Lloyd iteration) built on the CPU checker."""

    def empty(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype)

    def assign(self, x, n, dim, cen, k, assign, best):
        a, d = oracle.kmeans_assign(x.numpy(), cen.numpy())
        assign.copy_(torch.from_numpy(a)); best.copy_(torch.from_numpy(d))

    def accumulate(self, x, n, dim, assign, best, k, sums, counts, obj):
        s = np.zeros((k, dim), np.float64)
        np.add.at(s, assign.numpy(), x.numpy().astype(np.float64))
        sums.copy_(torch.from_numpy(s))
        counts.copy_(torch.from_numpy(np.bincount(assign.numpy(), minlength=k).astype(np.int32)))
        obj[0] = float(best.numpy().astype(np.float64).sum())

    def update(self, sums, counts, k, dim, cen):
        c = counts.numpy()
        new = cen.numpy().copy()
        nz = c > 0
        new[nz] = (sums.numpy()[nz] / c[nz, None]).astype(np.float32)
        cen.copy_(torch.from_numpy(new))
