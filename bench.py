#!/usr/bin/env python
"""Benchmark of the IVF-PQ search hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference's own CPU path (oracle/_ref)

One "step" = one batch of queries through coarse -> LUT -> ADC scan -> exact rerank -> id map.
Workload (default "c4"): IVF-PQ, 100M x 96 fp32 base from a 65,536-component Gaussian mixture with Zipf(1.1)
populations, nlist 65,536, PQ M=48 x 8 bit, batch 10,000, nprobe 128, k 100, rerank top-1000 from host-resident
fp32 rows.  Data are synthetic and seeded (counter-based generators on the GPU); the inverted lists are the
mixture components (a row's list is its generating component), centroids are the component centres, and the
PQ codebook is trained on a 1M-row sample.

Prints ONE JSON line.  `value` is queries/s with the queries already in HBM; `e2e` is queries/s through
psb_session_search with host (pinned) queries and host outputs.  `roofline` describes the ADC scan kernel;
`cpu_baseline` is the reference's CPU path timed on a bounded sample of the same batch on this host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # benchmark configuration "IVF-PQ at scale" (the one the headline metric is quoted on)
    "c4": dict(n=100_000_000, dim=96, nlist=65536, M=48, sigma=0.25, zipf=1.1, nq=10000, nprobe=128, topk=100,
               n_rerank=1000, seed=3, desc="IVF-PQ 100Mx96 nlist=65536 M=48 nprobe=128 k=100 rerank=1000 batch=10000"),
    # the same index in residual ADC mode (codebook trained on, and codes encoding, row - centroid[list])
    "c4r": dict(n=100_000_000, dim=96, nlist=65536, M=48, sigma=0.25, zipf=1.1, nq=10000, nprobe=128, topk=100,
                n_rerank=1000, seed=3, residual=True,
                desc="IVF-ResidualPQ 100Mx96 nlist=65536 M=48 nprobe=128 k=100 rerank=1000 batch=10000"),
    # benchmark configuration "IVF-Flat fp32" (the reference's own CPU-runnable case): lists from 10 Lloyd iterations
    "c1": dict(n=100_000, dim=128, nlist=256, M=0, sigma=0.3, zipf=None, nq=1000, nprobe=16, topk=10, n_rerank=0, seed=0, iters=10,
               desc="IVF-Flat 100kx128 (256-component mixture, sigma 0.3) nlist=256 from 10 Lloyd iterations, 1,000 queries, nprobe=16 k=10, exact L2"),
    # benchmark configuration "IVF-PQ fp32 1M"
    "c2": dict(n=1_000_000, dim=128, nlist=1024, M=32, sigma=0.25, zipf=None, nq=10000, nprobe=32, topk=10,
               n_rerank=100, seed=1, desc="IVF-PQ 1Mx128 nlist=1024 M=32 nprobe=32 k=10 rerank=100 batch=10000"),
    # benchmark configuration "index training" (secondary line: k-means assignment on the tensor-core filter, PQ on residuals)
    "c5": dict(n=10_000_000, dim=128, nlist=65536, components=4096, M=32, sigma=0.3, zipf=None, nq=0, nprobe=1, topk=1, n_rerank=0,
               seed=4, iters=20, pq_iters=25,
               desc="training: 10M x 128 rows (4,096-component mixture, sigma 0.3) -> k-means to 65,536 centroids (20 Lloyd iterations), "
                    "PQ M=32 x 8 bit on residuals (25 iterations), encode"),
    # secondary line: the 1-bit sign codec (TurboQuant) - database encoding and candidate search over sign-coded lists
    "sign": dict(n=20_000_000, dim=128, nlist=8192, M=0, sigma=0.0, zipf=None, nq=10000, nprobe=32, topk=512, n_rerank=0, seed=6,
                 desc="1-bit sign codec: 20M x 128 u8 rows in 8,192 lists, 10,000 queries x 32 probes, 512 candidates, float states"),
    # benchmark configuration "coarse stage only" (secondary line: tensor-core roofline of the fused coarse GEMM)
    "c3": dict(n=65536, dim=96, nlist=65536, M=8, sigma=0.0, zipf=None, nq=100000, nprobe=64, topk=64, n_rerank=0, seed=2,
               desc="coarse only: 100,000 queries x 65,536 centroids, d=96, unit-mean-norm N(0,1), top-64"),
}


_OUT_FD = None


def claim_stdout():
    """Keeps a private handle on stdout for the one JSON line and points fd 1 at stderr, so that whatever libraries
    print to stdout (NCCL's version banner, for one) cannot end up beside it."""
    global _OUT_FD
    if _OUT_FD is None:
        sys.stdout.flush()
        _OUT_FD = os.dup(1)
        os.dup2(2, 1)
        os.environ["PSB_BENCH_OUT_FD"] = str(_OUT_FD)  # this file may also be imported as a module beside __main__


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    fd = _OUT_FD if _OUT_FD is not None else int(os.environ.get("PSB_BENCH_OUT_FD", "1"))
    os.write(fd, data)


def log(*a):
    if int(os.environ.get("RANK", "0")) == 0:
        print("[bench]", *a, file=sys.stderr, flush=True)


def populations(n, nlist, zipf):
    w = np.ones(nlist) if not zipf else 1.0 / np.arange(1, nlist + 1) ** zipf
    w = w / w.sum()
    counts = np.floor(w * n).astype(np.int64)
    rem = int(n - counts.sum())
    order = np.argsort(-(w * n - counts), kind="stable")
    counts[order[:rem]] += 1
    offsets = np.zeros(nlist + 1, np.int64)
    offsets[1:] = np.cumsum(counts)
    return w, offsets


def coprime_multiplier(n):
    a = 2654435761 % n
    from math import gcd
    while gcd(a, n) != 1:
        a += 1
    return a


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def build_index(cfg, torch, api, device, row_lo=0, row_hi=None, gt_queries=None, gt_k=0):
    """Generates rows [row_lo,row_hi) of the synthetic base on the GPU, trains the PQ codebook, encodes, and
    returns host arrays.  Optionally accumulates exact ground truth for gt_queries over the generated rows."""
    n, dim, nlist, M = cfg["n"], cfg["dim"], cfg["nlist"], cfg["M"]
    seed = cfg["seed"]
    row_hi = n if row_hi is None else row_hi
    t0 = time.time()
    w, offsets = populations(n, nlist, cfg["zipf"])
    d_off = torch.from_numpy(offsets).cuda()
    centres = torch.empty((nlist, dim), dtype=torch.float32, device="cuda")
    api.gen_normal(seed * 1000 + 1, 0, nlist * dim, 1.0, centres, device=device)
    # PQ training sample: 64 evenly spaced blocks of rows (the same on every rank)
    blocks, per = 64, min(16384, max(1, n // 64))
    residual = bool(cfg.get("residual"))

    def coded(rows_t, r0, m):
        """What the PQ codes encode: the row itself, or in residual mode row - centroid[list(row)]."""
        if not residual:
            return rows_t[:m]
        torch.cuda.synchronize()  # the generators run on the default stream, torch on its own
        lists = torch.searchsorted(d_off[1:], torch.arange(r0, r0 + m, device="cuda"), right=True)
        out = (rows_t[:m] - centres[lists]).contiguous()
        torch.cuda.synchronize()
        return out

    sample = torch.empty((blocks * per, dim), dtype=torch.float32, device="cuda")
    for b in range(blocks):
        r0 = (n // blocks) * b
        api.gen_mixture_rows(centres, d_off, nlist, dim, cfg["sigma"], seed * 1000 + 2, r0, per, sample[b * per:],
                             device=device)
        if residual:
            sample[b * per:(b + 1) * per] = coded(sample[b * per:(b + 1) * per], r0, per)
    codebook = torch.empty((M, 256, dim // M), dtype=torch.float32, device="cuda")
    api.pq_train(sample, blocks * per, dim, M, 256, 8, seed * 1000 + 3, codebook, device=device)
    del sample
    rows = row_hi - row_lo
    vectors = np.empty((rows, dim), np.float32)
    codes = np.empty((rows, M), np.uint8)
    chunk = 2_000_000
    buf = torch.empty((min(chunk, rows), dim), dtype=torch.float32, device="cuda")
    cbuf = torch.empty((min(chunk, rows), M), dtype=torch.uint8, device="cuda")
    gt_d = gt_i = None
    for r0 in range(row_lo, row_hi, chunk):
        m = min(chunk, row_hi - r0)
        api.gen_mixture_rows(centres, d_off, nlist, dim, cfg["sigma"], seed * 1000 + 2, r0, m, buf, device=device)
        api.pq_encode(coded(buf, r0, m), m, dim, codebook, M, 256, cbuf, device=device)
        if gt_queries is not None:
            k = min(gt_k, m)
            ti = torch.empty((gt_queries.shape[0], k), dtype=torch.int32, device="cuda")
            td = torch.empty((gt_queries.shape[0], k), dtype=torch.float32, device="cuda")
            api.knn_exact(gt_queries, gt_queries.shape[0], buf, m, dim, k, ti, td, device=device)
            torch.cuda.synchronize()  # library calls without a stream run on the default stream, torch on its own
            ti = ti.long() + r0
            if gt_d is None:
                gt_d, gt_i = td, ti
            else:
                cd, ci = torch.cat([gt_d, td], 1), torch.cat([gt_i, ti], 1)
                o = torch.argsort(cd, dim=1, stable=True)[:, :gt_k]
                gt_d, gt_i = torch.gather(cd, 1, o), torch.gather(ci, 1, o)
        torch.cuda.synchronize()
        torch.from_numpy(vectors[r0 - row_lo:r0 - row_lo + m]).copy_(buf[:m])
        torch.from_numpy(codes[r0 - row_lo:r0 - row_lo + m]).copy_(cbuf[:m])
    del buf, cbuf
    a = coprime_multiplier(n)
    ids = (np.arange(row_lo, row_hi, dtype=np.int64) * a + 12345) % n
    index = dict(centroids=centres.cpu().numpy(), offsets=offsets, reordered_ids=ids, codes=codes,
                 codebook=codebook.cpu().numpy(), vectors=vectors, nlist=nlist)
    log("index built in %.1fs (%d rows, %.1f GB vectors on the host)" % (time.time() - t0, rows, vectors.nbytes / 1e9))
    return index, w, centres, (gt_i.cpu().numpy() if gt_i is not None else None)


def make_queries(cfg, torch, api, centres, w, device):
    rng = np.random.default_rng(cfg["seed"] * 1000 + 7)
    comp = rng.choice(cfg["nlist"], size=cfg["nq"], p=w)
    noise = torch.empty((cfg["nq"], cfg["dim"]), dtype=torch.float32, device="cuda")
    api.gen_normal(cfg["seed"] * 1000 + 8, 0, cfg["nq"] * cfg["dim"], cfg["sigma"], noise, device=device)
    torch.cuda.synchronize()
    return (centres[torch.from_numpy(comp).cuda()] + noise).contiguous()


def measure_h2d_gbs(torch, mbytes=512, reps=3):
    """Host -> device copy bandwidth of one large pinned buffer: the ceiling of any transport of the exact rows."""
    host = torch.empty(mbytes << 20, dtype=torch.uint8).pin_memory()
    dev = torch.empty(mbytes << 20, dtype=torch.uint8, device="cuda")
    dev.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        dev.copy_(host, non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    return round(reps * (mbytes << 20) / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1)


def recall_at(got, truth, k):
    hit = 0
    for g, t in zip(got[:, :k], truth[:, :k]):
        hit += len(set(g.tolist()) & set(t.tolist()))
    return hit / float(truth.shape[0] * k)


def cpu_reference_run(index, q_host, cfg, nsample, threads):
    """The reference's CPU path (coarse loop + ivfpq_fine_cpu_lut + ivfpq_rerank_cpu + ivfpq_map_ids) on nsample queries."""
    import oracle
    q = np.ascontiguousarray(q_host[:nsample])
    t0 = time.time()
    residual = bool(cfg.get("residual"))
    if oracle.have_ref():
        probes, _ = oracle.ref_coarse(q, index["centroids"], cfg["nprobe"], threads=threads)
        if residual:  # cpu_fine_kernel_pq_resid_cpu_lut_timed: stage 1 + exact rerank, then the id map
            r = oracle.ref_ivfrespq_search(index, q, probes, cfg["topk"], cfg["n_rerank"], threads=threads)
        else:
            r = oracle.ref_ivfpq_search(index, q, probes, cfg["topk"], cfg["n_rerank"], fine_threads=threads,
                                        rerank_threads=threads)
        kind = "reference"
    else:
        search = oracle.ivfrespq_search if residual else oracle.ivfpq_search
        r = search(index, q, cfg["nprobe"], cfg["topk"], cfg["n_rerank"])
        kind = "port"
    dt = time.time() - t0
    return r, dt, kind


def scan_roofline(cfg, c, S, scan_ms, launches_per_step, peaks, clocks, sm_count, world):
    """Roofline object of the dominant kernel, the ADC scan.  S = (row, query) pairs one launch scores, all ranks together.

    Tensor-core pre-filter scan (k_scan_tc): a bf16 GEMM of visiting queries against decoded code rows, so the bound is the
    tensor pipe: algorithmic FLOPs = 2 * S * dim per launch (executed: tiles * 2 * 128 * 128 * padded K).  The figure the
    scan used to be reported by - S * M code bytes per launch over the HBM peak - is kept beside it: it is a LOGICAL byte
    count (every visit of a row counted), and since a decoded row now serves 128 visiting queries it exceeds what HBM
    could deliver; the physical DRAM traffic is `traffic`.
    SIMT scans (k_scan_h / k_scan): the HBM-logical figure is the roofline, as before."""
    hbm = float(peaks.get("hbm_gbs", 6650.0)) * world
    logical = S * cfg["M"] / (scan_ms * 1e-3) / 1e9 if scan_ms > 0 else 0.0
    src = "measured" if peaks else "fallback"
    tiles = c.get("tc_tiles", 0) / max(1, c["scan_kernel_launches"]) * world  # per launch, all ranks (counters are one rank's)
    if tiles > 0:
        dim = cfg["dim"]
        kp = (dim + 4 + 15) // 16 * 16
        peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1590.0))) * world
        flops = 2.0 * S * dim
        achieved = flops / (scan_ms * 1e-3) / 1e12 if scan_ms > 0 else 0.0
        # DRAM bytes per launch: each decoded code row is read once per tile of up to 128 visitors - M code bytes + 8 bytes of
        # per-row terms - plus the survivors written to the pools; 5,019 bytes per 128-row tile in the ncu capture of this workload
        # cut to 8M rows x 2,000 queries (profiles/k_scan_tc_M48_c4-8Mrows-2000q.md), scaled here by the tiles this launch issues
        return dict(bound="tensor", kernel="k_scan_tc", achieved=round(achieved, 1), peak=peak, unit="TFLOP/s",
                    frac=round(achieved / peak, 4), peak_source=src + " (cuBLAS bf16, sustained)",
                    algorithmic_flops_per_launch=flops, executed_flops_per_launch=tiles * 2.0 * 128 * 128 * kp,
                    pairs_per_launch=int(S), tiles_per_launch=int(tiles), ms_per_launch=round(scan_ms, 3),
                    launches_per_step=launches_per_step,
                    traffic=int(5019.0 * tiles) if cfg["M"] == 48 else None,
                    traffic_source="ncu dram__bytes_read+write of a cut-down capture (8M rows, 2,000 queries), scaled by rows decoded",
                    hbm_logical=dict(achieved=round(logical, 1), peak=hbm, unit="GB/s", frac=round(logical / hbm, 4),
                                     algorithmic_bytes_per_launch=int(S * cfg["M"]),
                                     note="S x M code bytes per launch: logical bytes, every visit of a row counted; above the HBM "
                                          "peak because a decoded row serves up to 128 visiting queries"))
    return dict(bound="hbm", kernel="k_scan_h", achieved=round(logical, 1), peak=hbm, unit="GB/s", frac=round(logical / hbm, 4),
                peak_source=src, algorithmic_bytes_per_launch=int(S * cfg["M"]), rows_per_launch=int(S),
                ms_per_launch=round(scan_ms, 3), launches_per_step=launches_per_step,
                traffic=int(2.62 * S) if cfg["M"] == 48 else None,
                traffic_source="ncu dram__bytes_read+write of a cut-down capture (8M rows, 2,000 queries), scaled by rows scanned",
                lookups_per_clk_per_sm=round(S * cfg["M"] / (scan_ms * 1e-3) / (sm_count * world) / ((clocks.get("sm_mhz") or 1965.0) * 1e6), 2))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the base size (scaled-down runs)")
    ap.add_argument("--queries", type=int, default=0, help="override the batch size")
    ap.add_argument("--cpu-sample", type=int, default=0, help="queries in the CPU baseline sample (0 = auto)")
    ap.add_argument("--exact-mode", default="auto", choices=["auto", "mapped", "staged", "cached", "hybrid"],
                    help="rerank transport on one GPU: staged = host threads gather rows into pinned rings and cudaMemcpyAsync moves "
                         "them (no SM time spent on the transfer), mapped = kernels gather mapped host rows over PCIe; "
                         "auto = hybrid when a batch gathers at least 2 GB (the scan is then long enough to run beside the transfer), else mapped; "
                         "cached = the session copies the rows into device memory once (not the host-resident configuration the "
                         "headline metric names: an extra data point); hybrid = staged and mapped at once, --zero-copy-pct of every "
                         "sub-batch through the kernel")
    ap.add_argument("--zero-copy-pct", type=int, default=0, help="hybrid transport: share of each sub-batch gathered by the kernel (0 = library default)")
    ap.add_argument("--reserve-sms", type=int, default=24, help="N > 1: SMs the scan's persistent grid leaves to the exchange half "
                    "(the PCIe gather of the exact rows runs on that many SMs of its own, the collectives beside it)")
    ap.add_argument("--parts", type=int, default=4, help="N > 1: sub-batches per batch")
    ap.add_argument("--native-group", action="store_true", help="N > 1: drive the sharded step through the C ABI's psb_group_* (NCCL "
                    "communicators of its own) instead of the torch.distributed orchestration of paraselect_b200.multi")
    ap.add_argument("--local-cutoffs", action="store_true", help="N > 1: every rank places its admission cutoffs on its own rows only "
                    "(default: on the rows of all ranks, from exchanged sample records)")
    ap.add_argument("--serial", action="store_true", help="N = 1: no sub-batches (one scan launch per batch, then the rerank)")
    ap.add_argument("--pipeline-parts", type=int, default=0, help="N = 1: sub-batches per batch (0 = library default)")
    ap.add_argument("--cut-plan", type=int, default=0, help="N = 1, staged transport: sub-batch cut plan (see psb_options.even_cuts)")
    ap.add_argument("--gather-ctas", type=int, default=0, help="CTAs of the PCIe gather kernel beside a scan (0 = library default)")
    ap.add_argument("--n1-reserve-sms", type=int, default=-1, help="N = 1: SMs the scan leaves to the gather kernel (-1 = auto)")
    args = ap.parse_args()
    claim_stdout()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0

    import torch
    from paraselect_b200 import api
    from paraselect_b200 import build as psb_build
    if rank == 0:
        psb_build.ensure_built()
    cfg = dict(WORKLOADS[args.workload])
    if args.rows:
        cfg["n"] = args.rows
        cfg["nlist"] = max(16, min(cfg["nlist"], args.rows // 256))
        cfg["nprobe"] = min(cfg["nprobe"], cfg["nlist"])
    if args.queries:
        cfg["nq"] = args.queries
    auto_mode = args.exact_mode == "auto"
    args.auto_mode = auto_mode
    if args.exact_mode == "auto":
        gathered = cfg["nq"] * max(cfg["n_rerank"], cfg["topk"]) * cfg["dim"] * 4
        args.exact_mode = "hybrid" if gathered >= 2e9 else "mapped"
    if not torch.cuda.is_available() or api.device_count() < 1:
        raise SystemExit("bench.py needs a B200: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = local_rank
    if world > 1 and args.impl == "ours":
        import torch.distributed as dist
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # NCCL's banner and warnings go to stderr: stdout is one JSON line
        dist.init_process_group("nccl")
    if args.impl == "ours" and world > 1 and args.workload in ("c3", "c5", "sign"):
        raise SystemExit("workloads c3, c5 and sign are single-GPU lines")
    if args.impl == "ours" and world > 1:
        return multi_gpu_main(args, cfg, rank, world, local_rank)

    if args.workload == "c1":
        if world > 1:
            raise SystemExit("workload c1 is a single-GPU line")
        return flat_search(args, cfg, torch, api, device)
    if args.workload == "c3":
        return coarse_only(args, cfg, torch, api, device)
    if args.workload == "c5":
        return training(args, cfg, torch, api, device)
    if args.workload == "sign":
        return sign_codec(args, cfg, torch, api, device)

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        gt_n = 64
        # queries need the centres: build a tiny first pass for them
        w, offsets = populations(cfg["n"], cfg["nlist"], cfg["zipf"])
        centres = torch.empty((cfg["nlist"], cfg["dim"]), dtype=torch.float32, device="cuda")
        api.gen_normal(cfg["seed"] * 1000 + 1, 0, cfg["nlist"] * cfg["dim"], 1.0, centres, device=device)
        dq = make_queries(cfg, torch, api, centres, w, device)
        torch.cuda.synchronize()
        index, w, centres, gt = build_index(cfg, torch, api, device, gt_queries=dq[:gt_n].contiguous(), gt_k=cfg["topk"])
        nq, dim, nprobe, topk, R = cfg["nq"], cfg["dim"], cfg["nprobe"], cfg["topk"], cfg["n_rerank"]
        q_pinned = torch.empty((nq, dim), dtype=torch.float32).pin_memory()
        q_pinned.copy_(dq)
        torch.cuda.synchronize()
        q_host = q_pinned.numpy()

        if args.impl == "reference":
            return reference_arm(args, cfg, index, q_host, gt)

        h2d_gbs = measure_h2d_gbs(torch)
        t0 = time.time()
        def make_session(mode):
            return api.Session(index, n_rerank=R, device=device, max_batch=nq, stream=stream.cuda_stream, time_kernels=True,
                               residual=bool(cfg.get("residual")), gather_ctas=args.gather_ctas, serial_pipeline=args.serial,
                               pipeline_parts=args.pipeline_parts, even_cuts=args.cut_plan,
                               reserve_sms=max(0, args.n1_reserve_sms), zero_copy_pct=args.zero_copy_pct,
                               exact_mode={"staged": api.EXACT_HOST_STAGED, "cached": api.EXACT_HOST_CACHED,
                                           "hybrid": api.EXACT_HOST_HYBRID}.get(mode, api.EXACT_HOST_MAPPED))
        try:
            sess = make_session(args.exact_mode)
        except api.PsbError as e:
            if not (auto_mode and args.exact_mode == "hybrid"):
                raise
            # a host that does not let 38 GB of rows be registered: the staged transport needs no registration
            log("hybrid transport unavailable (%s): falling back to the staged transport" % e)
            args.exact_mode = "staged"
            sess = make_session("staged")
        log("session created in %.1fs" % (time.time() - t0))
        stage1 = min(R, cfg["n"]) if R > topk else topk
        d_probes = torch.empty((nq, nprobe), dtype=torch.int32, device="cuda")
        d_lut = torch.empty((nq, cfg["M"], 256), dtype=torch.float32, device="cuda")
        d_cand = torch.empty((nq, stage1), dtype=torch.int32, device="cuda")
        d_cdist = torch.empty((nq, stage1), dtype=torch.float32, device="cuda")
        d_ccnt = torch.empty((nq,), dtype=torch.int32, device="cuda")
        d_rows = torch.empty((nq, topk), dtype=torch.int32, device="cuda")
        d_dist = torch.empty((nq, topk), dtype=torch.float32, device="cuda")
        d_ids = torch.empty((nq, topk), dtype=torch.int64, device="cuda")

        def device_step():
            # device-resident queries -> device-resident ids/distances (sub-batches overlap the PCIe rerank with the scan)
            sess.search_device(dq, nq, nprobe, topk, d_ids, d_dist, d_probes)

        for _ in range(max(args.warmup, 3)):
            device_step()
        torch.cuda.synchronize()
        sess.counters(reset=True)
        sampler = ClockSampler(local_rank)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            device_step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_dev = e0.elapsed_time(e1) / args.steps
        c = sess.counters(reset=True)
        dev_ids = d_ids.cpu().numpy()

        # end to end: host queries -> host results through psb_session_search
        out_ids = torch.empty((nq, topk), dtype=torch.int64).pin_memory()
        out_dist = torch.empty((nq, topk), dtype=torch.float32).pin_memory()
        st = api.Stats()
        for _ in range(2):
            sess.search_raw(q_pinned.data_ptr(), nq, nprobe, topk, nq, out_ids.data_ptr(), out_dist.data_ptr(), st)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            sess.search_raw(q_pinned.data_ptr(), nq, nprobe, topk, nq, out_ids.data_ptr(), out_dist.data_ptr(), st)
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
        stats = st.as_dict()
        e2e_ids = out_ids.numpy().copy()
        e2e_dist = out_dist.numpy().copy()
        assert np.array_equal(dev_ids, e2e_ids), "stage-level and end-to-end results differ"

    launches = int(c["kernel_launches"] - 0)
    launches_per_step = max(1, c["scan_kernel_launches"]) / max(1, args.steps)  # one per sub-batch
    scan_ms = c["scan_kernel_ms"] / max(1, c["scan_kernel_launches"])
    S = c["pq_scanned_codes"] / max(1, args.steps) / launches_per_step  # rows per launch
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    roofline = scan_roofline(cfg, c, S, scan_ms, launches_per_step, peaks, clocks,
                             torch.cuda.get_device_properties(device).multi_processor_count, 1)

    # CPU baseline + parity on a bounded sample of the same batch
    cores = os.cpu_count() or 1
    ns = args.cpu_sample or 16
    ref, dt, kind = cpu_reference_run(index, q_host, cfg, ns, cores)
    if not args.cpu_sample and dt < 6.0:
        ns2 = int(min(512, nq, max(ns, ns * 12.0 / max(dt, 1e-3))))
        if ns2 >= 2 * ns:
            ns = ns2
            ref, dt, kind = cpu_reference_run(index, q_host, cfg, ns, cores)
    ids_equal = bool(np.array_equal(ref["indices"], e2e_ids[:ns]))
    rel = float(np.max(np.abs(ref["distances"] - e2e_dist[:ns]) / np.maximum(np.abs(ref["distances"]), 1e-30)))
    gtn = min(gt.shape[0], ns) if gt is not None else 0
    gt_ids = index["reordered_ids"][gt] if gt is not None else None
    parity = dict(sample_queries=ns, ids_equal=ids_equal, max_rel_dist_err=rel,
                  recall_at_k_gpu=recall_at(e2e_ids[:gtn], gt_ids[:gtn], topk) if gtn else None,
                  recall_at_k_cpu=recall_at(ref["indices"][:gtn], gt_ids[:gtn], topk) if gtn else None,
                  recall_at_10_gpu=recall_at(e2e_ids[:gtn], gt_ids[:gtn], min(10, topk)) if gtn else None,
                  recall_at_10_cpu=recall_at(ref["indices"][:gtn], gt_ids[:gtn], min(10, topk)) if gtn else None)
    line = dict(
        metric="QPS (IVF-PQ search, recall@k equal to the reference CPU path)", value=round(nq / (ms_dev * 1e-3), 1),
        unit="queries/s", n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=round(ms_dev, 3),
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
        config=dict(workload=args.workload, desc=cfg["desc"], rows=cfg["n"], dim=dim, nlist=cfg["nlist"], M=cfg["M"],
                    batch=nq, nprobe=nprobe, topk=topk, n_rerank=R, exact_rows="host-%s fp32" % args.exact_mode,
                    l2="inputs larger than L2 (codes %.1f GB)" % (index["codes"].nbytes / 1e9)),
        e2e=dict(value=round(nq / (ms_e2e * 1e-3), 1), unit="queries/s", ms_per_step=round(ms_e2e, 3),
                 h2d_bytes_per_step=int(stats["h2d_bytes"]), d2h_bytes_per_step=int(stats["d2h_bytes"]),
                 pcie_gather_bytes_per_step=int(nq * stage1 * dim * 4) if R > topk else 0),
        gpu_launches=launches, roofline=roofline,
        # the exact rerank moves nq * n_rerank rows from host memory per batch: what the end-to-end step is bound by
        transport=dict(bytes_per_step=int(nq * stage1 * dim * 4) if R > topk else 0,
                       achieved_gbs=round(nq * stage1 * dim * 4 / max(1e-9, stats["pq_rerank_ms"] * 1e-3) / 1e9, 1) if R > topk and stats["pq_rerank_ms"] > 0 else None,
                       pinned_h2d_copy_gbs=h2d_gbs, note="achieved = gathered bytes / rerank stage time (random rows of dim * 4 bytes); "
                       "pinned_h2d_copy_gbs = one large pinned copy on this host, the link's ceiling"),
        cpu_baseline=dict(value=round(ns / dt, 2), unit="queries/s", cores=cores, kind=kind,
                          sample="first %d queries of the batch, all %d host threads" % (ns, cores)),
        stages_ms=dict(coarse=round(stats["coarse_search_ms"], 3), lut=round(stats["pq_lut_build_ms"], 3),
                       scan=round(stats["pq_adc_scan_ms"], 3), rerank=round(stats["pq_rerank_ms"], 3),
                       map_ids=round(stats["pq_map_ids_ms"], 3), h2d=round(stats["h2d_ms"], 3), d2h=round(stats["d2h_ms"], 3)),
        counters=dict(scanned_codes_per_step=int(S * launches_per_step), admitted_per_step=int(c["threshold_candidates"] / max(1, args.steps)),
                      fallback_queries_per_step=c["fallback_queries"] / max(1, args.steps),
                      prefilter_survivors_per_step=int(c["prefilter_survivors"] / max(1, args.steps)),
                      tc_tiles_per_step=int(c["tc_tiles"] / max(1, args.steps)),
                      staged_host_gather_gbs=round(c["staged_gather_bytes"] / max(1e-9, c["staged_gather_ms"] * 1e-3) / 1e9, 1) if c["staged_gather_ms"] > 0 else None,
                      tc_issuer_wait_cycles_per_tile=dict(item=round(c["tc_wait_item_cycles"] / max(1, c["tc_tiles"]), 1),
                                                          rows=round(c["tc_wait_rows_cycles"] / max(1, c["tc_tiles"]), 1),
                                                          accumulator=round(c["tc_wait_acc_cycles"] / max(1, c["tc_tiles"]), 1))),
        parity=parity,
        result_checksum=int(np.bitwise_xor.reduce((e2e_ids.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)).ravel())
                            & np.uint64((1 << 62) - 1)),
        clocks=clocks)
    emit(line)
    sess.close()
    return 0


def pin_to_gpu_numa_node(torch, local_rank):
    """Keeps this rank's threads - and so the pages of the host arrays it is about to fill - on the NUMA node its GPU hangs
    off, so that the PCIe gather of the exact rows does not cross the socket interconnect.  Silently does nothing where the
    topology cannot be read."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        dev = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % dev).read())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    return None


def multi_gpu_main(args, cfg, rank, world, local_rank):
    """`bench.py --gpus N` for N > 1 (one process per GPU under torchrun)."""
    import torch
    import torch.distributed as dist
    numa_node = pin_to_gpu_numa_node(torch, local_rank)
    from paraselect_b200 import api, multi
    from paraselect_b200.multi import ShardedSearch, SessionEngine, stripe_layout

    device = local_rank
    n, dim, nlist, M = cfg["n"], cfg["dim"], cfg["nlist"], cfg["M"]
    nq, nprobe, topk, R = cfg["nq"], cfg["nprobe"], cfg["topk"], cfg["n_rerank"]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        w, offsets = populations(n, nlist, cfg["zipf"])
        gb, loff = stripe_layout(offsets, rank, world)
        t0 = time.time()
        index, centres = build_stripe(cfg, torch, api, device, offsets, gb, loff)
        log("rank 0 stripe built in %.1fs (%d rows)" % (time.time() - t0, index["codes"].shape[0]))
        dq = make_queries(cfg, torch, api, centres, w, device)
        q_pinned = torch.empty((nq, dim), dtype=torch.float32).pin_memory()
        q_pinned.copy_(dq)
        torch.cuda.synchronize()
        # The exchange half of a sub-batch (collectives, PCIe rerank) runs beside the next sub-batch's scan.  A collective's
        # CTA cannot share an SM with a scan CTA, so the scan's persistent grid leaves a few SMs free for it.
        reserve = args.reserve_sms
        # Rerank transport per rank: the gather kernel over mapped host rows.  The hybrid transport (host cores beside the kernel)
        # can be asked for with --exact-mode hybrid; with the cores shared between the ranks and every candidate first to be
        # looked up in the stripe it measured slower (two ranks: 98.5 ms against 89-91.5 ms per batch).
        mode = getattr(args, "exact_mode", "auto")
        cores = os.cpu_count() or 16
        if mode == "cached":
            exact_mode, zc_pct = api.EXACT_HOST_CACHED, 0
        elif mode == "mapped" or getattr(args, "auto_mode", True):
            exact_mode, zc_pct = api.EXACT_HOST_MAPPED, 0
        else:
            exact_mode = api.EXACT_HOST_HYBRID
            zc_pct = args.zero_copy_pct or int(round(100 * 28.0 / (28.0 + 32.0 / world)))
        sess = api.Session(index, n_rerank=R, device=device, max_batch=nq, stream=stream.cuda_stream, time_kernels=True,
                           list_global_begin=gb, reserve_sms=reserve, exact_mode=exact_mode, zero_copy_pct=zc_pct,
                           host_threads=max(2, min(64, cores // world)))
        width = min(R, n) if R > topk else topk
        search = ShardedSearch(SessionEngine(sess, torch), dist, world, nq, dim, M, 256, nprobe, topk, width, torch,
                               rerank=R > topk, parts=args.parts if nq >= 2048 else 1, shared_cutoff=not args.local_cutoffs)
        group = None
        if args.native_group:
            nccl_path, comms, destroy_comms = multi.raw_nccl_comms(dist, torch, 2)
            group = api.Group(sess, comms[0], comms[1], nq, nprobe, topk, nccl_library=nccl_path, parts=args.parts if nq >= 2048 else 1,
                              shared_cutoff=not args.local_cutoffs)
            g_ids = torch.empty((nq, topk), dtype=torch.int64, device="cuda")
            g_dist = torch.empty((nq, topk), dtype=torch.float32, device="cuda")

            def group_step(q):
                group.search_device(q, nq, nprobe, topk, g_ids, g_dist)
                return g_ids, g_dist
        run_step = group_step if group is not None else search.step
        search.step(dq, profile=True)  # first step in one piece: every workspace reaches its final size before streams overlap
        for _ in range(max(args.warmup, 3)):
            run_step(dq)
        torch.cuda.synchronize()
        sess.counters(reset=True)
        sampler = ClockSampler(local_rank)
        sampler.start()

        def timed(fn):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(args.steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            dist.barrier()
            ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device="cuda")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        ms_dev = timed(lambda: run_step(dq))
        c = sess.counters(reset=True)
        out_ids = torch.empty((nq, topk), dtype=torch.int64).pin_memory()
        out_dist = torch.empty((nq, topk), dtype=torch.float32).pin_memory()
        dq2 = torch.empty_like(dq)

        def e2e_step():
            dq2.copy_(q_pinned, non_blocking=True)
            ids, dd = run_step(dq2)
            out_ids.copy_(ids, non_blocking=True)
            out_dist.copy_(dd, non_blocking=True)
            stream.synchronize()

        e2e_step()
        ms_e2e = timed(e2e_step)
        search.step(dq, profile=True)
        torch.cuda.synchronize()
        stage_ms = search.stage_times()
        search.step(dq, trace=True)   # one pipelined step with events around the halves of every sub-batch: shows what overlaps
        torch.cuda.synchronize()
        timeline = search.timeline()
        clocks = sampler.stop()
        torch.cuda.synchronize()
        # totals over ranks
        tot = torch.tensor([float(c["pq_scanned_codes"]), float(c["scan_kernel_ms"]), float(c["scan_kernel_launches"]),
                            float(c["kernel_launches"]), float(c["fallback_queries"]), float(c["tc_tiles"]), float(c["prefilter_survivors"])], dtype=torch.float64, device="cuda")
        mx = tot.clone()
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        torch.cuda.synchronize()  # the collectives run on this block's stream: finish them before the host reads
        tot, mx = tot.cpu(), mx.cpu()
        ids_np = out_ids.numpy()
        checksum = int(np.bitwise_xor.reduce((ids_np.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)).ravel()) & np.uint64((1 << 62) - 1))
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        S = tot[0].item() / max(1, args.steps)                      # rows scanned per step, all ranks
        launches_per_step = max(1.0, mx[2].item()) / max(1, args.steps)  # one scan launch per sub-batch
        scan_ms = mx[1].item() / max(1.0, mx[2].item())             # slowest rank's scan kernel, per launch
        S = S / launches_per_step                                   # rows per launch, all ranks
        c_tot = dict(c, tc_tiles=tot[5].item() / world, scan_kernel_launches=max(1.0, mx[2].item()))
        roofline = scan_roofline(cfg, c_tot, S, scan_ms, launches_per_step, peaks, clocks,
                                 torch.cuda.get_device_properties(device).multi_processor_count, world)
        roofline["note"] = "aggregate over ranks: all ranks' work / slowest rank's kernel time, against world x peak"
        line = dict(
            metric="QPS (IVF-PQ search, recall@k equal to the reference CPU path)", value=round(nq / (ms_dev * 1e-3), 1),
            unit="queries/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=round(ms_dev, 3),
            higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
            config=dict(workload=args.workload, desc=cfg["desc"], rows=n, dim=dim, nlist=nlist, M=M, batch=nq, nprobe=nprobe,
                        topk=topk, n_rerank=R, exact_rows={api.EXACT_HOST_CACHED: "device-cached fp32", api.EXACT_HOST_MAPPED: "host-mapped fp32",
                                    api.EXACT_HOST_HYBRID: "host fp32, hybrid transport (%d %% through the gather kernel)" % zc_pct}[exact_mode], sharding="lists of at least %d x 4,096 rows striped over the %d ranks, shorter ones whole on rank (list mod %d)" % (world, world, world),
                        l2="inputs larger than L2 (codes %.2f GB per rank)" % (index["codes"].nbytes / 1e9)),
            e2e=dict(value=round(nq / (ms_e2e * 1e-3), 1), unit="queries/s", ms_per_step=round(ms_e2e, 3),
                     h2d_bytes_per_step=int(nq * dim * 4), d2h_bytes_per_step=int(nq * topk * 12),
                     pcie_gather_bytes_per_step=int(nq * width * dim * 4) if R > topk else 0),
            gpu_launches=int(tot[3].item()),
            roofline=roofline,
            counters=dict(scanned_codes_per_step=int(S * launches_per_step), fallback_queries_per_step=tot[4].item() / max(1, args.steps),
                          prefilter_survivors_per_step=tot[6].item() / max(1, args.steps), shared_cutoffs=bool(search.shared),
                          batches_searched_again=int(group.searched_again() if group is not None else search.redone),
                          driver="psb_group (C ABI)" if group is not None else "multi.ShardedSearch (torch.distributed)"),
            stages_ms_rank0=stage_ms, pipeline_timeline_ms_rank0=timeline, host_numa_node_rank0=numa_node, result_checksum=checksum, clocks=clocks)
        emit(line)
    if group is not None:
        group.close()
        destroy_comms()
    sess.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


def build_stripe(cfg, torch, api, device, offsets, gb, loff):
    """Generates the whole synthetic base chunk by chunk on this rank's GPU and keeps the rows of its stripe."""
    n, dim, nlist, M, seed = cfg["n"], cfg["dim"], cfg["nlist"], cfg["M"], cfg["seed"]
    d_off = torch.from_numpy(offsets).cuda()
    centres = torch.empty((nlist, dim), dtype=torch.float32, device="cuda")
    api.gen_normal(seed * 1000 + 1, 0, nlist * dim, 1.0, centres, device=device)
    blocks, per = 64, min(16384, max(1, n // 64))
    sample = torch.empty((blocks * per, dim), dtype=torch.float32, device="cuda")
    for b in range(blocks):
        api.gen_mixture_rows(centres, d_off, nlist, dim, cfg["sigma"], seed * 1000 + 2, (n // blocks) * b, per,
                             sample[b * per:], device=device)
    codebook = torch.empty((M, 256, dim // M), dtype=torch.float32, device="cuda")
    api.pq_train(sample, blocks * per, dim, M, 256, 8, seed * 1000 + 3, codebook, device=device)
    del sample
    rows = int(loff[-1])
    vectors = np.empty((rows, dim), np.float32)
    codes = np.empty((rows, M), np.uint8)
    ids = np.empty(rows, np.int64)
    a = coprime_multiplier(n)
    d_gb = torch.from_numpy(gb).cuda()
    d_len = torch.from_numpy(loff[1:] - loff[:-1]).cuda()
    chunk = 2_000_000
    buf = torch.empty((chunk, dim), dtype=torch.float32, device="cuda")
    cbuf = torch.empty((chunk, M), dtype=torch.uint8, device="cuda")
    at = 0
    for r0 in range(0, n, chunk):
        m = min(chunk, n - r0)
        g = torch.arange(r0, r0 + m, dtype=torch.int64, device="cuda")
        l = torch.searchsorted(d_gb, g, right=True) - 1
        lc = l.clamp(min=0)
        own = (l >= 0) & (g < d_gb[lc] + d_len[lc])
        sel = torch.nonzero(own).squeeze(1)
        k = int(sel.numel())
        if k == 0:
            continue
        api.gen_mixture_rows(centres, d_off, nlist, dim, cfg["sigma"], seed * 1000 + 2, r0, m, buf, device=device)
        torch.cuda.synchronize()  # the generator runs on the default stream, torch on its own
        mine = buf[:m].index_select(0, sel)
        torch.cuda.synchronize()
        api.pq_encode(mine, k, dim, codebook, M, 256, cbuf, device=device)
        torch.cuda.synchronize()
        torch.from_numpy(vectors[at:at + k]).copy_(mine)
        torch.from_numpy(codes[at:at + k]).copy_(cbuf[:k])
        ids[at:at + k] = ((sel.cpu().numpy() + r0) * a + 12345) % n
        at += k
    assert at == rows, (at, rows)
    index = dict(centroids=centres.cpu().numpy(), offsets=loff, reordered_ids=ids, codes=codes,
                 codebook=codebook.cpu().numpy(), vectors=vectors, nlist=nlist)
    return index, centres




def flat_search(args, cfg, torch, api, device):
    """Workload c1: IVF-Flat.  The reference's own CPU-runnable configuration; the library runs it with the rows resident in
    device memory.  A step = the batch of 1,000 queries through coarse -> exact fine scan -> id map."""
    import oracle
    n, dim, nlist, nq, nprobe, topk = cfg["n"], cfg["dim"], cfg["nlist"], cfg["nq"], cfg["nprobe"], cfg["topk"]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        w, offsets = populations(n, nlist, None)
        d_off = torch.from_numpy(offsets).cuda()
        centres = torch.empty((nlist, dim), dtype=torch.float32, device="cuda")
        api.gen_normal(cfg["seed"] * 1000 + 1, 0, nlist * dim, 1.0, centres, device=device, stream=st)
        x = torch.empty((n, dim), dtype=torch.float32, device="cuda")
        api.gen_mixture_rows(centres, d_off, nlist, dim, cfg["sigma"], cfg["seed"] * 1000 + 2, 0, n, x, device=device, stream=st)
        torch.cuda.synchronize()
        dq = make_queries(cfg, torch, api, centres, w, device)
        # the index: 10 Lloyd iterations from a seeded sample of rows (k-means on the GPU), rows reordered by list
        g = torch.Generator(device="cuda"); g.manual_seed(cfg["seed"])
        cen = x[torch.randperm(n, device="cuda", generator=g)[:nlist]].clone()
        assign = torch.empty((n,), dtype=torch.int32, device="cuda")
        api.kmeans_train(x, n, dim, cen, nlist, cfg["iters"], assign, device=device, stream=st)
        torch.cuda.synchronize()
        order = torch.argsort(assign.long(), stable=True)
        counts = torch.bincount(assign.long(), minlength=nlist).cpu().numpy()
        loff = np.zeros(nlist + 1, np.int64); loff[1:] = np.cumsum(counts)
        index = dict(centroids=cen.cpu().numpy(), offsets=loff, reordered_ids=order.cpu().numpy().astype(np.int64),
                     vectors=x[order].cpu().numpy())
        q_host = dq.cpu().numpy()
        cores = os.cpu_count() or 1

        def cpu_run(qs):
            t0 = time.time()
            if oracle.have_ref_train():
                r = oracle.ref_cpu_ivf_search(index["centroids"], index["offsets"], index["reordered_ids"], index["vectors"], qs, nprobe, topk)[:2]
                kind = "reference"
            else:
                r = oracle.ivfflat_search(index["centroids"], index["offsets"], index["reordered_ids"], index["vectors"], qs, nprobe, topk)
                kind = "port"
            return r, time.time() - t0, kind

        if args.impl == "reference":
            times = []
            for i in range(args.warmup + args.steps):
                _, dt, kind = cpu_run(q_host)   # the whole batch: this is the reference's own CPU-runnable case
                if i >= args.warmup:
                    times.append(dt)
            ms = 1e3 * float(np.mean(times))
            v = round(nq / (ms * 1e-3), 2)
            emit(dict(impl="reference", metric="QPS (IVF-Flat search, exact L2)", value=v, unit="queries/s", n_gpus=args.gpus,
                      steps=args.steps, warmup=args.warmup, ms_per_step=round(ms, 3), higher_is_better=True, scaling="strong",
                      vs_baseline=None, dtype="f32", data="synthetic", config=dict(workload="c1", desc=cfg["desc"]),
                      cpu_baseline=dict(value=v, unit="queries/s", cores=cores, kind=kind,
                                        sample="all %d queries per step (cpu_ivf_search on the physical cores)" % nq),
                      e2e=dict(value=v, unit="queries/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)))
            return 0
        sess = api.FlatSession(index, device=device, max_batch=nq, stream=st, time_kernels=True)
        d_ids = torch.empty((nq, topk), dtype=torch.int64, device="cuda")
        d_dist = torch.empty((nq, topk), dtype=torch.float32, device="cuda")
        reps = 20  # a step is short: time `reps` batches per step so the clock sampler sees the load
        for _ in range(max(args.warmup, 3)):
            sess.search_device(dq, nq, nprobe, topk, d_ids, d_dist)
        torch.cuda.synchronize()
        sess.counters(reset=True)
        sampler = ClockSampler(device)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps * reps):
            sess.search_device(dq, nq, nprobe, topk, d_ids, d_dist)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (args.steps * reps)
        c = sess.counters(reset=True)
        qp = torch.empty((nq, dim), dtype=torch.float32).pin_memory(); qp.copy_(dq)
        oi = torch.empty((nq, topk), dtype=torch.int64).pin_memory()
        od = torch.empty((nq, topk), dtype=torch.float32).pin_memory()
        stt = api.Stats()
        sess.search_raw(qp.data_ptr(), nq, nprobe, topk, nq, oi.data_ptr(), od.data_ptr(), stt)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps * reps):
            sess.search_raw(qp.data_ptr(), nq, nprobe, topk, nq, oi.data_ptr(), od.data_ptr(), stt)
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / (args.steps * reps)
        clocks = sampler.stop()
        stats = stt.as_dict()
        got_i, got_d = oi.numpy().copy(), od.numpy().copy()
        # exact ground truth for recall
        gi = torch.empty((nq, topk), dtype=torch.int32, device="cuda")
        gd = torch.empty((nq, topk), dtype=torch.float32, device="cuda")
        api.knn_exact(dq, nq, x, n, dim, topk, gi, gd, device=device, stream=st)
        torch.cuda.synchronize()
        truth = gi.cpu().numpy().astype(np.int64)
    (ri, rd), dt, kind = cpu_run(q_host)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    rows_per_launch = c["pq_scanned_codes"] / max(1, c["scan_kernel_launches"])
    scan_ms = c["scan_kernel_ms"] / max(1, c["scan_kernel_launches"])
    achieved = rows_per_launch * dim * 4 / (scan_ms * 1e-3) / 1e9 if scan_ms > 0 else 0.0
    emit(dict(metric="QPS (IVF-Flat search, exact L2)", value=round(nq / (ms * 1e-3), 1), unit="queries/s", n_gpus=1, steps=args.steps,
              warmup=max(args.warmup, 3), ms_per_step=round(ms, 4), higher_is_better=True, scaling="strong", vs_baseline=None,
              dtype="f32", data="synthetic",
              config=dict(workload="c1", desc=cfg["desc"], batches_per_step=reps,
                          l2="rows 51 MB: resident in L2 after the first batch (the configuration is the reference's CPU-sized case)"),
              e2e=dict(value=round(nq / (ms_e2e * 1e-3), 1), unit="queries/s", ms_per_step=round(ms_e2e, 4),
                       h2d_bytes_per_step=int(stats["h2d_bytes"]), d2h_bytes_per_step=int(stats["d2h_bytes"])),
              gpu_launches=int(c["kernel_launches"]),
              roofline=dict(bound="hbm", kernel="k_flat_scan_direct", achieved=round(achieved, 1), peak=peak, unit="GB/s",
                            frac=round(achieved / peak, 4), peak_source="measured" if peaks else "fallback",
                            algorithmic_bytes_per_launch=int(rows_per_launch * dim * 4), rows_per_launch=int(rows_per_launch),
                            ms_per_launch=round(scan_ms, 4), traffic=None,
                            note="bytes = probed rows x dim x 4; at this size the rows stay in L2, so the figure is an L2-fed rate"),
              cpu_baseline=dict(value=round(nq / dt, 2), unit="queries/s", cores=cores, kind=kind,
                                sample="all %d queries, cpu_ivf_search on the physical cores" % nq),
              parity=dict(sample_queries=nq, ids_equal=bool(np.array_equal(ri, got_i)), dist_equal=bool(np.array_equal(rd, got_d)),
                          recall_at_k_gpu=recall_at(got_i, truth, topk),
                          recall_at_k_cpu=recall_at(ri, truth, topk)),
              clocks=clocks))
    sess.close()
    return 0


def training(args, cfg, torch, api, device):
    """Secondary workload: index training.  A step = one Lloyd iteration (assignment of every row to its nearest of k
    centroids + centroid update); then PQ codebook training on the residuals and encoding of all rows, each timed once."""
    import oracle
    n, dim, k, comps, M = cfg["n"], cfg["dim"], cfg["nlist"], cfg["components"], cfg["M"]
    steps, warm = args.steps, max(args.warmup, 1)
    if args.impl == "reference":
        # the reference's assignment arithmetic (restated: the reference's k-means needs its CUDA build) on the host cores,
        # a bounded sample of rows per step against all k centroids
        rng = np.random.default_rng(cfg["seed"])
        ns = args.cpu_sample or 4096
        cen_h = rng.standard_normal((k, dim)).astype(np.float32)
        times = []
        for i in range(args.warmup + steps):
            rows = rng.standard_normal((ns, dim)).astype(np.float32)
            t0 = time.time()
            oracle.kmeans_assign(rows, cen_h)
            if i >= args.warmup:
                times.append(time.time() - t0)
        v = round(ns / float(np.mean(times)), 1)
        cores = os.cpu_count() or 1
        emit(dict(impl="reference", metric="k-means rows/s per Lloyd iteration (k = %d)" % k, value=v, unit="rows/s",
                  n_gpus=args.gpus, steps=steps, warmup=args.warmup, ms_per_step=round(1e3 * float(np.mean(times)), 3),
                  higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                  config=dict(workload="c5", desc=cfg["desc"]),
                  cpu_baseline=dict(value=v, unit="rows/s", cores=cores, kind="port",
                                    sample="assignment of %d rows per step against all %d centroids, all %d host threads" % (ns, k, cores)),
                  e2e=dict(value=v, unit="rows/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)))
        return 0
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        _, offsets = populations(n, comps, None)
        d_off = torch.from_numpy(offsets).cuda()
        centres = torch.empty((comps, dim), dtype=torch.float32, device="cuda")
        api.gen_normal(cfg["seed"] * 1000 + 1, 0, comps * dim, 1.0, centres, device=device, stream=st)
        x = torch.empty((n, dim), dtype=torch.float32, device="cuda")
        api.gen_mixture_rows(centres, d_off, comps, dim, cfg["sigma"], cfg["seed"] * 1000 + 2, 0, n, x, device=device, stream=st)
        g = torch.Generator(device="cuda"); g.manual_seed(cfg["seed"])
        init = x[torch.randperm(n, device="cuda", generator=g)[:k]].clone()  # seeded sampling without replacement
        assign = torch.empty((n,), dtype=torch.int32, device="cuda")
        cen = init.clone()
        api.kmeans_train(x, n, dim, cen, k, warm - 1, assign, device=device, stream=st)  # warm-up passes
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        # A step = one Lloyd iteration in steady state.  The first assignment of a training has no previous assignment to take
        # its bounds from and runs the filter GEMM twice; every later one runs it once.  Timed: a training of 1 + steps
        # assignments and one of 1 + 2 * steps; their difference is `steps` steady-state iterations, and what the shorter one
        # took beyond its steady-state iterations is the first one.
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed_training(iterations):
            cen.copy_(init)
            e0.record(stream)
            out = api.kmeans_train(x, n, dim, cen, k, iterations, assign, device=device, stream=st)
            e1.record(stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), out
        # each training twice, the faster one counts: the host thread that drives the launches shares its cores with other jobs
        ms_long = min(timed_training(2 * steps)[0] for _ in range(2))
        ms_short, obj = min((timed_training(steps) for _ in range(2)), key=lambda t: t[0])  # 1 + `steps` assignment passes
        ms = (ms_long - ms_short) / steps
        ms_first = ms_short - steps * ms
        clocks = sampler.stop()
        # end to end: host rows in, host centroids + assignment out
        xh = torch.empty((n, dim), dtype=torch.float32).pin_memory()
        xh.copy_(x)
        ch = torch.empty((k, dim), dtype=torch.float32).pin_memory()
        ah = torch.empty((n,), dtype=torch.int32).pin_memory()
        torch.cuda.synchronize()
        e0.record(stream)
        x.copy_(xh, non_blocking=True)
        cen.copy_(init)
        api.kmeans_train(x, n, dim, cen, k, steps, assign, device=device, stream=st)
        ch.copy_(cen, non_blocking=True); ah.copy_(assign, non_blocking=True)
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = (e0.elapsed_time(e1) - ms_first) / steps   # the same training from host rows to host centroids and assignment
        # PQ on the residuals x - centroid[assign], then encoding
        t0 = time.time()
        api.residual_rows(x, n, dim, cen, assign, x, device=device, stream=st)  # in place
        codebook = torch.empty((M, 256, dim // M), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        t1 = time.time()
        api.pq_train(x, n, dim, M, 256, cfg["pq_iters"], cfg["seed"] * 1000 + 3, codebook, device=device, stream=st)
        torch.cuda.synchronize()
        t2 = time.time()
        codes = torch.empty((n, M), dtype=torch.uint8, device="cuda")
        api.pq_encode(x, n, dim, codebook, M, 256, codes, device=device, stream=st)
        torch.cuda.synchronize()
        t3 = time.time()
        # CPU baseline + parity: one assignment pass of the reference arithmetic on a bounded sample of rows
        ns = args.cpu_sample or 4096
        rows = (x[:ns] + cen[assign[:ns].long()]).cpu().numpy()  # the sample's original rows
        cen_h = cen.cpu().numpy()
        c0 = time.time()
        oa, od = oracle.kmeans_assign(rows, cen_h)
        cdt = time.time() - c0
        x[:ns] += cen[assign[:ns].long()]
        chk = torch.empty((ns,), dtype=torch.int32, device="cuda")
        api.kmeans_train(x[:ns].contiguous(), ns, dim, cen.clone(), k, 0, chk, device=device, stream=st)
        torch.cuda.synchronize()
        assign_equal = bool(np.array_equal(chk.cpu().numpy(), oa))
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1590.0)))
    flops = 2.0 * n * k * dim
    cores = os.cpu_count() or 1
    line = dict(metric="k-means rows/s per Lloyd iteration (k = %d)" % k, value=round(n / (ms * 1e-3), 1), unit="rows/s", n_gpus=1,
                steps=steps, warmup=warm, ms_per_step=round(ms, 3), higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="bf16 filter + f32 exact", data="synthetic",
                config=dict(workload="c5", desc=cfg["desc"], l2="rows 5.1 GB, far above L2"),
                e2e=dict(value=round(n / (ms_e2e * 1e-3), 1), unit="rows/s", ms_per_step=round(ms_e2e, 3),
                         h2d_bytes_per_step=int(n * dim * 4 / steps), d2h_bytes_per_step=int((k * dim * 4 + n * 4) / steps)),
                gpu_launches=steps * (-(-n // 262144) * 5 + 5),  # per pass and chunk: row prep, bound, filter pass, refinement, fallback; then count, offsets, fill, sums, update
                first_iteration_ms=round(ms_first, 3),
                roofline=dict(bound="tensor", kernel="k_coarse_tc (assignment: one filter pass bounded by the previous assignment + exact refinement)",
                              achieved=round(flops / (ms * 1e-3) / 1e12, 1), peak=peak, unit="TFLOP/s",
                              frac=round(flops / (ms * 1e-3) / 1e12 / peak, 4), peak_source="measured (sustained)" if peaks else "fallback",
                              algorithmic_flops_per_step=flops, traffic=None,
                              note="whole steady-state Lloyd iteration (row preparation, bound, filter GEMM, refinement, accumulation, update) "
                                   "against one algorithmic 2nkd; the first iteration of a training runs the filter twice (first_iteration_ms)"),
                cpu_baseline=dict(value=round(ns / cdt, 1), unit="rows/s", cores=cores, kind="port",
                                  sample="one assignment pass of %d rows against all %d centroids" % (ns, k)),
                objective=[float(v) for v in obj], pq_train_s=round(t2 - t1, 3), pq_encode_s=round(t3 - t2, 3),
                residual_s=round(t1 - t0, 3), total_training_estimate_s=round((ms_first + ms * cfg["iters"]) * 1e-3 + (t3 - t0), 2),
                parity=dict(sample_rows=ns, assign_equal=assign_equal), clocks=clocks)
    emit(line)
    return 0


def sign_codec(args, cfg, torch, api, device):
    """Secondary workload: the 1-bit sign codec.  A step = query states + candidate search for one batch of queries over
    sign-coded lists (probes given); the database encoding is timed once.  Rows, centroids and queries are uniform / normal
    noise: the scan's work does not depend on the values."""
    import oracle
    n, dim, nlist, nq, nprobe, k = cfg["n"], cfg["dim"], cfg["nlist"], cfg["nq"], cfg["nprobe"], cfg["topk"]
    padded = api.sign_padded_dim(dim) if args.impl == "ours" else oracle.sign_padded_dim(dim)
    words = padded // 32
    rng = np.random.default_rng(cfg["seed"])
    sizes = rng.multinomial(n, rng.dirichlet(np.full(nlist, 3.0)))
    off_h = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    cen_h = (rng.standard_normal((nlist, dim)) * 20 + 100).astype(np.float32)
    q_h = (rng.standard_normal((nq, dim)) * 20 + 100).astype(np.float32)
    probes_h = np.stack([rng.permutation(nlist)[:nprobe] for _ in range(min(nq, 256))])
    probes_h = np.tile(probes_h, ((nq + probes_h.shape[0] - 1) // probes_h.shape[0], 1))[:nq].astype(np.int32)
    visits = int(sizes[probes_h].sum())
    cores = os.cpu_count() or 1

    def cpu_sample(ns, seed_rows=200_000):
        """The restatement on a bounded sample: ns queries against an index of the first lists holding ~seed_rows rows."""
        nl = max(nprobe, int(np.searchsorted(off_h, seed_rows)))
        rows = rng.integers(0, 256, (int(off_h[nl]), dim)).astype(np.uint8)
        codes, scales = oracle.sign_encode_database(rows, cen_h[:nl], off_h[:nl + 1], padded)
        pr = np.stack([rng.permutation(nl)[:nprobe] for _ in range(ns)]).astype(np.int32)
        t0 = time.time()
        st, nsq, _, _ = oracle.sign_encode_queries(q_h[:ns], cen_h[:nl], pr, padded)
        oracle.sign_candidates(0, codes, scales, off_h[:nl + 1], pr, k, states=st, norm_sq=nsq)
        dt = time.time() - t0
        v = int(np.diff(off_h[:nl + 1])[pr].sum())
        return ns / dt, v / dt, "%d queries x %d probes over %d rows, all %d host threads" % (ns, nprobe, rows.shape[0], cores)

    if args.impl == "reference":
        # the reference's scan is a GPU kernel: the restatement of its arithmetic on the host cores, a bounded sample per step
        times, vals = [], []
        for i in range(args.warmup + args.steps):
            qps, vps, sample = cpu_sample(args.cpu_sample or 64)
            if i >= args.warmup:
                times.append(1.0 / qps); vals.append(qps)
        v = round(float(np.mean(vals)), 2)
        emit(dict(impl="reference", metric="sign-codec candidate search queries/s", value=v, unit="queries/s", n_gpus=args.gpus,
                  steps=args.steps, warmup=args.warmup, ms_per_step=round(1e3 * (args.cpu_sample or 64) / v, 3), higher_is_better=True,
                  scaling="strong", vs_baseline=None, dtype="f32", data="synthetic", config=dict(workload="sign", desc=cfg["desc"]),
                  cpu_baseline=dict(value=v, unit="queries/s", cores=cores, kind="port", sample=sample),
                  e2e=dict(value=v, unit="queries/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)))
        return 0

    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    with torch.cuda.stream(stream):
        off = torch.from_numpy(off_h).cuda(); cen = torch.from_numpy(cen_h).cuda()
        codes = torch.empty((n, words), dtype=torch.int32, device="cuda")
        scales = torch.empty(n, dtype=torch.float32, device="cuda")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        enc_ms = []
        chunk = 4_000_000   # the corpus passes through the device in chunks, as a host-resident one would
        gen = torch.Generator(device="cuda"); gen.manual_seed(cfg["seed"])
        for start in range(0, n, chunk):
            m = min(chunk, n - start)
            rows = torch.randint(0, 256, (m, dim), dtype=torch.uint8, device="cuda", generator=gen)
            stream.synchronize()
            e0.record(stream)
            api.sign_encode_database(rows, 1, m, cen, off, nlist, dim, padded, codes, scales, row_offset=start, device=device, stream=sp)
            e1.record(stream)
            stream.synchronize()
            enc_ms.append(e0.elapsed_time(e1))
            if start == 0:   # the first chunk against the restatement, bit for bit
                ns = 4096
                scale = api.sign_rotation_scale(padded, device=device)
                wc, ws = oracle.sign_encode_database(rows[:ns].cpu().numpy(), cen_h, off_h, padded, scale=scale)
                enc_equal = bool(np.array_equal(codes[:ns].cpu().numpy().view(np.uint32), wc[:ns]) and
                                 np.array_equal(scales[:ns].cpu().numpy().view(np.uint32), ws[:ns].view(np.uint32)))
            del rows
        q = torch.from_numpy(q_h).cuda(); probes = torch.from_numpy(probes_h).cuda()
        st = torch.empty((nq * nprobe, padded), dtype=torch.float32, device="cuda")
        nsq = torch.empty(nq * nprobe, dtype=torch.float32, device="cuda")
        out_r = torch.empty((nq, k), dtype=torch.int32, device="cuda")
        out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda")

        def step():
            api.sign_encode_queries(q, cen, probes, nq, nprobe, nlist, dim, padded, d_states=st, d_norm_sq=nsq, device=device, stream=sp)
            api.sign_search_candidates(api.SIGN_FLOAT_STATES, codes, scales, off, nlist, probes, nq, nprobe, padded, k, out_r, out_d,
                                       d_states=st, d_norm_sq=nsq, device=device, stream=sp)
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        # the scan alone
        e0.record(stream)
        for _ in range(args.steps):
            api.sign_search_candidates(api.SIGN_FLOAT_STATES, codes, scales, off, nlist, probes, nq, nprobe, padded, k, out_r, out_d,
                                       d_states=st, d_norm_sq=nsq, device=device, stream=sp)
        e1.record(stream)
        stream.synchronize()
        scan_ms = e0.elapsed_time(e1) / args.steps
        # end to end: host queries and probe ids in, host candidate rows out
        qp = torch.empty((nq, dim), dtype=torch.float32).pin_memory(); qp.copy_(q)
        pp = torch.empty((nq, nprobe), dtype=torch.int32).pin_memory(); pp.copy_(probes)
        oi = torch.empty((nq, k), dtype=torch.int32).pin_memory()
        q2 = torch.empty_like(q); p2 = torch.empty_like(probes)

        def e2e_step():
            q2.copy_(qp, non_blocking=True); p2.copy_(pp, non_blocking=True)
            api.sign_encode_queries(q2, cen, p2, nq, nprobe, nlist, dim, padded, d_states=st, d_norm_sq=nsq, device=device, stream=sp)
            api.sign_search_candidates(api.SIGN_FLOAT_STATES, codes, scales, off, nlist, p2, nq, nprobe, padded, k, out_r, None,
                                       d_states=st, d_norm_sq=nsq, device=device, stream=sp)
            oi.copy_(out_r, non_blocking=True)
            stream.synchronize()
        e2e_step()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        stream.synchronize()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
        # parity on a sample of queries: codes and scales of the whole index from the device, candidates from the restatement
        ns = args.cpu_sample or 8
        scale = api.sign_rotation_scale(padded, device=device)
        codes_h = codes.cpu().numpy().view(np.uint32); scales_h = scales.cpu().numpy()
        w_st, w_nsq, _, _ = oracle.sign_encode_queries(q_h[:ns], cen_h, probes_h[:ns], padded, scale=scale)
        w_rows, w_dist = oracle.sign_candidates(0, codes_h, scales_h, off_h, probes_h[:ns], k, states=w_st, norm_sq=w_nsq)
        got_r, got_d = out_r[:ns].cpu().numpy(), out_d[:ns].cpu().numpy()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    qps_cpu, vps_cpu, sample = cpu_sample(256)
    bytes_per_launch = visits * (words * 4 + 4)
    achieved = bytes_per_launch / (scan_ms * 1e-3) / 1e9
    emit(dict(metric="sign-codec candidate search queries/s", value=round(nq / (ms * 1e-3), 1), unit="queries/s", n_gpus=1,
              steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=round(ms, 3), higher_is_better=True, scaling="strong",
              vs_baseline=None, dtype="f32 chains over 1-bit codes", data="synthetic",
              config=dict(workload="sign", desc=cfg["desc"], rows=n, queries=nq, row_visits_per_step=visits,
                          l2="codes + scales %.0f MB, larger than L2" % (n * (words * 4 + 4) / 1e6)),
              e2e=dict(value=round(nq / (ms_e2e * 1e-3), 1), unit="queries/s", ms_per_step=round(ms_e2e, 3),
                       h2d_bytes_per_step=nq * dim * 4 + nq * nprobe * 4, d2h_bytes_per_step=nq * k * 4),
              gpu_launches=2 * args.steps,
              roofline=dict(bound="hbm", kernel="k_sign_scan<4,0>", achieved=round(achieved, 1), peak=peak, unit="GB/s",
                            frac=round(achieved / peak, 4), peak_source="measured" if peaks else "fallback",
                            ms_per_launch=round(scan_ms, 3), algorithmic_bytes_per_launch=bytes_per_launch,
                            bytes_per_row_visit=words * 4 + 4, row_visits_per_s=round(visits / (scan_ms * 1e-3), 1), traffic=None,
                            note="instruction-issue bound, not memory bound: see profiles/"),
              encode=dict(rows=n, ms=round(float(np.sum(enc_ms)), 3), rows_per_s=round(n / (float(np.sum(enc_ms)) * 1e-3), 1),
                          gbs=round(n * (dim + words * 4 + 4) / (float(np.sum(enc_ms)) * 1e-3) / 1e9, 1), equal_to_checker=enc_equal),
              cpu_baseline=dict(value=round(qps_cpu, 2), unit="queries/s", cores=cores, kind="port", sample=sample,
                                row_visits_per_s=round(vps_cpu, 1)),
              parity=dict(sample_queries=ns, rows_equal=bool(np.array_equal(got_r, w_rows)),
                          scores_equal=bool(np.array_equal(got_d.view(np.uint32), w_dist.view(np.uint32)))),
              clocks=clocks))
    return 0


def coarse_only(args, cfg, torch, api, device):
    """Secondary workload: the coarse stage alone (queries x centroids squared L2 with per-query top-64)."""
    import oracle
    nq, nlist, dim, k = cfg["nq"], cfg["nlist"], cfg["dim"], cfg["nprobe"]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        c = torch.empty((nlist, dim), dtype=torch.float32, device="cuda")
        q = torch.empty((nq, dim), dtype=torch.float32, device="cuda")
        api.gen_normal(cfg["seed"] * 1000 + 1, 0, nlist * dim, 1.0, c, device=device)
        api.gen_normal(cfg["seed"] * 1000 + 2, 0, nq * dim, 1.0, q, device=device)
        torch.cuda.synchronize()  # the generators run on the default stream, torch on its own
        c /= c.norm(dim=1).mean()
        q /= q.norm(dim=1).mean()
        torch.cuda.synchronize()
        # a carrier index: one row per list, so that a session (which owns the coarse stage) can be created
        index = dict(centroids=c.cpu().numpy(), offsets=np.arange(nlist + 1, dtype=np.int64),
                     reordered_ids=np.arange(nlist, dtype=np.int64), codes=np.zeros((nlist, 8), np.uint8),
                     codebook=np.zeros((8, 256, dim // 8), np.float32), vectors=None, nlist=nlist)
        q_host = q.cpu().numpy()
        if args.impl == "reference":
            cores = os.cpu_count() or 1
            ns = args.cpu_sample or 256
            times = []
            for i in range(args.warmup + args.steps):
                t0 = time.time()
                if oracle.have_ref():
                    oracle.ref_coarse(q_host[i * ns:(i + 1) * ns], index["centroids"], k, threads=cores); kind = "reference"
                else:
                    oracle.coarse(q_host[i * ns:(i + 1) * ns], index["centroids"], k); kind = "port"
                if i >= args.warmup:
                    times.append(time.time() - t0)
            v = round(ns / float(np.mean(times)), 2)
            emit(dict(impl="reference", metric="coarse queries/s (top-64 of 65,536 centroids)", value=v,
                                  unit="queries/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                                  ms_per_step=round(1e3 * float(np.mean(times)), 3), higher_is_better=True, scaling="strong",
                                  vs_baseline=None, dtype="f32", data="synthetic", config=dict(workload="c3", desc=cfg["desc"]),
                                  cpu_baseline=dict(value=v, unit="queries/s", cores=cores, kind=kind,
                                                    sample="%d queries per step, all %d host threads" % (ns, cores)),
                                  e2e=dict(value=v, unit="queries/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)))
            return 0
        sess = api.Session(index, device=device, max_batch=nq, stream=stream.cuda_stream, time_kernels=True)
        ids = torch.empty((nq, k), dtype=torch.int32, device="cuda")
        dist = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        for _ in range(max(args.warmup, 3)):
            sess.stage_coarse(q, nq, k, ids, dist)
        torch.cuda.synchronize()
        sess.counters(reset=True)
        sampler = ClockSampler(device)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            sess.stage_coarse(q, nq, k, ids, dist)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        cnt = sess.counters(reset=True)
        # end to end: host queries in, host ids/distances out
        qp = torch.empty((nq, dim), dtype=torch.float32).pin_memory(); qp.copy_(q)
        oi = torch.empty((nq, k), dtype=torch.int32).pin_memory()
        od = torch.empty((nq, k), dtype=torch.float32).pin_memory()
        q2 = torch.empty_like(q)

        def e2e_step():
            q2.copy_(qp, non_blocking=True)
            sess.stage_coarse(q2, nq, k, ids, dist)
            oi.copy_(ids, non_blocking=True); od.copy_(dist, non_blocking=True)
            stream.synchronize()
        e2e_step()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
        got_i, got_d = oi.numpy().astype(np.int64), od.numpy().copy()
    cores = os.cpu_count() or 1
    ns = args.cpu_sample or 512
    t0 = time.time()
    if oracle.have_ref():
        ri, rd = oracle.ref_coarse(q_host[:ns], index["centroids"], k, threads=cores); kind = "reference"
    else:
        ri, rd = oracle.coarse(q_host[:ns], index["centroids"], k); kind = "port"
    dt = time.time() - t0
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops", 1590.0))
    flops = 2.0 * nq * nlist * dim
    gemm_ms = cnt["coarse_gemm_ms"] / max(1, cnt["coarse_gemm_launches"])  # one pass
    line = dict(metric="coarse queries/s (top-64 of 65,536 centroids)", value=round(nq / (ms * 1e-3), 1), unit="queries/s",
                n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=round(ms, 3), higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="bf16 filter + f32 exact", data="synthetic",
                config=dict(workload="c3", desc=cfg["desc"], l2="distance matrix never materialised; operands 64 MB"),
                e2e=dict(value=round(nq / (ms_e2e * 1e-3), 1), unit="queries/s", ms_per_step=round(ms_e2e, 3),
                         h2d_bytes_per_step=nq * dim * 4, d2h_bytes_per_step=nq * k * 8),
                gpu_launches=int(cnt["kernel_launches"]),
                roofline=dict(bound="tensor", kernel="k_coarse_tc (one of two passes)", achieved=round(flops / (gemm_ms * 1e-3) / 1e12, 1),
                              peak=peak, unit="TFLOP/s", frac=round(flops / (gemm_ms * 1e-3) / 1e12 / peak, 4),
                              peak_source="measured (burst)" if peaks else "fallback", ms_per_launch=round(gemm_ms, 3),
                              algorithmic_flops_per_launch=flops, executed_flops_per_launch=2.0 * nq * nlist * 128, traffic=None,
                              stage_achieved_tflops=round(flops / (ms * 1e-3) / 1e12, 1)),
                cpu_baseline=dict(value=round(ns / dt, 2), unit="queries/s", cores=cores, kind=kind,
                                  sample="first %d queries, all %d host threads" % (ns, cores)),
                # the reference's partial_sort leaves the order of equal distances open; ids are compared against the
                # restatement (ties by centroid id), distances against the reference's own output
                parity=dict(sample_queries=ns, ids_equal=bool(np.array_equal(oracle.coarse(q_host[:ns], index["centroids"], k)[0], got_i[:ns])),
                            ids_equal_reference_tie_order=bool(np.array_equal(ri, got_i[:ns])),
                            dist_equal=bool(np.array_equal(rd, got_d[:ns])),
                            coarse_fallback_queries=int(cnt["coarse_fallback_queries"])),
                clocks=clocks)
    emit(line)
    sess.close()
    return 0


def reference_arm(args, cfg, index, q_host, gt):
    """Times the reference's own CPU implementation on bounded samples of the batch (rank 0 only)."""
    cores = os.cpu_count() or 1
    ns = args.cpu_sample
    if not ns:
        # The fine stage parallelises over queries: give every host thread at least 8 of them, and grow the sample until a
        # step takes several seconds (the sizing of this library's own cpu_baseline leg), so the host cores are kept busy.
        _, dt0, _ = cpu_reference_run(index, q_host, cfg, 16, cores)
        ns = int(min(512, cfg["nq"], max(8 * cores, 16 * 8.0 / max(dt0, 1e-3))))
    times = []
    for i in range(args.warmup + args.steps):
        lo = (i * ns) % max(1, cfg["nq"] - ns + 1)
        _, dt, kind = cpu_reference_run(index, q_host[lo:lo + ns], cfg, ns, cores)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    v = round(ns / (ms * 1e-3), 2)
    line = dict(impl="reference", metric="QPS (IVF-PQ search, recall@k equal to the reference CPU path)", value=v,
                unit="queries/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=round(ms, 3),
                higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, desc=cfg["desc"], rows=cfg["n"], dim=cfg["dim"], nlist=cfg["nlist"],
                            M=cfg["M"], batch=cfg["nq"], nprobe=cfg["nprobe"], topk=cfg["topk"], n_rerank=cfg["n_rerank"]),
                cpu_baseline=dict(value=v, unit="queries/s", cores=cores, kind=kind,
                                  sample="%d queries of the batch per step, all %d host threads" % (ns, cores)),
                e2e=dict(value=v, unit="queries/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    emit(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
