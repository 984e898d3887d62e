// PQ lookup tables, the list-centric probe schedule, and the ADC scan with per-query selection.
//
// Pipeline per batch (all kernels on one stream, no host synchronisation in between):
//   k_build_lut        one table [M][K] per query, built once and shared by all probed lists
//   k_count_visitors   inverts (query, probe) -> per-list visitor counts (+ rows each query will scan)
//   k_scan_lists       exclusive scans: visitor offsets and work-item offsets per list
//   k_fill_visitors    per-list visitor arrays
//   k_seed_threshold   per query: ADC distances of a strided row sample (1/16 .. 1/64 of its rows) -> admission cutoff
//   k_scan<M,V>        persistent CTAs; work item = (list, chunk of rows, group of V visitors); each thread
//                      keeps one code row in registers and scores it for the V visitors whose tables sit
//                      interleaved in shared memory (one LDS.128 fetches 4 visitors' entries); rows with
//                      dist <= cutoff are appended to the query's pool
//   k_select_pool      per query: exact (distance,row) sort of the pool -> stage1_k candidates; flags
//                      pools that overflowed or came up short
//   k_exact_fallback   re-scans flagged queries exactly with a CTA-local running top-k (normally zero work)
//
// Arithmetic matches the CPU path bit for bit: table entries are the sequential non-fused fp32 sum of
// (q-c)^2 and ADC distances are the sequential fp32 sum over m = 0..M-1
// (reference: src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:51-63,76-80).
#include <string>
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"
#include "scan_common.cuh"

namespace psb {

using namespace scan;

namespace {

constexpr int kScanThreads = 512;
constexpr int kSeedThreads = 512;
constexpr int kSelectThreads = 1024;
constexpr int kFallbackThreads = 1024;

// ------------------------------------------------------------------------------------------------------
__global__ void k_build_lut(const float* __restrict__ queries, int dim, const float* __restrict__ codebook,
                            int m, int k, float* __restrict__ lut) {
    extern __shared__ float s_q[];
    const int q = blockIdx.x;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) s_q[i] = queries[(size_t)q * dim + i];
    __syncthreads();
    const int dsub = dim / m;
    const int total = m * k;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int sub = e / k;
        const float* c = codebook + (size_t)e * dsub;
        const float* qs = s_q + sub * dsub;
        float dist = 0.0f;
        for (int d = 0; d < dsub; ++d) {
            const float diff = __fsub_rn(qs[d], __ldg(c + d));
            dist = __fadd_rn(dist, __fmul_rn(diff, diff));
        }
        lut[(size_t)q * total + e] = dist;
    }
}

// Residual mode: one table per (query, probe) pair, built on q - centroid[probe] (fp32 subtraction, then the same
// sequential non-fused sum; reference: src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:440-451 and :113-128).
__global__ void k_build_lut_residual(const float* __restrict__ queries, int dim, const int* __restrict__ probes,
                                     int nprobe, const float* __restrict__ centroids, int nlist,
                                     const float* __restrict__ codebook, int m, int k, float* __restrict__ lut) {
    extern __shared__ float s_q[];
    const long long pair = blockIdx.x;
    const int q = (int)(pair / nprobe);
    const int l = probes[pair];
    if (l < 0 || l >= nlist) return;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        s_q[i] = __fsub_rn(queries[(size_t)q * dim + i], __ldg(centroids + (size_t)l * dim + i));
    __syncthreads();
    const int dsub = dim / m;
    const int total = m * k;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int sub = e / k;
        const float* c = codebook + (size_t)e * dsub;
        const float* qs = s_q + sub * dsub;
        float dist = 0.0f;
        for (int d = 0; d < dsub; ++d) {
            const float diff = __fsub_rn(qs[d], __ldg(c + d));
            dist = __fadd_rn(dist, __fmul_rn(diff, diff));
        }
        lut[(size_t)pair * total + e] = dist;
    }
}

// ------------------------------------------------------------------------------------------------------
// One warp per query: counts visitors per local list and the rows the query will scan.
__global__ void k_count_visitors(const int* __restrict__ probes, int nq, int nprobe,
                                 const long long* __restrict__ offsets, int nlist, int lb, int le,
                                 int* __restrict__ vis_count, long long* __restrict__ q_rows,
                                 unsigned long long* __restrict__ counters) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= nq) return;
    long long rows = 0;
    for (int p = lane; p < nprobe; p += 32) {
        const int l = probes[(size_t)warp * nprobe + p];
        if (l < lb || l >= le || l < 0 || l >= nlist) continue;
        atomicAdd(&vis_count[l], 1);
        rows += offsets[l + 1] - offsets[l];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rows += __shfl_xor_sync(0xffffffffu, rows, o);
    if (lane == 0) {
        q_rows[warp] = rows;
        atomicAdd(&counters[0], (unsigned long long)rows);
    }
}

// Single CTA: exclusive scans over the lists (visitor offsets, work-item offsets).
// A list with at least tc_min_vis visitors (tc_min_vis > 0) belongs to the tensor-core kernel: its work items (groups of
// tc_group visitors) are counted in item_off_tc and it gets none in item_off; every other list the other way round.
__device__ __forceinline__ void list_items(int v, long long rows, int group, int tc_group, int tc_min_vis, int chunk_rows,
                                           long long& simt, long long& tc) {
    simt = 0; tc = 0;
    if (v <= 0 || rows <= 0) return;
    const long long chunks = (rows + chunk_rows - 1) / chunk_rows;
    if (tc_min_vis > 0 && v >= tc_min_vis) tc = (long long)((v + tc_group - 1) / tc_group) * chunks;
    else simt = (long long)((v + group - 1) / group) * chunks;
}
__global__ void __launch_bounds__(1024) k_scan_lists(const int* __restrict__ vis_count, const long long* __restrict__ offsets, int nlist,
                             int group, int chunk_rows, int* __restrict__ vis_off,
                             long long* __restrict__ item_off, int* __restrict__ vis_cursor,
                             int tc_group, int tc_min_vis, long long* __restrict__ item_off_tc) {
    // Rounds of blockDim.x consecutive lists (coalesced reads and writes), each round one block-wide scan of the three
    // per-list counts; the running totals carry over in registers.
    __shared__ long long s_items[32], s_tc[32];
    __shared__ int s_vis[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    long long carry_items = 0, carry_tc = 0; int carry_vis = 0;
    for (int base = 0; base < nlist; base += blockDim.x) {
        const int l = base + threadIdx.x;
        int v = 0; long long si = 0, ti = 0;
        if (l < nlist) {
            v = vis_count[l];
            list_items(v, offsets[l + 1] - offsets[l], group, tc_group, tc_min_vis, chunk_rows, si, ti);
        }
        int iv = v; long long ii = si, it = ti;   // inclusive within the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int nv = __shfl_up_sync(0xffffffffu, iv, o);
            const long long ni = __shfl_up_sync(0xffffffffu, ii, o), nt = __shfl_up_sync(0xffffffffu, it, o);
            if (lane >= o) { iv += nv; ii += ni; it += nt; }
        }
        if (lane == 31) { s_vis[warp] = iv; s_items[warp] = ii; s_tc[warp] = it; }
        __syncthreads();
        int wv = 0; long long wi = 0, wt = 0, tv = 0, tti = 0, ttt = 0;   // exclusive warp offsets and the round's totals
        for (int w2 = 0; w2 < nwarps; ++w2) {
            const int cv = s_vis[w2]; const long long ci = s_items[w2], ct = s_tc[w2];
            if (w2 < warp) { wv += cv; wi += ci; wt += ct; }
            tv += cv; tti += ci; ttt += ct;
        }
        if (l < nlist) {
            vis_off[l] = carry_vis + wv + iv - v;
            item_off[l] = carry_items + wi + ii - si;
            if (item_off_tc) item_off_tc[l] = carry_tc + wt + it - ti;
            vis_cursor[l] = 0;
        }
        carry_vis += (int)tv; carry_items += tti; carry_tc += ttt;
        __syncthreads();   // the warp totals are rewritten next round
    }
    if (threadIdx.x == 0) {
        item_off[nlist] = carry_items; vis_off[nlist] = carry_vis;
        if (item_off_tc) item_off_tc[nlist] = carry_tc;
    }
}

__global__ void k_fill_visitors(const int* __restrict__ probes, int nq, int nprobe, int nlist, int lb, int le,
                                const int* __restrict__ vis_off, int* __restrict__ vis_cursor,
                                int* __restrict__ visitors, int pair_ids) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)nq * nprobe) return;
    const int l = probes[i];
    if (l < lb || l >= le || l < 0 || l >= nlist) return;
    const int pos = atomicAdd(&vis_cursor[l], 1);
    visitors[vis_off[l] + pos] = pair_ids ? (int)i : (int)(i / nprobe);  // table index: the pair in residual mode
}

// ------------------------------------------------------------------------------------------------------
// Where a residual-mode table (one per (query, probe) pair) comes from: the tables materialised in global memory, or - when
// lut is null - the query, the probed list's centroid and the codebook, from which the block builds it in shared memory
// with the arithmetic of k_build_lut_residual (fp32 subtraction, sequential non-fused sum over the sub-vector).
struct ResidualSource {
    const float* queries;    // [nq][dim]
    const float* centroids;  // [nlist][dim]
    const float* codebook;   // [m][k][dim / m]
    const float* row_bias;   // [shard rows] per-row correction |recon|^2 + 2 <centroid[list(row)], recon(row)> as fp32, or null
    const uint16_t* row_bias_u16;  // the same in the affine u16 form (value = rc_offset + rc_scale * u16), or null
    float rc_scale, rc_offset;
    int dim;
};
__device__ __forceinline__ void stage_residual_table(float* __restrict__ s_lut, const float* __restrict__ lut, const ResidualSource& rs,
                                                     int q, int p, int nprobe, int list, int m, int k) {
    const int mk = m * k;
    if (lut) {
        const float* src = lut + ((size_t)q * nprobe + p) * mk;
        for (int e = threadIdx.x; e < mk; e += blockDim.x) s_lut[e] = src[e];
        return;
    }
    const int dsub = rs.dim / m;
    const float* qv = rs.queries + (size_t)q * rs.dim;
    const float* cv = rs.centroids + (size_t)list * rs.dim;
    __shared__ float s_qres[256];  // q - centroid, staged once when it fits (the callers' barriers around this call order its reuse)
    const bool staged = rs.dim <= 256;
    if (staged) {
        for (int d = threadIdx.x; d < rs.dim; d += blockDim.x) s_qres[d] = __fsub_rn(__ldg(qv + d), __ldg(cv + d));
        __syncthreads();
    }
    for (int e = threadIdx.x; e < mk; e += blockDim.x) {
        const int sub = e / k;
        const float* c = rs.codebook + (size_t)e * dsub;
        float dist = 0.0f;
        for (int d = 0; d < dsub; ++d) {
            const float r = staged ? s_qres[sub * dsub + d] : __fsub_rn(__ldg(qv + sub * dsub + d), __ldg(cv + sub * dsub + d));
            const float diff = __fsub_rn(r, __ldg(c + d));
            dist = __fadd_rn(dist, __fmul_rn(diff, diff));
        }
        s_lut[e] = dist;
    }
}

// Per query: admission cutoff from a strided sample of the rows it will scan.
//   N = rows the query scans.  N <= pool capacity: cutoff = +inf (everything is admitted).
//   Otherwise every stride-th row of each probed list is scored, stride = clamp(stage1_k / 16, 16, 64), n_s rows in
//   all, and the cutoff is the r-th smallest sample distance with r = ceil(mu + 4 sqrt(mu) + 2), mu = stage1_k * n_s / N:
//   the stage1_k-th smallest of all N distances lies below it except with negligible probability, and about r * stride
//   rows (2-4 x stage1_k) pass it.  The selection kernel verifies that each pool holds at least stage1_k rows and did
//   not overflow; the exact fallback handles the rest.  The r smallest sample keys are kept with a running cutoff:
//   keys below it go to a 2048-entry buffer that is sorted and cut back to r whenever it could overflow.
constexpr int kSeedBuf = 2048;
template <int M>
__global__ void __launch_bounds__(kSeedThreads)
k_seed_threshold(const float* __restrict__ lut, const int* __restrict__ probes, int nprobe,
                 const long long* __restrict__ offsets, int nlist, int lb, int le,
                 const uint8_t* __restrict__ codes, long long row_base, int m, int k,
                 const long long* __restrict__ q_rows, int stage1_k, int pool_cap, float* __restrict__ thr,
                 int per_probe, int tree, float margin_sigma, float margin_add, const ResidualSource rs,
                 uint32_t* __restrict__ seed_out, int seed_keys) {
    // per_probe (residual mode): lut holds one table per (query, probe) pair; the probes are then sampled one after
    // the other, each with its own table staged in shared memory.
    extern __shared__ __align__(16) unsigned char s_seed_raw[];
    float* s_lut = reinterpret_cast<float*>(s_seed_raw);                                  // [m * k]
    uint32_t* s_keys = reinterpret_cast<uint32_t*>(s_seed_raw + (size_t)m * k * 4);       // [kSeedBuf]
    int* s_pref = reinterpret_cast<int*>(s_seed_raw + (size_t)m * k * 4 + kSeedBuf * 4);  // [nprobe + 1]
    __shared__ int s_warp[32];
    __shared__ int s_total, s_cnt;
    __shared__ uint32_t s_cut;
    const int q = blockIdx.x;
    const long long N = q_rows[q];
    const float inf = __int_as_float(0x7f800000);
    // sample record for the other shards (sharded search): keys, then stride, key count, rows scanned
    uint32_t* rec = seed_out ? seed_out + (size_t)q * (seed_keys + kSeedTail) : nullptr;
    auto empty_record = [&](int stride_) {   // nothing to tell: this shard does not take part in placing the cutoff
        if (!rec) return;
        for (int i = threadIdx.x; i < seed_keys; i += blockDim.x) rec[i] = 0xffffffffu;
        if (threadIdx.x == 0) { rec[seed_keys] = (uint32_t)stride_; rec[seed_keys + 1] = 0; rec[seed_keys + 2] = (uint32_t)N; rec[seed_keys + 3] = (uint32_t)(N >> 32); }
    };
    // (a shard that records for the others samples even what it would admit whole: its rows count towards the shared cutoff)
    if (N <= pool_cap && !rec) { if (threadIdx.x == 0) thr[q] = inf; return; }
    if (N <= 0) { if (threadIdx.x == 0) thr[q] = inf; empty_record(0); return; }
    int stride = stage1_k / 16;
    stride = stride < 16 ? 16 : (stride > 64 ? 64 : stride);
    if ((N + 65535) / 65536 > stride) stride = (int)((N + 65535) / 65536);  // at most ~64K samples per query
    // Residual mode without materialised tables: no per-probe staging.  With c the probed list's centroid,
    //     |(q - c) - recon|^2 = |q - c|^2 - 2 <q, recon> + (|recon|^2 + 2 <c, recon>),
    // so ONE dot-product table per query (built here) serves every probed list, plus a constant per probe and the per-row
    // correction of the index (the reference's shared-table form: src/search/kernels/fine/gpu_fine/pq_adc/
    // pq_query_lut_score.cuh:7-22, src/common/row_correction.h:37-45; fp32 or affine u16).  The sum is the same distance in a
    // different rounding; it only places the CUTOFF, whose exact value does not matter: the selection counts the rows whose
    // EXACT distance is within it and falls back to the exact scan when they are too few.
    const bool flat_bias = per_probe && lut == nullptr;
    float* s_pk = reinterpret_cast<float*>(s_pref + nprobe + 1);  // [nprobe] |q - c|^2 per probe (flat_bias only)
    if (!per_probe) {
        for (int e = threadIdx.x; e < m * k; e += blockDim.x) s_lut[e] = lut[(size_t)q * m * k + e];
    } else if (flat_bias) {
        const int dsub = rs.dim / m;
        const float* qv = rs.queries + (size_t)q * rs.dim;
        for (int e = threadIdx.x; e < m * k; e += blockDim.x) {
            const int sub = e / k;
            const float* c = rs.codebook + (size_t)e * dsub;
            float dot = 0.0f;
            for (int d = 0; d < dsub; ++d) dot = fmaf(__ldg(qv + sub * dsub + d), __ldg(c + d), dot);
            s_lut[e] = -2.0f * dot;
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int p = warp; p < nprobe; p += (int)(blockDim.x >> 5)) {
            const int l = probes[(size_t)q * nprobe + p];
            float acc = 0.0f;
            if (l >= 0 && l < nlist) {
                const float* cv = rs.centroids + (size_t)l * rs.dim;
                for (int d = lane; d < rs.dim; d += 32) { const float diff = __ldg(qv + d) - __ldg(cv + d); acc = fmaf(diff, diff, acc); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) s_pk[p] = acc;
        }
    }
    // samples per probe and their exclusive prefix
    int carry = 0;
    for (int p0 = 0; p0 < nprobe; p0 += blockDim.x) {
        const int p = p0 + threadIdx.x;
        int nj = 0;
        if (p < nprobe) {
            const int l = probes[(size_t)q * nprobe + p];
            if (!(l < lb || l >= le || l < 0 || l >= nlist)) nj = (int)((offsets[l + 1] - offsets[l] + stride - 1) / stride);
        }
        const int ex = block_exclusive_scan(nj, s_warp, &s_total);
        if (p < nprobe) s_pref[p] = carry + ex;
        carry += s_total;
        __syncthreads();
    }
    const int ns = carry;
    if (threadIdx.x == 0) { s_pref[nprobe] = ns; s_cnt = 0; s_cut = 0xffffffffu; }
    const float mu = (float)stage1_k * (float)ns / (float)N;
    int r = (int)ceilf(mu + margin_sigma * sqrtf(mu) + margin_add);
    if (rec) {
        // For the other shards: as many keys as the shared cutoff can ask of ONE shard - the case of a query whose near rows all
        // lie here.  c keys of stride s put the cutoff once c - sigma sqrt(c) - 2 >= mu (k_pick_cutoff), so c solves that, plus a
        // few for a larger stride elsewhere.
        float c = mu;
        for (int it = 0; it < 6; ++it) c = mu + margin_sigma * sqrtf(c) + 2.0f;
        r = (int)ceilf(c) + 8;
    }
    if ((r >= ns && !rec) || r + (int)blockDim.x > kSeedBuf) { if (threadIdx.x == 0) thr[q] = inf; empty_record(0); return; }
    __syncthreads();
    const bool staged_probes = per_probe && !flat_bias;  // one table per probe, staged one after the other
    const int nseg = staged_probes ? nprobe : 1;
    for (int sg = 0; sg < nseg; ++sg) {
        const int b0 = staged_probes ? s_pref[sg] : 0, b1 = staged_probes ? s_pref[sg + 1] : ns;  // uniform
        if (b0 == b1) continue;
        if (staged_probes) {
            __syncthreads();  // the previous probe's table is no longer read
            stage_residual_table(s_lut, lut, rs, q, sg, nprobe, probes[(size_t)q * nprobe + sg], m, k);
            __syncthreads();
        }
        for (int base = b0; base < b1; base += blockDim.x) {
            const int c_now = s_cnt;  // stable since the barrier that ended the previous round
            __syncthreads();
            if (c_now + (int)blockDim.x > kSeedBuf) {  // uniform
                for (int i = c_now + threadIdx.x; i < kSeedBuf; i += blockDim.x) s_keys[i] = 0xffffffffu;
                __syncthreads();
                block_bitonic_sort(s_keys, kSeedBuf);
                if (threadIdx.x == 0) { s_cnt = r; s_cut = s_keys[r - 1]; }  // c_now >= r here
                __syncthreads();
            }
            const int idx = base + threadIdx.x;
            if (idx < b1) {
                int lo = sg, hi = nprobe;  // largest p with s_pref[p] <= idx
                if (!staged_probes) {
                    lo = 0;
                    while (hi - lo > 1) {
                        const int mid = (lo + hi) >> 1;
                        if (s_pref[mid] <= idx) lo = mid; else hi = mid;
                    }
                }
                const int l = probes[(size_t)q * nprobe + lo];
                const long long row = offsets[l] + (long long)(idx - s_pref[lo]) * stride;
                const uint8_t* rp = codes + (size_t)(row - row_base) * m;
                float sd = adc_row<M>(rp, s_lut, m, k, tree != 0);
                if (flat_bias) {
                    const float corr = rs.row_bias ? __ldg(rs.row_bias + (row - row_base))
                                                   : fmaf(rs.rc_scale, (float)__ldg(rs.row_bias_u16 + (row - row_base)), rs.rc_offset);
                    sd = fmaxf(sd + s_pk[lo] + corr, 0.0f);
                }
                const uint32_t key = f2o(sd);
                if (key < s_cut) s_keys[atomicAdd(&s_cnt, 1)] = key;
            }
            __syncthreads();
        }
    }
    const int c = s_cnt;
    for (int i = c + threadIdx.x; i < kSeedBuf; i += blockDim.x) s_keys[i] = 0xffffffffu;
    __syncthreads();
    block_bitonic_sort(s_keys, kSeedBuf);
    if (threadIdx.x == 0) thr[q] = c >= r ? o2f(s_keys[r - 1]) : inf;
    if (rec) {   // the r smallest sample keys: no key beyond them can lie below a cutoff placed on all shards' samples
        const int have = c < r ? c : r;
        const int out = have < seed_keys ? have : seed_keys;
        for (int i = threadIdx.x; i < seed_keys; i += blockDim.x) rec[i] = i < out ? s_keys[i] : 0xffffffffu;
        if (threadIdx.x == 0) {
            rec[seed_keys] = (uint32_t)stride;
            rec[seed_keys + 1] = (uint32_t)out;
            rec[seed_keys + 2] = (uint32_t)N; rec[seed_keys + 3] = (uint32_t)(N >> 32);
        }
    }
}

// Sharded search: the cutoff of query q from the sample records of all shards.  A key of shard g stands for stride_g rows of
// that shard, so after the i smallest keys of the union the rows below key i number about A = sum stride, with variance at
// most B = sum stride^2 (each stride-th row is a sample).  The cutoff is the first key with A - sigma sqrt(B) - 2 max stride
// >= stage1_k: at least stage1_k rows of the shards together lie below it except with the probability of a sigma-deviation.
// A record ends where its shard stopped recording, not where its samples end; keys of other shards beyond that point still
// count rows that are there, so A only underestimates and the cutoff errs to the high side.  No such key (few rows): +inf,
// every shard admits all its rows.  A shard whose record is empty (it admits everything it scans anyway, or has too few rows
// to sample) adds nothing to the sum.
// The caller verifies the outcome - the candidates of all shards together must number stage1_k - so a cutoff placed too low
// costs a second pass, never a wrong answer.
constexpr int kPickThreads = 256;
__global__ void __launch_bounds__(kPickThreads)
k_pick_cutoff(const uint32_t* __restrict__ all, int shards, int nq, int seed_keys, int stage1_k, float sigma,
              float* __restrict__ thr, long long* __restrict__ rows_global) {
    extern __shared__ __align__(16) uint64_t s_pick[];   // [next_pow2(shards * seed_keys)] key << 32 | stride
    __shared__ unsigned int s_smax;
    const int q = blockIdx.x;
    const int words = seed_keys + kSeedTail;
    const int total = shards * seed_keys;
    const int n = next_pow2(max(total, 2));
    if (threadIdx.x == 0) s_smax = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        uint64_t e = ~0ull;
        if (i < total) {
            const int g = i / seed_keys, j = i - g * seed_keys;
            const uint32_t* rec = all + ((size_t)g * nq + q) * words;
            const int have = (int)rec[seed_keys + 1];
            if (j < have) {
                const uint32_t stride = rec[seed_keys];
                e = ((uint64_t)rec[j] << 32) | stride;
                if (j == 0) atomicMax(&s_smax, stride);
            }
        }
        s_pick[i] = e;
    }
    __syncthreads();
    block_bitonic_sort(s_pick, n);
    if (threadIdx.x == 0) {
        const float inf = __int_as_float(0x7f800000);
        const float smax = (float)s_smax;
        float A = 0.f, B = 0.f, cut = inf;
        for (int i = 0; i < total; ++i) {
            const uint64_t e = s_pick[i];
            if (e == ~0ull) break;
            const float st = (float)(uint32_t)e;
            A += st; B += st * st;
            if (A - sigma * sqrtf(B) - 2.0f * smax >= (float)stage1_k) { cut = o2f((uint32_t)(e >> 32)); break; }
        }
        thr[q] = cut;
        if (rows_global) {
            long long N = 0;
            for (int g = 0; g < shards; ++g) {
                const uint32_t* rec = all + ((size_t)g * nq + q) * words;
                N += (long long)(((uint64_t)rec[seed_keys + 3] << 32) | rec[seed_keys + 2]);
            }
            rows_global[q] = N;
        }
    }
}

// ------------------------------------------------------------------------------------------------------
template <int V> struct LutVec;
template <> struct LutVec<1> { using T = float; };
template <> struct LutVec<2> { using T = float2; };
template <> struct LutVec<4> { using T = float4; };

template <int V>
__device__ __forceinline__ void lut_add(float (&acc)[V], const float* __restrict__ s_lut, int e) {
    if constexpr (V == 1) {
        acc[0] = __fadd_rn(acc[0], s_lut[e]);
    } else if constexpr (V == 2) {
        const float2 x = reinterpret_cast<const float2*>(s_lut)[e];
        acc[0] = __fadd_rn(acc[0], x.x); acc[1] = __fadd_rn(acc[1], x.y);
    } else if constexpr (V == 4) {
        const float4 x = reinterpret_cast<const float4*>(s_lut)[e];
        acc[0] = __fadd_rn(acc[0], x.x); acc[1] = __fadd_rn(acc[1], x.y);
        acc[2] = __fadd_rn(acc[2], x.z); acc[3] = __fadd_rn(acc[3], x.w);
    } else {
        static_assert(V == 8, "visitor group");
        const float4 x = reinterpret_cast<const float4*>(s_lut)[2 * e];
        const float4 y = reinterpret_cast<const float4*>(s_lut)[2 * e + 1];
        acc[0] = __fadd_rn(acc[0], x.x); acc[1] = __fadd_rn(acc[1], x.y);
        acc[2] = __fadd_rn(acc[2], x.z); acc[3] = __fadd_rn(acc[3], x.w);
        acc[4] = __fadd_rn(acc[4], y.x); acc[5] = __fadd_rn(acc[5], y.y);
        acc[6] = __fadd_rn(acc[6], y.z); acc[7] = __fadd_rn(acc[7], y.w);
    }
}

template <int M, int V>
__global__ void __launch_bounds__(640, 1) k_scan(const ScanArgs a) {
    extern __shared__ __align__(16) float s_lut[];  // [m*k][V] visitor-interleaved
    __shared__ long long s_item;
    __shared__ int s_list, s_vq[V], s_pq[V];
    __shared__ float s_thr[V];
    const int mk = a.m * a.k;
    const long long total = a.item_off[a.nlist];
    for (;;) {
        __syncthreads();  // previous item fully consumed (tables, s_* words)
        if (threadIdx.x < 32) {
            long long item = 0;
            if (threadIdx.x == 0) item = (long long)atomicAdd(a.work_cursor, 1ull);
            item = __shfl_sync(0xffffffffu, item, 0);
            int l = -1;
            if (item < total) l = find_list(a.item_off, a.nlist, item);
            if (threadIdx.x == 0) { s_item = item; s_list = l; }
        }
        __syncthreads();
        const long long item = s_item;
        if (item >= total) break;
        const int l = s_list;
        const int nvis = a.vis_count[l];
        const int ngroups = (nvis + V - 1) / V;
        const long long local = item - a.item_off[l];
        const int group = (int)(local % ngroups);
        const long long chunk = local / ngroups;
        if (threadIdx.x < V) {
            const int vi = group * V + threadIdx.x;
            const int q = vi < nvis ? a.visitors[a.vis_off[l] + vi] : -1;  // table index
            const int pq = q >= 0 ? q / a.lut_div : -1;                     // query (pool, cutoff)
            s_vq[threadIdx.x] = q;
            s_pq[threadIdx.x] = pq;
            s_thr[threadIdx.x] = q >= 0 ? a.thr[pq] : -1.0f;  // distances are >= 0: -1 admits nothing
        }
        __syncthreads();
        int vq[V], pq[V]; float thr[V];
#pragma unroll
        for (int v = 0; v < V; ++v) { vq[v] = s_vq[v]; pq[v] = s_pq[v]; thr[v] = s_thr[v]; }
        // stage the V tables, interleaved by visitor (padding visitors reuse visitor 0's table)
        {
            const float* src[V];
#pragma unroll
            for (int v = 0; v < V; ++v) src[v] = a.lut + (size_t)(vq[v] >= 0 ? vq[v] : vq[0]) * mk;
            for (int e = threadIdx.x; e < mk; e += kScanThreads) {
#pragma unroll
                for (int v = 0; v < V; ++v) s_lut[e * V + v] = __ldg(src[v] + e);
            }
        }
        __syncthreads();
        const long long delta = a.row_delta ? a.row_delta[l] : 0;
        const long long r0 = a.offsets[l] + chunk * a.chunk_rows;
        const long long r1 = min(r0 + a.chunk_rows, a.offsets[l + 1]);
        for (long long r = r0 + threadIdx.x; r < r1; r += kScanThreads) {
            const uint8_t* row = a.codes + (size_t)(r - a.row_base) * a.m;
            float acc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = 0.0f;
            if constexpr (M > 0 && M % 16 == 0) {
                const uint4* p = reinterpret_cast<const uint4*>(row);
                uint4 c[M / 16];
#pragma unroll
                for (int w = 0; w < M / 16; ++w) c[w] = __ldg(p + w);
#pragma unroll
                for (int w = 0; w < M / 16; ++w) {
                    const uint32_t cw[4] = {c[w].x, c[w].y, c[w].z, c[w].w};
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        lut_add<V>(acc, s_lut, (w * 16 + j) * a.k + (int)((cw[j >> 2] >> ((j & 3) * 8)) & 255));
                }
            } else if constexpr (M > 0 && M % 4 == 0) {
                const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
                uint32_t c[M / 4];
#pragma unroll
                for (int w = 0; w < M / 4; ++w) c[w] = __ldg(p + w);
#pragma unroll
                for (int w = 0; w < M / 4; ++w)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        lut_add<V>(acc, s_lut, (w * 4 + j) * a.k + (int)((c[w] >> (j * 8)) & 255));
            } else {
                for (int j = 0; j < a.m; ++j) lut_add<V>(acc, s_lut, j * a.k + (int)__ldg(row + j));
            }
            if constexpr (M == 8 || M == 16) {
                if (a.tree) {  // pairwise-tree order: pair sums first (0 + x is exact), then the balanced tree
                    const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
                    float part[M / 2][V];
#pragma unroll
                    for (int w = 0; w < M / 4; ++w) {
                        const uint32_t c = __ldg(p + w);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int v = 0; v < V; ++v) part[w * 2 + h][v] = 0.0f;
                            lut_add<V>(part[w * 2 + h], s_lut, (w * 4 + 2 * h) * a.k + (int)((c >> (16 * h)) & 255));
                            lut_add<V>(part[w * 2 + h], s_lut, (w * 4 + 2 * h + 1) * a.k + (int)((c >> (16 * h + 8)) & 255));
                        }
                    }
#pragma unroll
                    for (int n = M / 2; n > 1; n >>= 1)
#pragma unroll
                        for (int j = 0; j < n / 2; ++j)
#pragma unroll
                            for (int v = 0; v < V; ++v) part[j][v] = __fadd_rn(part[2 * j][v], part[2 * j + 1][v]);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = part[0][v];
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (acc[v] <= thr[v]) {
                    const int slot = atomicAdd(&a.pool_cnt[pq[v]], 1);
                    if (slot < a.pool_cap) a.pool[(size_t)pq[v] * a.pool_cap + slot] = make_key(acc[v], (uint32_t)(r + delta));
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Per query: sort the pool by (distance,row), emit the first stage1_k.  A pool that overflowed, or that holds
// fewer than min(stage1_k, rows scanned) entries, sends the query to the exact fallback.
__global__ void __launch_bounds__(kSelectThreads)
k_select_pool(const uint64_t* __restrict__ pool, const int* __restrict__ pool_cnt, int pool_cap,
              const long long* __restrict__ q_rows, int stage1_k, int* __restrict__ out_rows,
              float* __restrict__ out_dist, int* __restrict__ out_count, int* __restrict__ fail_list,
              int* __restrict__ n_fail, unsigned long long* __restrict__ counters, const float* __restrict__ shared_cut) {
    extern __shared__ __align__(16) uint64_t s_keys[];
    const int q = blockIdx.x;
    const int c = pool_cnt[q];
    const long long N = q_rows[q];
    // shared_cut (sharded search): the cutoff was placed on all shards' rows, so this shard alone owes no stage1_k rows
    long long need = N < stage1_k ? N : stage1_k;
    if (shared_cut && shared_cut[q] < __int_as_float(0x7f800000)) need = 0;
    if (c > pool_cap || c < need) {
        if (threadIdx.x == 0) fail_list[atomicAdd(n_fail, 1)] = q;
        return;  // the fallback writes this query's outputs
    }
    if (threadIdx.x == 0) atomicAdd(&counters[1], (unsigned long long)c);
    const int n = next_pow2(max(c, 2));
    for (int i = threadIdx.x; i < n; i += blockDim.x) s_keys[i] = i < c ? pool[(size_t)q * pool_cap + i] : KEY_MAX;
    __syncthreads();
    block_bitonic_sort(s_keys, n);
    const int keep = c < stage1_k ? c : stage1_k;
    for (int i = threadIdx.x; i < stage1_k; i += blockDim.x) {
        const bool ok = i < keep;
        out_rows[(size_t)q * stage1_k + i] = ok ? (int)key_idx(s_keys[i]) : -1;
        if (out_dist) out_dist[(size_t)q * stage1_k + i] = ok ? key_dist(s_keys[i]) : FLT_MAX;
    }
    if (out_count && threadIdx.x == 0) out_count[q] = keep;
}

// Exact fallback for the queries the selection kernel flagged.  The unit of work is a running top-k over the rows of some
// of a query's probes, kept in a CTA-local buffer: keys below the current cutoff are appended, and the buffer is compacted
// (sorted, truncated to stage1_k, cutoff tightened) whenever it could overflow during the next block of rows.
// A flagged query usually scans millions of rows, so its probes are cut into kFallbackSplit ranges that different CTAs
// scan; every range leaves its sorted top-stage1_k in global memory and k_fallback_merge combines the ranges of a query.
// Only the first kFallbackCap flagged queries are split (the partial lists need memory); any beyond are scanned whole by
// one CTA each, as a last resort.
constexpr int kFallbackSplit = 16;
constexpr int kFallbackCap = 128;

// Leaves the sorted keys of probes [p_begin, p_end) of query q in s_keys (KEY_MAX padded) and returns how many are valid.
template <int M>
__device__ __forceinline__ int fallback_scan_probes(const float* __restrict__ lut, const int* __restrict__ probes, int nprobe,
                                                    int q, int p_begin, int p_end, const long long* __restrict__ offsets,
                                                    int nlist, int lb, int le, const uint8_t* __restrict__ codes,
                                                    long long row_base, const long long* __restrict__ row_delta, int m, int k,
                                                    int stage1_k, int buf_n, int per_probe, int tree, uint64_t* s_keys,
                                                    float* s_lut, int* s_cnt, uint64_t* s_cut, const ResidualSource& rs) {
    __syncthreads();  // the previous unit's readers of s_keys / s_lut are done
    if (!per_probe)
        for (int e = threadIdx.x; e < m * k; e += blockDim.x) s_lut[e] = lut[(size_t)q * m * k + e];
    if (threadIdx.x == 0) { *s_cnt = 0; *s_cut = KEY_MAX; }
    __syncthreads();
    for (int p = p_begin; p < p_end; ++p) {
        const int l = probes[(size_t)q * nprobe + p];
        if (l < lb || l >= le || l < 0 || l >= nlist) continue;
        const long long b = offsets[l], e = offsets[l + 1];
        if (per_probe && b < e) {  // residual mode: this probe's own table (uniform branch)
            __syncthreads();
            stage_residual_table(s_lut, lut, rs, q, p, nprobe, l, m, k);
            __syncthreads();
        }
        const long long delta = row_delta ? row_delta[l] : 0;
        for (long long base = b; base < e; base += blockDim.x) {
            const int c_now = *s_cnt;  // stable since the barrier that ended the previous block of rows
            __syncthreads();           // every thread has read it before any thread appends again
            if (c_now + (int)blockDim.x > buf_n) {  // uniform decision
                for (int i = c_now + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
                __syncthreads();
                block_bitonic_sort(s_keys, buf_n);
                if (threadIdx.x == 0) {
                    const int keep = c_now < stage1_k ? c_now : stage1_k;
                    *s_cnt = keep;
                    *s_cut = keep == stage1_k ? s_keys[stage1_k - 1] : KEY_MAX;
                }
                __syncthreads();
            }
            const long long r = base + threadIdx.x;
            if (r < e) {
                const float d = adc_row<M>(codes + (size_t)(r - row_base) * m, s_lut, m, k, tree != 0);
                const uint64_t key = make_key(d, (uint32_t)(r + delta));
                if (key < *s_cut) s_keys[atomicAdd(s_cnt, 1)] = key;
            }
            __syncthreads();
        }
    }
    const int c = *s_cnt;
    for (int i = c + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
    __syncthreads();
    block_bitonic_sort(s_keys, buf_n);
    return c < stage1_k ? c : stage1_k;
}

__device__ __forceinline__ void fallback_emit(const uint64_t* s_keys, int keep, int q, int stage1_k, int* __restrict__ out_rows,
                                              float* __restrict__ out_dist, int* __restrict__ out_count) {
    for (int i = threadIdx.x; i < stage1_k; i += blockDim.x) {
        const bool ok = i < keep;
        out_rows[(size_t)q * stage1_k + i] = ok ? (int)key_idx(s_keys[i]) : -1;
        if (out_dist) out_dist[(size_t)q * stage1_k + i] = ok ? key_dist(s_keys[i]) : FLT_MAX;
    }
    if (out_count && threadIdx.x == 0) out_count[q] = keep;
}

template <int M>
__global__ void __launch_bounds__(kFallbackThreads)
k_exact_fallback(const float* __restrict__ lut, const int* __restrict__ probes, int nprobe,
                 const long long* __restrict__ offsets, int nlist, int lb, int le,
                 const uint8_t* __restrict__ codes, long long row_base, const long long* __restrict__ row_delta,
                 int m, int k, int stage1_k, int buf_n, const int* __restrict__ fail_list, const int* __restrict__ n_fail, int* __restrict__ fail_cursor,
                 int* __restrict__ out_rows, float* __restrict__ out_dist, int* __restrict__ out_count,
                 unsigned long long* __restrict__ counters, int per_probe, int tree, uint64_t* __restrict__ partial,
                 const ResidualSource rs) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_raw);                 // [buf_n]
    float* s_lut = reinterpret_cast<float*>(s_raw + (size_t)buf_n * 8);   // [m*k]
    __shared__ int s_cnt, s_idx;
    __shared__ uint64_t s_cut;
    const int nf = *n_fail;
    const int nsplit = nf < kFallbackCap ? nf : kFallbackCap;        // queries whose probes are cut into ranges
    const int items = nsplit * kFallbackSplit + (nf - nsplit);        // then whole queries
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_idx = atomicAdd(fail_cursor, 1);
        __syncthreads();
        const int item = s_idx;
        if (item >= items) return;
        if (item < nsplit * kFallbackSplit) {
            const int f = item / kFallbackSplit, part = item % kFallbackSplit;
            const int q = fail_list[f];
            const int p0 = (int)((long long)nprobe * part / kFallbackSplit), p1 = (int)((long long)nprobe * (part + 1) / kFallbackSplit);
            fallback_scan_probes<M>(lut, probes, nprobe, q, p0, p1, offsets, nlist, lb, le, codes, row_base, row_delta, m, k,
                                    stage1_k, buf_n, per_probe, tree, s_keys, s_lut, &s_cnt, &s_cut, rs);
            uint64_t* out = partial + (size_t)item * stage1_k;  // KEY_MAX beyond the valid keys
            for (int i = threadIdx.x; i < stage1_k; i += blockDim.x) out[i] = s_keys[i];
        } else {
            const int q = fail_list[nsplit + (item - nsplit * kFallbackSplit)];
            const int keep = fallback_scan_probes<M>(lut, probes, nprobe, q, 0, nprobe, offsets, nlist, lb, le, codes, row_base,
                                                     row_delta, m, k, stage1_k, buf_n, per_probe, tree, s_keys, s_lut, &s_cnt, &s_cut, rs);
            fallback_emit(s_keys, keep, q, stage1_k, out_rows, out_dist, out_count);
            if (threadIdx.x == 0) atomicAdd(&counters[2], 1ull);
        }
    }
}

// Combines the kFallbackSplit sorted partial lists of each split query: the same running top-k, fed with keys.
__global__ void __launch_bounds__(kFallbackThreads)
k_fallback_merge(const uint64_t* __restrict__ partial, int stage1_k, int buf_n, const int* __restrict__ fail_list,
                 const int* __restrict__ n_fail, int* __restrict__ out_rows, float* __restrict__ out_dist,
                 int* __restrict__ out_count, unsigned long long* __restrict__ counters) {
    extern __shared__ __align__(16) unsigned char s_raw_m[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_raw_m);  // [buf_n]
    __shared__ int s_cnt;
    __shared__ uint64_t s_cut;
    const int nf = *n_fail;
    const int f = blockIdx.x;
    if (f >= nf || f >= kFallbackCap) return;
    const int q = fail_list[f];
    if (threadIdx.x == 0) { s_cnt = 0; s_cut = KEY_MAX; atomicAdd(&counters[2], 1ull); }
    __syncthreads();
    const long long total = (long long)kFallbackSplit * stage1_k;
    const uint64_t* src = partial + (size_t)f * kFallbackSplit * stage1_k;
    for (long long base = 0; base < total; base += blockDim.x) {
        const int c_now = s_cnt;
        __syncthreads();
        if (c_now + (int)blockDim.x > buf_n) {  // uniform
            for (int i = c_now + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
            __syncthreads();
            block_bitonic_sort(s_keys, buf_n);
            if (threadIdx.x == 0) {
                const int keep = c_now < stage1_k ? c_now : stage1_k;
                s_cnt = keep;
                s_cut = keep == stage1_k ? s_keys[stage1_k - 1] : KEY_MAX;
            }
            __syncthreads();
        }
        const long long i = base + threadIdx.x;
        if (i < total) {
            const uint64_t key = src[i];
            if (key < s_cut) s_keys[atomicAdd(&s_cnt, 1)] = key;  // KEY_MAX padding never passes
        }
        __syncthreads();
    }
    const int c = s_cnt;
    for (int i = c + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
    __syncthreads();
    block_bitonic_sort(s_keys, buf_n);
    fallback_emit(s_keys, c < stage1_k ? c : stage1_k, q, stage1_k, out_rows, out_dist, out_count);
}

// ------------------------------------------------------------------------------------------------------
// Half-precision pre-filter variant of the scan: 8 visitors per work item.
//
// The 8 visitors' tables sit in shared memory as fp16, interleaved [m][code][8 visitors] = 16 bytes per entry, so one
// LDS.128 fetches 8 table entries and four HADD2 accumulate them.  The fp16 sum only decides which (row, visitor)
// pairs CAN be below the visitor's cutoff; those few are re-scored exactly (sequential fp32 sum from the fp32 table
// in global memory) before they are admitted, so the pools - and everything downstream - are identical to the
// fp32 kernel's.  No pair with exact distance <= cutoff is dropped:
//   table entries are e = RD_half(lut * s) (rounded toward -inf, s a power of two chosen so that no sum overflows),
//   half sums round to nearest: S~ <= (sum e)(1+2^-11)^(M-1) <= s * D * (1 + M * 2^-11 + 1e-4)   (D = exact fp32 sum),
//   so D <= cutoff implies S~ <= T := RU_half(cutoff * s * (1 + M * 2^-11 + 1e-4)); the kernel keeps pairs with S~ <= T.

constexpr int kHalfGroup = 8;
constexpr int kQueuePerWarp = 64;

// Power-of-two scale of a half table: the largest s with u * s <= 30000, u = sum over m of the table's row maxima.
__device__ __forceinline__ float half_table_scale(float u) {
    int ex = 0;
    if (u > 0.0f && u < 3.0e38f) ex = (int)floorf(log2f(30000.0f / u));
    ex = ex < -40 ? -40 : (ex > 40 ? 40 : ex);
    float sc = exp2f((float)ex);
    while (u * sc > 30000.0f) sc *= 0.5f;  // guard against log2f rounding
    return sc;
}

// Residual mode: the fp32 table of a (query, probe) pair and its fp16 copy in one kernel, without reading the fp32 table
// back.  One CTA of 256 threads per pair; thread c computes codeword c's entry for every sub-quantiser and writes both
// copies at once.  The fp16 scale needs no pass over the entries: an entry is at most (|r_m| + max_c |cb[m][c]|)^2
// (r_m: the residual's sub-vector), so s = largest power of two with s * 1.001 * sum_m (|r_m| + cbmax[m])^2 <= 30000 keeps
// every fp16 sum finite; fp16 being a floating-point format, a scale a few times below the tightest one costs no precision.
// (The table's fp16 copy may differ from k_lut_to_half's, which scales by the exact row maxima; the scan's results do
// not depend on the scale, only on the entries being rounded down and re-scored exactly.)  Needs codebook_size <= 256.
template <int M>
__global__ void __launch_bounds__(256)
k_build_tables_residual(const float* __restrict__ queries, int dim, const int* __restrict__ probes, int nprobe,
                        const float* __restrict__ centroids, int nlist, const float* __restrict__ codebook, int k,
                        const float* __restrict__ cb_maxnorm, float* __restrict__ lut, __half* __restrict__ lut_h,
                        float* __restrict__ scale_out) {
    extern __shared__ float s_q[];  // [dim] residual
    __shared__ float s_term[M];
    __shared__ float s_scale;
    const long long pair = blockIdx.x;
    const int q = (int)(pair / nprobe);
    const int l = probes[pair];
    if (l < 0 || l >= nlist) return;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        s_q[i] = __fsub_rn(queries[(size_t)q * dim + i], __ldg(centroids + (size_t)l * dim + i));
    __syncthreads();
    const int dsub = dim / M;
    if (threadIdx.x < M) {
        float n2 = 0.0f;
        for (int d = 0; d < dsub; ++d) n2 += s_q[threadIdx.x * dsub + d] * s_q[threadIdx.x * dsub + d];
        const float t = sqrtf(n2) + cb_maxnorm[threadIdx.x];
        s_term[threadIdx.x] = t * t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float u = 0.0f;
        for (int j = 0; j < M; ++j) u += s_term[j];
        const float sc = half_table_scale(u * 1.001f);
        s_scale = sc;
        scale_out[pair] = sc;
    }
    __syncthreads();
    const float sc = s_scale;
    const int c = threadIdx.x;
    if (c >= k) return;
    float* out = lut + (size_t)pair * M * k;
    __half* out_h = lut_h + (size_t)pair * M * k;
#pragma unroll 4
    for (int j = 0; j < M; ++j) {
        const float* cb = codebook + ((size_t)j * k + c) * dsub;
        float e = 0.0f;
        for (int d = 0; d < dsub; ++d) {
            const float diff = __fsub_rn(s_q[j * dsub + d], __ldg(cb + d));
            e = __fadd_rn(e, __fmul_rn(diff, diff));
        }
        out[(size_t)j * k + c] = e;
        out_h[(size_t)j * k + c] = __float2half_rd(e * sc);
    }
}

// Per query: scale s (power of two) with sum_m max_c lut[m][c] * s <= 30000, and the fp16 table RD_half(lut * s).
__global__ void k_lut_to_half(const float* __restrict__ lut, int m, int k, __half* __restrict__ lut_h,
                              float* __restrict__ scale_out) {
    __shared__ unsigned int s_max[64 + 1];
    __shared__ float s_scale;
    const int q = blockIdx.x;
    const int mk = m * k;
    for (int i = threadIdx.x; i < m; i += blockDim.x) s_max[i] = 0u;
    __syncthreads();
    for (int e = threadIdx.x; e < mk; e += blockDim.x) {
        const float v = lut[(size_t)q * mk + e];
        atomicMax(&s_max[e / k], __float_as_uint(v > 0.0f ? v : 0.0f));  // non-negative floats order like their bits
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float u = 0.0f;
        for (int i = 0; i < m; ++i) u += __uint_as_float(s_max[i]);
        const float sc = half_table_scale(u);
        s_scale = sc;
        scale_out[q] = sc;
    }
    __syncthreads();
    const float sc = s_scale;
    for (int e = threadIdx.x; e < mk; e += blockDim.x)
        lut_h[(size_t)q * mk + e] = __float2half_rd(lut[(size_t)q * mk + e] * sc);
}

// Affine u8 quantisation of fp32 tables, per sub-quantiser (reference: quantize_query_codeword_dot_lut_u8_kernel,
// src/search/kernels/fine/gpu_fine/pq_adc/pq_query_lut.cu:37-97): scale = max((hi - lo) / 255, 1e-6),
// u8 = clamp(rint((v - lo) / scale), 0, 255), lo_sum = sum of lo, inflation = sum of scale * (0.5 plain | 1 residual).
// One CTA per table; sub-quantisers one after the other, block-wide min / max.
__global__ void __launch_bounds__(256)
k_lut_to_u8(const float* __restrict__ lut, int m, int k, int residual, uint8_t* __restrict__ q8, float* __restrict__ scales,
            float* __restrict__ lo_sum, float* __restrict__ inflation) {
    __shared__ float s_lo[8], s_hi[8];
    __shared__ float s_mlo, s_mscale;
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float ls = 0.0f, inf = 0.0f;  // thread 0 only
    for (int j = 0; j < m; ++j) {
        const float* row = lut + (t * m + j) * k;
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (int c = threadIdx.x; c < k; c += blockDim.x) { const float v = row[c]; lo = fminf(lo, v); hi = fmaxf(hi, v); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
            float scale = __fdiv_rn(__fsub_rn(hi, lo), 255.0f);
            if (scale < 1e-6f) scale = 1e-6f;
            s_mlo = lo; s_mscale = scale;
            scales[t * m + j] = scale;
            ls = __fadd_rn(ls, lo);
            inf = __fadd_rn(inf, __fmul_rn(scale, residual ? 1.0f : 0.5f));
        }
        __syncthreads();
        const float mlo = s_mlo, mscale = s_mscale;
        for (int c = threadIdx.x; c < k; c += blockDim.x) {
            float r = rintf(__fdiv_rn(__fsub_rn(row[c], mlo), mscale));
            r = r < 0.0f ? 0.0f : (r > 255.0f ? 255.0f : r);
            q8[(t * m + j) * k + c] = (uint8_t)r;
        }
    }
    if (threadIdx.x == 0) { lo_sum[t] = ls; inflation[t] = inf; }
}

struct ScanArgsH {
    ScanArgs a;
    const __half* lut_h;   // [nq][m*k]
    const float* scale;    // [nq]
};

template <int M>
// launch bound 640 (> the 512 threads launched) caps the kernel at 96 registers, which leaves register-file room for the
// rerank's gather kernel to run beside it on every SM.
__global__ void __launch_bounds__(640, 1) k_scan_h(const ScanArgsH ah) {
    const ScanArgs& a = ah.a;
    constexpr int V = kHalfGroup;
    extern __shared__ __align__(16) unsigned char s_raw_h[];
    uint4* s_lut = reinterpret_cast<uint4*>(s_raw_h);  // [m*k] entries of 8 halves
    const int mk = a.m * a.k;
    unsigned long long* s_queue = reinterpret_cast<unsigned long long*>(s_raw_h + (size_t)mk * 16);  // [warps][kQueuePerWarp]
    __shared__ long long s_item;
    __shared__ int s_list, s_vq[V], s_pq[V];
    __shared__ float s_thr[V], s_T[V];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* queue = s_queue + warp * kQueuePerWarp;
    const long long total = a.item_off[a.nlist];
    const float slack = 1.0f + (float)a.m * (1.0f / 2048.0f) + 1e-4f;

    // Exact re-score of one queued (row, visitor) pair and admission into the visitor's pool.
    auto rescore = [&](unsigned long long entry, long long delta) {
        const long long r = (long long)(entry >> 3);
        const int v = (int)(entry & 7);
        const int q = s_pq[v];
        const float* lq = a.lut + (size_t)s_vq[v] * mk;
        const uint8_t* row = a.codes + (size_t)(r - a.row_base) * a.m;
        float d = 0.0f;
        bool done = false;
        if constexpr (M == 8 || M == 16) {
            if (a.tree) { d = adc_row_tree<M>(row, lq, a.k); done = true; }
        }
        if (done) {
        } else if constexpr (M % 16 == 0) {
            const uint4* p = reinterpret_cast<const uint4*>(row);
#pragma unroll
            for (int w = 0; w < M / 16; ++w) {
                const uint4 c = __ldg(p + w);
                const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    d = __fadd_rn(d, __ldg(lq + (w * 16 + j) * a.k + (int)((cw[j >> 2] >> ((j & 3) * 8)) & 255)));
            }
        } else {
            const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
#pragma unroll
            for (int w = 0; w < M / 4; ++w) {
                const uint32_t c = __ldg(p + w);
#pragma unroll
                for (int j = 0; j < 4; ++j) d = __fadd_rn(d, __ldg(lq + (w * 4 + j) * a.k + (int)((c >> (j * 8)) & 255)));
            }
        }
        if (d <= s_thr[v]) {
            const int slot = atomicAdd(&a.pool_cnt[q], 1);
            if (slot < a.pool_cap) a.pool[(size_t)q * a.pool_cap + slot] = make_key(d, (uint32_t)(r + delta));
        }
    };

    for (;;) {
        __syncthreads();  // previous item fully consumed
        if (threadIdx.x < 32) {
            long long item = 0;
            if (threadIdx.x == 0) item = (long long)atomicAdd(a.work_cursor, 1ull);
            item = __shfl_sync(0xffffffffu, item, 0);
            int l = -1;
            if (item < total) l = find_list(a.item_off, a.nlist, item);
            if (threadIdx.x == 0) { s_item = item; s_list = l; }
        }
        __syncthreads();
        const long long item = s_item;
        if (item >= total) break;
        const int l = s_list;
        const int nvis = a.vis_count[l];
        const int ngroups = (nvis + V - 1) / V;
        const long long local = item - a.item_off[l];
        const int group = (int)(local % ngroups);
        const long long chunk = local / ngroups;
        if (threadIdx.x < V) {
            const int vi = group * V + threadIdx.x;
            const int q = vi < nvis ? a.visitors[a.vis_off[l] + vi] : -1;  // table index
            s_vq[threadIdx.x] = q;
            s_pq[threadIdx.x] = q >= 0 ? q / a.lut_div : -1;               // query (pool, cutoff)
            float t = -1.0f, T = -1.0f;  // padding visitors admit nothing
            if (q >= 0) {
                t = a.thr[q / a.lut_div];
                T = __half2float(__float2half_ru(t * ah.scale[q] * slack));  // +inf stays +inf
            }
            s_thr[threadIdx.x] = t;
            s_T[threadIdx.x] = T;
        }
        __syncthreads();
        float T[V];
#pragma unroll
        for (int v = 0; v < V; ++v) T[v] = s_T[v];
        // stage the 8 fp16 tables, two consecutive entries per thread and round
        {
            const int q0 = s_vq[0];
            const __half2* src[V];
#pragma unroll
            for (int v = 0; v < V; ++v)
                src[v] = reinterpret_cast<const __half2*>(ah.lut_h + (size_t)(s_vq[v] >= 0 ? s_vq[v] : q0) * mk);
            for (int e2 = threadIdx.x; e2 < mk / 2; e2 += kScanThreads) {
                uint32_t w[V];
#pragma unroll
                for (int v = 0; v < V; ++v) w[v] = __ldg(reinterpret_cast<const unsigned int*>(src[v] + e2));
                uint4 lo, hi;  // entry 2*e2 takes the low halves, entry 2*e2+1 the high halves
                lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
                lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
                lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
                lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
                s_lut[2 * e2] = lo;
                s_lut[2 * e2 + 1] = hi;
            }
        }
        __syncthreads();
        const long long delta = a.row_delta ? a.row_delta[l] : 0;
        const long long r0 = a.offsets[l] + chunk * a.chunk_rows;
        const long long r1 = min(r0 + a.chunk_rows, a.offsets[l + 1]);
        int qcount = 0;  // warp-uniform
        for (long long base = r0 + warp * 32; base < r1; base += kScanThreads) {
            const long long r = base + lane;
            const bool valid = r < r1;
            const uint8_t* row = a.codes + (size_t)((valid ? r : r0) - a.row_base) * a.m;
            __half2 acc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = __float2half2_rn(0.0f);
            if constexpr (M % 16 == 0) {
                const uint4* p = reinterpret_cast<const uint4*>(row);
                uint4 c[M / 16];
#pragma unroll
                for (int w = 0; w < M / 16; ++w) c[w] = __ldg(p + w);
#pragma unroll
                for (int w = 0; w < M / 16; ++w) {
                    const uint32_t cw[4] = {c[w].x, c[w].y, c[w].z, c[w].w};
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint4 x = s_lut[(w * 16 + j) * a.k + (int)((cw[j >> 2] >> ((j & 3) * 8)) & 255)];
                        acc[0] = __hadd2(acc[0], *reinterpret_cast<const __half2*>(&x.x));
                        acc[1] = __hadd2(acc[1], *reinterpret_cast<const __half2*>(&x.y));
                        acc[2] = __hadd2(acc[2], *reinterpret_cast<const __half2*>(&x.z));
                        acc[3] = __hadd2(acc[3], *reinterpret_cast<const __half2*>(&x.w));
                    }
                }
            } else {
                const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
                uint32_t c[M / 4];
#pragma unroll
                for (int w = 0; w < M / 4; ++w) c[w] = __ldg(p + w);
#pragma unroll
                for (int w = 0; w < M / 4; ++w)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 x = s_lut[(w * 4 + j) * a.k + (int)((c[w] >> (j * 8)) & 255)];
                        acc[0] = __hadd2(acc[0], *reinterpret_cast<const __half2*>(&x.x));
                        acc[1] = __hadd2(acc[1], *reinterpret_cast<const __half2*>(&x.y));
                        acc[2] = __hadd2(acc[2], *reinterpret_cast<const __half2*>(&x.z));
                        acc[3] = __hadd2(acc[3], *reinterpret_cast<const __half2*>(&x.w));
                    }
            }
            float f[V];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 t = __half22float2(acc[i]);
                f[2 * i] = t.x; f[2 * i + 1] = t.y;
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const bool pass = valid && f[v] <= T[v];
                const unsigned bal = __ballot_sync(0xffffffffu, pass);
                if (bal) {
                    if (pass) queue[qcount + __popc(bal & ((1u << lane) - 1u))] = ((unsigned long long)r << 3) | (unsigned)v;
                    qcount += __popc(bal);
                    __syncwarp();
                    if (qcount >= 32) {
                        rescore(queue[lane], delta);
                        const unsigned long long moved = (32 + lane < qcount) ? queue[32 + lane] : 0ull;
                        __syncwarp();
                        if (32 + lane < qcount) queue[lane] = moved;
                        qcount -= 32;
                        __syncwarp();
                    }
                }
            }
        }
        if (lane < qcount) rescore(queue[lane], delta);
        __syncwarp();
    }
}

template <int M>
psb_status run_scan_h(const ScanArgsH& ah, int sm_count, cudaStream_t s) {
    if constexpr (M <= 0 || M % 4 != 0) {
        return fail(PSB_INTERNAL, "half scan needs a templated M");
    } else {
        const size_t smem = (size_t)ah.a.m * ah.a.k * 16 + (size_t)(kScanThreads / 32) * kQueuePerWarp * 8;
        if (smem > 32 * 1024)
            PSB_CUDA(cudaFuncSetAttribute(k_scan_h<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int occ = 0;
        PSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_scan_h<M>, kScanThreads, smem));
        if (occ < 1) return fail(PSB_UNSUPPORTED_SHAPE, "half scan kernel does not fit an SM");
        k_scan_h<M><<<scan_grid(sm_count * occ, ah.a.reserve_ctas), kScanThreads, smem, s>>>(ah);
        count_launch();
        PSB_LAUNCH_CHECK();
        return PSB_OK;
    }
}

// The half pre-filter needs a templated M (a multiple of 4), K even, and 8 tables + queues within shared memory.
bool half_scan_fits(int m, int k) {
    const bool templated = m == 8 || m == 16 || m == 20 || m == 32 || m == 48 || m == 64;
    return templated && (k % 2 == 0) && (size_t)m * k * 16 + (kScanThreads / 32) * kQueuePerWarp * 8 <= 220 * 1024;
}

// The reference's residual CPU scan sums M = 16 and M = 8 (K = 256) rows as a balanced pairwise tree and every other
// shape sequentially (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:307-341); the plain mode is always sequential.
bool tree_order(const ScanIndex& ix) { return ix.residual && ix.k == 256 && (ix.m == 16 || ix.m == 8); }

template <typename F>
psb_status set_smem(F kernel, size_t bytes) {
    if (bytes > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return PSB_OK;
}

template <int M, int V>
psb_status run_scan_kernel(const ScanArgs& a, int sm_count, cudaStream_t s) {
    const size_t smem = (size_t)a.m * a.k * V * sizeof(float);
    PSB_TRY(set_smem(k_scan<M, V>, smem));
    int occ = 0;
    PSB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_scan<M, V>, kScanThreads, smem));
    if (occ < 1) return fail(PSB_UNSUPPORTED_SHAPE, "scan kernel does not fit an SM");
    k_scan<M, V><<<scan_grid(sm_count * occ, a.reserve_ctas), kScanThreads, smem, s>>>(a);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

// Visitor-group width: as many tables as fit ~200 KB of shared memory, 4 at most.
int pick_group(int m, int k) {
    const size_t one = (size_t)m * k * sizeof(float);
    if (4 * one <= 200 * 1024) return 4;
    if (2 * one <= 200 * 1024) return 2;
    return 1;
}

template <int M>
psb_status run_scan_m(const ScanArgs& a, int group, int sm_count, cudaStream_t s) {
    switch (group) {
        case 4: return run_scan_kernel<M, 4>(a, sm_count, s);
        case 2: return run_scan_kernel<M, 2>(a, sm_count, s);
        default: return run_scan_kernel<M, 1>(a, sm_count, s);
    }
}

// Safety margin of the sampled cutoff in standard deviations (ScanWorkspace::seed_sigma; 4 unless the caller set 2..10).
// Margin of a cutoff shared by several shards: a cutoff placed too low there costs the caller a second pass over the whole
// batch, so the margin is wider than for one shard, where the exact fallback repairs a single query.
float shared_cut_sigma(const ScanWorkspace& ws) { return ws.seed_sigma >= 6.f && ws.seed_sigma <= 10.f ? ws.seed_sigma : 6.0f; }
float seed_margin_sigma(const ScanWorkspace& ws) { return ws.seed_sigma >= 2.f && ws.seed_sigma <= 10.f ? ws.seed_sigma : 4.0f; }

template <int M>
psb_status run_seed(const ScanIndex& ix, const ScanWorkspace& ws, const float* d_lut, int nq, const int* d_probes,
                    int nprobe, int stage1_k, cudaStream_t s, const ResidualSource& rs) {
    const size_t smem = (size_t)ix.m * ix.k * sizeof(float) + kSeedBuf * sizeof(uint32_t) + ((size_t)nprobe + 1) * sizeof(int) +
                        (size_t)nprobe * sizeof(float);
    if (ix.residual && !d_lut && !rs.row_bias && !rs.row_bias_u16) return fail(PSB_INTERNAL, "residual scan without tables: the per-row correction is missing");
    PSB_TRY(set_smem(k_seed_threshold<M>, smem));
    PSB_TRY(prefer_max_shared(k_seed_threshold<M>));
    k_seed_threshold<M><<<nq, kSeedThreads, smem, s>>>(d_lut, d_probes, nprobe, ix.offsets, ix.nlist, ix.list_begin,
                                                         ix.list_end, ix.codes, ix.row_base, ix.m, ix.k, ws.q_rows,
                                                         stage1_k, ws.pool_cap, ws.thr, ix.residual ? 1 : 0,
                                                         tree_order(ix) ? 1 : 0, ws.phase == 1 ? shared_cut_sigma(ws) : seed_margin_sigma(ws),
                                                         seed_margin_sigma(ws) - 2.0f, rs, ws.phase == 1 ? ws.seed_export : nullptr, ws.seed_keys);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

template <int M>
psb_status run_fallback(const ScanIndex& ix, const ScanWorkspace& ws, const float* d_lut, const int* d_probes,
                        int nprobe, int stage1_k, int* d_rows, float* d_dist, int* d_count, int sm_count,
                        cudaStream_t s, const ResidualSource& rs) {
    int buf_n = 2 * 1024;
    while (buf_n < stage1_k + kFallbackThreads) buf_n <<= 1;
    const size_t smem = (size_t)buf_n * 8 + (size_t)ix.m * ix.k * sizeof(float);
    PSB_TRY(set_smem(k_exact_fallback<M>, smem));
    PSB_TRY(prefer_max_shared(k_exact_fallback<M>));
    k_exact_fallback<M><<<sm_count, kFallbackThreads, smem, s>>>(
        d_lut, d_probes, nprobe, ix.offsets, ix.nlist, ix.list_begin, ix.list_end, ix.codes, ix.row_base, ix.row_delta, ix.m, ix.k,
        stage1_k, buf_n, ws.fail_list, ws.n_fail, ws.fail_cursor, d_rows, d_dist, d_count, ws.counters,
        ix.residual ? 1 : 0, tree_order(ix) ? 1 : 0, ws.fallback_partial, rs);
    count_launch();
    PSB_LAUNCH_CHECK();
    const size_t msmem = (size_t)buf_n * 8;
    PSB_TRY(set_smem(k_fallback_merge, msmem));
    PSB_TRY(prefer_max_shared(k_fallback_merge));
    k_fallback_merge<<<kFallbackCap, kFallbackThreads, msmem, s>>>(ws.fallback_partial, stage1_k, buf_n, ws.fail_list, ws.n_fail,
                                                                  d_rows, d_dist, d_count, ws.counters);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

#define PSB_DISPATCH_M(m_value, CALL)                 \
    switch (m_value) {                                \
        case 8: { constexpr int MM = 8; CALL; } break;   \
        case 16: { constexpr int MM = 16; CALL; } break; \
        case 20: { constexpr int MM = 20; CALL; } break; \
        case 32: { constexpr int MM = 32; CALL; } break; \
        case 48: { constexpr int MM = 48; CALL; } break; \
        case 64: { constexpr int MM = 64; CALL; } break; \
        default: { constexpr int MM = 0; CALL; } break;  \
    }

}  // namespace

int seed_record_keys(int stage1_k, float sigma) {
    const float s = sigma >= 6.f && sigma <= 10.f ? sigma : 6.0f;   // the margin of the shared cutoff
    const float mu = (float)stage1_k / 16.0f + 16.0f;   // the smallest stride is 16; the ceilings of the per-list sample counts add a little
    float c = mu;
    for (int it = 0; it < 6; ++it) c = mu + s * std::sqrt(c) + 2.0f;
    const int r = (int)std::ceil(c) + 8;
    return (r + 31) / 32 * 32;
}

psb_status launch_build_lut(const float* d_queries, int nq, int dim, const float* d_codebook, int m, int k,
                            float* d_lut, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    PSB_TRY(prefer_max_shared(k_build_lut));
    k_build_lut<<<nq, 256, (size_t)dim * sizeof(float), s>>>(d_queries, dim, d_codebook, m, k, d_lut);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_lut_to_u8(const float* d_lut, long long tables, int m, int k, int residual, uint8_t* d_q8, float* d_scales,
                            float* d_lo_sum, float* d_inflation, cudaStream_t s) {
    if (tables <= 0) return PSB_OK;
    if (tables > 0x7fffffffLL) return fail(PSB_UNSUPPORTED_SHAPE, "too many tables in one call");
    k_lut_to_u8<<<(unsigned)tables, 256, 0, s>>>(d_lut, m, k, residual, d_q8, d_scales, d_lo_sum, d_inflation);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_build_lut_residual(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe,
                                     const float* d_centroids, int nlist, const float* d_codebook, int m, int k,
                                     float* d_lut, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    const long long pairs = (long long)nq * nprobe;
    if (pairs > 0x7fffffffLL) return fail(PSB_UNSUPPORTED_SHAPE, "too many (query, probe) pairs in one batch");
    PSB_TRY(prefer_max_shared(k_build_lut_residual));
    k_build_lut_residual<<<(unsigned)pairs, 256, (size_t)dim * sizeof(float), s>>>(d_queries, dim, d_probes, nprobe,
                                                                                   d_centroids, nlist, d_codebook, m, k, d_lut);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

template <int M>
psb_status run_build_tables_residual(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe,
                                     const float* d_centroids, int nlist, const float* d_codebook, int k,
                                     const float* d_cb_maxnorm, float* d_lut, void* d_lut_h, float* d_scale, cudaStream_t s) {
    if constexpr (M <= 0) {
        return fail(PSB_INTERNAL, "fused residual tables need a templated M");
    } else {
        PSB_TRY(prefer_max_shared(k_build_tables_residual<M>));
        k_build_tables_residual<M><<<(unsigned)((long long)nq * nprobe), 256, (size_t)dim * sizeof(float), s>>>(
            d_queries, dim, d_probes, nprobe, d_centroids, nlist, d_codebook, k, d_cb_maxnorm, d_lut, static_cast<__half*>(d_lut_h),
            d_scale);
        count_launch();
        PSB_LAUNCH_CHECK();
        return PSB_OK;
    }
}

size_t fallback_partial_bytes(int stage1_k) { return (size_t)kFallbackCap * kFallbackSplit * stage1_k * sizeof(uint64_t); }

bool residual_tables_fused(const ScanWorkspace& ws, int m, int k) {
    return ws.lut_h != nullptr && ws.scan_mode != 1 && half_scan_fits(m, k) && k <= 256;
}

psb_status launch_build_tables_residual(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe,
                                        const float* d_centroids, int nlist, const float* d_codebook, int m, int k,
                                        const float* d_cb_maxnorm, float* d_lut, const ScanWorkspace& ws, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    if ((long long)nq * nprobe > 0x7fffffffLL) return fail(PSB_UNSUPPORTED_SHAPE, "too many (query, probe) pairs in one batch");
    if (!d_cb_maxnorm) return fail(PSB_INTERNAL, "codeword norms missing");
    PSB_DISPATCH_M(m, PSB_TRY((run_build_tables_residual<MM>(d_queries, nq, dim, d_probes, nprobe, d_centroids, nlist, d_codebook,
                                                             k, d_cb_maxnorm, d_lut, ws.lut_h, ws.lut_scale, s))));
    return PSB_OK;
}

psb_status launch_scan(const ScanIndex& ix, const ScanWorkspace& ws, const float* d_lut, int nq,
                       const int* d_probes, int nprobe, int stage1_k, int* d_rows, float* d_dist,
                       int* d_count, int sm_count, cudaStream_t s, const float* d_queries) {
    if (nq <= 0) return PSB_OK;
    const long long tables = ix.residual ? (long long)nq * nprobe : nq;
    if (tables > 0x7fffffffLL) return fail(PSB_UNSUPPORTED_SHAPE, "too many (query, probe) pairs in one batch");
    // Tensor-core pre-filter: needs the queries, the centroids and the codebook, a supported shape, and a selection that fits.
    const bool tc_possible = d_queries != nullptr && ix.centroids != nullptr && ix.codebook != nullptr && ix.dim == ix.m * (ix.dim / ix.m) &&
                             ws.item_off_tc != nullptr && ws.work_cursor_tc != nullptr && ws.tc_status != nullptr &&
                             ix.row_aug != nullptr && scan_tc_supported(ix.dim, ix.m, ix.k) &&
                             (size_t)ws.pool_cap * 8 + (ix.residual ? (size_t)ix.dim * 4 : (size_t)ix.m * ix.k * 4) <= (size_t)226 * 1024;
    if (ws.scan_mode == 3 && !tc_possible) return fail(PSB_UNSUPPORTED_SHAPE, "the tensor-core scan does not support this call (shape, or no queries given)");
    const bool use_tc = tc_possible && (ws.scan_mode == 0 || ws.scan_mode == 3);
    const int tc_min_vis = use_tc ? (ws.tc_min_visitors > 0 ? ws.tc_min_visitors : 1) : 0;
    const bool simt_needed = !use_tc || tc_min_vis > 1;  // lists below the visitor limit stay with the SIMT scan
    // Without tables (d_lut null): residual mode only, and only when the tensor-core scan takes every list - the cutoff, the
    // re-scoring and the fallback then build what they need from the queries, the centroids and the codebook.
    if (!d_lut && !(ix.residual && use_tc && !simt_needed))
        return fail(PSB_INVALID_ARGUMENT, "the scan needs the lookup tables (they may be left out only in residual mode with the tensor-core scan)");
    const bool use_half = simt_needed && ws.lut_h != nullptr && ws.scan_mode != 1 && half_scan_fits(ix.m, ix.k);
    if (nq > ws.cap_queries || (use_half && tables > ws.cap_tables))
        return fail(PSB_INTERNAL, "scan workspace holds " + std::to_string(ws.cap_queries) + " queries / " + std::to_string(ws.cap_tables) +
                                      " tables, the call needs " + std::to_string(nq) + " / " + std::to_string(tables));
    const int group = use_half ? kHalfGroup : pick_group(ix.m, ix.k);
    if (ws.phase == 1 && (!ws.seed_export || ws.seed_keys <= 0)) return fail(PSB_INTERNAL, "scan phase 1 without a record buffer");
    if (ws.phase == 2 && (!ws.seed_all || ws.seed_shards <= 0 || ws.seed_keys <= 0)) return fail(PSB_INTERNAL, "scan phase 2 without the shards' records");
    ResidualSource rs;
    rs.queries = d_queries; rs.centroids = ix.centroids; rs.codebook = ix.codebook; rs.row_bias = ix.row_bias; rs.row_bias_u16 = ix.row_bias_u16; rs.rc_scale = ix.rc_scale; rs.rc_offset = ix.rc_offset; rs.dim = ix.dim;
    if (ws.phase != 2) {
    // schedule
    PSB_CUDA(cudaMemsetAsync(ws.vis_count, 0, sizeof(int) * (size_t)ix.nlist, s));
    PSB_CUDA(cudaMemsetAsync(ws.pool_cnt, 0, sizeof(int) * (size_t)nq, s));
    PSB_CUDA(cudaMemsetAsync(ws.n_fail, 0, sizeof(int), s));
    PSB_CUDA(cudaMemsetAsync(ws.fail_cursor, 0, sizeof(int), s));
    PSB_CUDA(cudaMemsetAsync(ws.work_cursor, 0, sizeof(unsigned long long), s));
    if (use_tc) PSB_CUDA(cudaMemsetAsync(ws.work_cursor_tc, 0, sizeof(unsigned long long), s));
    PSB_TRY(prefer_max_shared(k_count_visitors));
    k_count_visitors<<<(nq * 32 + 255) / 256, 256, 0, s>>>(d_probes, nq, nprobe, ix.offsets, ix.nlist, ix.list_begin,
                                                          ix.list_end, ws.vis_count, ws.q_rows, ws.counters);
    count_launch();
    PSB_LAUNCH_CHECK();
    PSB_TRY(prefer_max_shared(k_scan_lists));
    k_scan_lists<<<1, 1024, 0, s>>>(ws.vis_count, ix.offsets, ix.nlist, group, kScanChunkRows, ws.vis_off,
                                    ws.item_off, ws.vis_cursor, 128, tc_min_vis, use_tc ? ws.item_off_tc : nullptr);
    count_launch();
    PSB_LAUNCH_CHECK();
    const long long pairs = (long long)nq * nprobe;
    PSB_TRY(prefer_max_shared(k_fill_visitors));
    k_fill_visitors<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>(d_probes, nq, nprobe, ix.nlist, ix.list_begin,
                                                                    ix.list_end, ws.vis_off, ws.vis_cursor, ws.visitors,
                                                                    ix.residual ? 1 : 0);
    count_launch();
    PSB_LAUNCH_CHECK();
    // cutoff
    PSB_DISPATCH_M(ix.m, PSB_TRY((run_seed<MM>(ix, ws, d_lut, nq, d_probes, nprobe, stage1_k, s, rs))));
    }
    if (ws.phase == 1) return PSB_OK;
    if (ws.phase == 2) {   // the cutoff from every shard's sample records
        const int n = ws.seed_shards * ws.seed_keys;
        int np = 2;
        while (np < n) np <<= 1;
        const size_t smem = (size_t)np * sizeof(uint64_t);
        if (smem > (size_t)200 * 1024) return fail(PSB_UNSUPPORTED_SHAPE, "too many shards for the shared cutoff");
        PSB_TRY(set_smem(k_pick_cutoff, smem));
        PSB_TRY(prefer_max_shared(k_pick_cutoff));
        k_pick_cutoff<<<nq, kPickThreads, smem, s>>>(ws.seed_all, ws.seed_shards, nq, ws.seed_keys, stage1_k, shared_cut_sigma(ws), ws.thr,
                                                     ws.rows_global);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    // scan
    ScanArgs a;
    a.lut = d_lut; a.lut_div = ix.residual ? nprobe : 1; a.tree = tree_order(ix) ? 1 : 0; a.codes = ix.codes; a.offsets = ix.offsets; a.row_base = ix.row_base; a.row_delta = ix.row_delta;
    a.nlist = ix.nlist; a.m = ix.m; a.k = ix.k;
    a.vis_count = ws.vis_count; a.vis_off = ws.vis_off; a.visitors = ws.visitors; a.item_off = ws.item_off;
    a.thr = ws.thr; a.pool_cnt = ws.pool_cnt; a.pool = ws.pool; a.pool_cap = ws.pool_cap;
    a.work_cursor = ws.work_cursor; a.counters = ws.counters; a.chunk_rows = kScanChunkRows;
    a.reserve_ctas = ws.reserve_ctas;
    if (use_half && !ws.half_tables_ready && simt_needed) {
        PSB_TRY(prefer_max_shared(k_lut_to_half));
        k_lut_to_half<<<(unsigned)tables, 256, 0, s>>>(d_lut, ix.m, ix.k, reinterpret_cast<__half*>(ws.lut_h), ws.lut_scale);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    if (ws.ev_begin) PSB_CUDA(cudaEventRecord(ws.ev_begin, s));
    if (use_tc) {
        ScanTcLaunch L;
        L.queries = d_queries; L.centroids = ix.centroids; L.codebook = ix.codebook; L.probes = d_probes; L.row_aug = ix.row_aug;
        L.codes = ix.codes; L.offsets = ix.offsets; L.row_base = ix.row_base; L.nlist = ix.nlist; L.dim = ix.dim; L.m = ix.m; L.k = ix.k;
        L.lut_div = a.lut_div; L.residual = ix.residual; L.vis_count = ws.vis_count; L.vis_off = ws.vis_off; L.visitors = ws.visitors;
        L.item_off = ws.item_off_tc; L.thr = ws.thr; L.pool_cnt = ws.pool_cnt; L.pool = ws.pool; L.pool_cap = ws.pool_cap;
        L.work_cursor = ws.work_cursor_tc; L.counters = ws.counters; L.status = ws.tc_status; L.chunk_rows = kScanChunkRows;
        L.reserve_ctas = ws.reserve_ctas; L.sm_count = sm_count; L.wait_limit = ws.tc_wait_limit; L.skip_mma = ws.tc_skip_mma;
        PSB_TRY(launch_scan_tc(L, s));
    }
    if (simt_needed) {
        if (use_half) {
            ScanArgsH ah;
            ah.a = a; ah.lut_h = reinterpret_cast<const __half*>(ws.lut_h); ah.scale = ws.lut_scale;
            PSB_DISPATCH_M(ix.m, PSB_TRY((run_scan_h<MM>(ah, sm_count, s))));
        } else {
            PSB_DISPATCH_M(ix.m, PSB_TRY((run_scan_m<MM>(a, group, sm_count, s))));
        }
    }
    if (ws.ev_end) PSB_CUDA(cudaEventRecord(ws.ev_end, s));
    // selection
    if (use_tc) {  // pools may hold unscored survivors of the tensor-core filter: the selection re-scores them exactly
        SelectRescoreLaunch R;
        R.pool = ws.pool; R.pool_cnt = ws.pool_cnt; R.pool_cap = ws.pool_cap; R.q_rows = ws.q_rows; R.thr = ws.thr; R.stage1_k = stage1_k;
        R.lut = d_lut; R.queries = d_queries; R.centroids = ix.centroids; R.codebook = ix.codebook; R.probes = d_probes;
        R.nprobe = nprobe; R.dim = ix.dim; R.nlist = ix.nlist; R.codes = ix.codes; R.row_base = ix.row_base; R.row_delta = ix.row_delta;
        R.m = ix.m; R.k = ix.k; R.residual = ix.residual; R.tree = tree_order(ix);
        R.out_rows = d_rows; R.out_dist = d_dist; R.out_count = d_count; R.fail_list = ws.fail_list; R.n_fail = ws.n_fail;
        R.counters = ws.counters; R.shared_cut = ws.phase == 2;
        PSB_TRY(launch_select_rescore(R, nq, s));
    } else {
        const size_t smem = (size_t)ws.pool_cap * sizeof(uint64_t);
        PSB_TRY(set_smem(k_select_pool, smem));
        PSB_TRY(prefer_max_shared(k_select_pool));
        k_select_pool<<<nq, kSelectThreads, smem, s>>>(ws.pool, ws.pool_cnt, ws.pool_cap, ws.q_rows, stage1_k, d_rows,
                                                       d_dist, d_count, ws.fail_list, ws.n_fail, ws.counters,
                                                       ws.phase == 2 ? ws.thr : nullptr);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    PSB_DISPATCH_M(ix.m, PSB_TRY((run_fallback<MM>(ix, ws, d_lut, d_probes, nprobe, stage1_k, d_rows, d_dist, d_count,
                                                  sm_count, s, rs))));
    return PSB_OK;
}

}  // namespace psb
