// Exact rerank of the ADC candidates, id mapping and the multi-shard candidate merge.
//
//   k_gather_rows     copies each candidate's exact row (fp32 or u8) from the exact store - host memory mapped
//                     into the device address space and read over PCIe, or device memory - into a dense staging
//                     buffer in HBM; one warp per row, 16-byte loads.  Rows this session does not hold (other
//                     shards' rows, invalid ids) are skipped.
//   k_rerank_score    half-warps score staged rows in the accumulation order of the CPU kernel the reference uses
//                     (four 16-lane FMA accumulators, pairwise combine, halving tree:
//                     src/cpu/distance/fp32_l2_avx512.h:16-53); rows not held here score +inf
//   k_topk_select     one CTA per query: bitonic sort of (distance,row) keys, duplicate rows collapse, the first
//                     topk are written (reference semantics: src/search/ivf_common/ivf_host_rerank.cpp:152-177,
//                     src/search/ivf_common/ivf_exact_topk.h:12-22)
#include <cstdlib>
#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace {

__device__ __forceinline__ int cand_count(const int* counts, int q, int candidate_count) {
    if (!counts) return candidate_count;
    const int c = counts[q];
    return c < 0 ? 0 : (c > candidate_count ? candidate_count : c);
}

// Global (index-wide, list-contiguous) row -> row of this session's exact store, or -1 when not held here.
__device__ __forceinline__ long long local_row(const RowMap& mp, long long r) {
    if (r < 0) return -1;
    if (!mp.global_begin) {
        const long long l = r - mp.base;
        return (l >= 0 && l < mp.count) ? l : -1;
    }
    int lo = 0, hi = mp.nlist;  // largest list with global_begin[list] <= r
    if (r < mp.global_begin[0]) return -1;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (mp.global_begin[mid] <= r) lo = mid; else hi = mid;
    }
    const long long l = mp.local_offsets[lo] + (r - mp.global_begin[lo]);
    return l < mp.local_offsets[lo + 1] ? l : -1;
}

// Gathers candidate rows into the staging buffer.  A warp takes 32 candidates at a time: every lane resolves one candidate
// to a local row (for a striped shard that is a binary search of 16 dependent loads - done for 32 candidates at once), then
// the warp copies the rows four at a time, all four rows' loads issued before the first store, so that a few hundred KB
// of PCIe reads stay in flight even on a small grid.
template <int U = 4>
__device__ __forceinline__ void gather_rows_body(const unsigned char* __restrict__ src, const RowMap& mp, int row_bytes,
                                                 const int* __restrict__ cand, int nq, int candidate_count, int candidate_stride,
                                                 const int* __restrict__ counts, unsigned char* __restrict__ stage) {
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = (long long)nq * candidate_count;
    const uintptr_t both = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(stage);
    const bool vec16 = (row_bytes % 16) == 0 && (both % 16) == 0;
    const bool vec4 = (row_bytes % 4) == 0 && (both % 4) == 0;
    const int n16 = row_bytes / 16;
    for (long long base = warp0 * 32; base < total; base += nwarps * 32) {
        long long mine = -1;
        const long long w = base + lane;
        if (w < total) {
            const int q = (int)(w / candidate_count), i = (int)(w % candidate_count);
            if (i < cand_count(counts, q, candidate_count)) mine = local_row(mp, cand[(size_t)q * candidate_stride + i]);
        }
        if (vec16 && n16 <= 32) {
            // The rows held here, four at a time whatever their positions among the 32 candidates: on a shard most candidates
            // belong to other shards, and the reads in flight must not thin out with them.
            unsigned present = __ballot_sync(0xffffffffu, mine >= 0);
#pragma unroll 1
            while (present) {
                int at[U];
                long long r[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    at[u] = present ? __ffs(present) - 1 : -1;   // uniform across the warp
                    if (present) present &= present - 1;
                    r[u] = __shfl_sync(0xffffffffu, mine, at[u] < 0 ? 0 : at[u]);
                }
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (at[u] >= 0 && lane < n16) v[u] = reinterpret_cast<const uint4*>(src + (size_t)r[u] * row_bytes)[lane];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (at[u] >= 0 && lane < n16) reinterpret_cast<uint4*>(stage + (size_t)(base + at[u]) * row_bytes)[lane] = v[u];
            }
        } else {
            for (int k = 0; k < 32; ++k) {
                const long long row = __shfl_sync(0xffffffffu, mine, k);
                if (row < 0) continue;
                const unsigned char* sp = src + (size_t)row * row_bytes;
                unsigned char* d = stage + (size_t)(base + k) * row_bytes;
                if (vec16) {
                    for (int j = lane; j < n16; j += 32) reinterpret_cast<uint4*>(d)[j] = reinterpret_cast<const uint4*>(sp)[j];
                } else if (vec4) {
                    for (int j = lane; j < row_bytes / 4; j += 32) reinterpret_cast<uint32_t*>(d)[j] = reinterpret_cast<const uint32_t*>(sp)[j];
                } else {
                    for (int j = lane; j < row_bytes; j += 32) d[j] = sp[j];
                }
            }
        }
    }
}

__global__ void k_gather_rows(const unsigned char* __restrict__ src, RowMap mp, int row_bytes,
                              const int* __restrict__ cand, int nq, int candidate_count, int candidate_stride,
                              const int* __restrict__ counts, unsigned char* __restrict__ stage) {
    gather_rows_body(src, mp, row_bytes, cand, nq, candidate_count, candidate_stride, counts, stage);
}
// The same gather built to sit BESIDE a scan kernel that owns nearly a whole SM (one 576-thread CTA with ~55K registers and
// ~200 KB of shared memory): 128-thread CTAs capped at 40 registers and no shared memory, two of which fit into what the
// scan leaves of every SM.  Spread over all SMs they keep far more PCIe reads in flight than the link's bandwidth-delay
// product while taking almost no issue slots (their warps wait on loads).
__global__ void __launch_bounds__(256, 6) k_gather_rows_beside(const unsigned char* __restrict__ src, RowMap mp, int row_bytes,
                                                               const int* __restrict__ cand, int nq, int candidate_count,
                                                               int candidate_stride, const int* __restrict__ counts,
                                                               unsigned char* __restrict__ stage) {
    gather_rows_body(src, mp, row_bytes, cand, nq, candidate_count, candidate_stride, counts, stage);
}

// The same gather on SMs of its own: CTAs of 1,024 threads that also claim (without using it) nearly all the shared memory of
// an SM, so that no kernel with a shared-memory footprint - the scan, the cutoff sampling, the selections - shares an SM with
// them.  Reads of host memory stay in flight for microseconds; next to another kernel's warps they held up that kernel's own
// memory traffic (its stages ran at half speed), on separate SMs they do not.  Eight such CTAs keep ~800 KB of reads in
// flight.
__global__ void __launch_bounds__(1024, 1) k_gather_rows_owned(const unsigned char* __restrict__ src, RowMap mp, int row_bytes,
                                                               const int* __restrict__ cand, int nq, int candidate_count,
                                                               int candidate_stride, const int* __restrict__ counts,
                                                               unsigned char* __restrict__ stage) {
    gather_rows_body<8>(src, mp, row_bytes, cand, nq, candidate_count, candidate_stride, counts, stage);   // eight rows per warp in flight
}

// fp32 squared L2 by a half-warp (16 lanes), bit-identical to the AVX-512 kernel's order.
// All 16 lanes of the half-warp must call it together; hmask names exactly those lanes.
__device__ __forceinline__ float l2_halfwarp(const float* __restrict__ q, const float* __restrict__ v, int dim, int j,
                                             unsigned hmask) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int i = 0;
    for (; i + 64 <= dim; i += 64) {
        float d = __fsub_rn(q[i + j], v[i + j]); a0 = __fmaf_rn(d, d, a0);
        d = __fsub_rn(q[i + 16 + j], v[i + 16 + j]); a1 = __fmaf_rn(d, d, a1);
        d = __fsub_rn(q[i + 32 + j], v[i + 32 + j]); a2 = __fmaf_rn(d, d, a2);
        d = __fsub_rn(q[i + 48 + j], v[i + 48 + j]); a3 = __fmaf_rn(d, d, a3);
    }
    for (; i + 16 <= dim; i += 16) {
        const float d = __fsub_rn(q[i + j], v[i + j]); a0 = __fmaf_rn(d, d, a0);
    }
    float s = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
    s = __fadd_rn(s, __shfl_xor_sync(hmask, s, 8));
    s = __fadd_rn(s, __shfl_xor_sync(hmask, s, 4));
    s = __fadd_rn(s, __shfl_xor_sync(hmask, s, 2));
    s = __fadd_rn(s, __shfl_xor_sync(hmask, s, 1));
    for (; i < dim; ++i) { const float d = __fsub_rn(q[i], v[i]); s = __fmaf_rn(d, d, s); }
    return s;
}

__device__ __forceinline__ float l2_u8_halfwarp(const unsigned char* __restrict__ q, const unsigned char* __restrict__ v,
                                                int dim, int j, unsigned hmask) {
    int s = 0;
    for (int i = j; i < dim; i += 16) { const int d = (int)q[i] - (int)v[i]; s += d * d; }
    s += __shfl_xor_sync(hmask, s, 8);
    s += __shfl_xor_sync(hmask, s, 4);
    s += __shfl_xor_sync(hmask, s, 2);
    s += __shfl_xor_sync(hmask, s, 1);
    return (float)s;
}

constexpr int kScoreThreads = 256;
// grid (nq, ceil(candidate_count / 16 half-warps)): dist[q][i] = exact distance of candidate i, +inf when the row is
// invalid, beyond the query's count, or not held by this session.
__global__ void __launch_bounds__(kScoreThreads)
k_rerank_score(const unsigned char* __restrict__ stage, RowMap mp, int dim, int elem_bytes,
               const unsigned char* __restrict__ queries, const int* __restrict__ cand, int candidate_count,
               int candidate_stride, const int* __restrict__ counts, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) unsigned char s_q[];
    const int q = blockIdx.x;
    const int row_bytes = dim * elem_bytes;
    for (int i = threadIdx.x; i < row_bytes; i += blockDim.x) s_q[i] = queries[(size_t)q * row_bytes + i];
    __syncthreads();
    const int n = cand_count(counts, q, candidate_count);
    const int hw = threadIdx.x >> 4, j = threadIdx.x & 15;
    const unsigned hmask = 0xffffu << (threadIdx.x & 16);
    const int i = blockIdx.y * (kScoreThreads / 16) + hw;
    if (i >= candidate_count) return;
    float d = __int_as_float(0x7f800000);
    const long long row = i < n ? local_row(mp, cand[(size_t)q * candidate_stride + i]) : -1;
    if (row >= 0) {
        const unsigned char* v = stage + ((size_t)q * candidate_count + i) * row_bytes;
        d = elem_bytes == 4
            ? l2_halfwarp(reinterpret_cast<const float*>(s_q), reinterpret_cast<const float*>(v), dim, j, hmask)
            : l2_u8_halfwarp(s_q, v, dim, j, hmask);
    }
    if (j == 0) out_dist[(size_t)q * candidate_count + i] = d;
}

constexpr int kSelectThreads = 256;
// dist [nq][candidate_count] (dense), cand [nq][candidate_stride] global rows.
__global__ void __launch_bounds__(kSelectThreads)
k_topk_select(const float* __restrict__ dist, const int* __restrict__ cand, int candidate_count, int candidate_stride,
              const int* __restrict__ counts, int topk, int np, int* __restrict__ out_rows, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_raw);         // [np]
    int* s_rank = reinterpret_cast<int*>(s_raw + (size_t)np * 8);  // [np]
    __shared__ int s_warp[32];
    __shared__ int s_total;
    const int q = blockIdx.x;
    const int n = cand_count(counts, q, candidate_count);
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        uint64_t key = KEY_MAX;
        if (i < n) {
            const int row = cand[(size_t)q * candidate_stride + i];
            const float d = dist[(size_t)q * candidate_count + i];
            if (row >= 0 && d != __int_as_float(0x7f800000)) key = make_key(d, (uint32_t)row);
        }
        s_keys[i] = key;
    }
    __syncthreads();
    block_bitonic_sort(s_keys, np);
    // duplicates are adjacent (same row -> same distance -> same key): keep the first of each run
    int base = 0;
    for (int c0 = 0; c0 < np; c0 += blockDim.x) {
        const int i = c0 + threadIdx.x;
        int keep = 0;
        if (i < np) {
            const uint64_t key = s_keys[i];
            keep = key != KEY_MAX && (i == 0 || s_keys[i - 1] != key);
        }
        const int ex = block_exclusive_scan(keep, s_warp, &s_total);
        if (i < np) s_rank[i] = keep ? base + ex : -1;
        base += s_total;
        __syncthreads();
    }
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        const int r = s_rank[i];
        if (r >= 0 && r < topk) {
            out_rows[(size_t)q * topk + r] = (int)key_idx(s_keys[i]);
            out_dist[(size_t)q * topk + r] = key_dist(s_keys[i]);
        }
    }
    for (int r = base + threadIdx.x; r < topk; r += blockDim.x) {
        out_rows[(size_t)q * topk + r] = -1;
        out_dist[(size_t)q * topk + r] = FLT_MAX;
    }
}

// out[i] = original id of global row rows[i] when this session holds the row, else -1.
__global__ void k_map_ids(const int* __restrict__ rows, long long n, const long long* __restrict__ reordered, RowMap mp,
                          long long* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long l = local_row(mp, rows[i]);
    out[i] = l >= 0 ? reordered[l] : -1ll;
}

__global__ void k_widen_ids(const int* __restrict__ in, long long n, long long* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i];
}

__global__ void k_offset_rows(int* __restrict__ rows, long long n, int delta) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && rows[i] >= 0) rows[i] += delta;
}

// Per query: the k smallest (distance,row) of parts*k shard candidates.
__global__ void __launch_bounds__(1024)
k_merge(const int* __restrict__ rows, const float* __restrict__ dist, int parts, int nq, int k, int np,
        int* __restrict__ out_rows, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) uint64_t s_mkeys[];
    const int q = blockIdx.x;
    const int total = parts * k;
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        uint64_t key = KEY_MAX;
        if (i < total) {
            const int p = i / k, e = i % k;
            const size_t at = ((size_t)p * nq + q) * k + e;
            const int r = rows[at];
            if (r >= 0) key = make_key(dist[at], (uint32_t)r);
        }
        s_mkeys[i] = key;
    }
    __syncthreads();
    block_bitonic_sort(s_mkeys, np);
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const uint64_t key = s_mkeys[i];
        const bool ok = key != KEY_MAX;
        out_rows[(size_t)q * k + i] = ok ? (int)key_idx(key) : -1;
        out_dist[(size_t)q * k + i] = ok ? key_dist(key) : FLT_MAX;
    }
}

}  // namespace

psb_status launch_gather_rows(const void* src, const RowMap& mp, int dim, int elem_bytes, const int* d_candidates,
                              int nq, int candidate_count, int candidate_stride, const int* d_counts,
                              void* d_stage, cudaStream_t s, int sm_count, int compact_ctas, int owned_sms) {
    if (nq <= 0) return PSB_OK;
    const long long total = (long long)nq * candidate_count;
    PSB_TRY(prefer_max_shared(k_gather_rows));
    if (owned_sms > 0) {
        constexpr int kOwnedSmem = 200 * 1024;   // claimed, not used: keeps every kernel that needs shared memory off the SM
        PSB_TRY(prefer_max_shared(k_gather_rows_owned));
        PSB_CUDA(cudaFuncSetAttribute(k_gather_rows_owned, cudaFuncAttributeMaxDynamicSharedMemorySize, kOwnedSmem));
        long long blocks = (total * 32 + 1023) / 1024;
        if (blocks > owned_sms) blocks = owned_sms;
        k_gather_rows_owned<<<(unsigned)blocks, 1024, kOwnedSmem, s>>>(static_cast<const unsigned char*>(src), mp, dim * elem_bytes,
                                                                        d_candidates, nq, candidate_count, candidate_stride, d_counts,
                                                                        static_cast<unsigned char*>(d_stage));
    } else if (compact_ctas > 0) {
        // Beside a scan kernel on the other stream of the overlapped pipeline: small lean CTAs on every SM (compact_ctas of them).
        PSB_TRY(prefer_max_shared(k_gather_rows_beside));
        long long blocks = (total * 32 + 127) / 128;
        if (blocks > compact_ctas) blocks = compact_ctas;
        k_gather_rows_beside<<<(unsigned)blocks, 128, 0, s>>>(static_cast<const unsigned char*>(src), mp, dim * elem_bytes,
                                                              d_candidates, nq, candidate_count, candidate_stride, d_counts,
                                                              static_cast<unsigned char*>(d_stage));
    } else {
        long long blocks = (total * 32 + 255) / 256;
        if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
        k_gather_rows<<<(unsigned)blocks, 256, 0, s>>>(static_cast<const unsigned char*>(src), mp, dim * elem_bytes,
                                                       d_candidates, nq, candidate_count, candidate_stride, d_counts,
                                                       static_cast<unsigned char*>(d_stage));
    }
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_rerank_score(const void* d_stage, const RowMap& mp, int dim, int elem_bytes, const void* d_queries,
                               const int* d_candidates, int nq, int candidate_count, int candidate_stride,
                               const int* d_counts, float* d_out_dist, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    dim3 grid(nq, (candidate_count + kScoreThreads / 16 - 1) / (kScoreThreads / 16));
    PSB_TRY(prefer_max_shared(k_rerank_score));
    k_rerank_score<<<grid, kScoreThreads, (size_t)dim * elem_bytes, s>>>(
        static_cast<const unsigned char*>(d_stage), mp, dim, elem_bytes, static_cast<const unsigned char*>(d_queries),
        d_candidates, candidate_count, candidate_stride, d_counts, d_out_dist);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_topk_select(const float* d_dist, const int* d_candidates, int nq, int candidate_count,
                              int candidate_stride, const int* d_counts, int topk, int* d_out_rows,
                              float* d_out_dist, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    if (candidate_count > kMaxRerankWidth) return fail(PSB_UNSUPPORTED_SHAPE, "rerank accepts at most 4096 candidates per query");
    int np = 32;
    while (np < candidate_count) np <<= 1;
    const size_t smem = (size_t)np * 12;
    if (smem > 32 * 1024)
        PSB_CUDA(cudaFuncSetAttribute(k_topk_select, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_TRY(prefer_max_shared(k_topk_select));
    k_topk_select<<<nq, kSelectThreads, smem, s>>>(d_dist, d_candidates, candidate_count, candidate_stride, d_counts,
                                                   topk, np, d_out_rows, d_out_dist);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_map_ids(const int* d_rows, long long n, const long long* d_reordered, const RowMap& mp,
                          long long* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    PSB_TRY(prefer_max_shared(k_map_ids));
    k_map_ids<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_rows, n, d_reordered, mp, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_widen_ids(const int* d_in, long long n, long long* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    k_widen_ids<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_in, n, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_offset_rows(int* d_rows, long long n, int delta, cudaStream_t s) {
    if (n <= 0 || delta == 0) return PSB_OK;
    k_offset_rows<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_rows, n, delta);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_merge(const int* d_rows, const float* d_dist, int parts, int nq, int k, int* d_out_rows,
                        float* d_out_dist, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    const long long total = (long long)parts * k;
    if (total > 16384) return fail(PSB_UNSUPPORTED_SHAPE, "merge accepts at most 16384 candidates per query");
    int np = 2;
    while (np < total) np <<= 1;
    const size_t smem = (size_t)np * 8;
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_merge, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_merge<<<nq, 1024, smem, s>>>(d_rows, d_dist, parts, nq, k, np, d_out_rows, d_out_dist);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

}  // namespace psb
