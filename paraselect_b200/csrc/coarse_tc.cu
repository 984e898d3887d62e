// Coarse stage, tensor-core part: a bf16 tcgen05 GEMM (queries x centroids, fp32 accumulators in tensor memory,
// operands staged in shared memory by TMA) whose epilogue folds in the centroid norms and filters - it never
// writes the distance matrix.  Two passes over the same GEMM:
//   pass 1  epilogue keeps, per query and per group of G consecutive centroids, the minimum approximate distance
//           a = |c'|^2 - 2 q'.c'  (q', c' = inputs minus the mean centroid, rounded to bf16).  The nprobe-th smallest
//           group minimum T is an upper bound of the nprobe-th smallest approximate distance.
//   pass 2  epilogue appends every centroid with a <= T + 2E to the query's candidate list, E >= |a - exact| being
//           the bf16 rounding bound 4.1 * 2^-8 * |q'| * max|c'| (plus fp32 slack).  Every centroid of the exact top-nprobe
//           is then a candidate: the nprobe approximately-nearest have exact distance <= T + E, so the exact
//           nprobe-th distance is <= T + E and its members have a <= T + 2E.
// k_coarse_refine re-scores the candidates (typically 1.2-2 x nprobe) in the CPU path's arithmetic (sequential
// non-fused fp32, reference src/cpu/utils/cpu_distance.h:74-81) and sorts by (distance, id): results are bit-identical
// to the exact kernels in coarse.cu.  A query whose list overflowed is redone by k_coarse_exact_query.
//
// Reference counterpart: the fused fp16 GEMM + threshold admission + exact top-nprobe of
// src/search/kernels/coarse/runtime/kernels/wmma_body.cuh:45-248 and coarse_runtime.cu:121-149 (wmma, SM 12.0 only).
//
// Every wait on an mbarrier is bounded: after kWaitLimit polls the CTA raises a status word, releases its tensor
// memory and returns, and the host reports PSB_TIMEOUT.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace psb {
namespace {

using namespace tc;

constexpr int TQ = 128;          // queries per tile  (UMMA M)
constexpr int TCOL = 256;        // centroids per tile (UMMA N)
constexpr int KATOM = 64;        // bf16 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kCandCap = 2048;

// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = 256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCOL >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);

// Per group of G consecutive values of a 32-value chunk: out = -2 * max(w), i.e. the minimum of a = -2 w.
template <int G>
__device__ __forceinline__ void group_mins(const float (&v)[32], float* __restrict__ out) {
#pragma unroll
    for (int g = 0; g < 32 / G; ++g) {
        float t[G];
#pragma unroll
        for (int j = 0; j < G; ++j) t[j] = v[g * G + j];
#pragma unroll
        for (int w = G / 2; w >= 1; w >>= 1)  // pairwise tree: short dependency chains
#pragma unroll
            for (int j = 0; j < w; ++j) t[j] = fmaxf(t[j], t[j + w]);
        out[g] = -2.0f * t[0];
    }
}

struct TcArgs {
    int nq, nlist, katoms;  // katoms = padded dim / 64
    int ntiles;             // centroid tiles of TCOL
    int group;              // G: centroids per minimum in pass 1 (power of two <= 32)
    int lg_group;           // log2(G)
    int ngroups;            // minima per query row = ntiles * (TCOL / G)
    int nprobe;
    const float* cn2;       // [ntiles * TCOL] |c'|^2, +inf beyond nlist
    const float* qnorm;     // [nq] |q'|
    float cmax;             // max |c'|
    float* gmin;            // pass 1 out: [nq][ngroups]
    const float* seltop;    // pass 2 in: [nq][nprobe] ascending group minima (T = last)
    uint32_t* mask;         // pass 2 out: [nq][mwords] one bit per centroid (zeroed before the launch; only non-zero words are written)
    int mwords;             // ntiles * TCOL / 32
    int* status;            // [1] != 0 after a bounded wait gave up
    int cblocks, qtiles;    // work = cblocks (512 centroids each) x qtiles (128 queries each) tile pairs
    int* cand_cnt;          // pass 2, list form (nearest-centroid assignment with a known bound): [nq] candidates found so far
    int* cand_list;         //   [nq][cand_cap] their ids; null: the bit mask above is written instead
    int cand_cap;
    int wait_limit;         // polls before a wait gives up (0: kWaitLimit)
    int skip_loads;         // test hook of the time-out path: the producer issues no load at all, so nothing is in flight when
                            // the other roles give up
};

// Work split: the (centroid block, query tile) pairs are numbered block-major and CTA b takes the contiguous range
// [total * b / grid, total * (b + 1) / grid), so every CTA gets the same number of tile pairs (+-1) and reloads its
// resident centroid block at most once or twice.  A range is walked as segments of one centroid block each.
__device__ __forceinline__ void cta_range(const TcArgs& a, long long& l0, long long& l1) {
    const long long total = (long long)a.cblocks * a.qtiles;
    l0 = total * blockIdx.x / gridDim.x;
    l1 = total * (blockIdx.x + 1) / gridDim.x;
}
__device__ __forceinline__ int seg_count(const TcArgs& a, long long l0, long long l1) {
    return l1 > l0 ? (int)((l1 - 1) / a.qtiles - l0 / a.qtiles) + 1 : 0;
}
__device__ __forceinline__ void seg_get(const TcArgs& a, long long l0, long long l1, int i, int& cblock, int& t0, int& t1) {
    cblock = (int)(l0 / a.qtiles) + i;
    const long long b = (long long)cblock * a.qtiles;
    t0 = (int)((l0 > b ? l0 : b) - b);
    t1 = (int)((l1 < b + a.qtiles ? l1 : b + a.qtiles) - b);
}

// Persistent, warp-specialised kernel.  A work unit = one segment of the CTA's range: (block of 512 centroids, range of query tiles).  The unit's
// two centroid tiles (B operands) stay in shared memory while query tiles (A operand, 128 rows) stream through a
// two-stage ring; each query tile is multiplied against both centroid tiles into two tensor-memory accumulators, so
// the epilogue of one accumulator overlaps the MMAs of the other.
//   warps 0-15 epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31 (one query row per thread) and the 64
//              columns (w / 4) * 64 .. +63 of each accumulator, 32 columns per tcgen05.ld; folds |c'|^2 in;
//              pass 1: group minima -> gmin, pass 2: compare with the row's cut-off -> candidate list.
//              Sixteen warps because the epilogue (2+ instructions per matrix element), not the MMA, sets the pace.
//   warp 16    TMA producer (one lane)
//   warp 17    MMA issuer (one lane): 2 x katoms x 4 tcgen05.mma per query tile, tcgen05.commit -> mbarriers
constexpr int kStagesA = 2;
constexpr int kEpiWarps = 16;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kTcThreadsV2 = kEpiThreads + 64;
constexpr int kBlockCols = 2 * TCOL;  // centroids per work unit

// kAug: the operands carry 3 extra K slots (ones on the query side, minus the three-term bf16 split of |c'|^2 / 2 on the
// centroid side), so the accumulator already holds w = q'.c' - |c'|^2 / 2 and the epilogue needs no norm arithmetic.
template <bool kSecondPass, bool kAug>
__global__ void __launch_bounds__(kTcThreadsV2, 1)
k_coarse_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_c, const TcArgs a) {
    extern __shared__ __align__(1024) unsigned char s_tc[];
    unsigned char* s_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_tc) + 1023) & ~uintptr_t(1023));
    const size_t a_bytes = (size_t)a.katoms * TQ * 128, b_bytes = (size_t)a.katoms * TCOL * 128;
    unsigned char* s_a = s_base;                         // [kStagesA][katoms][TQ][128 B]
    unsigned char* s_b = s_base + kStagesA * a_bytes;    // [2][katoms][TCOL][128 B]
    __shared__ __align__(8) uint64_t a_full[kStagesA], a_empty[kStagesA], b_full, b_empty, acc_full[2], acc_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(16) float s_cn2[kBlockCols];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < kStagesA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
        mbar_init(&b_full, 1); mbar_init(&b_empty, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpiThreads); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&s_tmem, 2 * TCOL);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    long long l0, l1;
    cta_range(a, l0, l1);
    const int nunits = seg_count(a, l0, l1);
    const int wl = a.wait_limit > 0 ? a.wait_limit : kWaitLimit;
    int failed = 0;

    if (warp == kEpiWarps) {
        if (lane == 0 && !a.skip_loads) {
            uint32_t it = 0, un = 0;  // query tiles issued, units issued
            for (; (int)un < nunits && !failed; ++un) {
                int cblock, t0, t1;
                seg_get(a, l0, l1, (int)un, cblock, t0, t1);
                if (!mbar_wait(&b_empty, (un & 1u) ^ 1u, wl)) { failed = 1; break; }
                mbar_expect_tx(&b_full, (uint32_t)(2 * b_bytes));
                for (int h = 0; h < 2; ++h)
                    for (int ka = 0; ka < a.katoms; ++ka)
                        tma_load_2d(s_b + h * b_bytes + (size_t)ka * TCOL * 128, &map_c, ka * KATOM, cblock * kBlockCols + h * TCOL, &b_full);
                for (int t = t0; t < t1; ++t, ++it) {
                    const uint32_t st = it % kStagesA;
                    if (!mbar_wait(&a_empty[st], ((it / kStagesA) & 1u) ^ 1u, wl)) { failed = 1; break; }
                    mbar_expect_tx(&a_full[st], (uint32_t)a_bytes);
                    for (int ka = 0; ka < a.katoms; ++ka)
                        tma_load_2d(s_a + st * a_bytes + (size_t)ka * TQ * 128, &map_q, ka * KATOM, t * TQ, &a_full[st]);
                }
            }
        }
    } else if (warp == kEpiWarps + 1) {
        if (lane == 0) {
            uint32_t it = 0, un = 0, nacc[2] = {0, 0};
            for (; (int)un < nunits && !failed; ++un) {
                int cblock, t0, t1;
                seg_get(a, l0, l1, (int)un, cblock, t0, t1);
                (void)cblock;
                if (!mbar_wait(&b_full, un & 1u, wl)) { failed = 1; break; }
                for (int t = t0; t < t1 && !failed; ++t, ++it) {
                    const uint32_t st = it % kStagesA;
                    if (!mbar_wait(&a_full[st], (it / kStagesA) & 1u, wl)) { failed = 1; break; }
                    for (int h = 0; h < 2; ++h) {
                        if (!mbar_wait(&acc_empty[h], (nacc[h] & 1u) ^ 1u, wl)) { failed = 1; break; }
                        tc_fence_after();
                        const uint32_t sa = smem_u32(s_a + st * a_bytes), sb = smem_u32(s_b + h * b_bytes);
                        for (int ka = 0; ka < a.katoms; ++ka)
                            for (int kk = 0; kk < KATOM / UMMA_K; ++kk)
                                umma_bf16(tmem + (uint32_t)(h * TCOL), make_sw128_desc(sa + ka * TQ * 128 + kk * UMMA_K * 2),
                                          make_sw128_desc(sb + ka * TCOL * 128 + kk * UMMA_K * 2), kIdesc, (ka | kk) ? 1u : 0u);
                        umma_commit(&acc_full[h]);
                        ++nacc[h];
                    }
                    umma_commit(&a_empty[st]);  // stage reusable once both MMAs have read it
                }
                umma_commit(&b_empty);
            }
        }
    } else {
        // epilogue warps
        uint32_t nacc[2] = {0, 0};
        const int quad = warp & 3, part = warp >> 2;
        const int row = quad * 32 + lane;  // tensor-memory lane = row of the current query tile
        const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
        for (int u = 0; u < nunits; ++u) {  // every thread passes both barriers of every unit, failed or not
            int cblock, t0, t1;
            seg_get(a, l0, l1, u, cblock, t0, t1);
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");  // previous unit's readers of s_cn2 are done
            for (int i = tid; i < kBlockCols; i += kEpiThreads) s_cn2[i] = a.cn2[(size_t)cblock * kBlockCols + i];
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            for (int t = t0; t < t1 && !failed; ++t) {
                const int q = t * TQ + row;
                float cut = 0.0f;
                if (kSecondPass && q < a.nq) {
                    const float T = a.seltop[(size_t)q * a.nprobe + a.nprobe - 1];
                    const float qn = a.qnorm[q];
                    const float E = 4.1f * 0.00390625f * qn * a.cmax;  // |a - exact| <= 2 |q'.c' - qb.cb| <= 2 * 2.01 * 2^-8 |q'||c'|
                    cut = -0.5f * (T + 2.0f * E + 4e-5f * (qn + a.cmax) * (qn + a.cmax));  // candidates: w >= cut
                }
                const bool partial = (cblock + 1) * kBlockCols > a.nlist;  // block reaches past the last centroid
                for (int h = 0; h < 2; ++h) {
                    if (!mbar_wait(&acc_full[h], nacc[h] & 1u, wl)) { failed = 1; break; }
                    ++nacc[h];
                    tc_fence_after();
                    uint32_t r0[32], r1[32];
                    const int cb0 = part * 64;
                    __syncwarp();
                    tmem_ld32(lane_addr + (uint32_t)(h * TCOL + cb0), r0);
                    tmem_ld32(lane_addr + (uint32_t)(h * TCOL + cb0 + 32), r1);
                    tmem_ld_wait();
                    // the accumulators are in registers: hand the tensor memory back before the arithmetic
                    tc_fence_before();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[h])) : "memory");
                    if (q < a.nq) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int cb = cb0 + half * 32;
                            const int c0 = cblock * kBlockCols + h * TCOL + cb;
                            float v[32];  // w = q'.c' - |c'|^2 / 2 = -a / 2; -inf beyond the last centroid
                            const uint32_t* rr = half ? r1 : r0;
                            if (kAug) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[j]);
                                if (partial) {
#pragma unroll
                                    for (int j = 0; j < 32; ++j) if (c0 + j >= a.nlist) v[j] = __int_as_float(0xff800000);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    const float4 n4 = *reinterpret_cast<const float4*>(&s_cn2[h * TCOL + cb + j]);
                                    v[j] = fmaf(-0.5f, n4.x, __uint_as_float(rr[j]));
                                    v[j + 1] = fmaf(-0.5f, n4.y, __uint_as_float(rr[j + 1]));
                                    v[j + 2] = fmaf(-0.5f, n4.z, __uint_as_float(rr[j + 2]));
                                    v[j + 3] = fmaf(-0.5f, n4.w, __uint_as_float(rr[j + 3]));
                                }
                            }
                            if (!kSecondPass) {
                                float* out = a.gmin + (size_t)q * a.ngroups + (c0 >> a.lg_group);
                                switch (a.lg_group) {  // uniform
                                    case 5: group_mins<32>(v, out); break;
                                    case 4: group_mins<16>(v, out); break;
                                    case 3: group_mins<8>(v, out); break;
                                    case 2: group_mins<4>(v, out); break;
                                    case 1: group_mins<2>(v, out); break;
                                    default: group_mins<1>(v, out); break;
                                }
                            } else {
                                // one bit per centroid of this 32-column chunk; most chunks hold none and write nothing
                                uint32_t bits = 0;
#pragma unroll
                                for (int j = 0; j < 32; ++j) bits |= (v[j] >= cut ? 1u : 0u) << j;
                                if (bits) {
                                    if (a.cand_list) {   // a handful of candidates per row: a short list instead of a mask to scan
                                        while (bits) {
                                            const int j = __ffs((int)bits) - 1;
                                            bits &= bits - 1;
                                            const int pos = atomicAdd(&a.cand_cnt[q], 1);
                                            if (pos < a.cand_cap) a.cand_list[(size_t)q * a.cand_cap + pos] = c0 + j;
                                        }
                                    } else {
                                        a.mask[(size_t)q * a.mwords + (c0 >> 5)] = bits;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    if (failed) atomicExch(a.status, 1);
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (warp == 0) tmem_dealloc(tmem, 2 * TCOL);
}

// q' = q - mu as bf16 rows padded with zeros to dimp, and |q'|.
// aug: 0 = no extra slots, 1 = query rows (slots dim..dim+2 hold 1), 2 = centroid rows (slots hold minus the bf16
// three-term split of |c'|^2 / 2).
__global__ void k_tc_prep_rows(const float* __restrict__ x, int n, int dim, int dimp, const float* __restrict__ mu,
                               __nv_bfloat16* __restrict__ out, float* __restrict__ norm, float* __restrict__ sq, int aug) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n) return;
    float s = 0.0f;
    for (int d = lane; d < dimp; d += 32) {
        float v = 0.0f;
        if (d < dim) v = x[(size_t)warp * dim + d] - mu[d];
        if (!(aug && d >= dim && d < dim + 3)) out[(size_t)warp * dimp + d] = __float2bfloat16_rn(v);
        s += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        if (norm) norm[warp] = sqrtf(s);
        if (sq) sq[warp] = s;
        if (aug == 1) {
            for (int i = 0; i < 3; ++i) out[(size_t)warp * dimp + dim + i] = __float2bfloat16_rn(1.0f);
        } else if (aug == 2) {
            float rest = 0.5f * s;
            for (int i = 0; i < 3; ++i) {
                const __nv_bfloat16 h = __float2bfloat16_rn(rest);
                out[(size_t)warp * dimp + dim + i] = __hneg(h);
                rest -= __bfloat162float(h);
            }
        }
    }
}

__global__ void k_fill_inf(float* p, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = __int_as_float(0x7f800000);
}

// Per query row the k-th smallest of n <= 2048 values, written to out[q * out_stride + out_stride - 1].  One warp per row:
// the values sit in registers as order-preserving integer keys and the answer is found by bisection on the key (32
// counting rounds), which is exact.
constexpr int kKthPerLane = 64;
__global__ void __launch_bounds__(256)
k_kth_smallest(const float* __restrict__ vals, int nq, int n, int k, float* __restrict__ out, int out_stride) {
    const int q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (q >= nq) return;
    uint32_t key[kKthPerLane];
#pragma unroll
    for (int j = 0; j < kKthPerLane; ++j) {
        const int i = j * 32 + lane;
        key[j] = i < n ? f2o(vals[(size_t)q * n + i]) : 0xffffffffu;
    }
    uint32_t lo = 0u, hi = 0xffffffffu;
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        int c = 0;
#pragma unroll
        for (int j = 0; j < kKthPerLane; ++j) c += key[j] <= mid ? 1 : 0;
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= k) hi = mid; else lo = mid + 1;
    }
    if (lane == 0) out[(size_t)q * out_stride + out_stride - 1] = o2f(lo);
}

// Exact re-scoring of a query's candidates in the CPU path's arithmetic, sort by (distance, id), first nprobe out.
constexpr int kRefineThreads = 256;
__global__ void __launch_bounds__(kRefineThreads)
k_coarse_refine(const float* __restrict__ queries, const float* __restrict__ centroids, int dim, int nlist, int nprobe,
                const uint32_t* __restrict__ mask, int mwords, int* __restrict__ out_ids,
                float* __restrict__ out_dist, int* __restrict__ fail_list, int* __restrict__ n_fail) {
    extern __shared__ __align__(16) unsigned char s_ref[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_ref);                        // [kCandCap]
    float* s_q = reinterpret_cast<float*>(s_ref + (size_t)kCandCap * 8);         // [dim]
    int* s_cand = reinterpret_cast<int*>(s_ref + (size_t)kCandCap * 8 + (size_t)((dim + 3) & ~3) * 4);  // [kCandCap]
    __shared__ int s_n;
    const int q = blockIdx.x;
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    for (int w = threadIdx.x; w < mwords; w += blockDim.x) {  // the candidate bits of this query -> list of centroid ids
        uint32_t bits = mask[(size_t)q * mwords + w];
        while (bits) {
            const int j = __ffs((int)bits) - 1;
            bits &= bits - 1;
            const int pos = atomicAdd(&s_n, 1);
            if (pos < kCandCap) s_cand[pos] = w * 32 + j;
        }
    }
    __syncthreads();
    const int n = s_n;
    if (n > kCandCap || n < nprobe) {
        if (threadIdx.x == 0) {
            fail_list[atomicAdd(n_fail, 1)] = q;
            atomicAdd(n_fail + 3, 1);  // cumulative count of queries sent to the exact per-query kernel
        }
        return;
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) s_q[d] = queries[(size_t)q * dim + d];
    __syncthreads();
    const int np = next_pow2(max(n, 2));
    for (int i = threadIdx.x; i < np; i += blockDim.x) {
        uint64_t key = KEY_MAX;
        if (i < n) {
            const int c = s_cand[i];
            const float* cp = centroids + (size_t)c * dim;
            float sum = 0.0f;
            if ((dim & 3) == 0) {  // 16-byte loads: a row's 32-byte sectors are fetched once or twice, not eight times
                const float4* cp4 = reinterpret_cast<const float4*>(cp);
                const float4* q4 = reinterpret_cast<const float4*>(s_q);
                for (int d = 0; d < dim / 4; ++d) {
                    const float4 x = __ldg(cp4 + d);
                    const float4 y = q4[d];
                    float diff = __fsub_rn(y.x, x.x); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(y.y, x.y); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(y.z, x.z); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(y.w, x.w); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                }
            } else {
                for (int d = 0; d < dim; ++d) {
                    const float diff = __fsub_rn(s_q[d], __ldg(cp + d));
                    sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                }
            }
            key = make_key(sum, (uint32_t)c);
        }
        s_keys[i] = key;
    }
    __syncthreads();
    block_bitonic_sort(s_keys, np);
    for (int i = threadIdx.x; i < nprobe; i += blockDim.x) {
        out_ids[(size_t)q * nprobe + i] = (int)key_idx(s_keys[i]);
        if (out_dist) out_dist[(size_t)q * nprobe + i] = key_dist(s_keys[i]);
    }
}

// ---- nearest-centroid assignment with a bound known beforehand (Lloyd iterations after the first) -------------------------
// A row's distance to the centroid it was assigned to in the previous iteration, at that centroid's NEW position, bounds its
// distance to the nearest centroid from above.  With that bound in place of pass 1's group minimum the GEMM runs once: the
// candidates (every centroid whose bf16 estimate is within the bound plus the rounding slack - the nearest one and all its
// ties among them) go to a short per-row list, and k_coarse_refine1 picks the exact nearest in the CPU path's arithmetic.
constexpr int kAssignCap = 32;   // candidates kept per row (one per lane of the refining warp); more: the exact per-row kernel
// seltop[row] = (bound on the squared distance) - |q'|^2, the quantity pass 2 compares a = |c'|^2 - 2 q'.c' against.
__global__ void k_prev_bound(const float* __restrict__ rows, long long n, int dim, const float* __restrict__ centroids, int nlist,
                             const int* __restrict__ prev, const float* __restrict__ qnorm, float* __restrict__ seltop) {
    const long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    const int c = prev[r];
    float acc = 0.0f;
    const bool ok = c >= 0 && c < nlist;
    if (ok) {
        const float* x = rows + (size_t)r * dim;
        const float* cp = centroids + (size_t)c * dim;
        for (int d = lane; d < dim; d += 32) { const float diff = x[d] - __ldg(cp + d); acc = fmaf(diff, diff, acc); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        const float qn = qnorm[r];
        // a bound, not a result: one part in 1e5 covers the different summation order
        seltop[r] = ok ? acc * (1.0f + 1e-5f) - qn * qn : __int_as_float(0x7f800000);
    }
}
// One warp per row: lane i re-scores candidate i exactly (sequential non-fused fp32, the CPU path's arithmetic), the warp
// takes the smallest (distance, id).  No candidate or too many: the row goes to the exact per-row kernel.
__global__ void __launch_bounds__(256) k_coarse_refine1(const float* __restrict__ rows, const float* __restrict__ centroids, int dim,
                                                        long long n, const int* __restrict__ cand_cnt, const int* __restrict__ cand_list,
                                                        int* __restrict__ out_ids, float* __restrict__ out_dist,
                                                        int* __restrict__ fail_list, int* __restrict__ n_fail) {
    const long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    const int cnt = cand_cnt[r];
    if (cnt <= 0 || cnt > kAssignCap) {
        if (lane == 0) {
            fail_list[atomicAdd(n_fail, 1)] = (int)r;
            atomicAdd(n_fail + 3, 1);
        }
        return;
    }
    uint64_t key = KEY_MAX;
    if (lane < cnt) {
        const int c = cand_list[(size_t)r * kAssignCap + lane];
        const float* x = rows + (size_t)r * dim;
        const float* cp = centroids + (size_t)c * dim;
        float sum = 0.0f;
        if ((dim & 3) == 0) {
            const float4* cp4 = reinterpret_cast<const float4*>(cp);
            const float4* x4 = reinterpret_cast<const float4*>(x);
            for (int d = 0; d < dim / 4; ++d) {
                const float4 a = __ldg(cp4 + d);
                const float4 b = __ldg(x4 + d);
                float diff = __fsub_rn(b.x, a.x); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                diff = __fsub_rn(b.y, a.y); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                diff = __fsub_rn(b.z, a.z); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                diff = __fsub_rn(b.w, a.w); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
            }
        } else {
            for (int d = 0; d < dim; ++d) {
                const float diff = __fsub_rn(__ldg(x + d), __ldg(cp + d));
                sum = __fadd_rn(sum, __fmul_rn(diff, diff));
            }
        }
        key = make_key(sum, (uint32_t)c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other < key ? other : key;
    }
    if (lane == 0) {
        out_ids[r] = (int)key_idx(key);
        if (out_dist) out_dist[r] = key_dist(key);
    }
}

// Whole-row exact coarse search for the queries on the fail list: running cut-off buffer, one CTA per query.
constexpr int kExactThreads = 1024;
__global__ void __launch_bounds__(kExactThreads)
k_coarse_exact_query(const float* __restrict__ queries, const float* __restrict__ centroids, int dim, int nlist,
                     int nprobe, int buf_n, const int* __restrict__ fail_list, const int* __restrict__ n_fail,
                     int* __restrict__ cursor, int* __restrict__ out_ids, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) unsigned char s_ex[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_ex);                 // [buf_n]
    float* s_q = reinterpret_cast<float*>(s_ex + (size_t)buf_n * 8);     // [dim]
    __shared__ int s_cnt, s_idx;
    __shared__ uint64_t s_cut;
    const int nf = *n_fail;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_idx = atomicAdd(cursor, 1);
        __syncthreads();
        if (s_idx >= nf) return;
        const int q = fail_list[s_idx];
        for (int d = threadIdx.x; d < dim; d += blockDim.x) s_q[d] = queries[(size_t)q * dim + d];
        if (threadIdx.x == 0) { s_cnt = 0; s_cut = KEY_MAX; }
        __syncthreads();
        for (int base = 0; base < nlist; base += blockDim.x) {
            const int c_now = s_cnt;
            __syncthreads();
            if (c_now + (int)blockDim.x > buf_n) {  // uniform
                for (int i = c_now + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
                __syncthreads();
                block_bitonic_sort(s_keys, buf_n);
                if (threadIdx.x == 0) { s_cnt = nprobe; s_cut = s_keys[nprobe - 1]; }  // c_now >= nprobe here
                __syncthreads();
            }
            const int c = base + threadIdx.x;
            if (c < nlist) {
                const float* cp = centroids + (size_t)c * dim;
                float sum = 0.0f;
                for (int d = 0; d < dim; ++d) {
                    const float diff = __fsub_rn(s_q[d], __ldg(cp + d));
                    sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                }
                const uint64_t key = make_key(sum, (uint32_t)c);
                if (key < s_cut) s_keys[atomicAdd(&s_cnt, 1)] = key;
            }
            __syncthreads();
        }
        const int c = s_cnt;
        for (int i = c + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
        __syncthreads();
        block_bitonic_sort(s_keys, buf_n);
        for (int i = threadIdx.x; i < nprobe; i += blockDim.x) {
            const uint64_t key = s_keys[i];
            const bool ok = key != KEY_MAX;
            out_ids[(size_t)q * nprobe + i] = ok ? (int)key_idx(key) : -1;
            if (out_dist) out_dist[(size_t)q * nprobe + i] = ok ? key_dist(key) : FLT_MAX;
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

psb_status encode_rows_map(CUtensorMap* map, const void* base, long long rows, int dimp, int box_rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        PSB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (!p || qres != cudaDriverEntryPointSuccess) return fail(PSB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    const cuuint64_t gdim[2] = {(cuuint64_t)dimp, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)dimp * 2};
    const cuuint32_t box[2] = {(cuuint32_t)KATOM, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PSB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return PSB_OK;
}

}  // namespace

int coarse_tc_padded_dim(int dim) { return (dim + KATOM - 1) / KATOM * KATOM; }
int coarse_tc_tiles(int nlist) { return (nlist + kBlockCols - 1) / kBlockCols * 2; }  // whole 512-centroid blocks
int coarse_tc_cand_cap() { return kCandCap; }
int coarse_tc_mask_words(int nlist) { return coarse_tc_tiles(nlist) * TCOL / 32; }

int coarse_tc_group(int nlist, int nprobe) {
    int g = 32;
    while (g > 1 && nlist / g < 4 * nprobe) g >>= 1;
    return g;
}

bool coarse_tc_supported(int nq, int nlist, int dim, int nprobe) {
    const int dimp = coarse_tc_padded_dim(dim);
    return nq >= 64 && nlist >= 1024 && dimp <= 128 && nprobe <= 512 && nlist >= 8 * nprobe &&
           nlist / coarse_tc_group(nlist, nprobe) >= 4 * nprobe;
}

psb_status launch_tc_prep_centroids(const float* d_centroids, int nlist, int dim, const float* d_mu, void* d_cb,
                                    float* d_cn2, float* d_cnorm, cudaStream_t s) {
    const int dimp = coarse_tc_padded_dim(dim);
    const long long padded = (long long)coarse_tc_tiles(nlist) * TCOL;
    k_fill_inf<<<(unsigned)((padded + 255) / 256), 256, 0, s>>>(d_cn2, padded);
    count_launch();
    PSB_LAUNCH_CHECK();
    k_tc_prep_rows<<<(nlist * 32 + 255) / 256, 256, 0, s>>>(d_centroids, nlist, dim, dimp, d_mu,
                                                            static_cast<__nv_bfloat16*>(d_cb), d_cnorm, d_cn2,
                                                            dimp - dim >= 3 ? 2 : 0);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_coarse_tc(const CoarseTcIndex& ix, const CoarseTcWorkspace& ws, const float* d_queries, int nq,
                            int nprobe, int* d_ids, float* d_dist, int sm_count, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    const int dimp = coarse_tc_padded_dim(ix.dim);
    const int katoms = dimp / KATOM;
    const int ntiles = coarse_tc_tiles(ix.nlist);
    const int group = coarse_tc_group(ix.nlist, nprobe);
    const int ngroups = ntiles * (TCOL / group);
    const bool aug = dimp - ix.dim >= 3;
    // query side: centre, round to bf16, norms
    k_tc_prep_rows<<<(nq * 32 + 255) / 256, 256, 0, s>>>(d_queries, nq, ix.dim, dimp, ix.mu,
                                                         static_cast<__nv_bfloat16*>(ws.qb), ws.qnorm, nullptr, aug ? 1 : 0);
    count_launch();
    PSB_LAUNCH_CHECK();
    CUtensorMap map_q, map_c;
    PSB_TRY(encode_rows_map(&map_q, ws.qb, nq, dimp, TQ));
    PSB_TRY(encode_rows_map(&map_c, ix.cb, ix.nlist, dimp, TCOL));
    TcArgs a;
    a.nq = nq; a.nlist = ix.nlist; a.katoms = katoms; a.ntiles = ntiles; a.group = group; a.ngroups = ngroups;
    a.lg_group = 0;
    while ((1 << a.lg_group) < group) ++a.lg_group;
    a.nprobe = nprobe; a.cn2 = ix.cn2; a.qnorm = ws.qnorm; a.cmax = ix.cmax; a.gmin = ws.gmin; a.seltop = ws.seltop;
    a.mask = reinterpret_cast<uint32_t*>(ws.cand); a.mwords = coarse_tc_mask_words(ix.nlist); a.status = ws.status;
    a.cand_cnt = nullptr; a.cand_list = nullptr; a.cand_cap = 0;
    a.wait_limit = ws.test_wait_limit; a.skip_loads = ws.test_skip_loads;
    const size_t smem = (size_t)katoms * (kStagesA * TQ + 2 * TCOL) * 128 + 1024;
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    a.qtiles = (nq + TQ - 1) / TQ;
    a.cblocks = ntiles / 2;
    const long long pairs = (long long)a.cblocks * a.qtiles;
    const dim3 grid((unsigned)(pairs < sm_count ? pairs : sm_count));
    constexpr int kTcThreads = kTcThreadsV2;
    PSB_CUDA(cudaMemsetAsync(ws.cand, 0, sizeof(uint32_t) * (size_t)nq * a.mwords, s));
    PSB_CUDA(cudaMemsetAsync(ws.n_fail, 0, 2 * sizeof(int), s));  // n_fail, cursor
    if (ws.ev[0]) PSB_CUDA(cudaEventRecord(ws.ev[0], s));
    if (aug) k_coarse_tc<false, true><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    else k_coarse_tc<false, false><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    if (ws.ev[1]) PSB_CUDA(cudaEventRecord(ws.ev[1], s));
    count_launch();
    PSB_LAUNCH_CHECK();
    // pass 2 needs only T = the nprobe-th smallest group minimum of each query
    if (ngroups <= kKthPerLane * 32) {
        k_kth_smallest<<<(unsigned)(((long long)nq * 32 + 255) / 256), 256, 0, s>>>(ws.gmin, nq, ngroups, nprobe, ws.seltop, nprobe);
        count_launch();
        PSB_LAUNCH_CHECK();
    } else {
        PSB_TRY(launch_select_rows(ws.gmin, nq, ngroups, nprobe, ws.selids, ws.seltop, s));
    }
    if (ws.ev[2]) PSB_CUDA(cudaEventRecord(ws.ev[2], s));
    if (aug) k_coarse_tc<true, true><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    else k_coarse_tc<true, false><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    if (ws.ev[3]) PSB_CUDA(cudaEventRecord(ws.ev[3], s));
    count_launch();
    PSB_LAUNCH_CHECK();
    {
        const size_t rsmem = (size_t)kCandCap * 8 + (size_t)((ix.dim + 3) & ~3) * sizeof(float) + (size_t)kCandCap * sizeof(int);
        k_coarse_refine<<<nq, kRefineThreads, rsmem, s>>>(d_queries, ix.centroids, ix.dim, ix.nlist, nprobe,
                                                          reinterpret_cast<const uint32_t*>(ws.cand), a.mwords, d_ids, d_dist,
                                                          ws.fail_list, ws.n_fail);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    {
        int buf_n = 2048;
        while (buf_n < nprobe + kExactThreads) buf_n <<= 1;
        const size_t esmem = (size_t)buf_n * 8 + (size_t)ix.dim * sizeof(float);
        if (esmem > 32 * 1024)
            PSB_CUDA(cudaFuncSetAttribute(k_coarse_exact_query, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)esmem));
        k_coarse_exact_query<<<sm_count, kExactThreads, esmem, s>>>(d_queries, ix.centroids, ix.dim, ix.nlist, nprobe, buf_n,
                                                                    ws.fail_list, ws.n_fail, ws.n_fail + 1, d_ids, d_dist);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    return PSB_OK;
}

// Nearest centroid of every row when a previous assignment is known (d_prev [nq], may alias d_ids): ONE GEMM pass.
psb_status launch_coarse_tc_assign(const CoarseTcIndex& ix, const CoarseTcWorkspace& ws, const float* d_rows, int nq, const int* d_prev,
                                   int* d_ids, float* d_dist, int sm_count, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    const int dimp = coarse_tc_padded_dim(ix.dim);
    const int katoms = dimp / KATOM;
    const int ntiles = coarse_tc_tiles(ix.nlist);
    const bool aug = dimp - ix.dim >= 3;
    if (coarse_tc_mask_words(ix.nlist) < kAssignCap) return fail(PSB_INTERNAL, "candidate buffer too small for the list form");
    k_tc_prep_rows<<<(nq * 32 + 255) / 256, 256, 0, s>>>(d_rows, nq, ix.dim, dimp, ix.mu, static_cast<__nv_bfloat16*>(ws.qb), ws.qnorm,
                                                         nullptr, aug ? 1 : 0);
    count_launch();
    PSB_LAUNCH_CHECK();
    k_prev_bound<<<(unsigned)(((long long)nq * 32 + 255) / 256), 256, 0, s>>>(d_rows, nq, ix.dim, ix.centroids, ix.nlist, d_prev, ws.qnorm,
                                                                              ws.seltop);
    count_launch();
    PSB_LAUNCH_CHECK();
    CUtensorMap map_q, map_c;
    PSB_TRY(encode_rows_map(&map_q, ws.qb, nq, dimp, TQ));
    PSB_TRY(encode_rows_map(&map_c, ix.cb, ix.nlist, dimp, TCOL));
    TcArgs a;
    a.nq = nq; a.nlist = ix.nlist; a.katoms = katoms; a.ntiles = ntiles; a.group = 32; a.lg_group = 5; a.ngroups = ntiles * (TCOL / 32);
    a.nprobe = 1; a.cn2 = ix.cn2; a.qnorm = ws.qnorm; a.cmax = ix.cmax; a.gmin = ws.gmin; a.seltop = ws.seltop;
    a.mask = nullptr; a.mwords = coarse_tc_mask_words(ix.nlist); a.status = ws.status;
    a.cand_cnt = ws.cand_cnt; a.cand_list = ws.cand; a.cand_cap = kAssignCap;
    a.wait_limit = ws.test_wait_limit; a.skip_loads = ws.test_skip_loads;
    const size_t smem = (size_t)katoms * (kStagesA * TQ + 2 * TCOL) * 128 + 1024;
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    a.qtiles = (nq + TQ - 1) / TQ;
    a.cblocks = ntiles / 2;
    const long long pairs = (long long)a.cblocks * a.qtiles;
    const dim3 grid((unsigned)(pairs < sm_count ? pairs : sm_count));
    PSB_CUDA(cudaMemsetAsync(ws.cand_cnt, 0, sizeof(int) * (size_t)nq, s));
    PSB_CUDA(cudaMemsetAsync(ws.n_fail, 0, 2 * sizeof(int), s));  // n_fail, cursor
    if (ws.ev[2]) PSB_CUDA(cudaEventRecord(ws.ev[2], s));
    if (aug) k_coarse_tc<true, true><<<grid, kTcThreadsV2, smem, s>>>(map_q, map_c, a);
    else k_coarse_tc<true, false><<<grid, kTcThreadsV2, smem, s>>>(map_q, map_c, a);
    if (ws.ev[3]) PSB_CUDA(cudaEventRecord(ws.ev[3], s));
    count_launch();
    PSB_LAUNCH_CHECK();
    k_coarse_refine1<<<(unsigned)(((long long)nq * 32 + 255) / 256), 256, 0, s>>>(d_rows, ix.centroids, ix.dim, nq, ws.cand_cnt, ws.cand, d_ids,
                                                                                  d_dist, ws.fail_list, ws.n_fail);
    count_launch();
    PSB_LAUNCH_CHECK();
    {
        int buf_n = 2048;
        while (buf_n < 1 + kExactThreads) buf_n <<= 1;
        const size_t esmem = (size_t)buf_n * 8 + (size_t)ix.dim * sizeof(float);
        if (esmem > 32 * 1024)
            PSB_CUDA(cudaFuncSetAttribute(k_coarse_exact_query, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)esmem));
        k_coarse_exact_query<<<sm_count, kExactThreads, esmem, s>>>(d_rows, ix.centroids, ix.dim, ix.nlist, 1, buf_n, ws.fail_list, ws.n_fail,
                                                                    ws.n_fail + 1, d_ids, d_dist);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    return PSB_OK;
}

}  // namespace psb
