// Pieces shared by the ADC scan kernels (pq_scan.cu: SIMT scans, cutoff, selection, fallback; scan_tc.cu: the
// tensor-core pre-filter scan and the re-scoring selection): kernel argument block, work-item lookup, and the exact
// ADC row sums in the CPU path's summation orders.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace scan {

struct ScanArgs {
    const float* lut;          // [tables][m*k]
    int lut_div;               // visitor entry / lut_div = query (1: one table per query; nprobe: one per pair)
    int tree;                  // pairwise-tree ADC order (residual mode, M = 8 or 16, K = 256)
    const uint8_t* codes;
    const long long* offsets;
    long long row_base;
    const long long* row_delta;  // optional [nlist]: reported row = local row + row_delta[list]
    int nlist, m, k;
    const int* vis_count; const int* vis_off; const int* visitors;
    const long long* item_off;
    const float* thr;
    int* pool_cnt; uint64_t* pool; int pool_cap;
    unsigned long long* work_cursor;
    unsigned long long* counters;
    int chunk_rows;
    int reserve_ctas;          // host side only: CTAs left out of the persistent grid (see ScanWorkspace::reserve_ctas)
};

// Persistent grid: every SM slot, minus the CTAs the caller wants kept free for kernels of another stream.
inline unsigned scan_grid(int slots, int reserve) {
    const int g = slots - (reserve > 0 ? reserve : 0);
    return (unsigned)(g < 1 ? 1 : g);
}

// Largest l in [0, nlist) with item_off[l] <= item, found by warp 0 with a 32-ary search.
__device__ __forceinline__ int find_list(const long long* __restrict__ item_off, int nlist, long long item) {
    const int lane = threadIdx.x & 31;
    int lo = 0, hi = nlist;  // answer in [lo, hi)
    while (hi - lo > 1) {
        const int span = hi - lo;
        const int step = (span + 31) / 32;
        const int pos = min(lo + lane * step, hi - 1);
        const bool ok = item_off[pos] <= item;  // monotone: true for a prefix of the lanes
        const unsigned bal = __ballot_sync(0xffffffffu, ok);
        const int last = 31 - __clz((int)bal);  // lane 0 always true (item_off[lo] <= item)
        const int nlo = min(lo + last * step, hi - 1);
        const int nhi = min(nlo + step, hi);
        lo = nlo; hi = nhi;
    }
    return lo;
}


// ------------------------------------------------------------------------------------------------------
// ADC distance of one code row against a table in shared memory laid out [m][k] (one visitor).
// Balanced pairwise sum of n (a power of two) terms, earlier term on the left: the order the reference's residual
// CPU scan uses for M = 16 and M = 8 (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:226-259).
template <int N>
__device__ __forceinline__ float tree_sum(float (&t)[N]) {
#pragma unroll
    for (int n = N; n > 1; n >>= 1)
#pragma unroll
        for (int j = 0; j < n / 2; ++j) t[j] = __fadd_rn(t[2 * j], t[2 * j + 1]);
    return t[0];
}
template <int M>
__device__ __forceinline__ float adc_row_tree(const uint8_t* __restrict__ row, const float* __restrict__ lut, int k) {
    static_assert(M == 8 || M == 16, "tree order exists for M = 8 and 16");
    const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
    float t[M];
#pragma unroll
    for (int w = 0; w < M / 4; ++w) {
        const uint32_t c = __ldg(p + w);
#pragma unroll
        for (int j = 0; j < 4; ++j) t[w * 4 + j] = lut[(w * 4 + j) * k + ((c >> (j * 8)) & 255)];
    }
    return tree_sum<M>(t);
}

template <int M>
__device__ __forceinline__ float adc_row_1(const uint8_t* __restrict__ row, const float* __restrict__ s_lut, int k) {
    float acc = 0.0f;
    if constexpr (M % 16 == 0) {
        const uint4* p = reinterpret_cast<const uint4*>(row);
#pragma unroll
        for (int w = 0; w < M / 16; ++w) {
            const uint4 c = __ldg(p + w);
            const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int code = (cw[j >> 2] >> ((j & 3) * 8)) & 255;
                acc = __fadd_rn(acc, s_lut[(w * 16 + j) * k + code]);
            }
        }
    } else if constexpr (M % 4 == 0 && M > 0) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(row);
#pragma unroll
        for (int w = 0; w < M / 4; ++w) {
            const uint32_t c = __ldg(p + w);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc = __fadd_rn(acc, s_lut[(w * 4 + j) * k + ((c >> (j * 8)) & 255)]);
        }
    }
    return acc;
}
// Generic M (runtime), byte loads.
__device__ __forceinline__ float adc_row_dyn(const uint8_t* __restrict__ row, const float* __restrict__ s_lut,
                                             int m, int k) {
    float acc = 0.0f;
    for (int j = 0; j < m; ++j) acc = __fadd_rn(acc, s_lut[j * k + __ldg(row + j)]);
    return acc;
}
template <int M>
__device__ __forceinline__ float adc_row(const uint8_t* row, const float* s_lut, int m, int k, bool tree = false) {
    if constexpr (M == 8 || M == 16) { if (tree) return adc_row_tree<M>(row, s_lut, k); }
    if constexpr (M > 0) return adc_row_1<M>(row, s_lut, k);
    else return adc_row_dyn(row, s_lut, m, k);
}


// Residual-mode ADC distance of one code row WITHOUT a table: every entry is computed from the residual query (qres = q -
// centroid, [dim]) and the codeword as k_build_lut_residual would store it - the sequential non-fused sum over the
// sub-vector - and the entries are summed in the CPU path's order (sequential, or the pairwise tree for M = 8 / 16).
// Worth it when a table (m * k entries) would serve fewer than k rows.  cen != null: qres holds the query itself and the
// centroid is subtracted here (fp32, the same subtraction).
template <int M>
__device__ __forceinline__ float adc_row_direct(const uint8_t* __restrict__ row, const float* __restrict__ qres,
                                                const float* __restrict__ codebook, int m, int k, int dsub, bool tree,
                                                const float* __restrict__ cen = nullptr) {
    auto entry = [&](int j, int code) {
        const float* cb = codebook + ((size_t)j * k + code) * dsub;
        float e = 0.0f;
        for (int d = 0; d < dsub; ++d) {
            float qv = qres[j * dsub + d];
            if (cen) qv = __fsub_rn(qv, __ldg(cen + j * dsub + d));
            const float diff = __fsub_rn(qv, __ldg(cb + d));
            e = __fadd_rn(e, __fmul_rn(diff, diff));
        }
        return e;
    };
    if constexpr (M > 0 && M % 4 == 0) {
        // templated M: the code words are loaded first and the loop is unrolled, so the codeword loads of all sub-quantisers are
        // in flight together (a rolled loop would wait for one dependent load after the other)
        uint32_t cw[M / 4];
#pragma unroll
        for (int w = 0; w < M / 4; ++w) cw[w] = __ldg(reinterpret_cast<const uint32_t*>(row) + w);
        float t[M];
#pragma unroll
        for (int j = 0; j < M; ++j) t[j] = entry(j, (int)((cw[j >> 2] >> ((j & 3) * 8)) & 255u));
        if constexpr (M == 8 || M == 16) { if (tree) return tree_sum<M>(t); }
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < M; ++j) acc = __fadd_rn(acc, t[j]);
        return acc;
    } else {
        float acc = 0.0f;
        for (int j = 0; j < m; ++j) acc = __fadd_rn(acc, entry(j, (int)__ldg(row + j)));
        return acc;
    }
}

}  // namespace scan
}  // namespace psb
