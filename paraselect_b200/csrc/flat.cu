// IVF-Flat fine scan over device-resident rows: for every query the exact fp32 squared L2 distance to every row of its
// probed lists, and the topk nearest by (distance, row).
//
// One CTA per query.  Rows are staged through shared memory in tiles (coalesced loads, one padded row per thread afterwards),
// each thread sums one row in the CPU path's arithmetic - sequential, sub / mul / add without FMA, the reference's
// l2_distance_squared (src/cpu/utils/cpu_distance.h:74-81) - and a running top-k keeps the best: keys below the current cutoff
// are appended to a buffer that is sorted and cut back to topk whenever it could overflow.  Results equal the reference's
// cpu_ivf_search (src/cpu/search/cpu_search.h:226-332) with ties by row; the kernel reads each probed row once per visiting
// query, so its bound is HBM: bytes = sum over (query, probe) of rows * dim * 4.
//
// Reference counterpart: the GPU-resident fine kernels of src/search/kernels/fine/gpu_fine/resident/resident_full_l2_topk.cu:19-178
// behind ivfflat_search (src/search/ivfflat/ivfflat_search.cuh:41-51).
#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace {

constexpr int kFlatThreads = 256;
constexpr int kFlatTile = 128;  // rows per shared-memory tile

__global__ void __launch_bounds__(kFlatThreads)
k_flat_scan(const float* __restrict__ queries, int dim, const int* __restrict__ probes, int nprobe,
            const long long* __restrict__ offsets, int nlist, const float* __restrict__ rows, long long row_base, int topk,
            int buf_n, int* __restrict__ out_rows, float* __restrict__ out_dist, unsigned long long* __restrict__ counters) {
    extern __shared__ __align__(16) unsigned char s_flat[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_flat);                         // [buf_n]
    float* s_q = reinterpret_cast<float*>(s_flat + (size_t)buf_n * 8);             // [dim]
    float* s_tile = s_q + ((dim + 3) & ~3);                                         // [kFlatTile][dim + 1]
    __shared__ int s_cnt;
    __shared__ uint64_t s_cut;
    const int q = blockIdx.x;
    const int pitch = dim + 1;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) s_q[d] = queries[(size_t)q * dim + d];
    if (threadIdx.x == 0) { s_cnt = 0; s_cut = KEY_MAX; }
    __syncthreads();
    long long scanned = 0;
    for (int p = 0; p < nprobe; ++p) {
        const int l = probes[(size_t)q * nprobe + p];
        if (l < 0 || l >= nlist) continue;  // uniform
        const long long b = offsets[l], e = offsets[l + 1];
        scanned += e - b;
        for (long long r0 = b; r0 < e; r0 += kFlatTile) {
            const int n = (int)min((long long)kFlatTile, e - r0);
            const float* src = rows + (size_t)(r0 - row_base) * dim;
            for (int i = threadIdx.x; i < n * dim; i += blockDim.x) s_tile[(i / dim) * pitch + (i % dim)] = __ldg(src + i);
            const int c_now = s_cnt;  // stable since the barrier that ended the previous tile
            __syncthreads();
            if (c_now + kFlatTile > buf_n) {  // uniform
                for (int i = c_now + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
                __syncthreads();
                block_bitonic_sort(s_keys, buf_n);
                if (threadIdx.x == 0) {
                    const int keep = c_now < topk ? c_now : topk;
                    s_cnt = keep;
                    s_cut = keep == topk ? s_keys[topk - 1] : KEY_MAX;
                }
                __syncthreads();
            }
            if (threadIdx.x < n) {
                const float* t = s_tile + threadIdx.x * pitch;
                float sum = 0.0f;
                for (int d = 0; d < dim; ++d) {
                    const float diff = __fsub_rn(s_q[d], t[d]);
                    sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                }
                const uint64_t key = make_key(sum, (uint32_t)(r0 + threadIdx.x));
                if (key < s_cut) s_keys[atomicAdd(&s_cnt, 1)] = key;
            }
            __syncthreads();
        }
    }
    const int c = s_cnt;
    for (int i = c + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
    __syncthreads();
    block_bitonic_sort(s_keys, buf_n);
    for (int i = threadIdx.x; i < topk; i += blockDim.x) {
        const uint64_t key = s_keys[i];
        const bool ok = key != KEY_MAX;
        out_rows[(size_t)q * topk + i] = ok ? (int)key_idx(key) : -1;
        out_dist[(size_t)q * topk + i] = ok ? key_dist(key) : FLT_MAX;
    }
    if (threadIdx.x == 0 && counters) atomicAdd(&counters[0], (unsigned long long)scanned);
}

// The same scan without the shared-memory tile, for dim % 4 == 0 and 16-byte aligned rows: every thread reads its own row
// straight from global memory with 16-byte loads (a row is a run of whole 128-byte lines, and the lines of a warp's 32 rows
// stay in L1 from one load to the next), so all 256 threads score rows, nothing is staged and re-read, and a step needs
// barriers only for the key buffer.  Same arithmetic in the same order, same keys.
constexpr int kFlatStep = kFlatThreads;   // rows per step
__global__ void __launch_bounds__(kFlatThreads)
k_flat_scan_direct(const float* __restrict__ queries, int dim, const int* __restrict__ probes, int nprobe,
                   const long long* __restrict__ offsets, int nlist, const float* __restrict__ rows, long long row_base, int topk,
                   int buf_n, int* __restrict__ out_rows, float* __restrict__ out_dist, unsigned long long* __restrict__ counters) {
    extern __shared__ __align__(16) unsigned char s_flat[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_flat);                         // [buf_n]
    float4* s_q = reinterpret_cast<float4*>(s_flat + (size_t)buf_n * 8);           // [dim / 4]
    __shared__ int s_cnt;
    __shared__ uint64_t s_cut;
    const int q = blockIdx.x;
    const int dim4 = dim >> 2;
    for (int d = threadIdx.x; d < dim4; d += blockDim.x) s_q[d] = reinterpret_cast<const float4*>(queries + (size_t)q * dim)[d];
    if (threadIdx.x == 0) { s_cnt = 0; s_cut = KEY_MAX; }
    __syncthreads();
    long long scanned = 0;
    for (int p = 0; p < nprobe; ++p) {
        const int l = probes[(size_t)q * nprobe + p];
        if (l < 0 || l >= nlist) continue;  // uniform
        const long long b = offsets[l], e = offsets[l + 1];
        scanned += e - b;
        for (long long r0 = b; r0 < e; r0 += kFlatStep) {
            const int c_now = s_cnt;  // stable since the barrier that ended the previous step
            __syncthreads();
            if (c_now + kFlatStep > buf_n) {  // uniform
                for (int i = c_now + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
                __syncthreads();
                block_bitonic_sort(s_keys, buf_n);
                if (threadIdx.x == 0) {
                    const int keep = c_now < topk ? c_now : topk;
                    s_cnt = keep;
                    s_cut = keep == topk ? s_keys[topk - 1] : KEY_MAX;
                }
                __syncthreads();
            }
            const uint64_t cut = s_cut;
            const long long row = r0 + threadIdx.x;
            if (row < e) {
                const float4* src = reinterpret_cast<const float4*>(rows + (size_t)(row - row_base) * dim);
                float sum = 0.0f;
#pragma unroll 8
                for (int d = 0; d < dim4; ++d) {
                    const float4 v = __ldg(src + d);
                    const float4 qv = s_q[d];
                    float diff = __fsub_rn(qv.x, v.x); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(qv.y, v.y); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(qv.z, v.z); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                    diff = __fsub_rn(qv.w, v.w); sum = __fadd_rn(sum, __fmul_rn(diff, diff));
                }
                const uint64_t key = make_key(sum, (uint32_t)row);
                if (key < cut) s_keys[atomicAdd(&s_cnt, 1)] = key;
            }
            __syncthreads();
        }
    }
    const int c = s_cnt;
    for (int i = c + threadIdx.x; i < buf_n; i += blockDim.x) s_keys[i] = KEY_MAX;
    __syncthreads();
    block_bitonic_sort(s_keys, buf_n);
    for (int i = threadIdx.x; i < topk; i += blockDim.x) {
        const uint64_t key = s_keys[i];
        const bool ok = key != KEY_MAX;
        out_rows[(size_t)q * topk + i] = ok ? (int)key_idx(key) : -1;
        out_dist[(size_t)q * topk + i] = ok ? key_dist(key) : FLT_MAX;
    }
    if (threadIdx.x == 0 && counters) atomicAdd(&counters[0], (unsigned long long)scanned);
}

}  // namespace

psb_status launch_flat_scan(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe, const long long* d_offsets,
                            int nlist, const float* d_rows, long long row_base, int topk, int* d_out_rows, float* d_out_dist,
                            unsigned long long* d_counters, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    if (topk <= 0 || topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "flat scan supports topk in 1..2048");
    if (dim % 4 == 0 && reinterpret_cast<uintptr_t>(d_rows) % 16 == 0 && reinterpret_cast<uintptr_t>(d_queries) % 16 == 0) {
        int buf = 1024;
        while (buf < topk + kFlatStep) buf <<= 1;
        const size_t bytes = (size_t)buf * 8 + (size_t)dim * 4;
        if (bytes <= (size_t)220 * 1024) {
            if (bytes > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_flat_scan_direct, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
            k_flat_scan_direct<<<nq, kFlatThreads, bytes, s>>>(d_queries, dim, d_probes, nprobe, d_offsets, nlist, d_rows, row_base, topk,
                                                               buf, d_out_rows, d_out_dist, d_counters);
            count_launch();
            PSB_LAUNCH_CHECK();
            return PSB_OK;
        }
    }
    int buf_n = 1024;
    while (buf_n < topk + kFlatTile) buf_n <<= 1;
    const size_t smem = (size_t)buf_n * 8 + (size_t)((dim + 3) & ~3) * 4 + (size_t)kFlatTile * (dim + 1) * 4;
    if (smem > (size_t)220 * 1024) return fail(PSB_UNSUPPORTED_SHAPE, "flat scan: dim too large for the shared-memory tile");
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_flat_scan, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_flat_scan<<<nq, kFlatThreads, smem, s>>>(d_queries, dim, d_probes, nprobe, d_offsets, nlist, d_rows, row_base, topk, buf_n,
                                               d_out_rows, d_out_dist, d_counters);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

}  // namespace psb
