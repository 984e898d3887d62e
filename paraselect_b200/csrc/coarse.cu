// Coarse stage, exact part: fp32 squared-L2 distances in the CPU path's arithmetic (sequential, non-fused:
// sum += (q-c)*(q-c), reference src/cpu/utils/cpu_distance.h:74-81) and per-row selection of the k smallest
// (distance, id) pairs.  The tensor-core filter in coarse_tc.cu narrows the centroid set first; what it keeps
// is scored by the kernels here, so results are bit-identical with or without it.
#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace {

constexpr int BQ = 64, BC = 128, KC = 16, kDistThreads = 256;

// dist[q][c] for a BQ x BC tile; each thread owns 4 queries x 8 centroids.
__global__ void __launch_bounds__(kDistThreads)
k_coarse_dist_exact(const float* __restrict__ queries, int nq, const float* __restrict__ centroids, int nlist,
                    int dim, float* __restrict__ dist) {
    __shared__ __align__(16) float qs[KC][BQ];
    __shared__ __align__(16) float cs[KC][BC];
    const int q0 = blockIdx.y * BQ, c0 = blockIdx.x * BC;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    for (int d0 = 0; d0 < dim; d0 += KC) {
        for (int i = threadIdx.x; i < BQ * KC; i += kDistThreads) {
            const int row = i % BQ, d = i / BQ;
            qs[d][row] = (q0 + row < nq && d0 + d < dim) ? queries[(size_t)(q0 + row) * dim + d0 + d] : 0.0f;
        }
        for (int i = threadIdx.x; i < BC * KC; i += kDistThreads) {
            const int row = i % BC, d = i / BC;
            cs[d][row] = (c0 + row < nlist && d0 + d < dim) ? centroids[(size_t)(c0 + row) * dim + d0 + d] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < KC; ++d) {
            const float4 qv = *reinterpret_cast<const float4*>(&qs[d][ty * 4]);
            const float4 ca = *reinterpret_cast<const float4*>(&cs[d][tx * 8]);
            const float4 cb = *reinterpret_cast<const float4*>(&cs[d][tx * 8 + 4]);
            const float qa[4] = {qv.x, qv.y, qv.z, qv.w};
            const float cc[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float diff = __fsub_rn(qa[i], cc[j]);
                    acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(diff, diff));
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q0 + ty * 4 + i;
        if (q >= nq) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + tx * 8 + j;
            if (c < nlist) dist[(size_t)q * nlist + c] = acc[i][j];
        }
    }
}

// Per row: the k smallest (value, index) pairs, ascending.  64-bit radix select (8-bit digits, most significant
// first, stopping as soon as the chosen bucket is taken whole), gather, bitonic sort.
constexpr int kSelThreads = 512;
__global__ void __launch_bounds__(kSelThreads)
k_select_rows(const float* __restrict__ dist, int n, int k, int* __restrict__ out_ids, float* __restrict__ out_dist) {
    extern __shared__ __align__(16) uint64_t s_sel[];  // [pow2 >= k]
    __shared__ unsigned int s_hist[256];
    __shared__ uint64_t s_prefix;
    __shared__ unsigned int s_rank;
    __shared__ int s_done, s_cnt;
    const float* row = dist + (size_t)blockIdx.x * n;
    if (threadIdx.x == 0) { s_prefix = 0; s_rank = (unsigned)k; s_done = 0; s_cnt = 0; }
    uint64_t mask = 0;
    uint64_t cut = KEY_MAX;
    if (k < n) {
        for (int pass = 7; pass >= 0; --pass) {
            const int shift = pass * 8;
            for (int i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0;
            __syncthreads();
            if (s_done) break;
            const uint64_t prefix = s_prefix;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const uint64_t key = make_key(row[i], (uint32_t)i);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255], 1u);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                unsigned cum = 0;
                const unsigned rank = s_rank;
                for (int b = 0; b < 256; ++b) {
                    const unsigned h = s_hist[b];
                    if (cum + h >= rank) {
                        s_prefix = prefix | ((uint64_t)b << shift);
                        s_rank = rank - cum;
                        if (h == rank - cum) s_done = 1;  // the whole bucket is selected
                        break;
                    }
                    cum += h;
                }
            }
            mask |= 255ull << shift;
            __syncthreads();
        }
        __syncthreads();
        // keys <= cut are exactly the k smallest: cut = prefix with every undecided low bit set
        cut = s_prefix | ~mask;
    }
    const int np = next_pow2(max(k, 2));
    for (int i = threadIdx.x; i < np; i += blockDim.x) s_sel[i] = KEY_MAX;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const uint64_t key = make_key(row[i], (uint32_t)i);
        if (key <= cut) {
            const int slot = atomicAdd(&s_cnt, 1);
            if (slot < np) s_sel[slot] = key;
        }
    }
    __syncthreads();
    block_bitonic_sort(s_sel, np);
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const uint64_t key = s_sel[i];
        const bool ok = key != KEY_MAX;
        out_ids[(size_t)blockIdx.x * k + i] = ok ? (int)key_idx(key) : -1;
        if (out_dist) out_dist[(size_t)blockIdx.x * k + i] = ok ? key_dist(key) : FLT_MAX;
    }
}

}  // namespace

psb_status launch_coarse_dist_exact(const float* d_queries, int nq, const float* d_centroids, int nlist,
                                    int dim, float* d_dist, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    dim3 grid((nlist + BC - 1) / BC, (nq + BQ - 1) / BQ);
    k_coarse_dist_exact<<<grid, kDistThreads, 0, s>>>(d_queries, nq, d_centroids, nlist, dim, d_dist);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_select_rows(const float* d_dist, int nq, int n, int k, int* d_ids, float* d_out, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    if (k <= 0 || k > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "row selection supports 1..4096 results");
    int np = 2;
    while (np < k) np <<= 1;
    k_select_rows<<<nq, kSelThreads, (size_t)np * sizeof(uint64_t), s>>>(d_dist, n, k, d_ids, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

}  // namespace psb

// ---- coarse search without any allocation ---------------------------------------------------------------
// Some callers may not allocate device memory at the moment they need a coarse search: a serving thread that
// holds a fixed memory budget granted at start-up, code that runs under a memory pool it must not touch, or a
// plugin host that forbids cudaMalloc after initialisation because an allocation synchronises the device and
// can fail late.  For them the distance tile [nq][nlist] lives in the array below, which every GPU that loads
// this library holds until the process exits.
namespace psb {
namespace {
constexpr size_t kStaticCoarseFloats = (size_t)4 << 20;  // 4 Mi distances = 16 MiB: nq * nlist must not exceed it
static __device__ __align__(256) float g_coarse_scratch[kStaticCoarseFloats];
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};  // per device: the array's DEVICE address (the symbol itself is a host stand-in)
}  // namespace
}  // namespace psb

extern "C" psb_status psb_coarse_search_static(const float* d_queries, int nq, const float* d_centroids, int nlist,
                                               int dim, int nprobe, int* d_ids, float* d_dist, void* stream) {
    using namespace psb;
    if (!d_queries || !d_centroids || !d_ids || nq < 0 || nlist <= 0 || dim <= 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid coarse request");
    if (nprobe <= 0 || nprobe > nlist) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist");
    if (nprobe > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 is not supported");
    if ((size_t)nq * (size_t)nlist > kStaticCoarseFloats)
        return fail(PSB_UNSUPPORTED_SHAPE,
                    "psb_coarse_search_static: nq * nlist exceeds the 4,194,304 distances of the built-in scratch; "
                    "split the query batch or use psb_stage_coarse");
    if (nq == 0) return PSB_OK;
    int device = -1;
    PSB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(PSB_UNSUPPORTED_SHAPE, "device ordinal above 63");
    if (!g_scratch_ptr[device]) {
        // First call on this device: resolve the array's device address (this device is current).
        float* p = nullptr;
        PSB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_coarse_scratch));
        g_scratch_ptr[device] = p;
    }
    float* tile = g_scratch_ptr[device];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PSB_TRY(launch_coarse_dist_exact(d_queries, nq, d_centroids, nlist, dim, tile, st));
    return launch_select_rows(tile, nq, nlist, nprobe, d_ids, d_dist, st);
}
