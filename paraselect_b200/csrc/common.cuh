// Shared device helpers and host-side status plumbing for the sm_100a IVF-PQ search library.
#pragma once

#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/psb.h"

// NVTX ranges per stage, compiled in with -DPSB_USE_NVTX=1 (the names are the reference's stage names,
// src/utils/nsight_nvtx.h:17-38 and src/search/ivfpq/pipeline/ivfpq_pipeline.cu:41-71).  NVTX 3 is header-only: without a
// profiler attached a range costs one indirect call.
#if defined(PSB_USE_NVTX) && PSB_USE_NVTX
#include <nvtx3/nvToolsExt.h>
#include <nvtx3/nvToolsExtCudaRt.h>
namespace psb {
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};
inline void nvtx_name_stream(cudaStream_t s, const char* name) { nvtxNameCudaStreamA(s, name); }
inline constexpr bool kNvtxCompiled = true;
}  // namespace psb
#else
namespace psb {
struct NvtxRange {
    explicit NvtxRange(const char*) {}
};
inline void nvtx_name_stream(cudaStream_t, const char*) {}
inline constexpr bool kNvtxCompiled = false;
}  // namespace psb
#endif
#define PSB_RANGE_CAT2(a, b) a##b
#define PSB_RANGE_CAT(a, b) PSB_RANGE_CAT2(a, b)
#define PSB_RANGE(name) ::psb::NvtxRange PSB_RANGE_CAT(psb_nvtx_range_, __LINE__)(name)

namespace psb {

// ---- host: status and error text ---------------------------------------------------------------
std::string& last_error_ref();
psb_status fail(psb_status code, const std::string& message);
psb_status cuda_fail(cudaError_t err, const char* what, const char* file, int line);

#define PSB_CUDA(call)                                                              \
    do {                                                                            \
        cudaError_t psb_err__ = (call);                                             \
        if (psb_err__ != cudaSuccess) return psb::cuda_fail(psb_err__, #call, __FILE__, __LINE__); \
    } while (0)

#define PSB_TRY(call)                                \
    do {                                             \
        psb_status psb_st__ = (call);                \
        if (psb_st__ != PSB_OK) return psb_st__;     \
    } while (0)

#define PSB_LAUNCH_CHECK() PSB_CUDA(cudaGetLastError())

// Counts kernel launches issued by this library (reported through psb_stats.kernel_launches).
void count_launch(long long n = 1);
long long launches_total();

// ---- device: order-preserving float <-> uint32 ---------------------------------------------------
// bits & 0x80000000 ? ~bits : bits ^ 0x80000000 (radix-sortable float; same mapping as the reference's
// src/search/kernels/fine/gpu_fine/pq_adc/pq_candidate_cap_select.cu:19-28).
__host__ __device__ __forceinline__ uint32_t f2o(float f) {
#ifdef __CUDA_ARCH__
    uint32_t b = __float_as_uint(f);
#else
    uint32_t b; __builtin_memcpy(&b, &f, 4);
#endif
    return (b & 0x80000000u) ? ~b : (b ^ 0x80000000u);
}
__host__ __device__ __forceinline__ float o2f(uint32_t o) {
    uint32_t b = (o & 0x80000000u) ? (o ^ 0x80000000u) : ~o;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float f; __builtin_memcpy(&f, &b, 4); return f;
#endif
}
// Composite selection key: (distance, index) ascending == key ascending.
__host__ __device__ __forceinline__ uint64_t make_key(float d, uint32_t idx) {
    return (static_cast<uint64_t>(f2o(d)) << 32) | idx;
}
__host__ __device__ __forceinline__ float key_dist(uint64_t k) { return o2f(static_cast<uint32_t>(k >> 32)); }
__host__ __device__ __forceinline__ uint32_t key_idx(uint64_t k) { return static_cast<uint32_t>(k); }

constexpr uint64_t KEY_MAX = ~0ull;

#ifdef __CUDACC__
// Asks for the maximum shared-memory carve-out for a kernel, whether or not it uses much shared memory.  An SM runs kernels of
// one carve-out at a time; the scan, coarse and selection kernels need nearly all of it, so every kernel that may run beside
// them on the other stream of the overlapped pipeline (and the small kernels queued between them) asks for the same
// carve-out - otherwise the SMs drain between kernels instead of sharing.
template <typename F>
inline psb_status prefer_max_shared(F kernel) {
    PSB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    return PSB_OK;
}

// ---- device: block-wide bitonic sort of n (power of two) keys in shared memory, ascending ---------
template <typename K>
__device__ __forceinline__ void block_bitonic_sort(K* s, int n) {
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int p = i + j;
                const bool asc = (i & k) == 0;
                const K a = s[i], b = s[p];
                if ((a > b) == asc) { s[i] = b; s[p] = a; }
            }
            __syncthreads();
        }
    }
}

__device__ __forceinline__ int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Block-wide exclusive prefix sum of one int per thread (blockDim.x <= 1024, multiple of 32).
// warp_sums must hold 32 ints of shared memory.  Returns the exclusive prefix; *total gets the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        warp_sums[lane] = wi - w;  // exclusive warp offsets
        if (lane == 31 && total) *total = wi;
    }
    __syncthreads();
    const int r = warp_sums[warp] + incl - v;
    __syncthreads();
    return r;
}
#endif  // __CUDACC__

}  // namespace psb
