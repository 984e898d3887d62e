// Training and encoding kernels: PQ encode (nearest codeword per sub-vector), PQ codebook Lloyd updates,
// k-means accumulation / update, and the counter-based synthetic data generators used by the bench.
//
// Semantics follow the reference trainers: assignment = argmin of squared L2 with strict '<' so the lowest
// index wins ties (src/clustering/kmeans/kmeans_utils.cu:359-413, src/quantization/pq/pq_encode.cuh:24-40),
// update = mean of members, empty cluster keeps its centroid (src/clustering/kmeans/kmeans_utils.cu:267-284).
// Member sums are accumulated in fp64 so the result does not depend on the summation order.
#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace {

constexpr int kEncThreads = 256;

// One CTA encodes kEncThreads rows for every sub-quantiser; codes are staged in shared memory and written
// out as whole rows.
__global__ void __launch_bounds__(kEncThreads)
k_pq_encode(const float* __restrict__ data, long long n, int dim, const float* __restrict__ codebook, int m, int k,
            uint8_t* __restrict__ codes) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    const int dsub = dim / m;
    float* s_cb = reinterpret_cast<float*>(s_raw);                            // [k * dsub]
    uint8_t* s_codes = s_raw + (size_t)k * dsub * sizeof(float);              // [kEncThreads * m]
    const long long row = (long long)blockIdx.x * kEncThreads + threadIdx.x;
    for (int sub = 0; sub < m; ++sub) {
        __syncthreads();
        for (int i = threadIdx.x; i < k * dsub; i += kEncThreads) s_cb[i] = codebook[(size_t)sub * k * dsub + i];
        __syncthreads();
        if (row < n) {
            const float* x = data + (size_t)row * dim + (size_t)sub * dsub;
            float best = FLT_MAX; int bc = 0;
            for (int c = 0; c < k; ++c) {
                float dist = 0.0f;
                for (int d = 0; d < dsub; ++d) {
                    const float diff = __fsub_rn(__ldg(x + d), s_cb[c * dsub + d]);
                    dist = __fadd_rn(dist, __fmul_rn(diff, diff));
                }
                if (dist < best) { best = dist; bc = c; }
            }
            s_codes[threadIdx.x * m + sub] = (uint8_t)bc;
        }
    }
    __syncthreads();
    const long long row0 = (long long)blockIdx.x * kEncThreads;
    const long long rows_here = min((long long)kEncThreads, n - row0);
    for (long long i = threadIdx.x; i < rows_here * m; i += kEncThreads) codes[(size_t)row0 * m + i] = s_codes[i];
}

// Same result, rows staged in shared memory: the CTA's rows are read once with coalesced loads into a tile padded to
// dim + 1 floats per row (conflict-free when every thread reads its own row), each thread keeps its sub-vector in
// registers while it walks the 256 codewords (broadcast reads).  DSUB = 0: run-time sub-vector length.
template <int DSUB>
__global__ void __launch_bounds__(kEncThreads)
k_pq_encode_tile(const float* __restrict__ data, long long n, int dim, const float* __restrict__ codebook, int m, int k,
                 uint8_t* __restrict__ codes) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    const int dsub = DSUB > 0 ? DSUB : dim / m;
    const int pitch = dim + 1;
    float* s_x = reinterpret_cast<float*>(s_raw);                                            // [kEncThreads][pitch]
    float* s_cb = s_x + (size_t)kEncThreads * pitch;                                         // [k * dsub]
    uint8_t* s_codes = reinterpret_cast<uint8_t*>(s_cb + (size_t)k * dsub);                  // [kEncThreads * m]
    const long long row0 = (long long)blockIdx.x * kEncThreads;
    const long long rows_here = min((long long)kEncThreads, n - row0);
    for (long long i = threadIdx.x; i < rows_here * dim; i += kEncThreads) {
        const int r = (int)(i / dim), d = (int)(i % dim);
        s_x[(size_t)r * pitch + d] = data[(size_t)row0 * dim + i];
    }
    const bool live = threadIdx.x < rows_here;
    const float* xs = s_x + (size_t)threadIdx.x * pitch;
    for (int sub = 0; sub < m; ++sub) {
        __syncthreads();
        for (int i = threadIdx.x; i < k * dsub; i += kEncThreads) s_cb[i] = codebook[(size_t)sub * k * dsub + i];
        __syncthreads();
        if (live) {
            float best = FLT_MAX; int bc = 0;
            if constexpr (DSUB > 0) {
                float xr[DSUB];
#pragma unroll
                for (int d = 0; d < DSUB; ++d) xr[d] = xs[sub * DSUB + d];
#pragma unroll 4
                for (int c = 0; c < k; ++c) {
                    float dist = 0.0f;
#pragma unroll
                    for (int d = 0; d < DSUB; ++d) {
                        const float diff = __fsub_rn(xr[d], s_cb[c * DSUB + d]);
                        dist = __fadd_rn(dist, __fmul_rn(diff, diff));
                    }
                    if (dist < best) { best = dist; bc = c; }
                }
            } else {
                for (int c = 0; c < k; ++c) {
                    float dist = 0.0f;
                    for (int d = 0; d < dsub; ++d) {
                        const float diff = __fsub_rn(xs[sub * dsub + d], s_cb[c * dsub + d]);
                        dist = __fadd_rn(dist, __fmul_rn(diff, diff));
                    }
                    if (dist < best) { best = dist; bc = c; }
                }
            }
            s_codes[threadIdx.x * m + sub] = (uint8_t)bc;
        }
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < rows_here * m; i += kEncThreads) codes[(size_t)row0 * m + i] = s_codes[i];
}

__global__ void k_pq_accumulate(const float* __restrict__ data, long long n, int dim, const uint8_t* __restrict__ codes,
                                int m, int k, double* __restrict__ sums, int* __restrict__ counts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * m) return;
    const long long row = i / m; const int sub = (int)(i % m);
    const int dsub = dim / m;
    const int c = codes[i];
    atomicAdd(&counts[sub * k + c], 1);
    for (int d = 0; d < dsub; ++d)
        atomicAdd(&sums[((size_t)sub * k + c) * dsub + d], (double)data[(size_t)row * dim + sub * dsub + d]);
}

__global__ void k_mean_update(const double* __restrict__ sums, const int* __restrict__ counts, long long n_centres,
                              int width, float* __restrict__ centres) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_centres * width) return;
    const int c = counts[i / width];
    if (c > 0) centres[i] = (float)(sums[i] / (double)c);
}

// out[row] = data[row] - centroids[assign[row]] (fp32 subtraction): what residual-mode PQ is trained on and encodes.
__global__ void k_residual_rows(const float* __restrict__ data, long long n, int dim, const float* __restrict__ centroids,
                                const int* __restrict__ assign, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * dim) return;
    const long long row = i / dim;
    const int d = (int)(i - row * dim);
    out[i] = __fsub_rn(data[i], __ldg(centroids + (size_t)assign[row] * dim + d));
}

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Initial codewords: codeword (sub, c) = sub-vector of the row hash(seed, sub, c) mod n.
__global__ void k_pq_init(const float* __restrict__ data, long long n, int dim, int m, int k, uint64_t seed,
                          float* __restrict__ codebook) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * k) return;
    const int sub = i / k;
    const int dsub = dim / m;
    const uint64_t h = splitmix64(splitmix64(seed + 0x51ED27ull * (uint64_t)sub) + (uint64_t)i);
    const long long row = (long long)(h % (uint64_t)n);
    for (int d = 0; d < dsub; ++d) codebook[(size_t)i * dsub + d] = data[(size_t)row * dim + sub * dsub + d];
}

__global__ void k_kmeans_accumulate(const float* __restrict__ data, long long n, int dim, const int* __restrict__ assign,
                                    const float* __restrict__ best, double* __restrict__ sums, int* __restrict__ counts,
                                    double* __restrict__ obj) {
    // one warp per row
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= n) return;
    const int c = assign[w];
    for (int d = lane; d < dim; d += 32) atomicAdd(&sums[(size_t)c * dim + d], (double)data[(size_t)w * dim + d]);
    if (lane == 0) {
        atomicAdd(&counts[c], 1);
        if (obj && best) atomicAdd(obj, (double)best[w]);
    }
}

// Standard normal from a counter: Box-Muller on two 24-bit uniforms of one hashed 64-bit word.
__device__ __forceinline__ float normal_from(uint64_t seed, uint64_t counter) {
    const uint64_t h = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull));
    const float u1 = ((float)((h >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
    const float u2 = (float)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);            // [0,1)
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

__global__ void k_gen_mixture(const float* __restrict__ centres, const long long* __restrict__ offsets, int ncomp,
                              int dim, float sigma, uint64_t seed, long long row_begin, long long n,
                              float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * dim) return;
    const long long row = row_begin + i / dim;
    const int d = (int)(i % dim);
    int lo = 0, hi = ncomp;  // largest c with offsets[c] <= row
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offsets[mid] <= row) lo = mid; else hi = mid;
    }
    out[i] = centres[(size_t)lo * dim + d] + sigma * normal_from(seed, (uint64_t)row * (uint64_t)dim + (uint64_t)d);
}

__global__ void k_gen_normal(uint64_t seed, long long first, long long n, float scale, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = scale * normal_from(seed, (uint64_t)(first + i));
}

}  // namespace

psb_status launch_pq_encode(const float* d_data, long long n, int dim, const float* d_codebook, int m, int k,
                            uint8_t* d_codes, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    const int dsub = dim / m;
    const unsigned grid = (unsigned)((n + kEncThreads - 1) / kEncThreads);
    const size_t tile = (size_t)kEncThreads * (dim + 1) * sizeof(float) + (size_t)k * dsub * sizeof(float) + (size_t)kEncThreads * m;
    if (tile <= 200 * 1024) {  // rows staged in shared memory
        auto run = [&](auto kernel) -> psb_status {
            PSB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile));
            kernel<<<grid, kEncThreads, tile, s>>>(d_data, n, dim, d_codebook, m, k, d_codes);
            return PSB_OK;
        };
        switch (dsub) {
            case 2: PSB_TRY(run(k_pq_encode_tile<2>)); break;
            case 4: PSB_TRY(run(k_pq_encode_tile<4>)); break;
            case 8: PSB_TRY(run(k_pq_encode_tile<8>)); break;
            default: PSB_TRY(run(k_pq_encode_tile<0>)); break;
        }
        count_launch();
        PSB_LAUNCH_CHECK();
        return PSB_OK;
    }
    const size_t smem = (size_t)k * dsub * sizeof(float) + (size_t)kEncThreads * m;
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_pq_encode, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_pq_encode<<<grid, kEncThreads, smem, s>>>(d_data, n, dim, d_codebook, m, k, d_codes);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_pq_accumulate(const float* d_data, long long n, int dim, const uint8_t* d_codes, int m, int k,
                                double* d_sums, int* d_counts, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    k_pq_accumulate<<<(unsigned)((n * m + 255) / 256), 256, 0, s>>>(d_data, n, dim, d_codes, m, k, d_sums, d_counts);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_pq_update(const double* d_sums, const int* d_counts, int m, int k, int dsub, float* d_codebook,
                            cudaStream_t s) {
    const long long total = (long long)m * k * dsub;
    k_mean_update<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(d_sums, d_counts, (long long)m * k, dsub, d_codebook);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

// codebook[sub][c] = the sub-vector `sub` of data row rows[sub * k + c]
__global__ void k_pq_init_rows(const float* __restrict__ data, int dim, int m, int k, const long long* __restrict__ rows,
                               float* __restrict__ codebook) {
    const int dsub = dim / m;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)m * k * dsub) return;
    const int d = (int)(i % dsub);
    const long long e = i / dsub;   // sub * k + c
    const int sub = (int)(e / k);
    codebook[i] = data[(size_t)rows[e] * dim + (size_t)sub * dsub + d];
}

psb_status launch_pq_init_rows(const float* d_data, int dim, int m, int k, const long long* d_rows, float* d_codebook, cudaStream_t s) {
    const long long total = (long long)m * k * (dim / m);
    k_pq_init_rows<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(d_data, dim, m, k, d_rows, d_codebook);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_pq_init(const float* d_data, long long n, int dim, int m, int k, uint64_t seed,
                          float* d_codebook, cudaStream_t s) {
    k_pq_init<<<(m * k + 255) / 256, 256, 0, s>>>(d_data, n, dim, m, k, seed, d_codebook);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_kmeans_accumulate(const float* d_data, long long n, int dim, const int* d_assign,
                                    const float* d_best, double* d_sums, int* d_counts, double* d_obj,
                                    cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    k_kmeans_accumulate<<<(unsigned)((n * 32 + 255) / 256), 256, 0, s>>>(d_data, n, dim, d_assign, d_best, d_sums, d_counts, d_obj);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_kmeans_update(const double* d_sums, const int* d_counts, int k, int dim, float* d_centroids,
                                cudaStream_t s) {
    const long long total = (long long)k * dim;
    k_mean_update<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(d_sums, d_counts, k, dim, d_centroids);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_residual_rows(const float* d_data, long long n, int dim, const float* d_centroids, const int* d_assign,
                                float* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    k_residual_rows<<<(unsigned)((n * dim + 255) / 256), 256, 0, s>>>(d_data, n, dim, d_centroids, d_assign, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_gen_mixture(const float* d_centres, const long long* d_offsets, int ncomp, int dim, float sigma,
                              uint64_t seed, long long row_begin, long long n, float* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    const long long total = n * dim;
    k_gen_mixture<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(d_centres, d_offsets, ncomp, dim, sigma, seed, row_begin, n, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_gen_normal(uint64_t seed, long long first, long long n, float scale, float* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    k_gen_normal<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(seed, first, n, scale, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

}  // namespace psb
