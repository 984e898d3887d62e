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

// Assignment of the Lloyd iterations of PQ training: nearest codeword by |c|^2 - 2 x.c (the row's own |x|^2 is the same for every
// codeword and left out), four fused multiply-adds per codeword for DSUB = 4, four rows per thread sharing every codeword read.
// Less than half the instructions of the encoder's (x - c)^2 chain, which is kept for the final encoding: that one reproduces the
// reference encoder's arithmetic bit for bit, this one only has to pick a nearest codeword (the reference's trainer assigns
// with a TF32 GEMM: src/quantization/pq/pq_trainer.cu:97-170); the lowest index still wins an exact tie.
constexpr int kAssignRows = 4;   // rows per thread
template <int DSUB>
__global__ void __launch_bounds__(kEncThreads)
k_pq_assign_train(const float* __restrict__ data, long long n, int dim, const float* __restrict__ codebook, int m, int k,
                  uint8_t* __restrict__ codes) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    float* s_cb = reinterpret_cast<float*>(s_raw);                                   // [k][DSUB]: -2 c
    float* s_nrm = s_cb + (size_t)k * DSUB;                                          // [k]: |c|^2
    uint8_t* s_codes = reinterpret_cast<uint8_t*>(s_nrm + k);                        // [rows per CTA][m]
    constexpr int kRowsPerCta = kEncThreads * kAssignRows;
    const long long row0 = (long long)blockIdx.x * kRowsPerCta;
    const long long rows_here = min((long long)kRowsPerCta, n - row0);
    for (int sub = 0; sub < m; ++sub) {
        __syncthreads();
        for (int c = threadIdx.x; c < k; c += kEncThreads) {
            float nrm = 0.f;
#pragma unroll
            for (int d = 0; d < DSUB; ++d) {
                const float v = codebook[((size_t)sub * k + c) * DSUB + d];
                s_cb[c * DSUB + d] = -2.0f * v;
                nrm = fmaf(v, v, nrm);
            }
            s_nrm[c] = nrm;
        }
        __syncthreads();
        float x[kAssignRows][DSUB], best[kAssignRows];
        int bc[kAssignRows];
#pragma unroll
        for (int r = 0; r < kAssignRows; ++r) {
            const long long row = row0 + threadIdx.x + (long long)r * kEncThreads;
            best[r] = FLT_MAX; bc[r] = 0;
#pragma unroll
            for (int d = 0; d < DSUB; ++d) x[r][d] = row < n ? __ldg(data + (size_t)row * dim + (size_t)sub * DSUB + d) : 0.f;
        }
#pragma unroll 4
        for (int c = 0; c < k; ++c) {
            float cb[DSUB];
#pragma unroll
            for (int d = 0; d < DSUB; ++d) cb[d] = s_cb[c * DSUB + d];
            const float nrm = s_nrm[c];
#pragma unroll
            for (int r = 0; r < kAssignRows; ++r) {
                float dist = nrm;
#pragma unroll
                for (int d = 0; d < DSUB; ++d) dist = fmaf(x[r][d], cb[d], dist);
                if (dist < best[r]) { best[r] = dist; bc[r] = c; }
            }
        }
#pragma unroll
        for (int r = 0; r < kAssignRows; ++r) s_codes[(threadIdx.x + r * kEncThreads) * m + sub] = (uint8_t)bc[r];
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < rows_here * m; i += kEncThreads) codes[(size_t)row0 * m + i] = s_codes[i];
}

// Codeword sums without a global atomic per element: a CTA takes a range of rows and a group of subspaces, accumulates into
// fp64 sums and counts in shared memory (G subspaces x k codewords x dsub), and adds its non-zero entries to the global
// sums once at the end.  grid (row ranges, subspace groups); dynamic shared memory = G * k * (dsub * 8 + 4) bytes.
constexpr int kPqAccRows = 8192;
__global__ void __launch_bounds__(256) k_pq_accumulate(const float* __restrict__ data, long long n, int dim, const uint8_t* __restrict__ codes,
                                                       int m, int k, int group, double* __restrict__ sums, int* __restrict__ counts) {
    extern __shared__ __align__(16) unsigned char s_pq_raw[];
    const int dsub = dim / m;
    const int sub0 = blockIdx.y * group;
    const int g = min(group, m - sub0);
    double* s_sums = reinterpret_cast<double*>(s_pq_raw);                                  // [g][k][dsub]
    int* s_cnt = reinterpret_cast<int*>(s_pq_raw + (size_t)group * k * dsub * sizeof(double));  // [g][k]
    for (int i = threadIdx.x; i < g * k * dsub; i += blockDim.x) s_sums[i] = 0.0;
    for (int i = threadIdx.x; i < g * k; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();
    const long long r0 = (long long)blockIdx.x * kPqAccRows;
    const long long r1 = min(n, r0 + kPqAccRows);
    const long long pairs = (r1 - r0) * g;
    for (long long i = threadIdx.x; i < pairs; i += blockDim.x) {
        const long long row = r0 + i / g;
        const int j = (int)(i % g), sub = sub0 + j;
        const int c = codes[(size_t)row * m + sub];
        atomicAdd(&s_cnt[j * k + c], 1);
        const float* x = data + (size_t)row * dim + (size_t)sub * dsub;
        double* dst = s_sums + ((size_t)j * k + c) * dsub;
        for (int d = 0; d < dsub; ++d) atomicAdd(&dst[d], (double)x[d]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g * k; i += blockDim.x) {
        const int cnt = s_cnt[i];
        if (!cnt) continue;
        atomicAdd(&counts[(size_t)sub0 * k + i], cnt);
        for (int d = 0; d < dsub; ++d) atomicAdd(&sums[((size_t)sub0 * k + i) * dsub + d], s_sums[(size_t)i * dsub + d]);
    }
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

// ---- k-means accumulation: rows grouped by centroid, then one CTA sums each group --------------------------------------
// (the reference sorts by assignment and accumulates segment by segment for the same reason: src/clustering/kmeans/
// kmeans.cu:519-575, kmeans_utils.cu:541-574; per-element atomics onto k * dim fp64 words serialise on popular centroids).
// 1. k_km_count:   counts[c] (one int atomic per row) and the objective (one fp64 atomic per CTA)
// 2. k_km_offsets: exclusive prefix of the counts, one CTA in coalesced rounds
// 3. k_km_fill:    order[offset[c] + slot] = row (one int atomic per row)
// 4. k_km_sums:    CTA c sums its rows in fp64, eight rows at a time (one per warp), and writes sums[c][:] - no atomics; a
//                  group of at most 1,024 rows is sorted first, so that its sum does not depend on the order the slots were taken
constexpr int kKmSumThreads = 256;
__global__ void k_km_count(const int* __restrict__ assign, const float* __restrict__ best, long long n, int* __restrict__ counts,
                           double* __restrict__ obj) {
    __shared__ double s_part[8];
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    double b = 0.0;
    if (i < n) {
        atomicAdd(&counts[assign[i]], 1);
        if (best) b = (double)best[i];
    }
    if (!obj) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_part[w];
        atomicAdd(obj, t);
    }
}
__global__ void __launch_bounds__(1024) k_km_offsets(const int* __restrict__ counts, int k, int* __restrict__ offsets, int* __restrict__ cursor) {
    __shared__ int s_warp[32];
    __shared__ int s_total;
    int carry = 0;
    for (int base = 0; base < k; base += blockDim.x) {
        const int c = base + threadIdx.x;
        const int v = c < k ? counts[c] : 0;
        const int ex = block_exclusive_scan(v, s_warp, &s_total);
        if (c < k) { offsets[c] = carry + ex; cursor[c] = 0; }
        carry += s_total;
        __syncthreads();
    }
    if (threadIdx.x == 0) offsets[k] = carry;
}
__global__ void k_km_fill(const int* __restrict__ assign, long long n, const int* __restrict__ offsets, int* __restrict__ cursor,
                          int* __restrict__ order) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = assign[i];
    order[offsets[c] + atomicAdd(&cursor[c], 1)] = (int)i;
}
__global__ void __launch_bounds__(kKmSumThreads) k_km_sums(const float* __restrict__ data, int dim, const int* __restrict__ offsets,
                                                           int* __restrict__ order, double* __restrict__ sums) {
    __shared__ int s_rows[1024];
    __shared__ double s_part[kKmSumThreads / 32][256];
    const int c = blockIdx.x;
    const int b0 = offsets[c], cnt = offsets[c + 1] - b0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* rows = order + b0;
    if (cnt > 1 && cnt <= 1024) {   // canonical order for the usual, small group
        int np = 2;
        while (np < cnt) np <<= 1;
        for (int i = threadIdx.x; i < np; i += blockDim.x) s_rows[i] = i < cnt ? rows[i] : 0x7fffffff;
        __syncthreads();
        block_bitonic_sort(s_rows, np);
        rows = s_rows;
    }
    for (int d0 = 0; d0 < dim; d0 += 256) {   // 256 dimensions at a time: eight per lane
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = warp; j < cnt; j += kKmSumThreads / 32) {
            const float* x = data + (size_t)rows[j] * dim + d0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int d = lane + 32 * t;
                if (d0 + d < dim) acc[t] += (double)x[d];
            }
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) s_part[warp][lane + 32 * t] = acc[t];
        __syncthreads();
        for (int d = threadIdx.x; d < 256 && d0 + d < dim; d += blockDim.x) {
            double t = 0.0;
#pragma unroll
            for (int w = 0; w < kKmSumThreads / 32; ++w) t += s_part[w][d];
            sums[(size_t)c * dim + d0 + d] = t;
        }
        __syncthreads();
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

psb_status launch_pq_assign_train(const float* d_data, long long n, int dim, const float* d_codebook, int m, int k,
                                  uint8_t* d_codes, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    const int dsub = dim / m;
    const int rows_per_cta = kEncThreads * kAssignRows;
    const size_t smem = (size_t)k * (dsub + 1) * sizeof(float) + (size_t)rows_per_cta * m;
    if ((dsub != 2 && dsub != 4 && dsub != 8) || smem > (size_t)200 * 1024 || (reinterpret_cast<uintptr_t>(d_data) % 4))
        return launch_pq_encode(d_data, n, dim, d_codebook, m, k, d_codes, s);   // shapes this kernel is not built for
    const unsigned grid = (unsigned)((n + rows_per_cta - 1) / rows_per_cta);
    auto run = [&](auto kernel) -> psb_status {
        PSB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, kEncThreads, smem, s>>>(d_data, n, dim, d_codebook, m, k, d_codes);
        return PSB_OK;
    };
    switch (dsub) {
        case 2: PSB_TRY(run(k_pq_assign_train<2>)); break;
        case 4: PSB_TRY(run(k_pq_assign_train<4>)); break;
        default: PSB_TRY(run(k_pq_assign_train<8>)); break;
    }
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_pq_accumulate(const float* d_data, long long n, int dim, const uint8_t* d_codes, int m, int k,
                                double* d_sums, int* d_counts, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    const int dsub = dim / m;
    const size_t per_sub = (size_t)k * ((size_t)dsub * sizeof(double) + sizeof(int));
    int group = (int)std::max<size_t>(1, std::min<size_t>((size_t)m, ((size_t)96 * 1024) / per_sub));
    const size_t smem = (size_t)group * per_sub;
    if (smem > (size_t)200 * 1024) return fail(PSB_UNSUPPORTED_SHAPE, "PQ sub-vectors too wide for the accumulation kernel");
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_pq_accumulate, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)((n + kPqAccRows - 1) / kPqAccRows), (unsigned)((m + group - 1) / group));
    k_pq_accumulate<<<grid, 256, smem, s>>>(d_data, n, dim, d_codes, m, k, group, d_sums, d_counts);
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

psb_status launch_kmeans_accumulate(const float* d_data, long long n, int dim, const int* d_assign, const float* d_best, int k,
                                    double* d_sums, int* d_counts, double* d_obj, const KmeansAccumWs& ws, cudaStream_t s) {
    if (n > 0x7fffffffLL) return fail(PSB_UNSUPPORTED_SHAPE, "more than 2^31-1 rows in one accumulation");
    if (!ws.order || !ws.offsets || !ws.cursor) return fail(PSB_INTERNAL, "k-means accumulation workspace missing");
    // d_counts and *d_obj were zeroed by the caller; d_sums is written whole
    if (n > 0) {
        k_km_count<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_assign, d_best, n, d_counts, d_obj);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    k_km_offsets<<<1, 1024, 0, s>>>(d_counts, k, ws.offsets, ws.cursor);
    count_launch();
    PSB_LAUNCH_CHECK();
    if (n > 0) {
        k_km_fill<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_assign, n, ws.offsets, ws.cursor, ws.order);
        count_launch();
        PSB_LAUNCH_CHECK();
    }
    k_km_sums<<<k, kKmSumThreads, 0, s>>>(d_data, dim, ws.offsets, ws.order, d_sums);
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
