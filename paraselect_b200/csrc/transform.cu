// OPQ rotation of rows: y = R x for every row x, R row-major [out][in] as the reference stores it
// (src/transform/opq_transform.cu:124-163 runs it as one SGEMM; src/search/ivfpq/ivfpq_index.cu:205-217 applies it to the
// queries of a request before the PQ tables are built).  Here each output element is one fp32 chain
// acc = fma(R[o][i], x[i], acc), i = 0 .. dim-1 in order, so the result does not depend on the launch shape.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace psb {

namespace {

constexpr int kRotTile = 32;   // outputs per CTA, rows per CTA and the depth of one staged slab

// CTA (32, 8): thread (tx, ty) owns output o0 + tx of rows r0 + ty + {0, 8, 16, 24}.  R and x slabs of 32 inputs go through
// shared memory (R read coalesced along its rows, kept [o][i] with one word of padding: the inner loop's reads of
// s_r[tx][ii] are conflict-free and those of s_x[row][ii] are broadcasts).
__global__ void __launch_bounds__(256) k_rotate_rows(const float* __restrict__ in, const float* __restrict__ mat, long long n, int dim,
                                                      float* __restrict__ out) {
    __shared__ float s_r[kRotTile][kRotTile + 1];
    __shared__ float s_x[kRotTile][kRotTile + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int o0 = blockIdx.x * kRotTile;
    const long long r0 = (long long)blockIdx.y * kRotTile;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i0 = 0; i0 < dim; i0 += kRotTile) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int rr = ty + 8 * j;
            const int o = o0 + rr, i = i0 + tx;
            s_r[rr][tx] = (o < dim && i < dim) ? __ldg(mat + (size_t)o * dim + i) : 0.f;
            const long long row = r0 + rr;
            s_x[rr][tx] = (row < n && i < dim) ? __ldg(in + (size_t)row * dim + i) : 0.f;
        }
        __syncthreads();
        const int depth = min(kRotTile, dim - i0);   // no padded terms: a chain never sees an extra + 0 * 0
        for (int ii = 0; ii < depth; ++ii) {
            const float w = s_r[tx][ii];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(w, s_x[ty + 8 * j][ii], acc[j]);
        }
        __syncthreads();
    }
    if (o0 + tx < dim) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long row = r0 + ty + 8 * j;
            if (row < n) out[(size_t)row * dim + o0 + tx] = acc[j];
        }
    }
}

}  // namespace

psb_status launch_rotate_rows(const float* d_in, const float* d_matrix, long long n, int dim, float* d_out, cudaStream_t s) {
    if (n <= 0) return PSB_OK;
    const long long row_tiles = (n + kRotTile - 1) / kRotTile;
    if (row_tiles > 65535) {   // grid.y limit: slabs of rows
        const long long slab = 65535LL * kRotTile;
        for (long long r = 0; r < n; r += slab)
            PSB_TRY(launch_rotate_rows(d_in + (size_t)r * dim, d_matrix, std::min(slab, n - r), dim, d_out + (size_t)r * dim, s));
        return PSB_OK;
    }
    dim3 grid((dim + kRotTile - 1) / kRotTile, (unsigned)row_tiles), block(kRotTile, 8);
    k_rotate_rows<<<grid, block, 0, s>>>(d_in, d_matrix, n, dim, d_out);
    PSB_CUDA(cudaGetLastError());
    return PSB_OK;
}

}  // namespace psb
