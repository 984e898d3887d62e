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

namespace psb {
namespace {

constexpr int TQ = 128;          // queries per tile  (UMMA M)
constexpr int TCOL = 256;        // centroids per tile (UMMA N)
constexpr int KATOM = 64;        // bf16 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kTcThreads = 128;
constexpr int kWaitLimit = 1 << 22;
constexpr int kCandCap = 2048;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false after kWaitLimit unsuccessful polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = 256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCOL >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);

// Minima of consecutive groups of G values of a 32-value chunk.
template <int G>
__device__ __forceinline__ void group_mins(const float (&v)[32], float* __restrict__ out) {
#pragma unroll
    for (int g = 0; g < 32 / G; ++g) {
        float m = v[g * G];
#pragma unroll
        for (int j = 1; j < G; ++j) m = fminf(m, v[g * G + j]);
        out[g] = m;
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
    int* cand_cnt;          // pass 2 out: [nq]
    int* cand;              // pass 2 out: [nq][kCandCap]
    int* status;            // [1] != 0 after a bounded wait gave up
};

template <bool kSecondPass>
__global__ void __launch_bounds__(kTcThreads)
k_coarse_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_c, const TcArgs a) {
    extern __shared__ __align__(1024) unsigned char s_tc[];
    // layout: A = katoms blocks of [TQ rows][128 B], then B = katoms blocks of [TCOL rows][128 B]; 1024-byte aligned
    unsigned char* s_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_tc) + 1023) & ~uintptr_t(1023));
    unsigned char* s_a = s_base;
    unsigned char* s_b = s_base + (size_t)a.katoms * TQ * 128;
    __shared__ __align__(8) uint64_t bar_a, bar_b, bar_mma;
    __shared__ uint32_t s_tmem;
    __shared__ float s_cn2[TCOL];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int q0 = blockIdx.x * TQ;

    if (tid == 0) {
        mbar_init(&bar_a, 1); mbar_init(&bar_b, 1); mbar_init(&bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&s_tmem, TCOL);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    if (tid == 0) {
        mbar_expect_tx(&bar_a, (uint32_t)a.katoms * TQ * 128);
        for (int ka = 0; ka < a.katoms; ++ka) tma_load_2d(s_a + (size_t)ka * TQ * 128, &map_q, ka * KATOM, q0, &bar_a);
    }
    const int q = q0 + tid;  // this thread's query row = tensor-memory lane
    float cut = 0.0f;
    if (kSecondPass && q < a.nq) {
        const float T = a.seltop[(size_t)q * a.nprobe + a.nprobe - 1];
        const float qn = a.qnorm[q];
        const float E = 4.1f * 0.00390625f * qn * a.cmax;  // |a - exact| <= 2 |q'.c' - qb.cb| <= 2 * 2.01 * 2^-8 |q'||c'|
        cut = T + 2.0f * E + 4e-5f * (qn + a.cmax) * (qn + a.cmax);
    }
    bool a_ready = false;
    uint32_t phase = 0;
    int failed = 0;
    for (int t = blockIdx.y; t < a.ntiles; t += gridDim.y) {
        const int c0 = t * TCOL;
        if (tid == 0) {
            mbar_expect_tx(&bar_b, (uint32_t)a.katoms * TCOL * 128);
            for (int ka = 0; ka < a.katoms; ++ka) tma_load_2d(s_b + (size_t)ka * TCOL * 128, &map_c, ka * KATOM, c0, &bar_b);
        }
        for (int i = tid; i < TCOL; i += kTcThreads) s_cn2[i] = a.cn2[c0 + i];
        int bad = 0;
        if (tid == 0) {
            if (!a_ready) { if (!mbar_wait(&bar_a, 0)) bad = 1; a_ready = true; }
            if (!bad && !mbar_wait(&bar_b, phase)) bad = 1;
            if (!bad) {
                tc_fence_after();
                const uint32_t sa = smem_u32(s_a), sb = smem_u32(s_b);
                for (int ka = 0; ka < a.katoms; ++ka)
                    for (int kk = 0; kk < KATOM / UMMA_K; ++kk) {
                        const uint64_t da = make_sw128_desc(sa + ka * TQ * 128 + kk * UMMA_K * 2);
                        const uint64_t db = make_sw128_desc(sb + ka * TCOL * 128 + kk * UMMA_K * 2);
                        umma_bf16(tmem, da, db, kIdesc, (ka | kk) ? 1u : 0u);
                    }
                umma_commit(&bar_mma);
            }
        }
        bad = __syncthreads_or(bad);  // also publishes s_cn2
        if (!bad && !mbar_wait(&bar_mma, phase)) bad = 1;
        bad = __syncthreads_or(bad);
        if (bad) { failed = 1; break; }
        tc_fence_after();
        // epilogue: lane = query row, 256 fp32 accumulators = dot products with this tile's centroids
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
        for (int cb = 0; cb < TCOL; cb += 32) {
            uint32_t r[32];
            __syncwarp();
            tmem_ld32(lane_addr + (uint32_t)cb, r);
            tmem_ld_wait();
            if (q < a.nq) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = fmaf(-2.0f, __uint_as_float(r[j]), s_cn2[cb + j]);  // +inf beyond nlist
                if (!kSecondPass) {
                    float* out = a.gmin + (size_t)q * a.ngroups + ((c0 + cb) >> a.lg_group);
                    switch (a.lg_group) {  // uniform
                        case 5: group_mins<32>(v, out); break;
                        case 4: group_mins<16>(v, out); break;
                        case 3: group_mins<8>(v, out); break;
                        case 2: group_mins<4>(v, out); break;
                        case 1: group_mins<2>(v, out); break;
                        default: group_mins<1>(v, out); break;
                    }
                } else {
                    float m = v[0];
#pragma unroll
                    for (int j = 1; j < 32; ++j) m = fminf(m, v[j]);
                    if (m <= cut) {  // rare: some centroid of this chunk is a candidate
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (v[j] <= cut) {
                                const int pos = atomicAdd(&a.cand_cnt[q], 1);
                                if (pos < kCandCap) a.cand[(size_t)q * kCandCap + pos] = c0 + cb + j;
                            }
                        }
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();  // accumulators and s_cn2 consumed: the next tile may overwrite them
        phase ^= 1u;
    }
    if (tid == 0) {
        if (failed) {
            atomicExch(a.status, 1);
            mbar_wait(&bar_b, phase);  // best effort, bounded: let this CTA's own copies land before its memory is released
        }
        if (!a_ready) mbar_wait(&bar_a, 0);
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (warp == 0) tmem_dealloc(tmem, TCOL);
}

// q' = q - mu as bf16 rows padded with zeros to dimp, and |q'|.
__global__ void k_tc_prep_rows(const float* __restrict__ x, int n, int dim, int dimp, const float* __restrict__ mu,
                               __nv_bfloat16* __restrict__ out, float* __restrict__ norm, float* __restrict__ sq) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n) return;
    float s = 0.0f;
    for (int d = lane; d < dimp; d += 32) {
        float v = 0.0f;
        if (d < dim) v = x[(size_t)warp * dim + d] - mu[d];
        out[(size_t)warp * dimp + d] = __float2bfloat16_rn(v);
        s += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        if (norm) norm[warp] = sqrtf(s);
        if (sq) sq[warp] = s;
    }
}

__global__ void k_fill_inf(float* p, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = __int_as_float(0x7f800000);
}

// Exact re-scoring of a query's candidates in the CPU path's arithmetic, sort by (distance, id), first nprobe out.
constexpr int kRefineThreads = 256;
__global__ void __launch_bounds__(kRefineThreads)
k_coarse_refine(const float* __restrict__ queries, const float* __restrict__ centroids, int dim, int nlist, int nprobe,
                const int* __restrict__ cand_cnt, const int* __restrict__ cand, int* __restrict__ out_ids,
                float* __restrict__ out_dist, int* __restrict__ fail_list, int* __restrict__ n_fail) {
    extern __shared__ __align__(16) unsigned char s_ref[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_ref);                        // [kCandCap]
    float* s_q = reinterpret_cast<float*>(s_ref + (size_t)kCandCap * 8);         // [dim]
    const int q = blockIdx.x;
    const int n = cand_cnt[q];
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
            const int c = cand[(size_t)q * kCandCap + i];
            const float* cp = centroids + (size_t)c * dim;
            float sum = 0.0f;
            for (int d = 0; d < dim; ++d) {
                const float diff = __fsub_rn(s_q[d], __ldg(cp + d));
                sum = __fadd_rn(sum, __fmul_rn(diff, diff));
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
int coarse_tc_tiles(int nlist) { return (nlist + TCOL - 1) / TCOL; }
int coarse_tc_cand_cap() { return kCandCap; }

int coarse_tc_group(int nlist, int nprobe) {
    int g = 32;
    while (g > 1 && nlist / g < 4 * nprobe) g >>= 1;
    return g;
}

bool coarse_tc_supported(int nq, int nlist, int dim, int nprobe) {
    const int dimp = coarse_tc_padded_dim(dim);
    return nq >= 64 && nlist >= 1024 && dimp <= 256 && nprobe <= 512 && nlist >= 8 * nprobe &&
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
                                                            static_cast<__nv_bfloat16*>(d_cb), d_cnorm, d_cn2);
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
    // query side: centre, round to bf16, norms
    k_tc_prep_rows<<<(nq * 32 + 255) / 256, 256, 0, s>>>(d_queries, nq, ix.dim, dimp, ix.mu,
                                                         static_cast<__nv_bfloat16*>(ws.qb), ws.qnorm, nullptr);
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
    a.cand_cnt = ws.cand_cnt; a.cand = ws.cand; a.status = ws.status;
    const size_t smem = (size_t)katoms * (TQ + TCOL) * 128 + 1024;
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_CUDA(cudaFuncSetAttribute(k_coarse_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int qtiles = (nq + TQ - 1) / TQ;
    int slices = (4 * sm_count + qtiles - 1) / qtiles;
    slices = slices < 1 ? 1 : (slices > ntiles ? ntiles : slices);
    const dim3 grid(qtiles, slices);
    PSB_CUDA(cudaMemsetAsync(ws.cand_cnt, 0, sizeof(int) * (size_t)nq, s));
    PSB_CUDA(cudaMemsetAsync(ws.n_fail, 0, 2 * sizeof(int), s));  // n_fail, cursor
    if (ws.ev[0]) PSB_CUDA(cudaEventRecord(ws.ev[0], s));
    k_coarse_tc<false><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    if (ws.ev[1]) PSB_CUDA(cudaEventRecord(ws.ev[1], s));
    count_launch();
    PSB_LAUNCH_CHECK();
    PSB_TRY(launch_select_rows(ws.gmin, nq, ngroups, nprobe, ws.selids, ws.seltop, s));
    if (ws.ev[2]) PSB_CUDA(cudaEventRecord(ws.ev[2], s));
    k_coarse_tc<true><<<grid, kTcThreads, smem, s>>>(map_q, map_c, a);
    if (ws.ev[3]) PSB_CUDA(cudaEventRecord(ws.ev[3], s));
    count_launch();
    PSB_LAUNCH_CHECK();
    {
        const size_t rsmem = (size_t)kCandCap * 8 + (size_t)ix.dim * sizeof(float);
        k_coarse_refine<<<nq, kRefineThreads, rsmem, s>>>(d_queries, ix.centroids, ix.dim, ix.nlist, nprobe, ws.cand_cnt,
                                                          ws.cand, d_ids, d_dist, ws.fail_list, ws.n_fail);
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

}  // namespace psb
