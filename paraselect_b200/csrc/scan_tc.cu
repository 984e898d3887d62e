// ADC scan, tensor-core pre-filter (sm_100a tcgen05) and the re-scoring selection that follows it.
//
// The ADC distance of a code row against a query is |q - recon(row)|^2, recon(row) = the row's codewords laid side by
// side.  For a list visited by many queries that is a GEMM: a tile of 128 visiting queries (A operand, centred on the
// list's centroid and rounded to bf16) against code rows decoded on the fly into shared memory as bf16 (B operand, the
// same centring), fp32 accumulators in tensor memory.  The product only FILTERS: a (row, visitor) pair survives when its
// bf16 score cannot rule out an exact distance <= the visitor's cutoff; survivors go to the visitor's pool unscored and
// k_select_rescore computes their exact fp32 ADC distance in the CPU path's arithmetic before selecting.  The candidate
// sets and distances are therefore identical to the SIMT scans' (pq_scan.cu), which do one shared-memory lookup per
// (row, visitor, sub-quantiser); here a row is decoded once per 128 visitors.
//
// Bound.  q' = fl(q - c), r' = fl(recon - c) (residual mode: r' = recon, the codes already encode row - c); qt, rt their
// bf16 roundings (|qt - q'| <= 2^-9 |q'|, same for r).  With D the exact distance,
//     |qt - rt| <= sqrt(D) + b (|q'| + |r'|),  b = 2^-9 (1 + 1e-3),
// so D_cpu <= cutoff implies  |qt|^2 + |rt|^2 - 2 qt.rt <= (sqrt(cutoff (1 + 1e-5)) + b |q'| + b w)^2 + e (|q'| + w)^2,
// w = |rt| (1 + 2^-8) >= |r'|, e covering the fp32 accumulation of the tensor core and of the norms.  Split by operand:
//     qt.rt - U_row + H_vis * w_row >= P_vis,
//     U_row = (|rt|^2 - (b^2 + e) w^2) / 2,  H_vis = a b + e |q'|,  P_vis = (|qt|^2 - a^2 - e |q'|^2) / 2,  a = sqrt(cutoff') + b |q'|.
// The left side comes out of the tensor core in one piece: four extra K slots carry (1, 1, 1, H_vis rounded up) on the query
// side and (the three-term bf16 split of -U_row, w_row rounded up) on the row side, so the epilogue is one comparison per
// (row, visitor) against a per-thread constant.
//
// Reference counterparts: the tensor-core ADC experiments src/search/kernels/fine/gpu_fine/pq_adc/pq_codeword_fp16.cu:18 and
// pq_codeword_u8_pipeline.cuh:15-119; the exact distances follow src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:51-63,76-80
// and, in residual mode, src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:87-130,226-259,440-451.
//
// Every mbarrier wait is bounded: a role that gives up raises a CTA-wide flag, the other roles see it in their own wait
// loops, the CTA frees its tensor memory and returns, and the host reports PSB_TIMEOUT.
#include <cuda_bf16.h>
#include <algorithm>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "scan_common.cuh"
#include "tc_ptx.cuh"

namespace psb {

using namespace scan;
using namespace tc;

namespace {

constexpr int TV = 128;            // visitors per tile (UMMA M)
constexpr int TN = 128;            // code rows per tile (UMMA N)
constexpr int kDecodeGroups = 2;   // warps 0-7: two groups of four warps; group g decodes tiles g, g + 2, ... (one row per thread)
constexpr int kDecodeWarps = 4 * kDecodeGroups;
constexpr int kEpiGroups = 2;      // warps 8-15: two groups of four warps (one warp per tensor-memory lane quarter); group e reads
constexpr int kEpiWarps = 4 * kEpiGroups;           // the accumulators of tiles e, e + 2, ...
constexpr int kWarpMma = kDecodeWarps + kEpiWarps;  // warp 16: MMA issuer
constexpr int kWarpSched = kWarpMma + 1;            // warp 17: fetches work items ahead of the others
// 18 warps: 112 registers per thread, which the decode (two tiles of code words in flight) and the epilogue (two 32-column
// accumulator loads in flight) both need.
constexpr int kTcScanThreads = (kWarpSched + 1) * 32;
constexpr int kProducers = kDecodeWarps * 32;
constexpr int kItemRing = 4;       // work items in flight
constexpr int kQueueCap = 256;     // survivors a warp collects before it pushes them to the pools
constexpr int kAugSlots = 4;
constexpr float kBeta = 0.001953125f * 1.001f;  // 2^-9 (1 + 1e-3)

struct ItemDesc {
    long long r0, r1;   // scanned rows of the item
    int ntiles, stop;   // tiles of TN rows; stop: no more work
    int list, vis_base, nvis;  // list id, first visitor entry, visitors of this group (<= TV)
};

struct ScanTcArgs {
    ScanArgs a;               // a.item_off: the tensor-core work items (lists the SIMT scan leaves out)
    const float* queries;     // [nq][dim]
    const float* centroids;   // [nlist][dim] (residual mode)
    const float* codebook;    // [m][k][dsub]
    const uint2* row_aug;     // [rows of the shard]: the extra K slots of every code row (k_row_aug)
    int dim, kp, katoms;      // kp: padded K (multiple of 16), katoms: 128-byte swizzle atoms along K
    int na, ns;               // query-tile slots (1 or 2), row-tile stages = accumulators = decode warp groups in use (2 or 3)
    int residual;
    float eps;                // accumulation slack e
    int* status;              // != 0 after a bounded wait gave up
    int wait_limit;           // polls before a wait gives up (tests shorten it)
    int skip_mma;             // test hook: the MMA warp issues nothing, so every role waiting for a result runs into its limit
};

// Bounded wait that also leaves when another role of the CTA has given up.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int limit) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t bf16_bits_rn(float x) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t bf16_bits_up(float x) {  // x >= 0, finite: the smallest bf16 >= x
    return (__float_as_uint(x) + 0xFFFFu) >> 16;
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) { return bf16_bits_rn(lo) | (bf16_bits_rn(hi) << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// 16-byte chunk c of an operand row in the K-major 128-byte-swizzled layout: rowbase = operand + row * 128,
// xs = (row & 7) << 4, atom_stride = rows * 128.
__device__ __forceinline__ uint4* chunk_at(unsigned char* rowbase, uint32_t xs, int atom_stride, int c) {
    return reinterpret_cast<uint4*>(rowbase + (size_t)(c >> 3) * atom_stride + ((((uint32_t)c & 7u) << 4) ^ xs));
}

// The extra K slots of a code row from |rt|^2: minus the three-term bf16 split of U = (|rt|^2 - (b^2 + e) w^2) / 2 and w rounded up.
__device__ __forceinline__ uint2 row_aug_words(float rn, float cw2) {
    const float wv = sqrtf(rn) * 1.003908f;  // >= |r'| (1 + 2^-8, and the square root's rounding)
    float rest = 0.5f * (rn - cw2 * wv * wv);
    uint32_t u[3];
#pragma unroll
    for (int x = 0; x < 3; ++x) {
        const __nv_bfloat16 h = __float2bfloat16_rn(rest);
        u[x] = (uint32_t)__bfloat16_as_ushort(__hneg(h));
        rest -= __bfloat162float(h);
    }
    return make_uint2(u[0] | (u[1] << 16), u[2] | (bf16_bits_up(wv) << 16));
}

// Code words of one row held in registers (templated M), so that the next tile's row can be fetched while this one is decoded.
template <int M> struct RowCodes { uint32_t w[M > 0 ? M / 4 : 1]; };
template <int M>
__device__ __forceinline__ void load_codes(RowCodes<M>& c, const uint8_t* __restrict__ row) {
    if constexpr (M > 0 && M % 16 == 0) {
#pragma unroll
        for (int i = 0; i < M / 16; ++i) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(row) + i);
            c.w[4 * i] = x.x; c.w[4 * i + 1] = x.y; c.w[4 * i + 2] = x.z; c.w[4 * i + 3] = x.w;
        }
    } else if constexpr (M > 0) {
#pragma unroll
        for (int i = 0; i < M / 4; ++i) c.w[i] = __ldg(reinterpret_cast<const uint32_t*>(row) + i);
    }
}

// One code row -> its bf16 operand row (data chunks only).  s_tab: [m][k] entries of DSUB bf16.  Templated M: the code words
// come in registers; M = 0 (any m that is a multiple of 4): they are read from `row` as the loop goes.
template <int DSUB, int M>
__device__ __forceinline__ void decode_row(const RowCodes<M>& codes, const uint8_t* __restrict__ row, int m_rt, int k,
                                           const unsigned char* __restrict__ s_tab, unsigned char* rowbase, uint32_t xs, int atom_stride) {
    constexpr int EB = DSUB * 2;  // bytes per table entry
    const int kstride = k * EB;
    auto word = [&](uint32_t cw, int w) {  // code word w: sub-quantisers 4w .. 4w+3
        const unsigned char* t = s_tab + (size_t)(4 * w) * kstride;
        if constexpr (DSUB == 2) {  // four codewords of 2 -> chunk w
            uint4 o;
            o.x = *reinterpret_cast<const uint32_t*>(t + (cw & 255u) * EB);
            o.y = *reinterpret_cast<const uint32_t*>(t + kstride + ((cw >> 8) & 255u) * EB);
            o.z = *reinterpret_cast<const uint32_t*>(t + 2 * kstride + ((cw >> 16) & 255u) * EB);
            o.w = *reinterpret_cast<const uint32_t*>(t + 3 * kstride + (cw >> 24) * EB);
            *chunk_at(rowbase, xs, atom_stride, w) = o;
        } else if constexpr (DSUB == 4) {  // two codewords of 4 -> chunks 2w, 2w+1
            const uint2 e0 = *reinterpret_cast<const uint2*>(t + (cw & 255u) * EB);
            const uint2 e1 = *reinterpret_cast<const uint2*>(t + kstride + ((cw >> 8) & 255u) * EB);
            const uint2 e2 = *reinterpret_cast<const uint2*>(t + 2 * kstride + ((cw >> 16) & 255u) * EB);
            const uint2 e3 = *reinterpret_cast<const uint2*>(t + 3 * kstride + (cw >> 24) * EB);
            *chunk_at(rowbase, xs, atom_stride, 2 * w) = make_uint4(e0.x, e0.y, e1.x, e1.y);
            *chunk_at(rowbase, xs, atom_stride, 2 * w + 1) = make_uint4(e2.x, e2.y, e3.x, e3.y);
        } else {  // DSUB == 8: one codeword -> one chunk
            *chunk_at(rowbase, xs, atom_stride, 4 * w) = *reinterpret_cast<const uint4*>(t + (cw & 255u) * EB);
            *chunk_at(rowbase, xs, atom_stride, 4 * w + 1) = *reinterpret_cast<const uint4*>(t + kstride + ((cw >> 8) & 255u) * EB);
            *chunk_at(rowbase, xs, atom_stride, 4 * w + 2) = *reinterpret_cast<const uint4*>(t + 2 * kstride + ((cw >> 16) & 255u) * EB);
            *chunk_at(rowbase, xs, atom_stride, 4 * w + 3) = *reinterpret_cast<const uint4*>(t + 3 * kstride + (cw >> 24) * EB);
        }
    };
    if constexpr (M > 0) {
#pragma unroll
        for (int i = 0; i < M / 4; ++i) {
            word(codes.w[i], i);
            if ((i & 3) == 3) asm volatile("" ::: "memory");  // keeps later table loads below these stores: bounded register use
        }
    } else {
        for (int w = 0; w < (m_rt >> 2); ++w) word(__ldg(reinterpret_cast<const uint32_t*>(row) + w), w);
    }
}

// Persistent, warp-specialised kernel without CTA-wide barriers in its main loop.  Work item = (list, chunk of rows, group
// of up to 128 visiting queries); the roles hand items and tiles to one another through mbarriers:
//   warp 17     scheduler: takes items off the global cursor, resolves them, fills a ring of item descriptors
//   warps 0-7   producers: build the item's query tile (A operand, ring of `na` slots) and its per-visitor constants, then
//               decode code rows into the ring of `ns` row tiles (B operand), one tile in flight per warp group
//   warp 16     MMA issuer: kp / 16 tcgen05.mma per tile into accumulator `stage`, tcgen05.commit -> mbarriers
//   warps 8-15  epilogue: tcgen05.ld the accumulator (two 32-column loads in flight), one comparison per (visitor, row); survivors go to a per-warp queue in
//               shared memory that is pushed to the visitors' pools 32 at a time (one round of global atomics per push)
template <int DSUB, int M>
__global__ void __launch_bounds__(kTcScanThreads, 1) k_scan_tc(const ScanTcArgs g) {
    const ScanArgs& a = g.a;
    extern __shared__ __align__(1024) unsigned char s_dyn[];
    unsigned char* s_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_dyn) + 1023) & ~uintptr_t(1023));
    const int a_stride = TV * 128, b_stride = TN * 128;
    const size_t a_bytes = (size_t)g.katoms * a_stride, b_bytes = (size_t)g.katoms * b_stride;
    unsigned char* s_a = s_base;                             // [na][katoms][TV][128 B]
    unsigned char* s_b = s_a + g.na * a_bytes;               // [ns][katoms][TN][128 B]
    unsigned char* s_tab = s_b + g.ns * b_bytes;             // [m][k] entries of DSUB bf16: the codebook rounded to bf16
    __shared__ __align__(8) uint64_t item_full[kItemRing], item_empty[kItemRing], vis_full[kItemRing];
    __shared__ __align__(8) uint64_t a_full[2], a_empty[2], b_full[4], b_empty[4], acc_full[4], acc_empty[4];
    __shared__ ItemDesc s_desc[kItemRing];
    __shared__ float s_P[kItemRing][TV];
    __shared__ int s_pq[kItemRing][TV], s_hi[kItemRing][TV];
    __shared__ uint32_t s_queue[kEpiWarps][kQueueCap];
    __shared__ int s_qcnt[kEpiWarps];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunk_data = g.dim >> 3, nchunk = g.kp >> 3;
    const int limit = g.wait_limit;
    const int NA = g.na, NS = g.ns;
    const uint32_t tmem_cols = NS * TN <= 256 ? 256u : 512u;

    if (tid == 0) {
        for (int i = 0; i < kItemRing; ++i) {
            mbar_init(&item_full[i], 1);
            mbar_init(&item_empty[i], kProducers + 1 + kEpiWarps * 32);
            mbar_init(&vis_full[i], kProducers);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(&a_full[i], kProducers); mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&b_full[i], TN); mbar_init(&b_empty[i], 1);
            mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 128);  // the four warps of one epilogue group
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid < kEpiWarps) s_qcnt[tid] = 0;
    // the codebook rounded to bf16, once per CTA (all threads)
    for (int e = tid; e < a.m * a.k; e += kTcScanThreads) {
        const float* cb = g.codebook + (size_t)e * DSUB;
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_tab + (size_t)e * DSUB * 2);
#pragma unroll
        for (int d = 0; d < DSUB; d += 2) dst[d / 2] = pack_bf16x2_rn(__ldg(cb + d), __ldg(cb + d + 1));
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&s_tmem, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const long long total = a.item_off[a.nlist];
    volatile int* abort_flag = &s_abort;
    bool failed = false;
    unsigned long long passes = 0;

    if (warp == kWarpSched) {
        // ---- scheduler ----
        for (uint32_t n = 0;; ++n) {
            const int islot = n % kItemRing;
            if (!__all_sync(0xffffffffu, wait_or_abort(&item_empty[islot], ((n / kItemRing) & 1u) ^ 1u, abort_flag, limit))) { failed = true; break; }
            long long item = 0;
            if (lane == 0) item = (long long)atomicAdd(a.work_cursor, 1ull);
            item = __shfl_sync(0xffffffffu, item, 0);
            const bool stop = item >= total;
            int l = 0;
            if (!stop) l = find_list(a.item_off, a.nlist, item);
            if (lane == 0) {
                ItemDesc d;
                d.stop = stop ? 1 : 0; d.r0 = d.r1 = 0; d.ntiles = 0; d.list = l; d.vis_base = 0; d.nvis = 0;
                if (!stop) {
                    const int nvis = a.vis_count[l];
                    const int ngroups = (nvis + TV - 1) / TV;
                    const long long local = item - a.item_off[l];
                    const int group = (int)(local % ngroups);
                    const long long chunk = local / ngroups;
                    d.r0 = a.offsets[l] + chunk * a.chunk_rows;
                    d.r1 = min(d.r0 + a.chunk_rows, a.offsets[l + 1]);
                    d.ntiles = (int)((d.r1 - d.r0 + TN - 1) / TN);
                    d.vis_base = a.vis_off[l] + group * TV;
                    d.nvis = min(TV, nvis - group * TV);
                }
                s_desc[islot] = d;
                mbar_arrive(&item_full[islot]);  // release: the descriptor is visible to whoever sees the phase complete
            }
            __syncwarp();
            if (stop) break;
        }
    } else if (warp < kDecodeWarps) {
        // ---- producers ----
        const int grp = warp >> 2, lt = tid & (TN - 1);
        const uint32_t xs = (uint32_t)(lt & 7) << 4;
        uint32_t it0 = 0;
        for (uint32_t n = 0;; ++n) {
            const int islot = n % kItemRing;
            if (!__all_sync(0xffffffffu, wait_or_abort(&item_full[islot], (n / kItemRing) & 1u, abort_flag, limit))) { failed = true; break; }
            const ItemDesc d = s_desc[islot];
            if (d.stop) break;
            const int aslot = n % NA;
            if (!__all_sync(0xffffffffu, wait_or_abort(&a_empty[aslot], ((n / NA) & 1u) ^ 1u, abort_flag, limit))) { failed = true; break; }
            const float* cen = g.centroids + (size_t)d.list * g.dim;  // residual mode: the list's centroid (read through L1/L2)
            if (tid < 2 * TV) {  // query tile: two threads per visitor row
                const int i = tid >> 1, part = tid & 1;
                unsigned char* arow = s_a + aslot * a_bytes + (size_t)i * 128;
                const uint32_t axs = (uint32_t)(i & 7) << 4;
                const int vq = i < d.nvis ? a.visitors[d.vis_base + i] : -1;    // table index: the query, or the pair in residual mode
                const int pq = vq >= 0 ? vq / a.lut_div : -1;                    // query (pool, cutoff)
                float qn = 0.0f, n2 = 0.0f;  // |qt|^2, |q'|^2 over this thread's chunks
                float P = __int_as_float(0x7f800000), H = 0.0f;
                if (pq >= 0) {
                    const float* qrow = g.queries + (size_t)pq * g.dim;
                    for (int c = part; c < nchunk_data; c += 2) {
                        float4 x0 = __ldg(reinterpret_cast<const float4*>(qrow + c * 8));
                        float4 x1 = __ldg(reinterpret_cast<const float4*>(qrow + c * 8 + 4));
                        if (g.residual) {
                            const float4 c0 = __ldg(reinterpret_cast<const float4*>(cen + c * 8));
                            const float4 c1 = __ldg(reinterpret_cast<const float4*>(cen + c * 8 + 4));
                            x0.x = __fsub_rn(x0.x, c0.x); x0.y = __fsub_rn(x0.y, c0.y); x0.z = __fsub_rn(x0.z, c0.z); x0.w = __fsub_rn(x0.w, c0.w);
                            x1.x = __fsub_rn(x1.x, c1.x); x1.y = __fsub_rn(x1.y, c1.y); x1.z = __fsub_rn(x1.z, c1.z); x1.w = __fsub_rn(x1.w, c1.w);
                        }
                        const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        const uint32_t ow[4] = {pack_bf16x2_rn(v[0], v[1]), pack_bf16x2_rn(v[2], v[3]), pack_bf16x2_rn(v[4], v[5]),
                                                pack_bf16x2_rn(v[6], v[7])};
#pragma unroll
                        for (int j = 0; j < 8; ++j) n2 = fmaf(v[j], v[j], n2);
#pragma unroll
                        for (int j = 0; j < 4; ++j) { const float lo = bf16_lo(ow[j]), hi = bf16_hi(ow[j]); qn = fmaf(lo, lo, qn); qn = fmaf(hi, hi, qn); }
                        *chunk_at(arow, axs, a_stride, c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                } else {
                    for (int c = part; c < nchunk_data; c += 2) *chunk_at(arow, axs, a_stride, c) = make_uint4(0, 0, 0, 0);
                }
                qn += __shfl_xor_sync(0xffffffffu, qn, 1);
                n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
                if (pq >= 0) {
                    const float t = a.thr[pq];
                    if (t < 3.0e38f) {
                        const float nq = sqrtf(n2) * 1.000001f;
                        const float av = sqrtf(fmaxf(t, 0.0f) * 1.00001f) * 1.000001f + kBeta * nq;
                        P = 0.5f * (qn - (av * av + g.eps * nq * nq));
                        H = av * kBeta + g.eps * nq;
                    } else {
                        P = __int_as_float(0xff800000);  // no cutoff: every row of the list is a candidate
                    }
                }
                for (int c = nchunk_data + part; c < nchunk; c += 2) {  // the extra K slots (1, 1, 1, H), then zero padding
                    uint4 o = make_uint4(0, 0, 0, 0);
                    if (c == nchunk_data && pq >= 0) { o.x = 0x3F803F80u; o.y = 0x3F80u | (bf16_bits_up(H) << 16); }
                    *chunk_at(arow, axs, a_stride, c) = o;
                }
                if (part == 0) { s_P[islot][i] = P; s_pq[islot][i] = pq; s_hi[islot][i] = g.residual ? vq : d.list; }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // operand stores -> visible to the tensor core
            }
            mbar_arrive(&a_full[aslot]);
            mbar_arrive(&vis_full[islot]);
            // code rows of this warp group's tiles: tile k of the item has running number it0 + k and belongs to the group
            // (it0 + k) % NS - groups in use == stages, so a group meets the phases of its stage's barriers one after the
            // other, never two apart (parity waits could not tell those from each other).  The next tile's code words are
            // fetched before the current tile is decoded.
            int k = (int)(((uint32_t)grp + (uint32_t)NS - it0 % (uint32_t)NS) % (uint32_t)NS);
            RowCodes<M> cur, nxt;
            uint2 aug_cur = make_uint2(0, 0), aug_nxt = make_uint2(0, 0);
            auto fetch = [&](int kk, RowCodes<M>& c, uint2& aug) {
                const long long r = d.r0 + (long long)kk * TN + lt;
                if (kk < d.ntiles && r < d.r1) {
                    const size_t lr = (size_t)(r - a.row_base);
                    aug = __ldg(g.row_aug + lr);
                    load_codes<M>(c, a.codes + lr * a.m);
                }
            };
            if (grp < NS) fetch(k, cur, aug_cur);
            for (; grp < NS && k < d.ntiles; k += NS) {
                const uint32_t gi = it0 + (uint32_t)k;
                const uint32_t st = (uint32_t)grp, use = gi / (uint32_t)NS;
                fetch(k + NS, nxt, aug_nxt);
                if (!__all_sync(0xffffffffu, wait_or_abort(&b_empty[st], (use & 1u) ^ 1u, abort_flag, limit))) { failed = true; break; }
                unsigned char* rowbase = s_b + st * b_bytes + (size_t)lt * 128;
                const long long r = d.r0 + (long long)k * TN + lt;
                if (r < d.r1) {
                    decode_row<DSUB, M>(cur, a.codes + (size_t)(r - a.row_base) * a.m, a.m, a.k, s_tab, rowbase, xs, b_stride);
                    *chunk_at(rowbase, xs, b_stride, nchunk_data) = make_uint4(aug_cur.x, aug_cur.y, 0u, 0u);
                } else {
                    // past the end of the chunk: a row no visitor can admit (score -1e30)
                    for (int c = 0; c < nchunk_data; ++c) *chunk_at(rowbase, xs, b_stride, c) = make_uint4(0, 0, 0, 0);
                    *chunk_at(rowbase, xs, b_stride, nchunk_data) = make_uint4(bf16_bits_rn(-1.0e30f), 0u, 0u, 0u);
                }
                for (int c = nchunk_data + 1; c < nchunk; ++c) *chunk_at(rowbase, xs, b_stride, c) = make_uint4(0, 0, 0, 0);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&b_full[st]);
                cur = nxt; aug_cur = aug_nxt;
            }
            if (failed) break;
            it0 += (uint32_t)d.ntiles;
            mbar_arrive(&item_empty[islot]);
        }
    } else if (warp < kDecodeWarps + kEpiWarps) {
        // ---- epilogue: one visitor per thread (tensor-memory lane), all 128 rows of every second tile ----
        const int e = warp - kDecodeWarps, quad = warp & 3, eg = e >> 2;  // warp % 4 == quad: the tensor-memory lanes this warp may read
        const int i = quad * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
        uint32_t* queue = s_queue[e];
        uint32_t it0 = 0;
        for (uint32_t n = 0;; ++n) {
            const int islot = n % kItemRing;
            if (!__all_sync(0xffffffffu, wait_or_abort(&item_full[islot], (n / kItemRing) & 1u, abort_flag, limit))) { failed = true; break; }
            const ItemDesc d = s_desc[islot];
            if (d.stop) break;
            if (!__all_sync(0xffffffffu, wait_or_abort(&vis_full[islot], (n / kItemRing) & 1u, abort_flag, limit))) { failed = true; break; }
            const float P = s_P[islot][i];
            const uint32_t nrows = (uint32_t)(d.r1 - d.r0);  // rows of the item
            // pushes the queued survivors of this item to their visitors' pools
            auto flush = [&]() {
                const int cnt = min(s_qcnt[e], kQueueCap);
                for (int x = lane; x < cnt; x += 32) {
                    const uint32_t en = queue[x];
                    const int vi = (int)(en >> 24);
                    const int pq = s_pq[islot][vi];
                    const int slot = atomicAdd(&a.pool_cnt[pq], 1);
                    if (slot < a.pool_cap)
                        a.pool[(size_t)pq * a.pool_cap + slot] = ((uint64_t)(uint32_t)s_hi[islot][vi] << 32) | (uint32_t)(d.r0 + (en & 0xFFFFFFu));
                }
                __syncwarp();
                if (lane == 0) s_qcnt[e] = 0;
                __syncwarp();
            };
            // 32 accumulator columns (rows rel .. rel + 31 of the item) against this thread's visitor: the maximum by three-input
            // max, and only when it reaches the visitor's bound the hit mask and one queue entry per hit (no branch per column)
            auto scan32 = [&](const uint32_t (&v)[32], uint32_t rel) {
                float m0 = __uint_as_float(v[0]), m1 = __uint_as_float(v[1]);
#pragma unroll
                for (int j = 2; j < 32; j += 4) {
                    asm("max.f32 %0, %0, %1, %2;" : "+f"(m0) : "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])));
                    if (j + 3 < 32) asm("max.f32 %0, %0, %1, %2;" : "+f"(m1) : "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])));
                }
                if (fmaxf(m0, m1) >= P) {
                    uint32_t mask = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) mask |= (__uint_as_float(v[j]) >= P ? 1u : 0u) << j;
                    if (rel + 32 > nrows) mask &= rel < nrows ? (0xffffffffu >> (rel + 32 - nrows)) : 0u;  // padding rows of the last tile
                    while (mask) {
                        const uint32_t j = (uint32_t)__ffs((int)mask) - 1u;
                        mask &= mask - 1u;
                        ++passes;
                        const int pos = atomicAdd(&s_qcnt[e], 1);
                        if (pos < kQueueCap) {
                            queue[pos] = ((uint32_t)i << 24) | (rel + j);
                        } else {  // queue full (a visitor without cutoff admits whole lists): straight to the pool
                            const int pq = s_pq[islot][i];
                            const int slot = atomicAdd(&a.pool_cnt[pq], 1);
                            if (slot < a.pool_cap)
                                a.pool[(size_t)pq * a.pool_cap + slot] = ((uint64_t)(uint32_t)s_hi[islot][i] << 32) | (uint32_t)(d.r0 + rel + j);
                        }
                    }
                }
                __syncwarp();  // reconverged: the tcgen05 loads and waits that follow are warp-aligned
                if (s_qcnt[e] >= kQueueCap / 2) flush();  // warp-uniform
            };
            for (int k = 0; k < d.ntiles; ++k) {
                const uint32_t gi = it0 + (uint32_t)k;
                if ((int)(gi & 1u) != eg) continue;  // tiles alternate between the two epilogue groups
                const uint32_t st = gi % (uint32_t)NS, use = gi / (uint32_t)NS;
                if (!__all_sync(0xffffffffu, wait_or_abort(&acc_full[st], use & 1u, abort_flag, limit))) { failed = true; break; }
                tc_fence_after();
                const uint32_t rel0 = (uint32_t)k * TN;  // tile's first row, relative to r0
                const uint32_t col0 = lane_addr + st * TN;
                uint32_t va[32], vb[32];  // two loads in flight: the next 32 columns arrive while these are compared
                __syncwarp();
                tmem_ld32(col0, va);
                tmem_ld_wait();
                tmem_ld32(col0 + 32, vb);
                scan32(va, rel0);
                tmem_ld_wait();
                tmem_ld32(col0 + 64, va);
                scan32(vb, rel0 + 32);
                tmem_ld_wait();
                tmem_ld32(col0 + 96, vb);
                scan32(va, rel0 + 64);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(&acc_empty[st]);  // the accumulator is in registers: hand it back before the last comparisons
                scan32(vb, rel0 + 96);
            }
            if (failed) break;
            flush();
            it0 += (uint32_t)d.ntiles;
            mbar_arrive(&item_empty[islot]);
        }
    } else if (warp == kWarpMma) {
        // ---- MMA issuer (one lane) ----
        if (lane == 0) {
            // One thread issues everything, so its instruction count per tile is the pipeline's clock: the operand descriptors
            // of every slot and stage are built once (shared-memory addresses never change), a K step only adds a constant to
            // them (the address field counts 16-byte units; both operands have 16 KB swizzle atoms), and the K loop is unrolled.
            const uint32_t idesc = idesc_bf16(TV, TN);
            const uint64_t da0 = make_sw128_desc(smem_u32(s_a)), da1 = make_sw128_desc(smem_u32(s_a + a_bytes));
            const uint64_t db0 = make_sw128_desc(smem_u32(s_b)), db1 = make_sw128_desc(smem_u32(s_b + b_bytes)),
                           db2 = make_sw128_desc(smem_u32(s_b + 2 * b_bytes));
            const int nsteps = g.kp >> 4;  // <= 12
            uint32_t it0 = 0;
            long long w_item = 0, w_rows = 0, w_acc = 0;  // cycles spent waiting: for an item and its query tile, for decoded rows, for a free accumulator
            for (uint32_t n = 0;; ++n) {
                const int islot = n % kItemRing;
                long long t0 = clock64();
                if (!wait_or_abort(&item_full[islot], (n / kItemRing) & 1u, abort_flag, limit)) { failed = true; break; }
                const int ntiles = s_desc[islot].ntiles;
                if (s_desc[islot].stop) break;
                const int aslot = n % NA;
                if (!wait_or_abort(&a_full[aslot], (n / NA) & 1u, abort_flag, limit)) { failed = true; break; }
                w_item += clock64() - t0;
                const uint64_t da = aslot ? da1 : da0;
                for (int k = 0; k < ntiles; ++k) {
                    const uint32_t gi = it0 + (uint32_t)k;
                    const uint32_t st = gi % (uint32_t)NS, use = gi / (uint32_t)NS;
                    t0 = clock64();
                    if (!wait_or_abort(&b_full[st], use & 1u, abort_flag, limit)) { failed = true; break; }
                    const long long t1 = clock64();
                    if (!wait_or_abort(&acc_empty[st], (use & 1u) ^ 1u, abort_flag, limit)) { failed = true; break; }
                    w_rows += t1 - t0; w_acc += clock64() - t1;
                    if (g.skip_mma) continue;  // test hook: nothing is issued or committed, so the waiting roles give up
                    tc_fence_after();
                    const uint64_t db = st == 0 ? db0 : (st == 1 ? db1 : db2);
                    const uint32_t tacc = tmem + st * TN;
#pragma unroll
                    for (int s2 = 0; s2 < 12; ++s2) {
                        const uint64_t off = (uint64_t)((s2 >> 2) * 1024 + (s2 & 3) * 2);  // atom (16 KB) and 32-byte K step, in 16-byte units
                        if (s2 < nsteps) umma_bf16(tacc, da + off, db + off, idesc, s2 ? 1u : 0u);
                    }
                    umma_commit(&acc_full[st]);
                    umma_commit(&b_empty[st]);
                }
                if (failed) break;
                if (!g.skip_mma) umma_commit(&a_empty[aslot]);  // the query tile may be rebuilt once these MMAs have read it
                it0 += (uint32_t)ntiles;
                mbar_arrive(&item_empty[islot]);
            }
            // where the issuer's time went (diagnostics, summed over CTAs): waiting for items, decoded rows, accumulators; tiles
            atomicAdd(&a.counters[4], (unsigned long long)w_item);
            atomicAdd(&a.counters[5], (unsigned long long)w_rows);
            atomicAdd(&a.counters[6], (unsigned long long)w_acc);
            atomicAdd(&a.counters[7], (unsigned long long)it0);
        }
    }
    if (failed) { *abort_flag = 1; atomicExch(g.status, 1); }
    if (passes) atomicAdd(&a.counters[3], passes);
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (warp == 0) tmem_dealloc(tmem, tmem_cols);
}

// The extra K slots of every code row, computed once per index: |rt|^2 of the row's codewords rounded to bf16.
template <int DSUB>
__global__ void k_row_aug(const uint8_t* __restrict__ codes, long long rows, int m, int k, const float* __restrict__ codebook,
                          float cw2, uint2* __restrict__ out) {
    extern __shared__ float s_n2[];  // [m * k]: squared norm of every rounded codeword
    for (int e = threadIdx.x; e < m * k; e += blockDim.x) {
        float n2 = 0.0f;
#pragma unroll
        for (int d = 0; d < DSUB; ++d) {
            const float v = __bfloat162float(__float2bfloat16_rn(__ldg(codebook + (size_t)e * DSUB + d)));
            n2 = fmaf(v, v, n2);
        }
        s_n2[e] = n2;
    }
    __syncthreads();
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
        const uint8_t* row = codes + (size_t)r * m;
        float rn = 0.0f;
        for (int j = 0; j < m; ++j) rn += s_n2[j * k + __ldg(row + j)];
        out[r] = row_aug_words(rn, cw2);
    }
}

// ------------------------------------------------------------------------------------------------------
// Selection with re-scoring.  A pool entry is either an exact key (distance bits with the top bit set: written by the SIMT
// scans) or an unscored survivor of the tensor-core filter: (list id, or in residual mode the (query, probe) pair) << 32 |
// scanned row.  Unscored entries get their exact fp32 ADC distance here - plain mode from the query's fp32 table staged in
// shared memory, residual mode from the pair's residual and the codebook, both in the CPU path's summation order - and are
// dropped when it exceeds the cutoff.  Then the pool is sorted by (distance, row) and the first stage1_k rows go out.  A pool
// that overflowed, or holds fewer than min(stage1_k, rows scanned) entries within the cutoff, sends the query to the exact
// fallback.
constexpr int kRescoreThreads = 1024;

struct RescoreArgs {
    const uint64_t* pool; const int* pool_cnt; int pool_cap;
    const long long* q_rows; const float* thr; int stage1_k;
    const float* lut;          // plain mode: [nq][m * k]
    const float* queries; const float* centroids; const float* codebook; const int* probes; int nprobe, dim, nlist;  // residual mode
    const uint8_t* codes; long long row_base; const long long* row_delta;
    int m, k, residual, tree;
    int* out_rows; float* out_dist; int* out_count;
    int* fail_list; int* n_fail; unsigned long long* counters;
    int shared_cut;   // the cutoff covers the rows of all shards: this shard need not reach stage1_k rows
};

template <int M>
__global__ void __launch_bounds__(kRescoreThreads) k_select_rescore(const RescoreArgs g) {
    extern __shared__ __align__(16) unsigned char s_sel[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_sel);                      // [pool_cap]
    float* s_tab = reinterpret_cast<float*>(s_sel + (size_t)g.pool_cap * 8);   // plain: the table [m * k]; residual: the query [dim]
    __shared__ int s_valid;
    const int q = blockIdx.x;
    const int c = g.pool_cnt[q];
    const long long N = g.q_rows[q];
    long long need = N < g.stage1_k ? N : g.stage1_k;
    if (g.shared_cut && g.thr[q] < __int_as_float(0x7f800000)) need = 0;   // sharded search: the shards owe stage1_k rows together
    if (c > g.pool_cap || c < need) {
        if (threadIdx.x == 0) g.fail_list[atomicAdd(g.n_fail, 1)] = q;
        return;  // the fallback writes this query's outputs
    }
    const int mk = g.m * g.k;
    const int dsub = g.dim / g.m;
    if (!g.residual) {
        for (int e = threadIdx.x; e < mk; e += blockDim.x) s_tab[e] = g.lut[(size_t)q * mk + e];
    } else {
        for (int d = threadIdx.x; d < g.dim; d += blockDim.x) s_tab[d] = g.queries[(size_t)q * g.dim + d];
    }
    if (threadIdx.x == 0) s_valid = 0;
    __syncthreads();
    const float cut = g.thr[q];
    const int n = next_pow2(max(c, 2));
    int valid = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        uint64_t key = KEY_MAX;
        if (i < c) {
            const uint64_t e = g.pool[(size_t)q * g.pool_cap + i];
            if (e >> 63) {
                key = e;  // exact already, and within the cutoff
                ++valid;
            } else {
                const long long r = (long long)(uint32_t)e;
                const int hi = (int)(e >> 32);
                const uint8_t* row = g.codes + (size_t)(r - g.row_base) * g.m;
                float d;
                int l;
                if (!g.residual) {
                    l = hi;
                    d = adc_row<M>(row, s_tab, g.m, g.k, false);
                } else {
                    l = g.probes[hi];
                    const float* cen = g.centroids + (size_t)l * g.dim;
                    d = adc_row_direct<M>(row, s_tab, g.codebook, g.m, g.k, dsub, g.tree != 0, cen);
                }
                if (d <= cut) {
                    const long long delta = g.row_delta ? g.row_delta[l] : 0;
                    key = make_key(d, (uint32_t)(r + delta));
                    ++valid;
                }
            }
        }
        s_keys[i] = key;
    }
    if (valid) atomicAdd(&s_valid, valid);
    __syncthreads();
    const int nv = s_valid;
    if (nv < need) {
        if (threadIdx.x == 0) g.fail_list[atomicAdd(g.n_fail, 1)] = q;
        return;
    }
    if (threadIdx.x == 0) atomicAdd(&g.counters[1], (unsigned long long)nv);
    block_bitonic_sort(s_keys, n);
    const int keep = nv < g.stage1_k ? nv : g.stage1_k;
    for (int i = threadIdx.x; i < g.stage1_k; i += blockDim.x) {
        const bool ok = i < keep;
        g.out_rows[(size_t)q * g.stage1_k + i] = ok ? (int)key_idx(s_keys[i]) : -1;
        if (g.out_dist) g.out_dist[(size_t)q * g.stage1_k + i] = ok ? key_dist(s_keys[i]) : FLT_MAX;
    }
    if (g.out_count && threadIdx.x == 0) g.out_count[q] = keep;
}

// Shared-memory plan of k_scan_tc for a shape: query-tile slots, row-tile stages and the dynamic bytes; false when the
// shape is outside the kernel's range or does not fit.
bool tc_scan_plan(int dim, int m, int k, int* na, int* ns, size_t* bytes) {
    if (m <= 0 || dim <= 0 || dim % m != 0) return false;
    const int dsub = dim / m;
    if (!(dsub == 2 || dsub == 4 || dsub == 8) || dim % 8 != 0 || m % 4 != 0 || k > 256 || k < 1) return false;
    const int kp = (dim + kAugSlots + 15) / 16 * 16;
    const int katoms = (kp + 63) / 64;
    const size_t a_bytes = (size_t)katoms * TV * 128, b_bytes = (size_t)katoms * TN * 128, tab = (size_t)m * k * dsub * 2;
    const size_t budget = (size_t)218 * 1024;  // dynamic part; ~11 KB of static shared memory and the 1 KB alignment come on top
    for (int a_slots = 2; a_slots >= 1; --a_slots) {
        if (tab + a_slots * a_bytes + 2 * b_bytes > budget) continue;
        int stages = (int)((budget - tab - a_slots * a_bytes) / b_bytes);
        stages = stages > kDecodeGroups ? kDecodeGroups : stages;  // one decode warp group per stage
        *na = a_slots; *ns = stages; *bytes = tab + a_slots * a_bytes + stages * b_bytes + 1024;
        return true;
    }
    return false;
}

}  // namespace

bool scan_tc_supported(int dim, int m, int k) {
    int na, ns; size_t bytes;
    return tc_scan_plan(dim, m, k, &na, &ns, &bytes);
}

float scan_tc_eps(int dim) {
    const int kp = (dim + kAugSlots + 15) / 16 * 16;
    return (float)kp * (1.0f / 4194304.0f) * 2.0f;  // kp * 2^-22 * 2: tensor-core accumulation plus the fp32 norms
}

namespace {
// One CTA per (list, block of 1024 rows): the centroid sits in shared memory, every thread sums w (w + 2 c) over its row's codewords.
__global__ void __launch_bounds__(256) k_row_bias(const uint8_t* __restrict__ codes, const long long* __restrict__ offsets, long long row_base,
                                                  int list_begin, int list_end, int dim, int m, int k, const float* __restrict__ codebook,
                                                  const float* __restrict__ centroids, float* __restrict__ out) {
    extern __shared__ float s_cen[];  // [dim]
    const int dsub = dim / m;
    for (int l = list_begin + blockIdx.y; l < list_end; l += gridDim.y) {
        const long long b = offsets[l], e = offsets[l + 1];
        if ((long long)blockIdx.x * 1024 >= e - b) continue;
        __syncthreads();
        for (int d = threadIdx.x; d < dim; d += blockDim.x) s_cen[d] = centroids[(size_t)l * dim + d];
        __syncthreads();
        for (long long r0 = b + (long long)blockIdx.x * 1024; r0 < e; r0 += (long long)gridDim.x * 1024) {
            for (long long r = r0 + threadIdx.x; r < min(r0 + 1024, e); r += blockDim.x) {
                const uint8_t* row = codes + (size_t)(r - row_base) * m;
                float acc = 0.0f;
                for (int j = 0; j < m; ++j) {
                    const float* cb = codebook + ((size_t)j * k + __ldg(row + j)) * dsub;
                    for (int d = 0; d < dsub; ++d) { const float w = __ldg(cb + d); acc = fmaf(w, w + 2.0f * s_cen[j * dsub + d], acc); }
                }
                out[r - row_base] = acc;
            }
        }
    }
}
}  // namespace

psb_status launch_row_bias(const uint8_t* d_codes, const long long* d_offsets, long long row_base, int list_begin, int list_end,
                           int dim, int m, int k, const float* d_codebook, const float* d_centroids, float* d_out, cudaStream_t s) {
    if (list_end <= list_begin) return PSB_OK;
    const dim3 grid(64, (unsigned)std::min(list_end - list_begin, 1024));
    k_row_bias<<<grid, 256, (size_t)dim * sizeof(float), s>>>(d_codes, d_offsets, row_base, list_begin, list_end, dim, m, k, d_codebook,
                                                               d_centroids, d_out);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

psb_status launch_row_aug(const uint8_t* d_codes, long long rows, int dim, int m, int k, const float* d_codebook, void* d_out,
                          cudaStream_t s) {
    if (rows <= 0) return PSB_OK;
    const int dsub = dim / m;
    const float cw2 = kBeta * kBeta + scan_tc_eps(dim);
    const size_t smem = (size_t)m * k * sizeof(float);
    const unsigned grid = (unsigned)std::min<long long>((rows + 255) / 256, 148 * 16);
#define PSB_AUG(D)                                                                                                      \
    do {                                                                                                                \
        if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_row_aug<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        k_row_aug<D><<<grid, 256, smem, s>>>(d_codes, rows, m, k, d_codebook, cw2, static_cast<uint2*>(d_out));          \
    } while (0)
    if (dsub == 2) PSB_AUG(2);
    else if (dsub == 4) PSB_AUG(4);
    else if (dsub == 8) PSB_AUG(8);
    else return fail(PSB_UNSUPPORTED_SHAPE, "tensor-core scan does not support this shape");
#undef PSB_AUG
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

namespace {
template <int DSUB, int M>
psb_status run_scan_tc(const ScanTcArgs& g, unsigned grid, size_t smem, cudaStream_t s) {
    PSB_CUDA(cudaFuncSetAttribute(k_scan_tc<DSUB, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_scan_tc<DSUB, M><<<grid, kTcScanThreads, smem, s>>>(g);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}
}  // namespace

psb_status launch_scan_tc(const ScanTcLaunch& L, cudaStream_t s) {
    int na = 0, ns = 0;
    size_t smem = 0;
    if (!tc_scan_plan(L.dim, L.m, L.k, &na, &ns, &smem)) return fail(PSB_UNSUPPORTED_SHAPE, "tensor-core scan does not support this shape");
    if (!L.row_aug) return fail(PSB_INTERNAL, "tensor-core scan: the per-row terms are missing");
    ScanTcArgs g;
    g.a.lut = nullptr; g.a.lut_div = L.lut_div; g.a.tree = 0; g.a.codes = L.codes; g.a.offsets = L.offsets; g.a.row_base = L.row_base;
    g.a.row_delta = nullptr; g.a.nlist = L.nlist; g.a.m = L.m; g.a.k = L.k; g.a.vis_count = L.vis_count; g.a.vis_off = L.vis_off;
    g.a.visitors = L.visitors; g.a.item_off = L.item_off; g.a.thr = L.thr; g.a.pool_cnt = L.pool_cnt; g.a.pool = L.pool;
    g.a.pool_cap = L.pool_cap; g.a.work_cursor = L.work_cursor; g.a.counters = L.counters; g.a.chunk_rows = L.chunk_rows;
    g.a.reserve_ctas = L.reserve_ctas;
    g.queries = L.queries; g.centroids = L.centroids; g.codebook = L.codebook; g.row_aug = static_cast<const uint2*>(L.row_aug);
    g.dim = L.dim; g.kp = (L.dim + kAugSlots + 15) / 16 * 16; g.katoms = (g.kp + 63) / 64; g.na = na; g.ns = ns;
    g.residual = L.residual ? 1 : 0;
    g.eps = scan_tc_eps(L.dim);
    g.status = L.status; g.wait_limit = L.wait_limit > 0 ? L.wait_limit : kWaitLimit; g.skip_mma = L.skip_mma;
    const unsigned grid = scan_grid(L.sm_count, L.reserve_ctas);
    const int dsub = L.dim / L.m;
    if (dsub == 2) {
        switch (L.m) {
            case 16: return run_scan_tc<2, 16>(g, grid, smem, s);
            case 32: return run_scan_tc<2, 32>(g, grid, smem, s);
            case 48: return run_scan_tc<2, 48>(g, grid, smem, s);
            case 64: return run_scan_tc<2, 64>(g, grid, smem, s);
            default: return run_scan_tc<2, 0>(g, grid, smem, s);
        }
    } else if (dsub == 4) {
        switch (L.m) {
            case 8: return run_scan_tc<4, 8>(g, grid, smem, s);
            case 16: return run_scan_tc<4, 16>(g, grid, smem, s);
            case 32: return run_scan_tc<4, 32>(g, grid, smem, s);
            default: return run_scan_tc<4, 0>(g, grid, smem, s);
        }
    } else {
        switch (L.m) {
            case 8: return run_scan_tc<8, 8>(g, grid, smem, s);
            case 16: return run_scan_tc<8, 16>(g, grid, smem, s);
            default: return run_scan_tc<8, 0>(g, grid, smem, s);
        }
    }
}

namespace {
template <int M>
psb_status run_select_rescore(const RescoreArgs& g, int nq, cudaStream_t s) {
    const size_t smem = (size_t)g.pool_cap * 8 + (g.residual ? (size_t)g.dim * 4 : (size_t)g.m * g.k * 4);
    if (smem > (size_t)226 * 1024) return fail(PSB_UNSUPPORTED_SHAPE, "re-scoring selection does not fit shared memory");
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_select_rescore<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PSB_TRY(prefer_max_shared(k_select_rescore<M>));
    k_select_rescore<M><<<nq, kRescoreThreads, smem, s>>>(g);
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}
}  // namespace

psb_status launch_select_rescore(const SelectRescoreLaunch& L, int nq, cudaStream_t s) {
    if (nq <= 0) return PSB_OK;
    RescoreArgs g;
    g.pool = L.pool; g.pool_cnt = L.pool_cnt; g.pool_cap = L.pool_cap; g.q_rows = L.q_rows; g.thr = L.thr; g.stage1_k = L.stage1_k;
    g.lut = L.lut; g.queries = L.queries; g.centroids = L.centroids; g.codebook = L.codebook; g.probes = L.probes;
    g.nprobe = L.nprobe; g.dim = L.dim; g.nlist = L.nlist; g.codes = L.codes; g.row_base = L.row_base; g.row_delta = L.row_delta;
    g.m = L.m; g.k = L.k; g.residual = L.residual ? 1 : 0; g.tree = L.tree ? 1 : 0;
    g.out_rows = L.out_rows; g.out_dist = L.out_dist; g.out_count = L.out_count; g.fail_list = L.fail_list; g.n_fail = L.n_fail;
    g.counters = L.counters; g.shared_cut = L.shared_cut ? 1 : 0;
    switch (L.m) {
        case 8: return run_select_rescore<8>(g, nq, s);
        case 16: return run_select_rescore<16>(g, nq, s);
        case 32: return run_select_rescore<32>(g, nq, s);
        case 48: return run_select_rescore<48>(g, nq, s);
        case 64: return run_select_rescore<64>(g, nq, s);
        default: return run_select_rescore<0>(g, nq, s);
    }
}

}  // namespace psb
