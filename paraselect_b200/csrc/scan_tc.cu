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
constexpr int kDecodeWarps = 8;    // warps 0-7: decode code rows into the B stages
constexpr int kEpiWarps = 8;       // warps 8-15: read accumulators, compare, push survivors
constexpr int kWorkers = (kDecodeWarps + kEpiWarps) * 32;
constexpr int kTcScanThreads = kWorkers + 32;  // warp 16: MMA issuer
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kAugSlots = 4;
constexpr float kBeta = 0.001953125f * 1.001f;  // 2^-9 (1 + 1e-3)

struct ScanTcArgs {
    ScanArgs a;               // a.item_off: the tensor-core work items (lists the SIMT scan leaves out)
    const float* queries;     // [nq][dim]
    const float* centroids;   // [nlist][dim]
    const float* codebook;    // [m][k][dsub]
    const int* probes;        // residual mode: [nq * nprobe] list of every (query, probe) pair
    int dim, kp, katoms, tn;  // kp: padded K (multiple of 16), katoms: 128-byte swizzle atoms along K, tn: code rows per tile
    int residual;
    float eps;                // accumulation slack e
    int* status;              // != 0 after a bounded wait gave up
    int wait_limit;           // polls before a wait gives up (tests shorten it)
    int skip_mma;             // test hook: the MMA warp issues nothing, so every waiting role runs into its limit
};

// Bounded wait that also leaves when another role of the CTA has given up.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int limit) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ uint32_t bf16_bits_rn(float x) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t bf16_bits_up(float x) {  // x >= 0, finite: the smallest bf16 >= x
    return (__float_as_uint(x) + 0xFFFFu) >> 16;
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) { return bf16_bits_rn(lo) | (bf16_bits_rn(hi) << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Address of 16-byte chunk c of operand row `row` in a K-major 128-byte-swizzled operand of `rows` rows.
__device__ __forceinline__ unsigned char* chunk_ptr(unsigned char* base, int rows, int row, int c) {
    return base + (size_t)(c >> 3) * rows * 128 + (size_t)row * 128 + (size_t)(((c & 7) ^ (row & 7)) << 4);
}

template <int DSUB>
__global__ void __launch_bounds__(kTcScanThreads, 1) k_scan_tc(const ScanTcArgs g) {
    const ScanArgs& a = g.a;
    extern __shared__ __align__(1024) unsigned char s_dyn[];
    unsigned char* s_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_dyn) + 1023) & ~uintptr_t(1023));
    const size_t a_bytes = (size_t)g.katoms * TV * 128, b_bytes = (size_t)g.katoms * g.tn * 128;
    unsigned char* s_a = s_base;                    // [katoms][TV][128 B]
    unsigned char* s_b = s_base + a_bytes;          // [2][katoms][tn][128 B]
    unsigned char* s_tab = s_b + 2 * b_bytes;       // [m][k] entries of DSUB bf16: the list's centred codewords
    float* s_c = reinterpret_cast<float*>(s_tab + (size_t)a.m * a.k * DSUB * 2);  // [dim] centroid of the list
    __shared__ __align__(8) uint64_t b_full[2], b_empty[2], acc_full[2], acc_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ long long s_item;
    __shared__ int s_list, s_abort;
    __shared__ int s_vq[TV], s_pq[TV];
    __shared__ float s_P[TV];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunk_data = g.dim >> 3, nchunk = g.kp >> 3;
    const int limit = g.wait_limit;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&b_full[i], kDecodeThreads); mbar_init(&b_empty[i], 1);
            mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpiThreads);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&s_tmem, (uint32_t)(2 * g.tn));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const long long total = a.item_off[a.nlist];
    const uint32_t idesc = idesc_bf16(TV, g.tn);
    volatile int* abort_flag = &s_abort;
    uint32_t it = 0;      // tiles this role has been through (all roles count alike)
    int tab_list = -1;    // list whose codewords s_tab holds (-2: the list-independent residual table)
    bool failed = false;
    unsigned long long passes = 0;

    for (;;) {
        __syncthreads();  // every role is done with the previous item: operands, tables and s_* words may be rewritten
        if (warp == 0) {
            long long item = 0;
            if (lane == 0) item = (long long)atomicAdd(a.work_cursor, 1ull);
            item = __shfl_sync(0xffffffffu, item, 0);
            int l = -1;
            if (item < total) l = find_list(a.item_off, a.nlist, item);
            if (lane == 0) { s_item = item; s_list = l; }
        }
        __syncthreads();
        if (*abort_flag) break;
        const long long item = s_item;
        if (item >= total) break;
        const int l = s_list;
        const int nvis = a.vis_count[l];
        const int ngroups = (nvis + TV - 1) / TV;
        const long long local = item - a.item_off[l];
        const int group = (int)(local % ngroups);
        const long long chunk = local / ngroups;
        const long long r0 = a.offsets[l] + chunk * a.chunk_rows;
        const long long r1 = min(r0 + a.chunk_rows, a.offsets[l + 1]);
        const int ntiles = (int)((r1 - r0 + g.tn - 1) / g.tn);

        // ---- set-up by the 512 worker threads: centroid, codeword table, query tile, per-visitor constants ----
        if (tid < kWorkers) {
            for (int d = tid; d < g.dim; d += kWorkers) s_c[d] = __ldg(g.centroids + (size_t)l * g.dim + d);
            asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory");
            const int want = g.residual ? -2 : l;
            if (tab_list != want) {  // uniform
                const int entries = a.m * a.k;
                for (int e = tid; e < entries; e += kWorkers) {
                    const int sub = e / a.k;
                    const float* cb = g.codebook + (size_t)e * DSUB;
                    uint32_t w[DSUB / 2];
#pragma unroll
                    for (int d = 0; d < DSUB; d += 2) {
                        float x0 = __ldg(cb + d), x1 = __ldg(cb + d + 1);
                        if (!g.residual) { x0 = __fsub_rn(x0, s_c[sub * DSUB + d]); x1 = __fsub_rn(x1, s_c[sub * DSUB + d + 1]); }
                        w[d / 2] = pack_bf16x2_rn(x0, x1);
                    }
                    uint32_t* dst = reinterpret_cast<uint32_t*>(s_tab + (size_t)e * DSUB * 2);
#pragma unroll
                    for (int d = 0; d < DSUB / 2; ++d) dst[d] = w[d];
                }
                tab_list = want;
            }
            // query tile: four threads per visitor row
            const int i = tid >> 2, part = tid & 3;
            const int vi = group * TV + i;
            const int vq = vi < nvis ? a.visitors[a.vis_off[l] + vi] : -1;   // table index: the query, or the pair in residual mode
            const int pq = vq >= 0 ? vq / a.lut_div : -1;                     // query (pool, cutoff)
            float qn = 0.0f, n2 = 0.0f;  // |qt|^2 over this thread's chunks, |q'|^2
            float P = __int_as_float(0x7f800000), H = 0.0f;
            const float* qrow = g.queries + (size_t)(pq >= 0 ? pq : 0) * g.dim;
            if (pq >= 0) {
                for (int c = part; c < nchunk_data; c += 4) {
                    const float4 x0 = __ldg(reinterpret_cast<const float4*>(qrow + c * 8));
                    const float4 x1 = __ldg(reinterpret_cast<const float4*>(qrow + c * 8 + 4));
                    const float4 c0 = *reinterpret_cast<const float4*>(s_c + c * 8);
                    const float4 c1 = *reinterpret_cast<const float4*>(s_c + c * 8 + 4);
                    const float v[8] = {__fsub_rn(x0.x, c0.x), __fsub_rn(x0.y, c0.y), __fsub_rn(x0.z, c0.z), __fsub_rn(x0.w, c0.w),
                                        __fsub_rn(x1.x, c1.x), __fsub_rn(x1.y, c1.y), __fsub_rn(x1.z, c1.z), __fsub_rn(x1.w, c1.w)};
                    uint4 o;
                    o.x = pack_bf16x2_rn(v[0], v[1]); o.y = pack_bf16x2_rn(v[2], v[3]);
                    o.z = pack_bf16x2_rn(v[4], v[5]); o.w = pack_bf16x2_rn(v[6], v[7]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) n2 = fmaf(v[j], v[j], n2);
                    const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) { const float lo = bf16_lo(ow[j]), hi = bf16_hi(ow[j]); qn = fmaf(lo, lo, qn); qn = fmaf(hi, hi, qn); }
                    *reinterpret_cast<uint4*>(chunk_ptr(s_a, TV, i, c)) = o;
                }
            } else {
                for (int c = part; c < nchunk_data; c += 4) *reinterpret_cast<uint4*>(chunk_ptr(s_a, TV, i, c)) = make_uint4(0, 0, 0, 0);
            }
            qn += __shfl_xor_sync(0xffffffffu, qn, 1); qn += __shfl_xor_sync(0xffffffffu, qn, 2);
            n2 += __shfl_xor_sync(0xffffffffu, n2, 1); n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
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
            for (int c = nchunk_data + part; c < nchunk; c += 4) {  // the extra K slots, then zero padding
                uint4 o = make_uint4(0, 0, 0, 0);
                if (c == nchunk_data && pq >= 0) { o.x = 0x3F803F80u; o.y = 0x3F80u | (bf16_bits_up(H) << 16); }  // 1, 1, 1, H
                *reinterpret_cast<uint4*>(chunk_ptr(s_a, TV, i, c)) = o;
            }
            if (part == 0) { s_vq[i] = g.residual ? vq : l; s_pq[i] = pq; s_P[i] = P; }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // operand stores -> visible to the tensor core
        }
        __syncthreads();

        if (warp < kDecodeWarps) {
            // ---- decode: thread j fills operand row j of every tile ----
            const float cw2 = kBeta * kBeta + g.eps;
            for (int t = 0; t < ntiles && !failed; ++t, ++it) {
                const uint32_t st = it & 1u;
                if (!__all_sync(0xffffffffu, wait_or_abort(&b_empty[st], ((it >> 1) & 1u) ^ 1u, abort_flag, limit))) { failed = true; break; }
                unsigned char* sb = s_b + st * b_bytes;
                if (tid < g.tn) {
                    const long long r = r0 + (long long)t * g.tn + tid;
                    if (r < r1) {
                        const uint8_t* row = a.codes + (size_t)(r - a.row_base) * a.m;
                        float rn = 0.0f;
                        const int words = a.m >> 2;
                        for (int w0 = 0; w0 < words; w0 += 4) {
                            uint32_t cw[4];
                            if ((a.m & 15) == 0) {
                                const uint4 c4 = __ldg(reinterpret_cast<const uint4*>(row) + (w0 >> 2));
                                cw[0] = c4.x; cw[1] = c4.y; cw[2] = c4.z; cw[3] = c4.w;
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j) cw[j] = w0 + j < words ? __ldg(reinterpret_cast<const uint32_t*>(row) + w0 + j) : 0u;
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int w = w0 + j;  // code word w holds sub-quantisers 4w .. 4w+3
                                if (w < words) {
                                    if constexpr (DSUB == 2) {  // four codewords of 2 -> one chunk
                                        uint32_t o[4];
#pragma unroll
                                        for (int b = 0; b < 4; ++b) {
                                            const int code = (cw[j] >> (8 * b)) & 255;
                                            o[b] = *reinterpret_cast<const uint32_t*>(s_tab + ((size_t)(4 * w + b) * a.k + code) * 4);
                                            const float lo = bf16_lo(o[b]), hi = bf16_hi(o[b]);
                                            rn = fmaf(lo, lo, rn); rn = fmaf(hi, hi, rn);
                                        }
                                        *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, w)) = make_uint4(o[0], o[1], o[2], o[3]);
                                    } else if constexpr (DSUB == 4) {  // two codewords of 4 -> one chunk
#pragma unroll
                                        for (int h = 0; h < 2; ++h) {
                                            const int c0 = (cw[j] >> (16 * h)) & 255, c1 = (cw[j] >> (16 * h + 8)) & 255;
                                            const uint2 e0 = *reinterpret_cast<const uint2*>(s_tab + ((size_t)(4 * w + 2 * h) * a.k + c0) * 8);
                                            const uint2 e1 = *reinterpret_cast<const uint2*>(s_tab + ((size_t)(4 * w + 2 * h + 1) * a.k + c1) * 8);
                                            const uint32_t o[4] = {e0.x, e0.y, e1.x, e1.y};
#pragma unroll
                                            for (int b = 0; b < 4; ++b) { const float lo = bf16_lo(o[b]), hi = bf16_hi(o[b]); rn = fmaf(lo, lo, rn); rn = fmaf(hi, hi, rn); }
                                            *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, 2 * w + h)) = make_uint4(o[0], o[1], o[2], o[3]);
                                        }
                                    } else {  // DSUB == 8: one codeword -> one chunk
#pragma unroll
                                        for (int b = 0; b < 4; ++b) {
                                            const int code = (cw[j] >> (8 * b)) & 255;
                                            const uint4 e = *reinterpret_cast<const uint4*>(s_tab + ((size_t)(4 * w + b) * a.k + code) * 16);
                                            const uint32_t o[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
                                            for (int x = 0; x < 4; ++x) { const float lo = bf16_lo(o[x]), hi = bf16_hi(o[x]); rn = fmaf(lo, lo, rn); rn = fmaf(hi, hi, rn); }
                                            *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, 4 * w + b)) = e;
                                        }
                                    }
                                }
                            }
                        }
                        // the extra K slots: minus the three-term split of U, then w rounded up
                        const float wv = sqrtf(rn) * 1.003908f;  // >= |r'| (1 + 2^-8 and the square root's rounding)
                        float rest = 0.5f * (rn - cw2 * wv * wv);
                        uint32_t u[3];
#pragma unroll
                        for (int x = 0; x < 3; ++x) {
                            const __nv_bfloat16 h = __float2bfloat16_rn(rest);
                            u[x] = (uint32_t)__bfloat16_as_ushort(__hneg(h));
                            rest -= __bfloat162float(h);
                        }
                        *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, nchunk_data)) =
                            make_uint4(u[0] | (u[1] << 16), u[2] | (bf16_bits_up(wv) << 16), 0u, 0u);
                    } else {
                        // past the end of the chunk: a row no visitor can admit (score -1e30)
                        for (int c = 0; c < nchunk_data; ++c) *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, c)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, nchunk_data)) = make_uint4(bf16_bits_rn(-1.0e30f), 0u, 0u, 0u);
                    }
                    for (int c = nchunk_data + 1; c < nchunk; ++c) *reinterpret_cast<uint4*>(chunk_ptr(sb, g.tn, tid, c)) = make_uint4(0, 0, 0, 0);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&b_full[st])) : "memory");
            }
        } else if (warp < kDecodeWarps + kEpiWarps) {
            // ---- epilogue: one visitor per thread (tensor-memory lane), half of the tile's columns per warp ----
            const int e = warp - kDecodeWarps, quad = e & 3, half = e >> 2;  // warp % 4 == quad: the lanes this warp may read
            const int i = quad * 32 + lane;
            const float P = s_P[i];
            const int pq = s_pq[i];
            const uint64_t hi_word = (uint64_t)(uint32_t)s_vq[i] << 32;
            const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
            const int cols = g.tn >> 1;  // per warp
            for (int t = 0; t < ntiles && !failed; ++t, ++it) {
                const uint32_t acc = it & 1u;
                if (!__all_sync(0xffffffffu, wait_or_abort(&acc_full[acc], (it >> 1) & 1u, abort_flag, limit))) { failed = true; break; }
                tc_fence_after();
                const long long rbase = r0 + (long long)t * g.tn + half * cols;
                for (int cb = 0; cb < cols; cb += 64) {
                    uint32_t v0[32], v1[32];
                    __syncwarp();
                    tmem_ld32(lane_addr + (uint32_t)(acc * g.tn + half * cols + cb), v0);
                    tmem_ld32(lane_addr + (uint32_t)(acc * g.tn + half * cols + cb + 32), v1);
                    tmem_ld_wait();
                    if (cb + 64 >= cols) {  // the accumulator is in registers: hand it back before the comparisons
                        tc_fence_before();
                        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
                    }
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint32_t* v = hh ? v1 : v0;
                        float m = __uint_as_float(v[0]);
#pragma unroll
                        for (int j = 1; j < 32; ++j) m = fmaxf(m, __uint_as_float(v[j]));
                        if (m >= P) {  // rare: a survivor among these 32 rows
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const long long r = rbase + cb + hh * 32 + j;
                                if (__uint_as_float(v[j]) >= P && r < r1) {  // r >= r1: padding rows of the last tile
                                    const int slot = atomicAdd(&a.pool_cnt[pq], 1);
                                    if (slot < a.pool_cap) a.pool[(size_t)pq * a.pool_cap + slot] = hi_word | (uint32_t)r;
                                    ++passes;
                                }
                            }
                        }
                    }
                }
            }
        } else if (lane == 0) {
            // ---- MMA issuer ----
            for (int t = 0; t < ntiles && !failed; ++t, ++it) {
                const uint32_t st = it & 1u;
                if (!wait_or_abort(&b_full[st], (it >> 1) & 1u, abort_flag, limit)) { failed = true; break; }
                if (!wait_or_abort(&acc_empty[st], ((it >> 1) & 1u) ^ 1u, abort_flag, limit)) { failed = true; break; }
                if (g.skip_mma) continue;  // test hook: nothing is issued, nothing completes, every waiting role gives up
                tc_fence_after();
                const uint32_t sa = smem_u32(s_a), sb = smem_u32(s_b + st * b_bytes);
                for (int ka = 0; ka < g.katoms; ++ka) {
                    const int ksteps = min(4, (g.kp - ka * 64) >> 4);
                    for (int kk = 0; kk < ksteps; ++kk)
                        umma_bf16(tmem + (uint32_t)(st * g.tn), make_sw128_desc(sa + ka * TV * 128 + kk * 32),
                                  make_sw128_desc(sb + ka * g.tn * 128 + kk * 32), idesc, (ka | kk) ? 1u : 0u);
                }
                umma_commit(&acc_full[st]);
                umma_commit(&b_empty[st]);
            }
        }
        if (failed) *abort_flag = 1;
    }
    if (failed) atomicExch(g.status, 1);
    if (passes) atomicAdd(&a.counters[3], passes);
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (warp == 0) tmem_dealloc(tmem, (uint32_t)(2 * g.tn));
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
};

// One table entry computed directly: the sequential non-fused sum over the sub-vector (what k_build_lut_residual stores).
__device__ __forceinline__ float entry_direct(const float* __restrict__ qres, const float* __restrict__ cb, int dsub) {
    float e = 0.0f;
    for (int d = 0; d < dsub; ++d) {
        const float diff = __fsub_rn(qres[d], __ldg(cb + d));
        e = __fadd_rn(e, __fmul_rn(diff, diff));
    }
    return e;
}

template <int M>
__global__ void __launch_bounds__(kRescoreThreads) k_select_rescore(const RescoreArgs g) {
    extern __shared__ __align__(16) unsigned char s_sel[];
    uint64_t* s_keys = reinterpret_cast<uint64_t*>(s_sel);                      // [pool_cap]
    float* s_tab = reinterpret_cast<float*>(s_sel + (size_t)g.pool_cap * 8);   // plain: the table [m * k]; residual: the query [dim]
    __shared__ int s_valid;
    const int q = blockIdx.x;
    const int c = g.pool_cnt[q];
    const long long N = g.q_rows[q];
    const long long need = N < g.stage1_k ? N : g.stage1_k;
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
                    float t[M > 0 ? M : 1];
                    float acc = 0.0f;
                    for (int j = 0; j < g.m; ++j) {
                        float qres[8];  // dsub <= 8 on this path
                        for (int x = 0; x < dsub; ++x) qres[x] = __fsub_rn(s_tab[j * dsub + x], __ldg(cen + j * dsub + x));
                        const float en = entry_direct(qres, g.codebook + ((size_t)j * g.k + __ldg(row + j)) * dsub, dsub);
                        if constexpr (M == 8 || M == 16) { if (g.tree) { t[j] = en; continue; } }
                        acc = __fadd_rn(acc, en);
                    }
                    if constexpr (M == 8 || M == 16) { if (g.tree) acc = tree_sum<M>(t); }
                    d = acc;
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

size_t tc_scan_smem(int dim, int m, int k, int tn) {
    const int dsub = dim / m;
    const int kp = (dim + kAugSlots + 15) / 16 * 16;
    const int katoms = (kp + 63) / 64;
    return (size_t)katoms * TV * 128 + 2 * (size_t)katoms * tn * 128 + (size_t)m * k * dsub * 2 + (size_t)dim * 4 + 1024;
}

}  // namespace

// Rows per tile: 256 when the operands fit, else 128; 0 = the shape is outside this kernel's range.
int scan_tc_tile_rows(int dim, int m, int k) {
    if (m <= 0 || dim % m != 0) return 0;
    const int dsub = dim / m;
    if (!(dsub == 2 || dsub == 4 || dsub == 8) || dim % 8 != 0 || m % 4 != 0 || k > 256 || k < 1) return 0;
    for (int tn : {256, 128})
        if (tc_scan_smem(dim, m, k, tn) <= (size_t)222 * 1024) return tn;  // dynamic part; ~2 KB of static shared memory come on top
    return 0;
}

psb_status launch_scan_tc(const ScanTcLaunch& L, cudaStream_t s) {
    const int tn = scan_tc_tile_rows(L.dim, L.m, L.k);
    if (tn == 0) return fail(PSB_UNSUPPORTED_SHAPE, "tensor-core scan does not support this shape");
    ScanTcArgs g;
    g.a.lut = nullptr; g.a.lut_div = L.lut_div; g.a.tree = 0; g.a.codes = L.codes; g.a.offsets = L.offsets; g.a.row_base = L.row_base;
    g.a.row_delta = nullptr; g.a.nlist = L.nlist; g.a.m = L.m; g.a.k = L.k; g.a.vis_count = L.vis_count; g.a.vis_off = L.vis_off;
    g.a.visitors = L.visitors; g.a.item_off = L.item_off; g.a.thr = L.thr; g.a.pool_cnt = L.pool_cnt; g.a.pool = L.pool;
    g.a.pool_cap = L.pool_cap; g.a.work_cursor = L.work_cursor; g.a.counters = L.counters; g.a.chunk_rows = L.chunk_rows;
    g.a.reserve_ctas = L.reserve_ctas;
    g.queries = L.queries; g.centroids = L.centroids; g.codebook = L.codebook; g.probes = L.probes;
    g.dim = L.dim; g.kp = (L.dim + kAugSlots + 15) / 16 * 16; g.katoms = (g.kp + 63) / 64; g.tn = tn; g.residual = L.residual ? 1 : 0;
    g.eps = (float)g.kp * (1.0f / 4194304.0f) * 2.0f;  // kp * 2^-22 * 2: tensor-core accumulation plus the fp32 norms
    g.status = L.status; g.wait_limit = L.wait_limit > 0 ? L.wait_limit : kWaitLimit; g.skip_mma = L.skip_mma;
    const size_t smem = tc_scan_smem(L.dim, L.m, L.k, tn);
    const unsigned grid = scan_grid(L.sm_count, L.reserve_ctas);
    const int dsub = L.dim / L.m;
#define PSB_TC_LAUNCH(D)                                                                                              \
    do {                                                                                                              \
        PSB_CUDA(cudaFuncSetAttribute(k_scan_tc<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));         \
        k_scan_tc<D><<<grid, kTcScanThreads, smem, s>>>(g);                                                           \
    } while (0)
    if (dsub == 2) PSB_TC_LAUNCH(2);
    else if (dsub == 4) PSB_TC_LAUNCH(4);
    else PSB_TC_LAUNCH(8);
#undef PSB_TC_LAUNCH
    count_launch();
    PSB_LAUNCH_CHECK();
    return PSB_OK;
}

namespace {
template <int M>
psb_status run_select_rescore(const RescoreArgs& g, int nq, cudaStream_t s) {
    const size_t smem = (size_t)g.pool_cap * 8 + (g.residual ? (size_t)g.dim * 4 : (size_t)g.m * g.k * 4);
    if (smem > (size_t)226 * 1024) return fail(PSB_UNSUPPORTED_SHAPE, "re-scoring selection does not fit shared memory");
    if (smem > 32 * 1024) PSB_CUDA(cudaFuncSetAttribute(k_select_rescore<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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
    g.counters = L.counters;
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
