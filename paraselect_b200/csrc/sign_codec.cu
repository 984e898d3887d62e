// TurboQuant 1-bit residual codec: random sign flips and a Walsh-Hadamard rotation, one sign bit per rotated dimension and one
// scale per row, and the candidate search over sign-coded lists.
//
//   k_sign_encode   one warp per row.  The reference runs one CTA of padded_dim threads per row with the values in shared
//                   memory and a __syncthreads() per butterfly width (src/quantization/turboquant/turboquant_1bit_encode.cu:
//                   33-110); here lane l holds elements l, l+32, l+64, ... in registers, widths below 32 are lane exchanges and
//                   widths from 32 up are register pairs.  Every butterfly still computes (lhs + rhs, lhs - rhs) on the same
//                   pairs, the per-row statistic goes through the same two shuffle-down trees, so the bits are the same; a row
//                   costs no barrier and the loads of 8 rows per CTA are in flight together.
//   k_sign_scan     one CTA per (query, slice of its probes): rows of the probed lists are scored against the state of their
//                   (query, probe) - one chain over d = 0..dim-1 of +-state[d] for float states, a popcount for sign-coded
//                   ones (src/quantization/turboquant/turboquant_1bit_score.cuh:17-72) - and the candidate_count smallest
//                   (score, row) keys are kept in shared memory: a row enters the buffer only below the current cutoff, a full
//                   buffer is cut back to candidate_count by a radix selection, and the survivors are sorted once at the end.
//                   For float states a table of partial sums gives every row a score with a known error bound first; only
//                   rows that could be below the cutoff get the exact chain (see the kernel).  The reference sorts every
//                   group of 8 chunks of 2,048 rows and merges the groups' lists per query
//                   (turboquant_1bit_grouped_scan.cu:92-190, 45-90); the result, the exact candidate_count smallest keys in
//                   ascending order, is the same.
//   k_sign_merge    joins the slices of one query when its probes were split over several CTAs (few queries).
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace psb {

namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ uint32_t sign_mix(uint32_t v) {   // turboquant_1bit_encode.cu:13-19
    v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu;
    return v ^ (v >> 16);
}

// Lane 0 gets what lane 0 of a warp holds after `for delta = 16..1: v += shfl_down(v, delta)`.
__device__ __forceinline__ float tree32(float v) {
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) v = __fadd_rn(v, __shfl_down_sync(kFull, v, delta));
    return v;
}

// Sum of one value per element in the order of the reference's block reduction: a tree per 32 elements, then the same tree
// over the group sums (zero beyond the last group).  Valid on lane 0.
template <int J>
__device__ __forceinline__ float block_order_sum(const float (&x)[J], int lane) {
    float g = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
        const float t = __shfl_sync(kFull, tree32(x[j]), 0);
        if (lane == j) g = t;
    }
    return tree32(g);
}

// v[j] = element lane + 32 j of the (zero padded) row on entry, of the rotated row on return.
template <int J>
__device__ __forceinline__ void rotate_in_warp(float (&v)[J], int lane, uint32_t seed, float scale) {
#pragma unroll
    for (int j = 0; j < J; ++j)
        if (sign_mix(seed ^ (uint32_t)(lane + 32 * j)) & 1u) v[j] = -v[j];
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const float o = __shfl_xor_sync(kFull, v[j], w);
            v[j] = (lane & w) ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);   // right: lhs - rhs, left: lhs + rhs
        }
    }
#pragma unroll
    for (int wj = 1; wj < J; wj <<= 1) {
#pragma unroll
        for (int j = 0; j < J; ++j)
            if ((j & wj) == 0) {
                const float lhs = v[j], rhs = v[j | wj];
                v[j] = __fadd_rn(lhs, rhs);
                v[j | wj] = __fsub_rn(lhs, rhs);
            }
    }
#pragma unroll
    for (int j = 0; j < J; ++j) v[j] = __fmul_rn(v[j], scale);
}

struct SignEncodeArgs {
    int kind;                    // 0 rows as given, 1 database rows minus their list's centroid, 2 (query, probe) residuals
    const void* rows;            // kind 0/2: fp32 [n][dim] (kind 2: the queries); kind 1: u8 or fp32 rows
    int elem_bytes;              // kind 1: 1 or 4
    long long n;                 // rows / states to encode
    const float* centroids;      // kind 1/2
    const long long* offsets;    // kind 1: [nlist + 1]
    const int* probes;           // kind 2: [n]
    int nlist, nprobe, dim, padded;
    uint32_t seed;
    long long row_offset;        // kind 1: global row of rows[0]
    float* rotated;              // [n][padded] or null
    uint32_t* codes;             // [.][padded / 32] or null
    float* norms;                // kind 0/2: sqrt(sum x^2); kind 1: L1 scale
    float* norm_sq;              // kind 0/2: sum x^2
};

template <int J>
__global__ void __launch_bounds__(256) k_sign_encode(const SignEncodeArgs a) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const float scale = rsqrtf((float)a.padded);   // on the device from a run-time value, as the reference's kernel takes it
    // A warp takes a run of consecutive rows: consecutive database rows mostly share a list, whose bounds are then at hand.
    const long long per_warp = (a.n + nwarps - 1) / nwarps;
    const long long r_end = min(a.n, (warp0 + 1) * per_warp);
    int held_list = 0;
    long long held_beg = 0, held_end = -1;
    for (long long r = warp0 * per_warp; r < r_end; ++r) {
        long long out_row = r;
        const float* cen = nullptr;
        const float* src_f = nullptr;
        const unsigned char* src_b = nullptr;
        bool live = true;
        if (a.kind == 0) {
            src_f = static_cast<const float*>(a.rows) + (size_t)r * a.dim;
        } else if (a.kind == 1) {
            out_row = r + a.row_offset;
            if (out_row < held_beg || out_row >= held_end) {
                int lo = 0, hi = a.nlist;   // the list of the global row (turboquant_1bit_encode.cu:21-31)
                while (lo + 1 < hi) {
                    const int mid = lo + (hi - lo) / 2;
                    if (a.offsets[mid] <= out_row) lo = mid; else hi = mid;
                }
                held_list = lo; held_beg = a.offsets[lo]; held_end = a.offsets[lo + 1];
            }
            cen = a.centroids + (size_t)held_list * a.dim;
            if (a.elem_bytes == 1) src_b = static_cast<const unsigned char*>(a.rows) + (size_t)r * a.dim;
            else src_f = static_cast<const float*>(a.rows) + (size_t)r * a.dim;
        } else {
            const int list = a.probes[r];
            live = list >= 0 && list < a.nlist;
            src_f = static_cast<const float*>(a.rows) + (size_t)(r / a.nprobe) * a.dim;
            cen = a.centroids + (size_t)(live ? list : 0) * a.dim;
        }
        float v[J], stat[J];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int d = lane + 32 * j;
            float x = 0.f;
            if (live && d < a.dim) {
                x = src_b ? (float)src_b[d] : src_f[d];
                if (cen) x = __fsub_rn(x, cen[d]);
            }
            v[j] = x;
            stat[j] = __fmul_rn(x, x);
        }
        rotate_in_warp<J>(v, lane, a.seed, scale);
#pragma unroll
        for (int j = 0; j < J; ++j) {
            if (a.rotated) a.rotated[(size_t)out_row * (32 * J) + lane + 32 * j] = v[j];
            const unsigned word = __ballot_sync(kFull, v[j] >= 0.0f);
            if (a.codes && lane == 0) a.codes[(size_t)out_row * J + j] = word;
            if (a.kind == 1) stat[j] = fabsf(v[j]);
        }
        if (a.norms || a.norm_sq) {   // uniform
            const float sum = block_order_sum<J>(stat, lane);
            if (lane == 0) {
                if (a.kind == 1) {
                    if (a.norms) a.norms[out_row] = __fdiv_rn(sum, (float)(32 * J));
                } else {
                    if (a.norm_sq) a.norm_sq[out_row] = sum;
                    if (a.norms) a.norms[out_row] = __fsqrt_rn(sum);
                }
            }
        }
    }
}

// The same encoding with one row per THREAD, for padded_dim <= 128 and rows whose length is a multiple of four elements: the
// whole (zero padded) row sits in registers, every butterfly is two register operations and nothing is exchanged between
// lanes (the warp-per-row kernel above spends 49 shuffles per row).  Every value goes through the same operations on the
// same operands - the sign flip, the (lhs + rhs, lhs - rhs) pairs width by width, the scale, the two reduction trees of the
// statistic taken as register trees - so the bits are the same.  A thread reads its row with 16-byte (fp32) or 4-byte (u8)
// loads; the row is a run of whole sectors, read once.
constexpr int kLaneEncThreads = 128;

// What lane 0 of a warp would hold after the shuffle-down tree over t[0..32): t[p] += t[p + delta], delta = 16 .. 1.
__device__ __forceinline__ float tree32_regs(float (&t)[32]) {
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) {
#pragma unroll
        for (int p = 0; p < delta; ++p) t[p] = __fadd_rn(t[p], t[p + delta]);
    }
    return t[0];
}

template <int P>
__global__ void __launch_bounds__(kLaneEncThreads, 2) k_sign_encode_lane(const SignEncodeArgs a) {
    __shared__ uint32_t s_flip[P];   // 0x80000000 where the rotation flips the sign of dimension d
    for (int d = threadIdx.x; d < P; d += kLaneEncThreads) s_flip[d] = (sign_mix(a.seed ^ (uint32_t)d) & 1u) ? 0x80000000u : 0u;
    __syncthreads();
    const float scale = rsqrtf((float)a.padded);   // on the device from a run-time value, as the reference's kernel takes it
    const int dim4 = a.dim >> 2;
    // A thread takes a run of consecutive rows: consecutive database rows mostly share a list, whose bounds are then at hand
    // (the search is 16 dependent loads).
    const long long threads = (long long)gridDim.x * kLaneEncThreads;
    const long long per_thread = (a.n + threads - 1) / threads;
    const long long r_begin = ((long long)blockIdx.x * kLaneEncThreads + threadIdx.x) * per_thread;
    const long long r_end = min(a.n, r_begin + per_thread);
    int held_list = 0;
    long long held_beg = 0, held_end = -1;
    const bool bytes16 = (a.dim & 15) == 0 && (reinterpret_cast<uintptr_t>(a.rows) & 15) == 0;   // u8 rows in 16-byte loads
    for (long long r = r_begin; r < r_end; ++r) {
        long long out_row = r;
        const float* cen = nullptr;
        const float* src_f = nullptr;
        const unsigned char* src_b = nullptr;
        bool live = true;
        if (a.kind == 0) {
            src_f = static_cast<const float*>(a.rows) + (size_t)r * a.dim;
        } else if (a.kind == 1) {
            out_row = r + a.row_offset;
            if (out_row < held_beg || out_row >= held_end) {
                int lo = 0, hi = a.nlist;   // the list of the global row (turboquant_1bit_encode.cu:21-31)
                while (lo + 1 < hi) {
                    const int mid = lo + (hi - lo) / 2;
                    if (a.offsets[mid] <= out_row) lo = mid; else hi = mid;
                }
                held_list = lo; held_beg = a.offsets[lo]; held_end = a.offsets[lo + 1];
            }
            cen = a.centroids + (size_t)held_list * a.dim;
            if (a.elem_bytes == 1) src_b = static_cast<const unsigned char*>(a.rows) + (size_t)r * a.dim;
            else src_f = static_cast<const float*>(a.rows) + (size_t)r * a.dim;
        } else {
            const int list = a.probes[r];
            live = list >= 0 && list < a.nlist;
            src_f = static_cast<const float*>(a.rows) + (size_t)(r / a.nprobe) * a.dim;
            cen = a.centroids + (size_t)(live ? list : 0) * a.dim;
        }
        float v[P];
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int d4 = 0; d4 < P / 4; ++d4) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live && d4 < dim4) {
                if (src_b) {
                    uint32_t word;
                    if (bytes16) {   // uniform; the 16-byte load of group d4 / 4 serves four passes of this loop
                        if ((d4 & 3) == 0) packed = __ldg(reinterpret_cast<const uint4*>(src_b) + (d4 >> 2));
                        word = (d4 & 3) == 0 ? packed.x : (d4 & 3) == 1 ? packed.y : (d4 & 3) == 2 ? packed.z : packed.w;
                    } else {
                        word = __ldg(reinterpret_cast<const uint32_t*>(src_b) + d4);
                    }
                    x = make_float4((float)(word & 255u), (float)((word >> 8) & 255u), (float)((word >> 16) & 255u), (float)(word >> 24));
                } else {
                    x = __ldg(reinterpret_cast<const float4*>(src_f) + d4);
                }
                if (cen) {
                    const float4 c = __ldg(reinterpret_cast<const float4*>(cen) + d4);
                    x.x = __fsub_rn(x.x, c.x); x.y = __fsub_rn(x.y, c.y); x.z = __fsub_rn(x.z, c.z); x.w = __fsub_rn(x.w, c.w);
                }
            }
            v[4 * d4] = x.x; v[4 * d4 + 1] = x.y; v[4 * d4 + 2] = x.z; v[4 * d4 + 3] = x.w;
        }
        float sum = 0.f;
        if (a.kind != 1 && (a.norms || a.norm_sq)) {   // sum of squares of the row as given, group trees then the tree over groups
            float g[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) g[i] = 0.f;
#pragma unroll
            for (int w = 0; w < P / 32; ++w) {
                float t[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) t[i] = __fmul_rn(v[32 * w + i], v[32 * w + i]);
                g[w] = tree32_regs(t);
            }
            sum = tree32_regs(g);
        }
#pragma unroll
        for (int d = 0; d < P; ++d) v[d] = __uint_as_float(__float_as_uint(v[d]) ^ s_flip[d]);
#pragma unroll
        for (int width = 1; width < P; width <<= 1) {
#pragma unroll
            for (int t = 0; t < P / 2; ++t) {
                const int left = (t / width) * (width << 1) + (t % width), right = left + width;
                const float lhs = v[left], rhs = v[right];
                v[left] = __fadd_rn(lhs, rhs);
                v[right] = __fsub_rn(lhs, rhs);
            }
        }
#pragma unroll
        for (int d = 0; d < P; ++d) v[d] = __fmul_rn(v[d], scale);
        if (a.rotated) {
            float4* out = reinterpret_cast<float4*>(a.rotated + (size_t)out_row * P);
#pragma unroll
            for (int d4 = 0; d4 < P / 4; ++d4) out[d4] = make_float4(v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
        }
        if (a.codes) {
#pragma unroll
            for (int w = 0; w < P / 32; ++w) {
                uint32_t word = 0u;
#pragma unroll
                for (int b = 0; b < 32; ++b) word |= v[32 * w + b] >= 0.0f ? (1u << b) : 0u;
                a.codes[(size_t)out_row * (P / 32) + w] = word;
            }
        }
        if (a.kind == 1) {
            if (a.norms) {
                float g[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) g[i] = 0.f;
#pragma unroll
                for (int w = 0; w < P / 32; ++w) {
                    float t[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) t[i] = fabsf(v[32 * w + i]);
                    g[w] = tree32_regs(t);
                }
                a.norms[out_row] = __fdiv_rn(tree32_regs(g), (float)P);
            }
        } else {
            if (a.norm_sq) a.norm_sq[out_row] = sum;
            if (a.norms) a.norms[out_row] = __fsqrt_rn(sum);
        }
    }
}

__global__ void k_sign_scale(int padded, float* out) { *out = rsqrtf((float)padded); }

// ---- candidate search ------------------------------------------------------------------------------------------

constexpr int kScanThreads = 256;
constexpr int kScanRows = 4;                      // rows per thread per step
constexpr int kScanStep = kScanThreads * kScanRows;
constexpr int kSignMaxCandidates = 8192;
constexpr int kMergeMaxKeys = 16384;

struct SignScanArgs {
    const float* states;          // float states [nq * nprobe][dim]
    const float* norm_sq;         // [nq * nprobe]
    const uint32_t* state_codes;  // sign-coded states [nq * nprobe][dim / 32]
    const float* norms;           // [nq * nprobe]
    const uint32_t* codes;        // [rows][dim / 32]
    const float* row_params;      // [rows]: reconstruction scale (float states) or norm (sign-coded states)
    const long long* offsets;     // [nlist + 1]
    const int* probes;            // [nq][nprobe]
    int nlist, nq, nprobe, dim, k, kp2, cap, split;
    uint64_t* partial;            // [nq][split][k] when split > 1
    int* rows_out;                // [nq][k]
    float* dist_out;              // [nq][k] or null
};

template <int W> struct CodeWords { uint32_t w[W]; };

template <int W>
__device__ __forceinline__ CodeWords<W> load_code(const uint32_t* __restrict__ codes, long long row) {
    CodeWords<W> c;
    if constexpr (W == 1) {
        c.w[0] = __ldg(codes + row);
    } else if constexpr (W == 2) {
        const uint2 t = __ldg(reinterpret_cast<const uint2*>(codes) + row);
        c.w[0] = t.x; c.w[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < W / 4; ++i) {
            const uint4 t = __ldg(reinterpret_cast<const uint4*>(codes) + row * (W / 4) + i);
            c.w[4 * i] = t.x; c.w[4 * i + 1] = t.y; c.w[4 * i + 2] = t.z; c.w[4 * i + 3] = t.w;
        }
    }
    return c;
}

// dot + v when the sign bit is set, dot - v when it is clear: one bit test into a predicate and two predicated adds.  Building
// +-v with a shift and an exclusive-or instead costs two integer operations per dimension, which run at half the rate of the
// adds; measured, this form is the faster of the two by a few percent.
__device__ __forceinline__ float sign_step(float dot, float v, uint32_t word, uint32_t mask) {
    asm("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t"
        "and.b32 t, %1, %2;\n\t"
        "setp.ne.u32 p, t, 0;\n\t"
        "@p add.rn.f32 %0, %0, %3;\n\t"
        "@!p sub.rn.f32 %0, %0, %3;\n\t}"
        : "+f"(dot)
        : "r"(word), "r"(mask), "f"(v));
    return dot;
}

// Shared scratch of the selection: a 256-bin histogram, the warp sums of its scan, and a few words.
struct SignSelectScratch {
    int hist[256];
    int warp_sums[32];
    int bucket, need, moved, filled;
    unsigned long long differ;
};

// Cuts the buffer back to its k smallest keys, keys[0..k) in no particular order, and moves the cutoff to the k-th smallest.
// A radix selection over the bytes of the keys (most significant first, bytes that all keys share skipped) finds the k-th
// key in a few passes over the buffer; keys beyond position k that stay are parked in `spill` and dropped into the places of
// keys within the first k that go.  A full sort of the buffer here cost two thirds of the instructions of the popcount scan
// and a fifth of those of the float scan.  Called by all threads of the CTA (blockDim.x == 256).
__device__ __forceinline__ void sign_compact(uint64_t* keys, uint64_t* spill, int k, int* s_cnt, unsigned long long* s_thr,
                                             SignSelectScratch* sc) {
    const int n = *s_cnt;
    const int tid = threadIdx.x;
    __syncthreads();
    if (n <= k) return;   // uniform
    if (tid == 0) sc->differ = 0ull;
    __syncthreads();
    const uint64_t first = keys[0];
    uint64_t diff = 0;
    for (int i = tid; i < n; i += kScanThreads) diff |= keys[i] ^ first;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) diff |= __shfl_xor_sync(kFull, diff, o);
    if ((tid & 31) == 0 && diff) atomicOr(&sc->differ, (unsigned long long)diff);
    __syncthreads();
    const unsigned long long differ = sc->differ;
    // keys are distinct unless a query names a list twice; all equal: any k of them will do
    int shift = differ ? 56 - 8 * (__clzll((long long)differ) / 8) : -8;
    uint64_t prefix = shift >= 0 && shift < 56 ? first & (~0ull << (shift + 8)) : 0ull;
    int need = k;
    for (; shift >= 0; shift -= 8) {
        sc->hist[tid] = 0;
        __syncthreads();
        const uint64_t above = shift == 56 ? 0ull : ~0ull << (shift + 8);
        for (int i = tid; i < n; i += kScanThreads) {
            const uint64_t key = keys[i];
            if ((key & above) == prefix) atomicAdd(&sc->hist[(int)((key >> shift) & 255u)], 1);
        }
        __syncthreads();
        const int c = sc->hist[tid];
        const int before = block_exclusive_scan(c, sc->warp_sums, nullptr);
        if (before < need && need <= before + c) { sc->bucket = tid; sc->need = need - before; }
        __syncthreads();
        prefix |= (uint64_t)sc->bucket << shift;
        need = sc->need;
        __syncthreads();
    }
    const uint64_t kth = differ ? prefix : first;
    if (tid == 0) { sc->moved = 0; sc->filled = 0; }
    __syncthreads();
    // keys below the k-th first, then keys equal to it (more than one only when a query names a list twice): the places that
    // come free go to the parked keys in this order
    for (int pass = 0; pass < 2; ++pass) {
        for (int i = k + tid; i < n; i += kScanThreads) {
            const uint64_t key = keys[i];
            if (pass == 0 ? key < kth : key == kth) {
                const int pos = atomicAdd(&sc->moved, 1);
                if (pos < k) spill[pos] = key;
            }
        }
        __syncthreads();
    }
    const int moved = sc->moved < k ? sc->moved : k;
    for (int j = tid; j < k; j += kScanThreads) {
        if (keys[j] > kth) {
            const int pos = atomicAdd(&sc->filled, 1);
            keys[j] = pos < moved ? spill[pos] : KEY_MAX;   // pos < moved always, for distinct keys
        }
    }
    if (tid == 0) { *s_cnt = k; *s_thr = kth; }
    __syncthreads();
}

// The kept keys in ascending order in keys[0..n), n = min(held, k).
__device__ __forceinline__ int sign_finish(uint64_t* keys, uint64_t* spill, int k, int kp2, int* s_cnt, unsigned long long* s_thr,
                                           SignSelectScratch* sc) {
    sign_compact(keys, spill, k, s_cnt, s_thr, sc);
    const int n = *s_cnt;
    __syncthreads();
    for (int i = n + threadIdx.x; i < kp2; i += kScanThreads) keys[i] = KEY_MAX;
    __syncthreads();
    block_bitonic_sort(keys, kp2);
    return n;
}

// The exact scores of up to kScanRows rows per thread, each against the float state `state[r]` points to (global memory: the
// rows of a thread may belong to different probes): one chain over d = 0..dim-1 per row, the chains interleaved.
template <int W>
__device__ __forceinline__ void exact_float_scores(const CodeWords<W> (&c)[kScanRows], const float (&param)[kScanRows],
                                                   const float* const (&state)[kScanRows], const float (&norm_sq)[kScanRows],
                                                   float (&score)[kScanRows]) {
    float dot[kScanRows];
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) dot[r] = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
#pragma unroll
        for (int bit = 0; bit < 32; ++bit) {
#pragma unroll
            for (int r = 0; r < kScanRows; ++r) dot[r] = sign_step(dot[r], __ldg(state[r] + 32 * w + bit), c[r].w[w], 1u << bit);
        }
    }
    const float dimf = (float)(32 * W);
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) {
        const float s = param[r];
        score[r] = __fmaf_rn(-__fmul_rn(2.0f, s), dot[r], __fmaf_rn(__fmul_rn(dimf, s), s, norm_sq[r]));
    }
}

// The signed sum of a row from a table of the 16 possible sums of every group of four dimensions: dim / 4 look-ups instead of
// dim additions.  The order of the additions differs from the chain's, so the value may differ from the exact dot in the last
// bits; the caller allows for that.  lut[g * 16 + v], v = the four sign bits of group g: the 16 entries of a group lie in 16
// different banks, so a warp's look-ups never collide.
template <int W>
__device__ __forceinline__ float table_dot(const CodeWords<W>& c, const float* lut) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const uint32_t word = c.w[w];
#pragma unroll
        for (int t = 0; t < 8; t += 2) {
            a0 += lut[(8 * w + t) * 16 + ((word >> (4 * t)) & 15u)];
            a1 += lut[(8 * w + t + 1) * 16 + ((word >> (4 * t + 4)) & 15u)];
        }
    }
    return a0 + a1;
}

constexpr int kQueueCap = 2 * kScanStep;   // rows waiting for their exact score

// Scan of one (query, slice of probes) per CTA.
//
// Sign-coded states (MODE 1): every row's score is a popcount; keys below the cutoff go to the buffer.
//
// Float states (MODE 0): a row's score is first taken from the table (table_dot), and only rows whose score could still be
// below the cutoff - the table score minus a bound on its error against the exact chain - are queued, (row, probe), for the
// exact chain.  The queue is worked off 1,024 rows at a time, four interleaved chains per thread on all threads, whenever it
// holds that many (and once at the end), so the chains - 128 dependent additions each - always run with full warps.  Until
// the first cutoff exists every row is queued.  A queued row is tested against the cutoff of the time its exact score is
// taken; cutoffs only fall, so nothing is lost by waiting.
// Error bound of the table score: with A = sum |state[d]|, every partial sum on either path is at most A in magnitude and
// every rounding at most 2^-24 of it; the chain has dim <= 256 roundings, the table path fewer than 80 (3 per entry,
// dim / 4 + 1 additions), so |table - chain| < 336 * 2^-24 * A < 2^-15 * A for every dim here.  The queue test uses
// 2^-14 * A (twice that) on the dot and 2^-20 relative on the final fused multiply-adds.
template <int W, int MODE>
__global__ void __launch_bounds__(kScanThreads, W > 4 ? 2 : (MODE == 1 ? 6 : 4)) k_sign_scan(const SignScanArgs a) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(s_raw);
    uint64_t* spill = keys + a.cap;                                       // k keys
    float* s_state = reinterpret_cast<float*>(spill + ((a.k + 1) & ~1));  // 256 floats: the state (MODE 0), 16-byte aligned
    float* s_lut = s_state + 256;                                         // W * 128 floats: the table (MODE 0)
    __shared__ SignSelectScratch s_sel;
    __shared__ uint32_t s_qrow[MODE == 0 ? kQueueCap : 1];
    __shared__ uint16_t s_qprobe[MODE == 0 ? kQueueCap : 1];
    __shared__ int s_qn;
    __shared__ int s_cnt;
    __shared__ unsigned long long s_thr;
    const int q = blockIdx.x / a.split, slice = blockIdx.x % a.split;
    const int tid = threadIdx.x;
    const float dimf = (float)(32 * W);
    if (tid == 0) { s_cnt = 0; s_thr = KEY_MAX; s_qn = 0; }
    __syncthreads();

    // MODE 0: takes the exact scores of queued rows, 1,024 per round; with `all` also the last, partial round.  Called by
    // all threads after a barrier that follows the last append to the queue.
    auto work_off_queue = [&](bool all) {
        const int queued = s_qn;
        int done = 0;
        while (queued - done >= (all ? 1 : kScanStep)) {
            const int take = min(kScanStep, queued - done);
            const int held = s_cnt;
            __syncthreads();
            if (held > a.cap - kScanStep) sign_compact(keys, spill, a.k, &s_cnt, &s_thr, &s_sel);   // uniform
            const unsigned long long thr = s_thr;
            CodeWords<W> c[kScanRows];
            float param[kScanRows], norm_sq[kScanRows], score[kScanRows];
            const float* state[kScanRows];
            uint32_t row[kScanRows];
            bool ok[kScanRows];
#pragma unroll
            for (int r = 0; r < kScanRows; ++r) {   // four consecutive entries per thread: whole warps work or rest
                const int at = kScanRows * tid + r;
                ok[r] = at < take;
                row[r] = 0u; param[r] = 0.f; norm_sq[r] = 0.f; state[r] = a.states;
#pragma unroll
                for (int w = 0; w < W; ++w) c[r].w[w] = 0u;
                if (ok[r]) {
                    row[r] = s_qrow[done + at];
                    const long long st = (long long)q * a.nprobe + s_qprobe[done + at];
                    c[r] = load_code<W>(a.codes, row[r]);
                    param[r] = __ldg(a.row_params + row[r]);
                    norm_sq[r] = __ldg(a.norm_sq + st);
                    state[r] = a.states + (size_t)st * (32 * W);
                }
            }
            if (ok[0]) {
                exact_float_scores<W>(c, param, state, norm_sq, score);
#pragma unroll
                for (int r = 0; r < kScanRows; ++r) {
                    if (!ok[r]) continue;
                    const uint64_t key = make_key(score[r], row[r]);
                    if (key < thr) keys[atomicAdd(&s_cnt, 1)] = key;   // room for a whole round was made above
                }
            }
            __syncthreads();
            done += take;
        }
        const int rest = queued - done;   // < 1,024 <= done whenever done > 0: source and destination do not overlap
        if (done > 0) {
            for (int i = tid; i < rest; i += kScanThreads) { s_qrow[i] = s_qrow[done + i]; s_qprobe[i] = s_qprobe[done + i]; }
            __syncthreads();
            if (tid == 0) s_qn = rest;
            __syncthreads();
        }
    };

    for (int p = slice; p < a.nprobe; p += a.split) {
        const long long st = (long long)q * a.nprobe + p;
        const int list = a.probes[st];
        if (list < 0 || list >= a.nlist) continue;   // uniform
        __syncthreads();
        float abs_sum = 0.f;   // MODE 0: sum |state[d]|, rounded up a little
        uint32_t qcode[W];     // MODE 1: the state's sign words
        if (MODE == 0) {
            for (int d = tid; d < 32 * W; d += kScanThreads) s_state[d] = a.states[(size_t)st * (32 * W) + d];
            __syncthreads();
            for (int e = tid; e < W * 128; e += kScanThreads) {   // entry v of group g: ((+-x0 +- x1) +- x2) +- x3
                const int g = e >> 4, v = e & 15;
                const float* x = s_state + 4 * g;
                float t = (v & 1) ? x[0] : -x[0];
                t += (v & 2) ? x[1] : -x[1];
                t += (v & 4) ? x[2] : -x[2];
                t += (v & 8) ? x[3] : -x[3];
                s_lut[e] = t;
            }
            const int lane = tid & 31;
#pragma unroll
            for (int j = 0; j < W; ++j) abs_sum += fabsf(s_state[lane + 32 * j]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) abs_sum += __shfl_xor_sync(kFull, abs_sum, o);
            abs_sum *= 1.001f;
        }
#pragma unroll
        for (int w = 0; w < W; ++w) qcode[w] = MODE == 1 ? __ldg(a.state_codes + (size_t)st * W + w) : 0u;   // same in every thread
        const float qparam = MODE == 0 ? a.norm_sq[st] : a.norms[st];
        __syncthreads();
        const long long beg = a.offsets[list], end = a.offsets[list + 1];
        for (long long row0 = beg; row0 < end; row0 += kScanStep) {
            unsigned long long thr;
            if (MODE == 1) {
                const int held = s_cnt;   // settled: the previous step ended with a barrier
                __syncthreads();          // ... and nobody appends before everybody has read it
                if (held > a.cap - kScanStep) sign_compact(keys, spill, a.k, &s_cnt, &s_thr, &s_sel);   // uniform
            }
            thr = s_thr;   // MODE 0: changed only inside work_off_queue, between barriers
            CodeWords<W> c[kScanRows];
            float param[kScanRows];
            bool ok[kScanRows];
            long long rows[kScanRows];
#pragma unroll
            for (int r = 0; r < kScanRows; ++r) {
                rows[r] = row0 + r * kScanThreads + tid;
                ok[r] = rows[r] < end;
                if (ok[r]) { c[r] = load_code<W>(a.codes, rows[r]); param[r] = __ldg(a.row_params + rows[r]); }
                else {
#pragma unroll
                    for (int w = 0; w < W; ++w) c[r].w[w] = 0u;
                    param[r] = 0.f;
                }
            }
            if (MODE == 0) {
                const bool have_cut = thr != KEY_MAX;   // uniform
                const float cut = key_dist(thr);
                const float dot_slack = abs_sum * (1.0f / 16384.0f);
                bool filled = false;   // one of this thread's rows took the queue's 1,024th place
#pragma unroll
                for (int r = 0; r < kScanRows; ++r) {
                    if (!ok[r]) continue;
                    bool queue = true;
                    if (have_cut) {
                        const float s = param[r], two_s = fabsf(2.0f * s);
                        const float base = __fmaf_rn(__fmul_rn(dimf, s), s, qparam);
                        const float rough = __fmaf_rn(-__fmul_rn(2.0f, s), table_dot<W>(c[r], s_lut), base);
                        const float slack = two_s * dot_slack + (fabsf(base) + two_s * abs_sum) * (1.0f / 1048576.0f);
                        queue = !(rough - slack > cut);   // NaN queues too
                    }
                    if (queue) {
                        const int at = atomicAdd(&s_qn, 1);   // at most 1,024 join a queue that held fewer than 1,024
                        s_qrow[at] = (uint32_t)rows[r];
                        s_qprobe[at] = (uint16_t)p;
                        filled |= at == kScanStep - 1;
                    }
                }
                // The queue held fewer than 1,024 rows before this step, so it holds that many now exactly when that place
                // was taken in this step: every thread learns it from the barrier itself (reading the counter after the
                // barrier would race with the next step's appends).
                if (__syncthreads_or(filled)) work_off_queue(false);
            } else {
#pragma unroll
                for (int r = 0; r < kScanRows; ++r) {
                    if (!ok[r]) continue;
                    int h = 0;
#pragma unroll
                    for (int w = 0; w < W; ++w) h += __popc(qcode[w] ^ c[r].w[w]);
                    const float cosine = __fdiv_rn(__fsub_rn(dimf, __fmul_rn(2.0f, (float)h)), dimf);
                    const float dn = param[r];
                    const float score = __fmaf_rn(-__fmul_rn(__fmul_rn(2.0f, qparam), dn), cosine, __fmaf_rn(dn, dn, __fmul_rn(qparam, qparam)));
                    const uint64_t key = make_key(score, (uint32_t)rows[r]);
                    if (key < thr) keys[atomicAdd(&s_cnt, 1)] = key;   // room for a whole step was checked above
                }
                __syncthreads();
            }
        }
    }
    __syncthreads();
    if (MODE == 0) work_off_queue(true);
    const int n = sign_finish(keys, spill, a.k, a.kp2, &s_cnt, &s_thr, &s_sel);
    if (a.split > 1) {
        uint64_t* out = a.partial + ((size_t)q * a.split + slice) * a.k;
        for (int i = tid; i < a.k; i += kScanThreads) out[i] = i < n ? keys[i] : KEY_MAX;
    } else {
        for (int i = tid; i < a.k; i += kScanThreads) {
            a.rows_out[(size_t)q * a.k + i] = i < n ? (int)key_idx(keys[i]) : -1;
            if (a.dist_out) a.dist_out[(size_t)q * a.k + i] = i < n ? key_dist(keys[i]) : FLT_MAX;
        }
    }
}

__global__ void __launch_bounds__(kScanThreads) k_sign_merge(const uint64_t* __restrict__ partial, int split, int k, int cap,
                                                             int* __restrict__ rows_out, float* __restrict__ dist_out) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(s_raw);
    const int q = blockIdx.x, n = split * k;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) keys[i] = i < n ? partial[(size_t)q * n + i] : KEY_MAX;
    __syncthreads();
    block_bitonic_sort(keys, cap);
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const uint64_t key = keys[i];
        rows_out[(size_t)q * k + i] = key == KEY_MAX ? -1 : (int)key_idx(key);
        if (dist_out) dist_out[(size_t)q * k + i] = key == KEY_MAX ? FLT_MAX : key_dist(key);
    }
}

int pow2_at_least(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

template <int J>
psb_status run_encode(const SignEncodeArgs& a, int sm_count, cudaStream_t s) {
    const long long ctas = std::min<long long>((a.n + 7) / 8, (long long)sm_count * 16);
    k_sign_encode<J><<<(unsigned)ctas, 256, 0, s>>>(a);
    PSB_LAUNCH_CHECK();
    count_launch();
    return PSB_OK;
}

template <int P>
psb_status run_encode_lane(const SignEncodeArgs& a, int sm_count, cudaStream_t s) {
    const long long ctas = std::min<long long>((a.n + kLaneEncThreads - 1) / kLaneEncThreads, (long long)sm_count * 8);
    k_sign_encode_lane<P><<<(unsigned)ctas, kLaneEncThreads, 0, s>>>(a);
    PSB_LAUNCH_CHECK();
    count_launch();
    return PSB_OK;
}

psb_status dispatch_encode(const SignEncodeArgs& args, int padded, int sm_count, cudaStream_t s) {
    if (args.n <= 0) return PSB_OK;
    SignEncodeArgs a = args;
    a.padded = padded;
    // one row per thread where the row fits the registers and its loads can be 16 (fp32) / 4 (u8) bytes wide
    const bool u8 = a.kind == 1 && a.elem_bytes == 1;
    const bool wide = a.dim % 4 == 0 && reinterpret_cast<uintptr_t>(a.rows) % (u8 ? 4 : 16) == 0 &&
                      (!a.centroids || reinterpret_cast<uintptr_t>(a.centroids) % 16 == 0) &&
                      (!a.rotated || reinterpret_cast<uintptr_t>(a.rotated) % 16 == 0);
    if (wide && padded <= 128) {
        switch (padded) {
            case 32: return run_encode_lane<32>(a, sm_count, s);
            case 64: return run_encode_lane<64>(a, sm_count, s);
            case 128: return run_encode_lane<128>(a, sm_count, s);
        }
    }
    switch (padded) {
        case 32: return run_encode<1>(a, sm_count, s);
        case 64: return run_encode<2>(a, sm_count, s);
        case 128: return run_encode<4>(a, sm_count, s);
        case 256: return run_encode<8>(a, sm_count, s);
    }
    return fail(PSB_INVALID_ARGUMENT, "padded_dim must be 32, 64, 128 or 256");
}

template <int W, int MODE>
psb_status run_scan(const SignScanArgs& a, size_t smem, cudaStream_t s) {
    PSB_TRY(prefer_max_shared(k_sign_scan<W, MODE>));
    PSB_CUDA(cudaFuncSetAttribute(k_sign_scan<W, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_sign_scan<W, MODE><<<(unsigned)(a.nq * a.split), kScanThreads, smem, s>>>(a);
    PSB_LAUNCH_CHECK();
    count_launch();
    return PSB_OK;
}

template <int MODE>
psb_status dispatch_scan(const SignScanArgs& a, size_t smem, cudaStream_t s) {
    switch (a.dim) {
        case 32: return run_scan<1, MODE>(a, smem, s);
        case 64: return run_scan<2, MODE>(a, smem, s);
        case 128: return run_scan<4, MODE>(a, smem, s);
        case 256: return run_scan<8, MODE>(a, smem, s);
    }
    return fail(PSB_INVALID_ARGUMENT, "padded_dim must be 32, 64, 128 or 256");
}

bool sign_shape_ok(int dim, int padded) {
    return dim > 0 && dim <= padded && (padded == 32 || padded == 64 || padded == 128 || padded == 256);
}

}  // namespace

int sign_padded_dim(int dim) {   // src/search/ivf_res_turboquant/ivf_res_turboquant_search.cu:24-29
    if (dim <= 0) return -1;
    int p = 32;
    while (p < dim) p <<= 1;
    return p > 256 ? -1 : p;
}

psb_status launch_sign_scale(int padded_dim, float* d_out, cudaStream_t s) {
    k_sign_scale<<<1, 1, 0, s>>>(padded_dim, d_out);
    PSB_LAUNCH_CHECK();
    count_launch();
    return PSB_OK;
}

psb_status launch_sign_rotate(const float* d_rows, long long n, int dim, int padded_dim, uint32_t seed, float* d_rotated,
                              uint32_t* d_codes, float* d_norms, float* d_norm_sq, int sm_count, cudaStream_t s) {
    if (!sign_shape_ok(dim, padded_dim)) return fail(PSB_INVALID_ARGUMENT, "sign codec: dim must be in 1..padded_dim, padded_dim 32, 64, 128 or 256");
    SignEncodeArgs a{};
    a.kind = 0; a.rows = d_rows; a.n = n; a.dim = dim; a.seed = seed;
    a.rotated = d_rotated; a.codes = d_codes; a.norms = d_norms; a.norm_sq = d_norm_sq;
    return dispatch_encode(a, padded_dim, sm_count, s);
}

psb_status launch_sign_encode_database(const void* d_rows, int elem_bytes, long long n, const float* d_centroids,
                                       const long long* d_offsets, int nlist, int dim, int padded_dim, uint32_t seed,
                                       long long row_offset, uint32_t* d_codes, float* d_scales, int sm_count, cudaStream_t s) {
    if (!sign_shape_ok(dim, padded_dim)) return fail(PSB_INVALID_ARGUMENT, "sign codec: dim must be in 1..padded_dim, padded_dim 32, 64, 128 or 256");
    SignEncodeArgs a{};
    a.kind = 1; a.rows = d_rows; a.elem_bytes = elem_bytes; a.n = n; a.centroids = d_centroids; a.offsets = d_offsets;
    a.nlist = nlist; a.dim = dim; a.seed = seed; a.row_offset = row_offset; a.codes = d_codes; a.norms = d_scales;
    return dispatch_encode(a, padded_dim, sm_count, s);
}

psb_status launch_sign_encode_queries(const float* d_queries, const float* d_centroids, const int* d_probes, int nq, int nprobe,
                                      int nlist, int dim, int padded_dim, uint32_t seed, float* d_states, float* d_norm_sq,
                                      uint32_t* d_state_codes, float* d_norms, int sm_count, cudaStream_t s) {
    if (!sign_shape_ok(dim, padded_dim)) return fail(PSB_INVALID_ARGUMENT, "sign codec: dim must be in 1..padded_dim, padded_dim 32, 64, 128 or 256");
    SignEncodeArgs a{};
    a.kind = 2; a.rows = d_queries; a.n = (long long)nq * nprobe; a.centroids = d_centroids; a.probes = d_probes;
    a.nlist = nlist; a.nprobe = nprobe; a.dim = dim; a.seed = seed;
    a.rotated = d_states; a.codes = d_state_codes; a.norms = d_norms; a.norm_sq = d_norm_sq;
    return dispatch_encode(a, padded_dim, sm_count, s);
}

psb_status launch_sign_candidates(int mode, const float* d_states, const float* d_norm_sq, const uint32_t* d_state_codes,
                                  const float* d_norms, const uint32_t* d_codes, const float* d_row_params,
                                  const long long* d_offsets, int nlist, const int* d_probes, int nq, int nprobe, int padded_dim,
                                  int candidate_count, int* d_rows_out, float* d_dist_out, int sm_count, cudaStream_t s) {
    if (!sign_shape_ok(padded_dim, padded_dim)) return fail(PSB_INVALID_ARGUMENT, "sign codec: padded_dim must be 32, 64, 128 or 256");
    if (nprobe > 65535) return fail(PSB_INVALID_ARGUMENT, "sign codec: at most 65,535 probes per query");
    if (candidate_count <= 0 || candidate_count > kSignMaxCandidates)
        return fail(PSB_INVALID_ARGUMENT, "sign codec: candidate_count must be in 1..8192");
    if (reinterpret_cast<uintptr_t>(d_codes) % 16) return fail(PSB_INVALID_ARGUMENT, "sign codec: the code array must be 16-byte aligned");
    if (nq <= 0) return PSB_OK;
    SignScanArgs a{};
    a.states = d_states; a.norm_sq = d_norm_sq; a.state_codes = d_state_codes; a.norms = d_norms;
    a.codes = d_codes; a.row_params = d_row_params; a.offsets = d_offsets; a.probes = d_probes;
    a.nlist = nlist; a.nq = nq; a.nprobe = nprobe; a.dim = padded_dim; a.k = candidate_count;
    const int kp2 = pow2_at_least(candidate_count);
    a.kp2 = kp2;
    a.cap = std::max(2 * kp2, 2 * kScanStep);   // a whole step always fits after a cut back to candidate_count
    // Few queries: the probes of one query go to several CTAs so that the grid covers the SMs twice over.
    int split = 1;
    if (nq < 2 * sm_count) split = std::min(nprobe, (2 * sm_count + nq - 1) / nq);
    split = std::max(1, std::min(split, kMergeMaxKeys / kp2));
    a.split = split;
    a.rows_out = d_rows_out; a.dist_out = d_dist_out;
    uint64_t* partial = nullptr;
    if (split > 1) {
        PSB_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&partial), sizeof(uint64_t) * (size_t)nq * split * candidate_count, s));
        a.partial = partial;
    }
    const size_t smem = sizeof(uint64_t) * ((size_t)a.cap + ((candidate_count + 1) & ~1)) + sizeof(float) * (256 + 1024);
    psb_status rc = mode == 0 ? dispatch_scan<0>(a, smem, s) : dispatch_scan<1>(a, smem, s);
    if (rc == PSB_OK && split > 1) {
        const int mcap = pow2_at_least(split * candidate_count);
        const size_t msmem = sizeof(uint64_t) * (size_t)mcap;
        cudaError_t e = cudaFuncSetAttribute(k_sign_merge, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)msmem);
        if (e == cudaSuccess) {
            k_sign_merge<<<(unsigned)nq, kScanThreads, msmem, s>>>(partial, split, candidate_count, mcap, d_rows_out, d_dist_out);
            e = cudaGetLastError();
            count_launch();
        }
        if (e != cudaSuccess) rc = cuda_fail(e, "k_sign_merge", __FILE__, __LINE__);
    }
    if (partial) {
        const cudaError_t e = cudaFreeAsync(partial, s);
        if (rc == PSB_OK && e != cudaSuccess) rc = cuda_fail(e, "cudaFreeAsync", __FILE__, __LINE__);
    }
    return rc;
}

}  // namespace psb
