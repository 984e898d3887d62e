// psb_group: one rank of a sharded search, driven from C.  Every rank (one process or thread per GPU) holds a session over its
// shard of the index (psb_options.list_global_begin) and two NCCL communicators of the caller's over the same ranks; a search
// runs the stage calls of the session and the exchanges between the ranks, sub-batch by sub-batch on two streams:
//
//   main stream   coarse (replicated) | tables, sampling, [all-gather of sample records], scan with the shared cutoff  (front i+1)
//   second stream all-to-all of packed candidates -> merge of my query slice -> all-gather of the merged rows ->
//                 exact scoring of the candidates held here -> all-reduce MIN -> top-k -> ids of the rows held here  (back i)
//
// and closes with one all-reduce MAX of the ids.  The reference has no sharded search (its search is single-GPU:
// src/search/ivfpq/pipeline/ivfpq_pipeline.cu:8-116); what it does per batch is what every rank does here on its shard.
// NCCL is not linked: its entry points are looked up in the copy of the library the caller's process already holds (the one
// that created the communicators), so no second copy is ever loaded.
#include <dlfcn.h>

#include <algorithm>
#include <cstdint>
#include <memory>
#include <new>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace psb {
namespace {

// ---- the few NCCL entry points used, by their public C signatures -------------------------------------------
using nccl_comm = void*;
enum : int { kNcclInt32 = 2, kNcclUint32 = 3, kNcclInt64 = 4, kNcclUint64 = 5, kNcclFloat32 = 7 };   // ncclDataType_t
enum : int { kNcclMax = 2, kNcclMin = 3 };                                                             // ncclRedOp_t
struct NcclApi {
    void* lib = nullptr;
    int (*all_reduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*all_gather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
    int (*send)(const void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*recv)(void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*group_start)() = nullptr;
    int (*group_end)() = nullptr;
    int (*comm_count)(nccl_comm, int*) = nullptr;
    int (*comm_rank)(nccl_comm, int*) = nullptr;
    const char* (*error_string)(int) = nullptr;

    psb_status load(const char* path) {
        const char* name = (path && *path) ? path : "libnccl.so.2";
        lib = dlopen(name, RTLD_NOW | RTLD_NOLOAD);          // the copy already in the process, if any
        if (!lib) lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return fail(PSB_INVALID_ARGUMENT, std::string("cannot open the NCCL library ") + name + ": " + dlerror());
        auto sym = [&](const char* s) { return dlsym(lib, s); };
        all_reduce = reinterpret_cast<decltype(all_reduce)>(sym("ncclAllReduce"));
        all_gather = reinterpret_cast<decltype(all_gather)>(sym("ncclAllGather"));
        send = reinterpret_cast<decltype(send)>(sym("ncclSend"));
        recv = reinterpret_cast<decltype(recv)>(sym("ncclRecv"));
        group_start = reinterpret_cast<decltype(group_start)>(sym("ncclGroupStart"));
        group_end = reinterpret_cast<decltype(group_end)>(sym("ncclGroupEnd"));
        comm_count = reinterpret_cast<decltype(comm_count)>(sym("ncclCommCount"));
        comm_rank = reinterpret_cast<decltype(comm_rank)>(sym("ncclCommUserRank"));
        error_string = reinterpret_cast<decltype(error_string)>(sym("ncclGetErrorString"));
        if (!all_reduce || !all_gather || !send || !recv || !group_start || !group_end || !comm_count || !comm_rank || !error_string)
            return fail(PSB_INVALID_ARGUMENT, std::string(name) + " lacks an NCCL entry point this library uses");
        return PSB_OK;
    }
    psb_status check(int rc, const char* what) const {
        if (rc == 0) return PSB_OK;
        return fail(PSB_CUDA_ERROR, std::string("NCCL ") + what + ": " + (error_string ? error_string(rc) : "error"));
    }
};
#define PSB_NCCL(g, call, what) PSB_TRY((g)->nccl.check((g)->nccl.call, what))

struct Buf {
    void* p = nullptr;
    size_t bytes = 0;
    ~Buf() { if (p) cudaFree(p); }
    psb_status reserve(size_t need) {
        if (need <= bytes) return PSB_OK;
        if (p) cudaFree(p);
        p = nullptr; bytes = 0;
        PSB_CUDA(cudaMalloc(&p, need ? need : 1));
        bytes = need;
        return PSB_OK;
    }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

// ---- small kernels of the exchange -------------------------------------------------------------------------------
// One 64-bit word per candidate: distance bits << 32 | row (the order of the words is the order of (distance, row) for the
// non-negative distances of this path).  Rows [m, padded) of the send buffer are padding queries: (FLT_MAX, -1).
__global__ void k_pack_candidates(const float* __restrict__ dist, const int* __restrict__ rows, long long valid, long long total,
                                  unsigned long long* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const unsigned int d = i < valid ? (unsigned int)__float_as_int(dist[i]) : 0x7f7fffffu;
    const unsigned int r = i < valid ? (unsigned int)rows[i] : 0xffffffffu;
    out[i] = ((unsigned long long)d << 32) | r;
}
__global__ void k_unpack_candidates(const unsigned long long* __restrict__ in, long long total, int* __restrict__ rows,
                                    float* __restrict__ dist) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const unsigned long long w = in[i];
    rows[i] = (int)(unsigned int)w;
    dist[i] = __int_as_float((int)(unsigned int)(w >> 32));
}
// Verification of the shared cutoffs on my slice of the queries: a finite cutoff must have left min(width, rows scanned)
// candidates among all shards.  One warp per query; *low becomes non-zero when a query came back short.
__global__ void k_check_short(const int* __restrict__ merged, int width, const long long* __restrict__ scanned,
                              const float* __restrict__ cut, int nq, int* __restrict__ low) {
    const int q = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (q >= nq) return;
    int have = 0;
    for (int i = lane; i < width; i += 32) have += merged[(size_t)q * width + i] >= 0 ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) have += __shfl_xor_sync(0xffffffffu, have, o);
    const long long need = scanned[q] < width ? scanned[q] : width;
    if (lane == 0 && have < need && cut[q] < __int_as_float(0x7f800000)) atomicOr(low, 1);
}
// No rerank: the first topk columns of the merged candidates are the result.
__global__ void k_take_columns(const int* __restrict__ rows, const float* __restrict__ dist, int width, int topk, long long nq,
                               int* __restrict__ out_rows, float* __restrict__ out_dist) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nq * topk) return;
    const long long q = i / topk;
    const int c = (int)(i % topk);
    out_rows[i] = rows[(size_t)q * width + c];
    out_dist[i] = dist[(size_t)q * width + c];
}

inline unsigned blocks_for(long long n, int threads = 256) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace
}  // namespace psb

using namespace psb;

struct psb_group {
    psb_session* s = nullptr;
    nccl_comm comm = nullptr, comm_samples = nullptr;
    int rank = 0, world = 1, max_batch = 0, parts = 4;
    bool shared_cutoff = true;
    NcclApi nccl;
    SessionShape shape;
    cudaStream_t main = nullptr, aux = nullptr;
    cudaEvent_t ev_fronts[32] = {}, ev_back = nullptr;
    Buf probes, lut, l_rows, l_dist, l_cnt, s_key, r_key, g_rows, g_dist, mg_rows, mg_dist, all_rows, all_dist, p_dist, o_rows, smp, smp_all,
        cut, n_scan, low;
    long long searched_again = 0;
    ~psb_group() {
        if (aux) { cudaStreamSynchronize(aux); cudaStreamDestroy(aux); }
        for (auto e : ev_fronts) if (e) cudaEventDestroy(e);
        if (ev_back) cudaEventDestroy(ev_back);
    }
};

namespace {

psb_status group_front(psb_group* g, const float* dq, int q0, int m, int nprobe, int width, bool shared) {
    psb_session* s = g->s;
    const int dim = g->shape.dim;
    const float* q = dq + (size_t)q0 * dim;
    float* lut = g->shape.residual ? nullptr : g->lut.as<float>();
    int* probes = g->probes.as<int>() + (size_t)q0 * nprobe;
    int* rows = g->l_rows.as<int>() + (size_t)q0 * width;
    float* dist = g->l_dist.as<float>() + (size_t)q0 * width;
    int* cnt = g->l_cnt.as<int>() + q0;
    if (lut) PSB_TRY(psb_stage_build_lut(s, q, m, lut));
    if (!shared) return psb_stage_scan_queries(s, q, lut, m, probes, nprobe, width, rows, dist, cnt);
    const int words = psb_scan_sample_words(s, width);
    PSB_TRY(psb_stage_scan_sample(s, q, lut, m, probes, nprobe, width, g->smp.as<uint32_t>()));
    PSB_NCCL(g, all_gather(g->smp.p, g->smp_all.p, (size_t)m * words, kNcclUint32, g->comm_samples, g->main), "all-gather of the sample records");
    return psb_stage_scan_shared(s, q, lut, m, probes, nprobe, width, g->smp_all.as<uint32_t>(), g->world, rows, dist, cnt,
                                 g->cut.as<float>() + q0, reinterpret_cast<int64_t*>(g->n_scan.as<long long>() + q0));
}

psb_status group_back(psb_group* g, const float* dq, int q0, int m, int topk, int width, bool rerank, bool shared, long long* d_ids,
                      float* d_dist) {
    psb_session* s = g->s;
    const int w = g->world, dim = g->shape.dim;
    cudaStream_t st = g->aux;
    const int ms = (m + w - 1) / w;                       // queries per slice (the last slice may be padded)
    const long long slice = (long long)ms * width;
    const int* l_rows = g->l_rows.as<int>() + (size_t)q0 * width;
    const float* l_dist = g->l_dist.as<float>() + (size_t)q0 * width;
    k_pack_candidates<<<blocks_for(slice * w), 256, 0, st>>>(l_dist, l_rows, (long long)m * width, slice * w, g->s_key.as<unsigned long long>());
    PSB_LAUNCH_CHECK();
    // all-to-all: slice p of my candidates goes to rank p, I receive my slice from everyone
    PSB_NCCL(g, group_start(), "group start");
    for (int p = 0; p < w; ++p) {
        PSB_NCCL(g, send(g->s_key.as<unsigned long long>() + (size_t)p * slice, (size_t)slice, kNcclUint64, p, g->comm, st), "send");
        PSB_NCCL(g, recv(g->r_key.as<unsigned long long>() + (size_t)p * slice, (size_t)slice, kNcclUint64, p, g->comm, st), "receive");
    }
    PSB_NCCL(g, group_end(), "group end");
    k_unpack_candidates<<<blocks_for(slice * w), 256, 0, st>>>(g->r_key.as<unsigned long long>(), slice * w, g->g_rows.as<int>(), g->g_dist.as<float>());
    PSB_LAUNCH_CHECK();
    PSB_TRY(psb_stage_merge(s, g->g_rows.as<int>(), g->g_dist.as<float>(), w, ms, width, g->mg_rows.as<int>(), g->mg_dist.as<float>()));
    if (shared) {
        const int a = std::min(q0 + g->rank * ms, q0 + m), b = std::min(a + ms, q0 + m);
        if (b > a) {
            k_check_short<<<blocks_for((long long)(b - a) * 32), 256, 0, st>>>(g->mg_rows.as<int>(), width, g->n_scan.as<long long>() + a,
                                                                                g->cut.as<float>() + a, b - a, g->low.as<int>());
            PSB_LAUNCH_CHECK();
        }
    }
    PSB_NCCL(g, all_gather(g->mg_rows.p, g->all_rows.p, (size_t)slice, kNcclInt32, g->comm, st), "all-gather of the merged rows");
    int* o_rows = g->o_rows.as<int>() + (size_t)q0 * topk;
    float* o_dist = d_dist + (size_t)q0 * topk;
    if (rerank) {
        float* p_dist = g->p_dist.as<float>() + (size_t)q0 * width;
        PSB_TRY(psb_stage_rerank_partial(s, dq + (size_t)q0 * dim, m, g->all_rows.as<int>(), width, width, nullptr, p_dist));
        PSB_NCCL(g, all_reduce(p_dist, p_dist, (size_t)m * width, kNcclFloat32, kNcclMin, g->comm, st), "all-reduce of the exact distances");
        PSB_TRY(psb_stage_select_topk(s, p_dist, g->all_rows.as<int>(), m, width, width, nullptr, topk, o_rows, o_dist));
    } else {   // the merged ADC distances of every slice go round with the rows
        PSB_NCCL(g, all_gather(g->mg_dist.p, g->all_dist.p, (size_t)slice, kNcclFloat32, g->comm, st), "all-gather of the merged distances");
        k_take_columns<<<blocks_for((long long)m * topk), 256, 0, st>>>(g->all_rows.as<int>(), g->all_dist.as<float>(), width, topk, m, o_rows, o_dist);
        PSB_LAUNCH_CHECK();
    }
    return psb_stage_map_ids(s, o_rows, (int64_t)m * topk, reinterpret_cast<int64_t*>(d_ids) + (size_t)q0 * topk);
}

psb_status group_step(psb_group* g, const float* dq, int nq, int nprobe, int topk, int width, bool rerank, bool shared, long long* d_ids,
                      float* d_dist) {
    psb_session* s = g->s;
    PSB_TRY(psb_session_set_stream(s, nullptr, 0));
    if (shared) PSB_CUDA(cudaMemsetAsync(g->low.p, 0, sizeof(int), g->main));
    PSB_TRY(psb_stage_coarse(s, dq, nq, nprobe, g->probes.as<int>(), nullptr));
    // sub-batches: the exchange half is the longer one, a small first sub-batch lets it start early
    int cuts[33];
    int parts = nq >= 2048 ? g->parts : 1;
    if (parts == 4 && nq >= 4096) {
        cuts[0] = 0; cuts[1] = (int)(0.10 * nq); cuts[2] = (int)(0.40 * nq); cuts[3] = (int)(0.70 * nq); cuts[4] = nq;
    } else {
        const int sb = (nq + parts - 1) / parts;
        parts = (nq + sb - 1) / sb;
        for (int i = 0; i <= parts; ++i) cuts[i] = std::min(i * sb, nq);
    }
    // The front half of sub-batch i + 1 is queued BEFORE the back half of sub-batch i: a back half may keep this thread busy (the
    // host's share of a hybrid rerank transport), and the GPU must not run dry meanwhile.
    psb_status rc = PSB_OK;
    for (int i = 0; i <= parts && rc == PSB_OK; ++i) {
        if (i < parts && cuts[i + 1] > cuts[i]) {
            rc = group_front(g, dq, cuts[i], cuts[i + 1] - cuts[i], nprobe, width, shared);
            if (rc != PSB_OK) break;
            PSB_CUDA(cudaEventRecord(g->ev_fronts[i], g->main));
        }
        if (i >= 1 && cuts[i] > cuts[i - 1]) {
            PSB_CUDA(cudaStreamWaitEvent(g->aux, g->ev_fronts[i - 1], 0));
            rc = psb_session_set_stream(s, g->aux, 1);
            if (rc == PSB_OK) rc = group_back(g, dq, cuts[i - 1], cuts[i] - cuts[i - 1], topk, width, rerank, shared, d_ids, d_dist);
            const psb_status back = psb_session_set_stream(s, nullptr, 0);
            if (rc == PSB_OK) rc = back;
        }
    }
    PSB_TRY(rc);
    PSB_CUDA(cudaEventRecord(g->ev_back, g->aux));
    PSB_CUDA(cudaStreamWaitEvent(g->main, g->ev_back, 0));
    // every rank wrote the ids of the rows it holds, -1 elsewhere
    PSB_NCCL(g, all_reduce(d_ids, d_ids, (size_t)nq * topk, kNcclInt64, kNcclMax, g->comm, g->main), "all-reduce of the ids");
    return PSB_OK;
}

}  // namespace

extern "C" {

psb_status psb_group_create(psb_session* session, void* nccl_comm_main, void* nccl_comm_samples, const char* nccl_library,
                            int max_batch, int nprobe, int topk, psb_group** out) {
    if (!out) return fail(PSB_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!session || !nccl_comm_main || max_batch <= 0 || nprobe <= 0 || topk <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid group request");
    if (nprobe > kMaxProbe || topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 or topk above 2048");
    std::unique_ptr<psb_group> g(new (std::nothrow) psb_group());
    if (!g) return fail(PSB_OUT_OF_MEMORY, "host allocation failed");
    g->s = session;
    g->comm = nccl_comm_main;
    g->comm_samples = nccl_comm_samples ? nccl_comm_samples : nccl_comm_main;
    g->shape = session_shape(session);
    if (g->shape.flat) return fail(PSB_INVALID_ARGUMENT, "an IVF-Flat session cannot join a group");
    if (g->shape.exact_elem == 1) return fail(PSB_UNSUPPORTED_SHAPE, "u8 exact rows are not supported by the group search");
    PSB_CUDA(cudaSetDevice(g->shape.device));
    PSB_TRY(g->nccl.load(nccl_library));
    PSB_TRY(g->nccl.check(g->nccl.comm_count(g->comm, &g->world), "communicator size"));
    PSB_TRY(g->nccl.check(g->nccl.comm_rank(g->comm, &g->rank), "communicator rank"));
    int w2 = 0, r2 = 0;
    PSB_TRY(g->nccl.check(g->nccl.comm_count(g->comm_samples, &w2), "communicator size"));
    PSB_TRY(g->nccl.check(g->nccl.comm_rank(g->comm_samples, &r2), "communicator rank"));
    if (w2 != g->world || r2 != g->rank) return fail(PSB_INVALID_ARGUMENT, "the two communicators must span the same ranks in the same order");
    g->max_batch = max_batch;
    g->main = g->shape.stream;
    int lo = 0, hi = 0;
    PSB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    PSB_CUDA(cudaStreamCreateWithPriority(&g->aux, cudaStreamNonBlocking, lo));
    for (auto& e : g->ev_fronts) PSB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    PSB_CUDA(cudaEventCreateWithFlags(&g->ev_back, cudaEventDisableTiming));
    const int width = std::max(g->shape.n_rerank > topk ? std::min(g->shape.n_rerank, kMaxStage1) : topk, topk);
    const int w = g->world;
    const size_t nq = (size_t)max_batch, ms = (nq + w - 1) / w, slab = (size_t)w * ms * width;
    PSB_TRY(g->probes.reserve(sizeof(int) * nq * nprobe));
    if (!g->shape.residual) PSB_TRY(g->lut.reserve(sizeof(float) * nq * g->shape.m * g->shape.k));
    PSB_TRY(g->l_rows.reserve(sizeof(int) * nq * width));
    PSB_TRY(g->l_dist.reserve(sizeof(float) * nq * width));
    PSB_TRY(g->l_cnt.reserve(sizeof(int) * nq));
    PSB_TRY(g->s_key.reserve(sizeof(unsigned long long) * slab));
    PSB_TRY(g->r_key.reserve(sizeof(unsigned long long) * slab));
    PSB_TRY(g->g_rows.reserve(sizeof(int) * slab));
    PSB_TRY(g->g_dist.reserve(sizeof(float) * slab));
    PSB_TRY(g->mg_rows.reserve(sizeof(int) * ms * width));
    PSB_TRY(g->mg_dist.reserve(sizeof(float) * ms * width));
    PSB_TRY(g->all_rows.reserve(sizeof(int) * slab));
    PSB_TRY(g->all_dist.reserve(sizeof(float) * slab));
    PSB_TRY(g->p_dist.reserve(sizeof(float) * nq * width));
    PSB_TRY(g->o_rows.reserve(sizeof(int) * nq * topk));
    const int words = psb_scan_sample_words(session, width);
    PSB_TRY(g->smp.reserve(sizeof(uint32_t) * nq * words));
    PSB_TRY(g->smp_all.reserve(sizeof(uint32_t) * nq * words * w));
    PSB_TRY(g->cut.reserve(sizeof(float) * nq));
    PSB_TRY(g->n_scan.reserve(sizeof(long long) * nq));
    PSB_TRY(g->low.reserve(sizeof(int)));
    *out = g.release();
    return PSB_OK;
}

psb_status psb_group_set(psb_group* g, int parts, int shared_cutoff) {
    if (!g || parts < 1 || parts > 32) return fail(PSB_INVALID_ARGUMENT, "parts must be in 1..32");
    g->parts = parts;
    g->shared_cutoff = shared_cutoff != 0;
    return PSB_OK;
}

psb_status psb_group_search_device(psb_group* g, const float* d_queries, int nq, const psb_search_params* params, int64_t* d_indices,
                                   float* d_distances) {
    PSB_RANGE("ivfpq_group_search");
    if (!g || !d_queries || !params || !d_indices || !d_distances) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nq <= 0 || nq > g->max_batch) return fail(PSB_INVALID_ARGUMENT, "nq must be in 1..max_batch of the group");
    const int nprobe = params->nprobe, topk = params->topk;
    if (nprobe <= 0 || topk <= 0 || (size_t)nq * nprobe * sizeof(int) > g->probes.bytes || (size_t)nq * topk * sizeof(int) > g->o_rows.bytes)
        return fail(PSB_INVALID_ARGUMENT, "nprobe / topk beyond what the group was created for");
    if (params->distance != 0) return fail(PSB_INVALID_ARGUMENT, "only squared L2 is supported");
    PSB_CUDA(cudaSetDevice(g->shape.device));
    const bool rerank = g->shape.exact_elem != 0 && g->shape.n_rerank > topk;
    if (g->shape.residual && !rerank) return fail(PSB_INVALID_ARGUMENT, "residual mode always reranks");
    const int width = rerank ? std::min(g->shape.n_rerank, kMaxStage1) : topk;
    if ((size_t)nq * width * sizeof(int) > g->l_rows.bytes) return fail(PSB_INVALID_ARGUMENT, "topk beyond what the group was created for");
    const bool shared = g->shared_cutoff && g->world > 1;
    long long* ids = reinterpret_cast<long long*>(d_indices);
    PSB_TRY(group_step(g, d_queries, nq, nprobe, topk, width, rerank, shared, ids, d_distances));
    if (shared) {   // one word for the whole batch: did any rank see a query come back short?  Then once more, per-shard cutoffs.
        PSB_NCCL(g, all_reduce(g->low.p, g->low.p, 1, kNcclInt32, kNcclMax, g->comm, g->main), "all-reduce of the verification word");
        int low = 0;
        PSB_CUDA(cudaMemcpyAsync(&low, g->low.p, sizeof(int), cudaMemcpyDeviceToHost, g->main));
        PSB_CUDA(cudaStreamSynchronize(g->main));
        if (low) {
            ++g->searched_again;
            PSB_TRY(group_step(g, d_queries, nq, nprobe, topk, width, rerank, false, ids, d_distances));
        }
    }
    return PSB_OK;
}

long long psb_group_searched_again(const psb_group* g) { return g ? g->searched_again : 0; }

psb_status psb_group_destroy(psb_group* g) {
    if (g) cudaSetDevice(g->shape.device);
    delete g;
    return PSB_OK;
}

}  // extern "C"
