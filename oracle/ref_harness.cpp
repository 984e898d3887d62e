// TEST INFRASTRUCTURE, not product code.
//
// C-ABI shim around the reference's own CPU implementation of the IVF-PQ
// search path.  The reference translation units are compiled where they lie
// in the reference checkout (see oracle/Makefile); nothing from them is copied
// here.  This file only fills the reference's context structs and calls:
//   - coarse probe selection: the scalar loop of src/cpu/search/cpu_search.h:261-271
//     (l2_distance_squared from src/cpu/utils/cpu_distance.h:74-81 + std::partial_sort
//     by distance only), re-written here because cpu_search.h as a whole needs the
//     CUDA toolchain's CUB headers;
//   - ivfpq_fine_cpu_lut      src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:25
//   - ivfpq_rerank_cpu        src/search/ivfpq/stage/ivfpq_rerank_cpu.cpp:14
//   - ivfpq_map_ids           src/search/ivfpq/stage/ivfpq_map_ids.cpp:4
//   - ivf_rerank_host         src/search/ivf_common/ivf_host_rerank.cpp:55
//   - cpu_fine_kernel_pq_resid_cpu_lut_timed (residual ADC mode, stage 1 + exact rerank)
//                             src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:594
#include "search/ivfpq/ivfpq_search_context.h"
#include "search/ivfpq/stage/ivfpq_stages.cuh"
#include "search/ivf_common/ivf_host_rerank.h"
#include "search/ivfrespq/ivfrespq_search.cuh"
#include "search/ivfrespq/stage/ivfrespq_cpu_rerank.h"
#include "search/ivfrespq/stage/ivfrespq_pq_storage.h"
#include "cpu/distance/distance_dispatch.h"
#include "cpu/utils/cpu_distance.h"
#include "cpu/utils/cpu_affinity.h"

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>
#include <omp.h>

// The search context owns a unique_ptr<coarse::Workspace> that the CPU path
// never constructs; the destructor still needs a definition to link.
namespace paraselect::coarse {
struct Workspace::Impl {};
Workspace::~Workspace() = default;
}  // namespace paraselect::coarse

namespace {
thread_local std::string g_err;
double now_ms() {
    return std::chrono::duration<double, std::milli>(
        std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

extern "C" {

const char* psbref_last_error() { return g_err.c_str(); }

const char* psbref_fp32_isa() { return paraselect::cpu_distance::selected_fp32_l2_isa_name(); }

int psbref_physical_cores() { return paraselect::get_physical_core_count(); }

// Scalar coarse stage of the CPU path: all-centroid squared L2, partial sort by
// distance only (tie order unspecified, as in the reference).
int psbref_coarse(const float* queries, int nq, const float* centroids, int nlist, int dim,
                  int nprobe, int64_t* out_ids, float* out_dist, int threads) {
    if (!queries || !centroids || nprobe <= 0 || nprobe > nlist) { g_err = "bad coarse args"; return 1; }
    struct Pair { float dist; int64_t idx; };
#pragma omp parallel num_threads(threads > 0 ? threads : omp_get_max_threads())
    {
        std::vector<Pair> tmp((size_t)nlist);
#pragma omp for schedule(static)
        for (int qi = 0; qi < nq; ++qi) {
            const float* query = queries + (size_t)qi * dim;
            for (int cid = 0; cid < nlist; ++cid)
                tmp[(size_t)cid] = {l2_distance_squared(query, centroids + (size_t)cid * dim, dim), (int64_t)cid};
            std::partial_sort(tmp.begin(), tmp.begin() + nprobe, tmp.end(),
                              [](const Pair& a, const Pair& b) { return a.dist < b.dist; });
            for (int p = 0; p < nprobe; ++p) {
                out_ids[(size_t)qi * nprobe + p] = tmp[(size_t)p].idx;
                if (out_dist) out_dist[(size_t)qi * nprobe + p] = tmp[(size_t)p].dist;
            }
        }
    }
    return 0;
}

// Plain IVF-PQ chain of the reference's serial pipeline (fine -> rerank -> map ids)
// for queries whose probes are given.  The fine stage is single-threaded in the
// reference; fine_threads > 1 splits the query batch into independent contexts.
// times_ms[0..2] = fine, rerank, map.  stage1_out (optional) = [nq][stage1_k] rows.
int psbref_ivfpq_search(const float* centroids, int nlist, int dim,
                        const int64_t* offsets, const int64_t* reordered_ids, int64_t n_vectors,
                        const uint8_t* codes, const float* codebook, int pq_m, int pq_k,
                        const float* rerank_fp32,
                        const float* queries, int nq, const int64_t* probes,
                        int nprobe, int topk, int n_rerank,
                        int fine_threads, int rerank_threads,
                        int64_t* out_indices, float* out_distances, int* stage1_out,
                        double* times_ms, long long* scanned_codes) {
    try {
        const bool rerank = rerank_fp32 != nullptr && n_rerank > topk;
        const int stage1_k = rerank ? (int)std::min<int64_t>(n_rerank, n_vectors) : topk;
        if (fine_threads <= 0) fine_threads = 1;
        fine_threads = std::min(fine_threads, std::max(1, nq));
        std::vector<long long> off((size_t)nlist + 1);
        std::vector<int> cnt((size_t)nlist);
        for (int i = 0; i <= nlist; ++i) off[(size_t)i] = offsets[i];
        for (int i = 0; i < nlist; ++i) cnt[(size_t)i] = (int)(offsets[i + 1] - offsets[i]);
        std::vector<std::string> errs((size_t)fine_threads);
        std::vector<double> t_fine((size_t)fine_threads, 0.0), t_rr((size_t)fine_threads, 0.0), t_map((size_t)fine_threads, 0.0);
        std::vector<long long> scanned((size_t)fine_threads, 0);
        // Fine stage: one context per slice (contexts are not shareable).
        std::vector<IVFPQSearchContext> ctxs((size_t)fine_threads);
        for (int t = 0; t < fine_threads; ++t) {
            const int q0 = (int)((long long)nq * t / fine_threads), q1 = (int)((long long)nq * (t + 1) / fine_threads);
            IVFPQSearchContext& ctx = ctxs[(size_t)t];
            ctx.index.coarse = {centroids, nlist, dim};
            ctx.index.lists = {offsets, reordered_ids, nlist, n_vectors};
            ctx.index.storage.rerank_fp32 = rerank_fp32;
            ctx.index.storage.pq.codes = codes;
            ctx.index.storage.pq.codebook = codebook;
            ctx.index.storage.pq.subvectors = pq_m;
            ctx.index.storage.pq.codebook_size = pq_k;
            ctx.queries = {queries, nullptr, nq, dim};
            ctx.params.nprobe = nprobe; ctx.params.topk = topk; ctx.params.batch_size = std::max(1, q1 - q0);
            ctx.output = {out_indices, out_distances, nullptr};
            ctx.options.n_rerank = n_rerank;
            ctx.options.rerank_dtype = rerank ? IVFExactRerankDType::FP32 : IVFExactRerankDType::Disabled;
            ctx.options.cpu_rerank_threads = rerank_threads;
            ctx.pq_rerank_enabled = rerank ? 1 : 0;
            ctx.pq_stage1_k = stage1_k;
            ctx.query_batch_size = std::max(1, q1 - q0);
            ctx.cluster_offsets = off;
            ctx.cluster_counts = cnt;
            const size_t bn = (size_t)std::max(0, q1 - q0);
            ctx.top_nprobe_batch.assign(probes + (size_t)q0 * nprobe, probes + (size_t)q1 * nprobe);
            ctx.topk_local_idx_batch.assign(bn * topk, -1);
            ctx.rerank_candidate_idx_batch.assign(bn * stage1_k, -1);
            ctx.rerank_candidate_count_batch.assign(bn, stage1_k);
        }
        const double f0 = now_ms();
#pragma omp parallel for num_threads(fine_threads) schedule(static, 1)
        for (int t = 0; t < fine_threads; ++t) {
            const int q0 = (int)((long long)nq * t / fine_threads), q1 = (int)((long long)nq * (t + 1) / fine_threads);
            if (q1 <= q0) continue;
            try {
                ivfpq_fine_cpu_lut(&ctxs[(size_t)t], q0, q1 - q0);
                scanned[(size_t)t] = ctxs[(size_t)t].pq_scanned_codes_total;
            } catch (const std::exception& e) { errs[(size_t)t] = e.what(); }
        }
        const double f1 = now_ms();
        for (auto& e : errs) if (!e.empty()) { g_err = e; return 2; }
        // Rerank owns its own thread pool and a process-wide mutex: run slices serially.
        for (int t = 0; t < fine_threads; ++t) {
            const int q0 = (int)((long long)nq * t / fine_threads), q1 = (int)((long long)nq * (t + 1) / fine_threads);
            if (q1 <= q0) continue;
            IVFPQSearchContext& ctx = ctxs[(size_t)t];
            if (stage1_out && rerank)
                std::memcpy(stage1_out + (size_t)q0 * stage1_k, ctx.rerank_candidate_idx_batch.data(),
                            sizeof(int) * (size_t)(q1 - q0) * stage1_k);
            const double a = now_ms();
            ivfpq_rerank_cpu(&ctx, q0, q1 - q0);
            const double b = now_ms();
            ivfpq_map_ids(&ctx, q0, q1 - q0);
            const double c = now_ms();
            t_rr[(size_t)t] = b - a; t_map[(size_t)t] = c - b;
            if (stage1_out && !rerank)
                for (int q = 0; q < q1 - q0; ++q)
                    for (int i = 0; i < stage1_k; ++i)
                        stage1_out[(size_t)(q0 + q) * stage1_k + i] = ctx.topk_local_idx_batch[(size_t)q * topk + i];
        }
        if (times_ms) {
            times_ms[0] = f1 - f0; times_ms[1] = 0; times_ms[2] = 0;
            for (int t = 0; t < fine_threads; ++t) { times_ms[1] += t_rr[(size_t)t]; times_ms[2] += t_map[(size_t)t]; }
        }
        if (scanned_codes) { *scanned_codes = 0; for (auto s : scanned) *scanned_codes += s; }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 3; }
}

// Direct call of the shared exact-rerank operator (fp32 or u8 rows).
int psbref_rerank_host(const float* base_fp32, const uint8_t* base_u8, int64_t count, int dim,
                       const float* queries_fp32, const uint8_t* queries_u8,
                       const int* candidates, int batch_n, int candidate_count, int candidate_stride,
                       int topk, const int* candidate_counts, int threads, int prefetch,
                       int* out_ids, float* out_dist) {
    try {
        paraselect::search::IVFHostStorageView st;
        st.fp32 = base_fp32; st.u8 = base_u8; st.count = count; st.dim = dim;
        ivf_rerank_host(st, queries_u8, queries_fp32, base_fp32 != nullptr, candidates, batch_n,
                        candidate_count, candidate_stride, topk, out_ids, out_dist, threads, false,
                        prefetch, nullptr, candidate_counts);
        return 0;
    } catch (const std::invalid_argument& e) { g_err = e.what(); return 1; }
    catch (const std::exception& e) { g_err = e.what(); return 2; }
}

// Residual ADC mode: the reference's CPU stage-1 + exact rerank for queries whose probes are given
// (query-balanced scheduler, row-major codes, fp32 rerank rows), then the id map through reordered_ids.
// out_local [nq][topk] = list-contiguous rows (-1 padded), out_indices (optional) = mapped ids.
int psbref_ivfrespq_search(const float* centroids, int nlist, int dim,
                           const int64_t* offsets, const int64_t* reordered_ids, int64_t n_vectors,
                           const uint8_t* codes, const float* codebook, int pq_m, int pq_k,
                           const float* rerank_fp32, const float* queries, int nq, const int64_t* probes,
                           int nprobe, int topk, int n_rerank, int threads,
                           int* out_local, int64_t* out_indices, float* out_distances,
                           double* times_ms, long long* scanned_codes) {
    try {
        std::vector<long long> off((size_t)nlist + 1);
        std::vector<int> cnt((size_t)nlist);
        for (int i = 0; i <= nlist; ++i) off[(size_t)i] = offsets[i];
        for (int i = 0; i < nlist; ++i) cnt[(size_t)i] = (int)(offsets[i + 1] - offsets[i]);
        const paraselect::cpu_fine::CpuPqCodeStorageView storage = paraselect::cpu_fine::make_pq_row_major_storage(
            codes, off.data(), cnt.data(), pq_m, nlist, (int)n_vectors);
        paraselect::cpu_fine::PQResidCpuLUTTiming timing;
        std::fill(out_local, out_local + (size_t)nq * topk, -1);
        (void)paraselect::cpu_fine::cpu_fine_kernel_pq_resid_cpu_lut_timed(
            nullptr, off.data(), cnt.data(), storage, codebook, centroids, nullptr, queries, nullptr, rerank_fp32, 1,
            probes, nq, dim, nlist, nprobe, topk, n_rerank, pq_m, pq_k, threads, out_local, out_distances,
            paraselect::search::IVFResPQCpuScheduler::QueryBalanced, 1, &timing);
        if (out_indices)
            for (size_t i = 0; i < (size_t)nq * topk; ++i) {
                const int r = out_local[i];
                out_indices[i] = (r >= 0 && r < n_vectors) ? (reordered_ids ? reordered_ids[r] : (int64_t)r) : -1;
            }
        if (times_ms) { times_ms[0] = timing.adc_lut_scan_ms; times_ms[1] = timing.rerank_ms; times_ms[2] = 0; }
        if (scanned_codes) *scanned_codes = timing.scanned_codes;
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 3; }
}

}  // extern "C"
