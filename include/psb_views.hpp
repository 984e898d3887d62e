/*
 * psb_views.hpp - header-only C++ shim: ParaSelect's own entry points for the IVF search hot path, implemented on the
 * C ABI of psb.h.
 *
 * A caller of the reference keeps its code as it is - it fills the reference's request structs and calls
 *     paraselect::search::ivfrespq_search(request, stats)        src/search/ivfrespq/ivfrespq_search.cuh:114-116
 *     paraselect::search::IVFResPQSession(request).search(stats)  src/search/ivfrespq/ivfrespq_search.cuh:120-133
 *     paraselect::search::ivfflat_search(request, stats)          src/search/ivfflat/ivfflat_search.cuh:49-51
 *     paraselect::search::ivf_res_turboquant::Index / SearchWorkspace   (when that header is included too)
 *                                                                 src/search/ivf_res_turboquant/ivf_res_turboquant_search.cuh:25-112
 * - includes this header AFTER the reference's headers, and links libpsb.so in place of the reference's search
 * libraries.  The definitions below take the place of the reference's .cu implementations of those declarations.
 *
 * What maps: the views (field for field), nprobe / topk / batch_size, options.n_rerank, the ADC distance mode
 * (PQAdcDistanceMode::Plain / ::Residual), host or device-resident exact rows.  What the hot path does not cover is
 * refused with std::invalid_argument instead of being ignored: other residual codecs, PCA refinement, file-backed exact
 * rows, the candidate-only request, cosine distance.  Failures of the library surface as exceptions
 * (std::invalid_argument where the reference throws it, std::runtime_error otherwise); nothing aborts or resets the device.
 */
#ifndef PSB_VIEWS_HPP
#define PSB_VIEWS_HPP

#include <algorithm>
#include <memory>
#include <stdexcept>
#include <string>

#include "psb.h"

#if !defined(PARASELECT_CUDA_IVFRESPQ_SEARCH_CUH) || !defined(PARASELECT_CUDA_IVFFLAT_SEARCH_CUH)
#error "include the reference's search/ivfrespq/ivfrespq_search.cuh and search/ivfflat/ivfflat_search.cuh before psb_views.hpp"
#endif

namespace paraselect::search {

namespace psb_shim {

inline void check(psb_status st) {
    if (st == PSB_OK) return;
    const std::string msg = psb_last_error();
    if (st == PSB_INVALID_ARGUMENT) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

// IVFResPQIndexView -> psb_index_view (the same pointers; nothing is copied).
inline psb_index_view index_view(const IVFResPQIndexView& ix, int* exact_mode) {
    psb_index_view v{};
    v.coarse.centroids = ix.coarse.centroids; v.coarse.nlist = ix.coarse.nlist; v.coarse.dim = ix.coarse.dim;
    v.lists.offsets = reinterpret_cast<const int64_t*>(ix.lists.offsets);
    v.lists.reordered_ids = reinterpret_cast<const int64_t*>(ix.lists.reordered_ids);
    v.lists.nlist = ix.lists.nlist; v.lists.n_vectors = ix.lists.n_vectors;
    v.pq.codes = ix.storage.pq.codes; v.pq.code_storage = ix.storage.pq.code_storage; v.pq.codebook = ix.storage.pq.codebook;
    v.pq.subvectors = ix.storage.pq.subvectors; v.pq.codebook_size = ix.storage.pq.codebook_size;
    const IVFExactStorageView& ex = ix.storage.assets.exact;
    *exact_mode = PSB_EXACT_HOST_STAGED;
    switch (ex.kind) {
        case IVFExactStorageKind::None: break;
        case IVFExactStorageKind::Host:
            v.exact.fp32 = ex.host.fp32; v.exact.u8 = ex.host.u8; v.exact.count = ex.host.count; v.exact.dim = ex.host.dim;
            v.exact.source_rows = ex.host.source_rows;
            break;
        case IVFExactStorageKind::Resident:
            v.exact.fp32 = ex.resident.fp32; v.exact.u8 = ex.resident.u8; v.exact.count = ex.resident.count; v.exact.dim = ex.resident.dim;
            *exact_mode = PSB_EXACT_RESIDENT;
            break;
        default: throw std::invalid_argument("psb shim: file-backed exact rows are not part of this path");
    }
    if (ix.storage.host_rows) throw std::invalid_argument("psb shim: a PQ-row -> exact-row mapping is not supported");
    return v;
}

inline psb_options options(const IVFResPQSearchOptions& o, const IVFSearchParams& p, int exact_mode) {
    if (o.residual_codec != ResidualCodecKind::PQ) throw std::invalid_argument("psb shim: only the PQ residual codec is on this path");
    if (o.pca_backend != IVFRefineBackend::None) throw std::invalid_argument("psb shim: PCA refinement is not on this path");
    psb_options opt{};
    opt.n_rerank = o.n_rerank;
    opt.exact_mode = exact_mode;
    opt.max_batch = p.batch_size > 0 ? p.batch_size : 0;
    opt.adc_mode = o.pq_distance_mode == PQAdcDistanceMode::Residual ? 1 : 0;
    return opt;
}

inline void fill_stats(const psb_stats& s, IVFSearchStats* out) {
    if (!out) return;
    out->total_time_ms = s.total_ms;
    out->avg_batch_time_ms = s.batches > 0 ? s.total_ms / s.batches : 0.0;
    out->coarse_search_ms = s.coarse_search_ms;
    // the field names of the reference's stats collector (src/search/ivfpq/pipeline/ivfpq_pipeline.cu:41-71,84-103)
    out->numeric_fields["coarse_search"] = s.coarse_search_ms;
    out->numeric_fields["pq_lut_build"] = s.pq_lut_build_ms;
    out->numeric_fields["pq_adc_scan"] = s.pq_adc_scan_ms;
    out->numeric_fields["pq_rerank"] = s.pq_rerank_ms;
    out->numeric_fields["pq_map_ids"] = s.pq_map_ids_ms;
    out->numeric_fields["pq_scanned_codes"] = (double)s.pq_scanned_codes;
    out->numeric_fields["pq_adc_lookups"] = (double)s.pq_adc_lookups;
    out->string_fields["search_impl"] = "psb_b200";
}

inline psb_query_batch_view query_view(const IVFQueryBatchView& q) {
    psb_query_batch_view v{};
    v.fp32 = q.fp32; v.u8 = q.u8; v.count = q.count; v.dim = q.dim; v.fp16 = q.fp16;
    return v;
}
inline psb_search_params params(const IVFSearchParams& p) {
    psb_search_params v{};
    v.nprobe = p.nprobe; v.topk = p.topk; v.batch_size = p.batch_size; v.distance = p.distance; v.fp16_coarse = p.fp16_coarse ? 1 : 0;
    return v;
}
inline psb_search_output_view output_view(const IVFSearchOutputView& o) {
    psb_search_output_view v{};
    v.indices = reinterpret_cast<int64_t*>(o.indices); v.distances = o.distances; v.coarse_ids = o.coarse_ids;
    return v;
}

}  // namespace psb_shim

// ---- IVFResPQSession: prepare once, search many --------------------------------------------------------------
struct IVFResPQSession::Impl {
    psb_session* session = nullptr;
    IVFResPQSearchRequest request;
    ~Impl() { psb_session_destroy(session); }
};

inline IVFResPQSession::IVFResPQSession(const IVFResPQSearchRequest& request) : impl_(new Impl()) {
    impl_->request = request;
    int exact_mode = 0;
    const psb_index_view ix = psb_shim::index_view(request.index, &exact_mode);
    const psb_options opt = psb_shim::options(request.options, request.params, exact_mode);
    psb_shim::check(psb_session_create(&ix, &opt, &impl_->session));
}
inline IVFResPQSession::IVFResPQSession(const IVFResPQCandidateRequest&) : impl_(nullptr) {
    throw std::invalid_argument("psb shim: the candidate-only request is not part of this path");
}
inline int IVFResPQSession::candidate_count() const { return 0; }
inline IVFResPQSession::~IVFResPQSession() = default;
inline void IVFResPQSession::search(IVFSearchStats* stats) {
    const psb_query_batch_view q = psb_shim::query_view(impl_->request.queries);
    const psb_search_params p = psb_shim::params(impl_->request.params);
    const psb_search_output_view o = psb_shim::output_view(impl_->request.output);
    psb_stats st{};
    psb_shim::check(psb_session_search(impl_->session, &q, &p, &o, &st));
    psb_shim::fill_stats(st, stats);
}

inline void ivfrespq_search(const IVFResPQSearchRequest& request, IVFSearchStats* stats) {
    IVFResPQSession session(request);
    session.search(stats);
}

// ---- ivfflat_search ---------------------------------------------------------------------------------------------
inline void ivfflat_search(const IVFFlatSearchRequest& request, IVFSearchStats* stats) {
    const IVFFlatStorageView& sv = request.index.storage;
    if (!sv.rowmajor_fp32) throw std::invalid_argument("psb shim: IVF-Flat needs row-major fp32 host rows");
    psb_flat_index_view ix{};
    ix.coarse.centroids = request.index.coarse.centroids; ix.coarse.nlist = request.index.coarse.nlist; ix.coarse.dim = request.index.coarse.dim;
    ix.lists.offsets = reinterpret_cast<const int64_t*>(request.index.lists.offsets);
    ix.lists.reordered_ids = reinterpret_cast<const int64_t*>(request.index.lists.reordered_ids);
    ix.lists.nlist = request.index.lists.nlist; ix.lists.n_vectors = request.index.lists.n_vectors;
    ix.rowmajor_fp32 = sv.rowmajor_fp32;
    psb_options opt{};
    opt.max_batch = request.params.batch_size > 0 ? request.params.batch_size : 0;
    psb_flat_session* s = nullptr;
    psb_shim::check(psb_flat_session_create(&ix, &opt, &s));
    std::unique_ptr<psb_flat_session, psb_status (*)(psb_flat_session*)> guard(s, psb_flat_session_destroy);
    const psb_query_batch_view q = psb_shim::query_view(request.queries);
    const psb_search_params p = psb_shim::params(request.params);
    const psb_search_output_view o = psb_shim::output_view(request.output);
    psb_stats st{};
    psb_shim::check(psb_flat_session_search(s, &q, &p, &o, &st));
    psb_shim::fill_stats(st, stats);
}

}  // namespace paraselect::search

// ---- IVFResTurboQuant (1-bit sign codec) -------------------------------------------------------------------------
// Only when the caller has included the reference's search/ivf_res_turboquant/ivf_res_turboquant_search.cuh: the member
// functions that header declares (src/search/ivf_res_turboquant/ivf_res_turboquant_search.cuh:25-112) are defined here on
// psb_sign_*.  The object keeps the reference's members - device copies of centroids, list offsets, sign codes and scales -
// and the caller links the CUDA runtime, as it does with the reference.  Differences: candidate_count up to
// PSB_SIGN_MAX_CANDIDATES (any value, not only powers of two); `exact_selection` changes nothing (the selection is always
// exact); SearchTiming gets total_ms only.
#ifdef PARASELECT_IVF_RES_TURBOQUANT_SEARCH_CUH
#include <chrono>
#include <vector>

namespace paraselect::search::ivf_res_turboquant {

namespace psb_sign_shim {
inline void cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("psb shim: ") + what + ": " + cudaGetErrorString(e));
}
inline int device() {
    if (psb_device_count() <= 0) throw std::runtime_error("psb shim: no CUDA device is usable; this library has no CPU path");
    int dev = 0;
    cuda(cudaGetDevice(&dev), "cudaGetDevice");
    return dev;
}
template <class T>
inline void renew(T** p, std::size_t count) {
    if (*p) cudaFree(*p);
    *p = nullptr;
    cuda(cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)), "cudaMalloc");
}
template <class T>
inline void drop(T** p) {
    if (*p) cudaFree(*p);
    *p = nullptr;
}
}  // namespace psb_sign_shim

inline Index::~Index() { release(); }

inline void Index::release() {
    psb_sign_shim::drop(&d_centroids_); psb_sign_shim::drop(&d_cluster_offsets_);
    psb_sign_shim::drop(&d_codes_); psb_sign_shim::drop(&d_reconstruction_scales_);
    n_vectors_ = n_clusters_ = dim_ = padded_dim_ = words_per_code_ = 0;
}

inline void Index::build_u8(const std::uint8_t* host_vectors, const float* host_centroids, const long long* host_cluster_offsets,
                            int n_vectors, int n_clusters, int dim, std::uint32_t rotation_seed) {
    if (!host_vectors || !host_centroids || !host_cluster_offsets || n_vectors <= 0 || n_clusters <= 0 || dim <= 0)
        throw std::invalid_argument("IVFResTurboQuant index build received invalid input");
    const int padded = psb_sign_padded_dim(dim);
    if (padded < 0) throw std::invalid_argument("IVFResTurboQuant supports dimensions <= 256");
    const int dev = psb_sign_shim::device();
    release();
    n_vectors_ = n_vectors; n_clusters_ = n_clusters; dim_ = dim; padded_dim_ = padded; words_per_code_ = padded / 32;
    rotation_seed_ = rotation_seed;
    std::uint8_t* d_chunk = nullptr;
    try {
        const std::size_t chunk_rows = std::min<std::size_t>((std::size_t)n_vectors, (std::size_t)1 << 20);
        psb_sign_shim::renew(&d_chunk, chunk_rows * (std::size_t)dim);
        psb_sign_shim::renew(&d_centroids_, (std::size_t)n_clusters * dim);
        psb_sign_shim::renew(&d_cluster_offsets_, (std::size_t)n_clusters + 1);
        psb_sign_shim::renew(&d_codes_, (std::size_t)n_vectors * words_per_code_);
        psb_sign_shim::renew(&d_reconstruction_scales_, (std::size_t)n_vectors);
        psb_sign_shim::cuda(cudaMemcpy(d_centroids_, host_centroids, (std::size_t)n_clusters * dim * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
        psb_sign_shim::cuda(cudaMemcpy(d_cluster_offsets_, host_cluster_offsets, ((std::size_t)n_clusters + 1) * sizeof(long long), cudaMemcpyHostToDevice), "cudaMemcpy");
        for (std::size_t start = 0; start < (std::size_t)n_vectors; start += chunk_rows) {
            const std::size_t count = std::min(chunk_rows, (std::size_t)n_vectors - start);
            psb_sign_shim::cuda(cudaMemcpy(d_chunk, host_vectors + start * dim, count * dim, cudaMemcpyHostToDevice), "cudaMemcpy");
            ::paraselect::search::psb_shim::check(psb_sign_encode_database(
                d_chunk, 1, (int64_t)count, d_centroids_, reinterpret_cast<const int64_t*>(d_cluster_offsets_), n_clusters, dim, padded,
                rotation_seed, (int64_t)start, d_codes_, d_reconstruction_scales_, dev, nullptr));
            psb_sign_shim::cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        }
        cudaFree(d_chunk);
    } catch (...) {
        if (d_chunk) cudaFree(d_chunk);
        release();
        throw;
    }
}

inline void Index::build_cached_u32(const std::uint32_t* host_codes, const float* host_scales, const float* host_centroids,
                                    const long long* host_cluster_offsets, int n_vectors, int n_clusters, int dim) {
    if (!host_codes || !host_scales || !host_centroids || !host_cluster_offsets || n_vectors <= 0 || n_clusters <= 0 || dim <= 0 ||
        dim % 32 != 0 || psb_sign_padded_dim(dim) < 0)
        throw std::invalid_argument("IVFResTurboQuant cached build received invalid input");
    psb_sign_shim::device();
    release();
    n_vectors_ = n_vectors; n_clusters_ = n_clusters; dim_ = dim; padded_dim_ = psb_sign_padded_dim(dim);
    words_per_code_ = padded_dim_ / 32; rotation_seed_ = PSB_SIGN_ROTATION_SEED;
    try {
        psb_sign_shim::renew(&d_centroids_, (std::size_t)n_clusters * dim);
        psb_sign_shim::renew(&d_cluster_offsets_, (std::size_t)n_clusters + 1);
        psb_sign_shim::renew(&d_codes_, (std::size_t)n_vectors * words_per_code_);
        psb_sign_shim::renew(&d_reconstruction_scales_, (std::size_t)n_vectors);
        psb_sign_shim::cuda(cudaMemcpy(d_centroids_, host_centroids, (std::size_t)n_clusters * dim * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
        psb_sign_shim::cuda(cudaMemcpy(d_cluster_offsets_, host_cluster_offsets, ((std::size_t)n_clusters + 1) * sizeof(long long), cudaMemcpyHostToDevice), "cudaMemcpy");
        psb_sign_shim::cuda(cudaMemcpy(d_codes_, host_codes, (std::size_t)n_vectors * words_per_code_ * sizeof(std::uint32_t), cudaMemcpyHostToDevice), "cudaMemcpy");
        psb_sign_shim::cuda(cudaMemcpy(d_reconstruction_scales_, host_scales, (std::size_t)n_vectors * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
    } catch (...) {
        release();
        throw;
    }
}

inline SearchWorkspace::~SearchWorkspace() { release(); }

inline void SearchWorkspace::release() {
    psb_sign_shim::drop(&d_queries_); psb_sign_shim::drop(&d_probe_ids_); psb_sign_shim::drop(&d_rotated_query_states_);
    psb_sign_shim::drop(&d_query_norm_sq_); psb_sign_shim::drop(&d_packed_query_states_); psb_sign_shim::drop(&d_query_norms_);
    psb_sign_shim::drop(&d_chunks_); psb_sign_shim::drop(&d_groups_); psb_sign_shim::drop(&d_query_group_starts_);
    psb_sign_shim::drop(&d_query_group_counts_); psb_sign_shim::drop(&d_group_indices_); psb_sign_shim::drop(&d_group_distances_);
    psb_sign_shim::drop(&d_candidate_ids_); psb_sign_shim::drop(&d_candidate_distances_);
    query_capacity_ = probe_capacity_ = chunk_capacity_ = group_capacity_ = 0;
    group_items_capacity_ = 0;
}

// Members used here: d_queries_, d_rotated_query_states_ / d_query_norm_sq_ (float states) or d_packed_query_states_ /
// d_query_norms_ (sign-coded states), d_query_group_starts_ as the int32 probe ids the library takes (ids outside the index
// become -1 and are skipped, as the reference skips them), d_candidate_ids_; group_items_capacity_ tracks the candidate buffer.
inline void SearchWorkspace::search_candidates(const Index& index, const float* host_queries, const long long* host_probe_ids,
                                               const long long* host_cluster_offsets, int n_queries, int n_probes,
                                               int* host_candidate_ids, int candidate_count, SearchTiming* timing,
                                               turboquant::TurboQuant1BitScoreMode score_mode, bool /*exact_selection*/) {
    if (!host_queries || !host_probe_ids || !host_cluster_offsets || !host_candidate_ids || n_queries <= 0 || n_probes <= 0 ||
        candidate_count <= 0 || candidate_count > kMaxCandidateCount || index.n_vectors_ <= 0)
        throw std::invalid_argument("IVFResTurboQuant search received invalid input");
    const auto begin = std::chrono::steady_clock::now();
    const int dev = psb_sign_shim::device();
    const std::size_t states = (std::size_t)n_queries * n_probes;
    std::vector<int> probes(states);
    bool any = false;
    for (std::size_t i = 0; i < states; ++i) {
        const long long c = host_probe_ids[i];
        const bool ok = c >= 0 && c < index.n_clusters_ && host_cluster_offsets[c + 1] > host_cluster_offsets[c];
        probes[i] = (c >= 0 && c < index.n_clusters_) ? (int)c : -1;
        any = any || ok;
    }
    if (!any) throw std::runtime_error("IVFResTurboQuant search generated no scan work");
    const bool float_states = score_mode == turboquant::TurboQuant1BitScoreMode::MseFloatQuery;
    if (n_queries > query_capacity_) {
        psb_sign_shim::renew(&d_queries_, (std::size_t)n_queries * index.dim_);
        query_capacity_ = n_queries;
    }
    if ((int)states > probe_capacity_) {
        psb_sign_shim::renew(&d_query_group_starts_, states);
        psb_sign_shim::renew(&d_rotated_query_states_, states * index.padded_dim_);
        psb_sign_shim::renew(&d_query_norm_sq_, states);
        psb_sign_shim::renew(&d_packed_query_states_, states * index.words_per_code_);
        psb_sign_shim::renew(&d_query_norms_, states);
        probe_capacity_ = (int)states;
    }
    const std::size_t items = (std::size_t)n_queries * candidate_count;
    if (items > group_items_capacity_) {
        psb_sign_shim::renew(&d_candidate_ids_, items);
        group_items_capacity_ = items;
    }
    psb_sign_shim::cuda(cudaMemcpy(d_queries_, host_queries, (std::size_t)n_queries * index.dim_ * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
    psb_sign_shim::cuda(cudaMemcpy(d_query_group_starts_, probes.data(), states * sizeof(int), cudaMemcpyHostToDevice), "cudaMemcpy");
    using ::paraselect::search::psb_shim::check;
    check(psb_sign_encode_queries(d_queries_, index.d_centroids_, d_query_group_starts_, n_queries, n_probes, index.n_clusters_, index.dim_,
                                  index.padded_dim_, index.rotation_seed_, float_states ? d_rotated_query_states_ : nullptr,
                                  float_states ? d_query_norm_sq_ : nullptr, float_states ? nullptr : d_packed_query_states_,
                                  float_states ? nullptr : d_query_norms_, dev, nullptr));
    check(psb_sign_search_candidates(float_states ? PSB_SIGN_FLOAT_STATES : PSB_SIGN_CODED_STATES, d_rotated_query_states_, d_query_norm_sq_,
                                     d_packed_query_states_, d_query_norms_, index.d_codes_, index.d_reconstruction_scales_,
                                     reinterpret_cast<const int64_t*>(index.d_cluster_offsets_), index.n_clusters_, d_query_group_starts_,
                                     n_queries, n_probes, index.padded_dim_, candidate_count, d_candidate_ids_, nullptr, dev, nullptr));
    psb_sign_shim::cuda(cudaMemcpy(host_candidate_ids, d_candidate_ids_, items * sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
    if (timing) {
        *timing = SearchTiming{};
        timing->total_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - begin).count();
    }
}

}  // namespace paraselect::search::ivf_res_turboquant
#endif  // PARASELECT_IVF_RES_TURBOQUANT_SEARCH_CUH

#endif  // PSB_VIEWS_HPP
