/*
 * psb_views.hpp - header-only C++ shim: ParaSelect's own entry points for the IVF search hot path, implemented on the
 * C ABI of psb.h.
 *
 * A caller of the reference keeps its code as it is - it fills the reference's request structs and calls
 *     paraselect::search::ivfrespq_search(request, stats)        src/search/ivfrespq/ivfrespq_search.cuh:114-116
 *     paraselect::search::IVFResPQSession(request).search(stats)  src/search/ivfrespq/ivfrespq_search.cuh:120-133
 *     paraselect::search::ivfflat_search(request, stats)          src/search/ivfflat/ivfflat_search.cuh:49-51
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

#endif  // PSB_VIEWS_HPP
