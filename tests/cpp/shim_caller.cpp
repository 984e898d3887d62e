// TEST INFRASTRUCTURE.  A caller written against the reference's own headers - request structs filled the way the reference's
// callers fill them, then ivfrespq_search / IVFResPQSession / ivfflat_search - built with include/psb_views.hpp in place of
// the reference's implementation.  It has to compile and link unchanged; without a GPU the calls must surface the library's
// "no device" status as an exception, not fall back to anything.
#include "search/ivfrespq/ivfrespq_search.cuh"
#include "search/ivfflat/ivfflat_search.cuh"
#include "search/ivf_res_turboquant/ivf_res_turboquant_search.cuh"
#include "psb_views.hpp"

#include <cstdio>
#include <vector>

using namespace paraselect::search;

int main() {
    const int nlist = 4, dim = 8, n = 64, M = 4, K = 16, nq = 3, topk = 5, nprobe = 2;
    std::vector<float> centroids((size_t)nlist * dim, 0.f), codebook((size_t)M * K * (dim / M), 0.f), rows((size_t)n * dim, 0.f);
    std::vector<float> queries((size_t)nq * dim, 0.f), dist((size_t)nq * topk);
    std::vector<idx_t> offsets = {0, 16, 32, 48, 64}, ids((size_t)n), out((size_t)nq * topk);
    std::vector<uint8_t> codes((size_t)n * M, 0);
    for (int i = 0; i < n; ++i) ids[(size_t)i] = i;

    IVFResPQSearchRequest req;
    req.index.coarse = {centroids.data(), nlist, dim};
    req.index.lists.offsets = offsets.data();
    req.index.lists.reordered_ids = ids.data();
    req.index.lists.nlist = nlist;
    req.index.lists.n_vectors = n;
    req.index.storage.pq.codes = codes.data();
    req.index.storage.pq.codebook = codebook.data();
    req.index.storage.pq.subvectors = M;
    req.index.storage.pq.codebook_size = K;
    IVFHostStorageView host;
    host.fp32 = rows.data(); host.count = n; host.dim = dim;
    req.index.storage.assets.exact = IVFExactStorageView::from_host(host);
    req.queries.fp32 = queries.data(); req.queries.count = nq; req.queries.dim = dim;
    req.params.nprobe = nprobe; req.params.topk = topk; req.params.batch_size = nq;
    req.output.indices = out.data(); req.output.distances = dist.data();
    req.options.n_rerank = 20;
    req.options.pq_distance_mode = PQAdcDistanceMode::Plain;

    int rc = 0;
    try {
        IVFSearchStats stats;
        ivfrespq_search(req, &stats);
        IVFResPQSession session(req);
        session.search(&stats);
        std::printf("SEARCH_OK %d\n", (int)stats.numeric_fields.count("pq_adc_scan"));
    } catch (const std::invalid_argument& e) {
        std::printf("INVALID_ARGUMENT %s\n", e.what()); rc = 2;
    } catch (const std::runtime_error& e) {
        std::printf("RUNTIME_ERROR %s\n", e.what()); rc = 3;
    }
    try {  // a bad request must come back as std::invalid_argument, as from the reference
        IVFResPQSearchRequest bad = req;
        bad.params.nprobe = nlist + 1;
        ivfrespq_search(bad, nullptr);
    } catch (const std::invalid_argument& e) {
        std::printf("BAD_REQUEST_REFUSED\n");
    } catch (const std::runtime_error& e) {
        std::printf("BAD_REQUEST_RUNTIME %s\n", e.what());
    }
    IVFFlatSearchRequest freq;
    freq.index.coarse = req.index.coarse;
    freq.index.lists = req.index.lists;
    freq.index.storage.rowmajor_fp32 = rows.data();
    freq.queries = req.queries; freq.params = req.params; freq.output = req.output;
    try {
        ivfflat_search(freq, nullptr);
        std::printf("FLAT_OK\n");
    } catch (const std::runtime_error& e) {
        std::printf("FLAT_RUNTIME_ERROR %s\n", e.what());
    }
    // the 1-bit sign codec index of the reference, its members defined by the shim
    {
        const int sdim = 32, srows = 200, slists = 4, k = 16;
        std::vector<std::uint8_t> vec((size_t)srows * sdim);
        for (size_t i = 0; i < vec.size(); ++i) vec[i] = (std::uint8_t)((i * 37 + (i >> 5) * 11) & 255);
        std::vector<float> cen((size_t)slists * sdim, 100.f), q((size_t)2 * sdim, 90.f);
        std::vector<long long> off = {0, 50, 50, 120, 200}, pr = {0, 3, 2, 7};
        std::vector<int> cand((size_t)2 * k, -2);
        try {
            ivf_res_turboquant::Index index;
            index.build_u8(vec.data(), cen.data(), off.data(), srows, slists, sdim);
            ivf_res_turboquant::SearchWorkspace ws;
            ivf_res_turboquant::SearchTiming timing;
            ws.search_candidates(index, q.data(), pr.data(), off.data(), 2, 2, cand.data(), k, &timing);
            bool ok = index.bytes_per_vector() == 8;
            for (int i = 0; i < k; ++i) ok = ok && cand[(size_t)i] >= 0 && cand[(size_t)i] < srows;                       // lists 0 and 3: 130 rows
            for (int i = 0; i < k; ++i) ok = ok && cand[(size_t)k + i] >= 50 && cand[(size_t)k + i] < 120;                // list 2 only (7 is skipped)
            std::printf(ok ? "SIGN_OK\n" : "SIGN_WRONG\n");
        } catch (const std::invalid_argument& e) {
            std::printf("SIGN_INVALID_ARGUMENT %s\n", e.what());
        } catch (const std::runtime_error& e) {
            std::printf("SIGN_RUNTIME_ERROR %s\n", e.what());
        }
        try {
            ivf_res_turboquant::Index index;
            index.build_u8(vec.data(), cen.data(), off.data(), srows, slists, 300);
        } catch (const std::invalid_argument&) {
            std::printf("SIGN_BAD_REQUEST_REFUSED\n");
        } catch (const std::runtime_error& e) {
            std::printf("SIGN_BAD_REQUEST_RUNTIME %s\n", e.what());
        }
    }
    return rc;
}
