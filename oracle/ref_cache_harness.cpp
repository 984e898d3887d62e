// TEST INFRASTRUCTURE: C entry points around the reference's own cache code (dataset/cache/cluster_cache.cpp,
// dataset/cache/residual_pq_cache.cpp, dataset/cache/cache_manifest.h), compiled in place from the reference checkout.
// Nothing of the product links this.
#include <cstdint>
#include <cstring>
#include <exception>
#include <cstdio>
#include <string>

#include "dataset/cache/cache_manifest.h"
#include "dataset/cache/cluster_cache.h"
#include "dataset/cache/plain_pq_cache.h"
#include "dataset/cache/residual_pq_cache.h"
#include "dataset/cache/turboquant_cache.h"

using namespace paraselect::dataset;

namespace {
void put(char* dst, int cap, const std::string& s) {
    if (!dst || cap <= 0) return;
    std::strncpy(dst, s.c_str(), (size_t)cap - 1);
    dst[cap - 1] = 0;
}
PQCacheRequest pq_request(int n, int dim, int nlist, const char* layout, int m, int k, int iters, int residual, int train_rows) {
    PQCacheRequest r;
    if (residual) {
        r.n_vectors = n; r.dim = dim; r.n_lists = nlist; r.pq_m = m; r.pq_k = k; r.pq_iters = iters;
    } else {
        r = make_plain_pq_cache_request(n, dim, nlist, m, k, iters, train_rows);
    }
    r.cluster_layout_id = layout;
    return r;
}
}  // namespace

extern "C" {

// ClusterCache::save; entry_out receives the published directory's layout id.
int ref_cluster_save(const char* root, const char* dataset, int n, int nlist, int dim, const char* recipe_json, const float* centroids,
                     const int64_t* reordered, const int* counts, const int64_t* offsets) {
    try {
        ClusterCache cache(root);
        ClusterCacheSpec spec{n, nlist, dim, recipe_json, ""};
        cache.save(dataset, spec, centroids, reinterpret_cast<const idx_t*>(reordered), counts, reinterpret_cast<const idx_t*>(offsets), nlist);
        return 0;
    } catch (const std::exception&) { return 1; }
}

// ClusterCache::try_load; returns 0 on a hit (arrays filled), 2 on a miss, 1 after an exception.
int ref_cluster_load(const char* root, const char* dataset, int n, int nlist, int dim, const char* recipe_json, const char* layout_in,
                     float* centroids, int64_t* reordered, int* counts, int64_t* offsets, char* entry_out, char* layout_out, int cap) {
    try {
        ClusterCache cache(root);
        ClusterCacheSpec spec{n, nlist, dim, recipe_json, layout_in ? layout_in : ""};
        const auto r = cache.try_load(dataset, spec);
        if (!r.hit) return 2;
        std::memcpy(centroids, r.centroids.data(), r.centroids.size() * sizeof(float));
        std::memcpy(reordered, r.reordered_indices.data(), r.reordered_indices.size() * sizeof(int64_t));
        std::memcpy(counts, r.cluster_counts.data(), r.cluster_counts.size() * sizeof(int));
        std::memcpy(offsets, r.cluster_offsets.data(), r.cluster_offsets.size() * sizeof(int64_t));
        put(entry_out, cap, r.entry_dir);
        put(layout_out, cap, r.layout_id);
        return 0;
    } catch (const std::exception&) { return 1; }
}

int ref_pq_save(const char* root, const char* dataset, int n, int dim, int nlist, const char* layout, int m, int k, int iters, int residual,
                int train_rows, const float* codebook, const uint8_t* codes) {
    try {
        ResidualPQCache cache(root, dataset);
        cache.save(pq_request(n, dim, nlist, layout, m, k, iters, residual, train_rows), codebook, codes);
        return 0;
    } catch (const std::exception&) { return 1; }
}

int ref_pq_load(const char* root, const char* dataset, int n, int dim, int nlist, const char* layout, int m, int k, int iters, int residual,
                int train_rows, float* codebook, uint8_t* codes, char* entry_out, int cap) {
    try {
        ResidualPQCache cache(root, dataset);
        const auto r = cache.try_load(pq_request(n, dim, nlist, layout, m, k, iters, residual, train_rows));
        if (!r.hit) return 2;
        std::memcpy(codebook, r.codebook.data(), r.codebook.size() * sizeof(float));
        std::memcpy(codes, r.codes.data(), r.codes.size());
        put(entry_out, cap, r.entry_dir);
        return 0;
    } catch (const std::exception&) { return 1; }
}

// cache_manifest::storage_id of a manifest given as JSON text.
int ref_storage_id(const char* manifest_json, char* out, int cap) {
    try { put(out, cap, cache_manifest::storage_id(cache_manifest::Json::parse(manifest_json))); return 0; }
    catch (const std::exception&) { return 1; }
}
// cache_manifest::matches(actual, expected) on JSON text: 1 / 0, -1 after an exception.
int ref_manifest_matches(const char* actual_json, const char* expected_json) {
    try { return cache_manifest::matches(cache_manifest::Json::parse(actual_json), cache_manifest::Json::parse(expected_json)) ? 1 : 0; }
    catch (const std::exception&) { return -1; }
}


// TurboQuantCache: publish_staged over payload files written here in the reference's binary layout (u32 n, u32 dim, data), and
// try_map.  `staged` must exist; it is renamed to the canonical entry.
static int write_payload(const std::string& path, uint32_t n, uint32_t dim, const void* data, size_t elem) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return 1;
    const uint32_t header[2] = {n, dim};
    const bool ok = std::fwrite(header, sizeof(header), 1, f) == 1 && std::fwrite(data, elem, (size_t)n * dim, f) == (size_t)n * dim;
    return (std::fclose(f) == 0 && ok) ? 0 : 1;
}
static TurboQuantCacheRequest sign_request(int n, int dim, int nlist, int seed, const char* layout) {
    TurboQuantCacheRequest r;
    r.n_vectors = n; r.dim = dim; r.n_lists = nlist; r.rotation_seed = seed; r.cluster_layout_id = layout;
    return r;
}
int ref_sign_cache_publish(const char* root, const char* dataset, const char* staged, int n, int dim, int nlist, int seed, const char* layout,
                           const uint32_t* codes, const float* scales) {
    try {
        const auto spec = sign_request(n, dim, nlist, seed, layout);
        if (write_payload(std::string(staged) + "/codes.u32bin", (uint32_t)n, (uint32_t)spec.words_per_code(), codes, sizeof(uint32_t))) return 1;
        if (write_payload(std::string(staged) + "/scales.f32bin", (uint32_t)n, 1u, scales, sizeof(float))) return 1;
        TurboQuantCache cache(root, dataset);
        cache.publish_staged(staged, spec);
        return 0;
    } catch (const std::exception&) { return 1; }
}
int ref_sign_cache_map(const char* root, const char* dataset, int n, int dim, int nlist, int seed, const char* layout, uint32_t* codes,
                       float* scales, char* entry_out, int cap) {
    try {
        TurboQuantCache cache(root, dataset);
        const auto r = cache.try_map(sign_request(n, dim, nlist, seed, layout));
        if (!r.hit) return 2;
        std::memcpy(codes, r.codes.data(), r.codes.size() * sizeof(uint32_t));
        std::memcpy(scales, r.scales.data(), r.scales.size() * sizeof(float));
        put(entry_out, cap, r.entry_dir);
        return 0;
    } catch (const std::exception&) { return 1; }
}

}  // extern "C"
