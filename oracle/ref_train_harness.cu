// TEST INFRASTRUCTURE, not product code.
//
// Exposes more of the reference's own CPU code through a C ABI for the tests: the IVF-Flat search and coarse loop
// (src/cpu/search/cpu_search.h:226-332), the CPU Lloyd k-means (src/cpu/clustering/cpu_kmeans.h:27-143) and the CPU PQ
// trainer / encoder (src/quantization/pq/pq_kmeans.cpp:12-74, src/quantization/pq/pq_quantizer_cpu.cpp:26-68).  The
// reference headers pull in CUB, so this file is compiled by nvcc as host code (no kernel is launched, no GPU is needed);
// the reference sources are compiled where they lie and nothing is copied from them.
#include "utils/pch.h"
#include "cpu/search/cpu_search.h"
#include "cpu/clustering/cpu_kmeans.h"
#include "quantization/pq/pq_quantizer.cuh"
#include "quantization/pq/pq_kmeans.h"
#include "transform/opq_cache.cuh"

#include <cstdint>
#include <cstring>
#include <random>
#include <vector>

bool g_ivf_debug_index_range = false;  // declared extern by the reference's pch.h

extern "C" {

// cpu_ivf_search on list-contiguous base rows; out_ids / out_dist [nq][topk], coarse_ids / coarse_dist [nq][nprobe] (optional).
int psbref_cpu_ivf_search(const float* queries, int nq, int dim, const float* base, const float* centroids, int nlist,
                          const int64_t* offsets, const int64_t* reordered_ids, int nprobe, int topk, int64_t* out_ids,
                          float* out_dist, int64_t* coarse_ids, float* coarse_dist) {
    std::vector<idx_t> off(offsets, offsets + nlist + 1);
    std::vector<int> counts((size_t)nlist);
    for (int l = 0; l < nlist; ++l) counts[(size_t)l] = (int)(offsets[l + 1] - offsets[l]);
    ClusterInfo info{off.data(), counts.data(), nlist};
    std::vector<idx_t*> oi((size_t)nq), ci((size_t)nq);
    std::vector<float*> od((size_t)nq), cd((size_t)nq);
    std::vector<idx_t> ids((size_t)nq * topk), cids((size_t)nq * nprobe);
    std::vector<float> cdist((size_t)nq * nprobe);
    for (int q = 0; q < nq; ++q) {
        oi[(size_t)q] = ids.data() + (size_t)q * topk; od[(size_t)q] = out_dist + (size_t)q * topk;
        ci[(size_t)q] = cids.data() + (size_t)q * nprobe; cd[(size_t)q] = cdist.data() + (size_t)q * nprobe;
    }
    std::vector<idx_t> rid;
    if (reordered_ids) rid.assign(reordered_ids, reordered_ids + offsets[nlist]);
    cpu_ivf_search(nq, dim, nlist, nprobe, topk, queries, base, centroids, info, L2_DISTANCE, oi.data(), od.data(), ci.data(), cd.data(),
                   reordered_ids ? rid.data() : nullptr);
    for (size_t i = 0; i < ids.size(); ++i) out_ids[i] = (int64_t)ids[i];
    if (coarse_ids) for (size_t i = 0; i < cids.size(); ++i) coarse_ids[i] = (int64_t)cids[i];
    if (coarse_dist) std::memcpy(coarse_dist, cdist.data(), sizeof(float) * cdist.size());
    return 0;
}

// cpu_kmeans_lloyd: centroids [k][dim] in/out, assign [n] out (the assignment of the LAST iteration, made against the centroids
// that iteration started from), objective of that iteration.
int psbref_cpu_kmeans_lloyd(const float* data, int n, int dim, int k, int iters, float* centroids, int* assign, float* objective) {
    KMeansCase cfg{};
    cfg.n = n; cfg.dim = dim; cfg.k = k; cfg.iters = iters; cfg.minibatch_iters = 0; cfg.seed = 0; cfg.dist = L2_DISTANCE;
    cpu_kmeans_lloyd(cfg, data, assign, centroids, objective);
    return 0;
}

// PQQuantizerCPU: train (25 iterations, seeds 42 + m) on data [n][dim], codebook [M][K][dim / M] out, codes [n][M] out.
int psbref_pq_train_encode(const float* data, int n, int dim, int M, int K, float* codebook, uint8_t* codes) {
    ivf::PQQuantizerCPU pq(M, K);
    pq.train(data, n, dim);
    if (pq.get_sub_dim() == 0) return 1;
    std::memcpy(codebook, pq.get_codebooks().data(), sizeof(float) * pq.get_codebooks().size());
    pq.encode(data, n, dim, codes);
    return 0;
}

// The initial codeword rows pq_kmeans_subspace draws for a seed: K draws of std::uniform_int_distribution<int>(0, n - 1) from
// std::mt19937(seed) (src/quantization/pq/pq_kmeans.cpp:25-31), made here with the same standard-library calls.
int psbref_pq_init_rows(int n, int K, unsigned seed, int* rows) {
    std::mt19937 gen(seed);
    std::uniform_int_distribution<int> dist(0, n - 1);
    for (int k = 0; k < K; ++k) rows[k] = dist(gen);
    return 0;
}

// pq_kmeans_subspace itself on one sub-space.
int psbref_pq_kmeans_subspace(const float* sub, int n, int dsub, int K, int iters, unsigned seed, float* out) {
    ivf::pq_kmeans_subspace(sub, n, dsub, K, iters, seed, out);
    return 0;
}

// The reference's OPQ rotation file (transform/opq_cache.cu): save under its own key, and load.
int psbref_opq_save(const char* dir, const char* dataset, int n, int train_n, int dim, int m, int k, int opq_iters, int pq_iters,
                    unsigned seed, const float* rotation, char* key_out, int cap) {
    try {
        paraselect::transform::OPQTrainSpec spec;
        spec.n = train_n; spec.dim = dim; spec.pq_m = m; spec.pq_k = k; spec.opq_iters = opq_iters; spec.pq_iters = pq_iters; spec.seed = seed;
        const std::string key = paraselect::transform::make_opq_cache_key(dataset, n, dim, spec);
        paraselect::transform::save_opq_rotation_cache(dir, key, spec, std::vector<float>(rotation, rotation + (size_t)dim * dim));
        if (key_out && cap > 0) { std::strncpy(key_out, key.c_str(), (size_t)cap - 1); key_out[cap - 1] = 0; }
        return 0;
    } catch (const std::exception&) { return 1; }
}
int psbref_opq_load(const char* dir, const char* key, int dim, float* rotation) {
    std::vector<float> r;
    if (!paraselect::transform::load_opq_rotation_cache(dir, key, dim, r)) return 2;
    std::memcpy(rotation, r.data(), r.size() * sizeof(float));
    return 0;
}

}  // extern "C"
