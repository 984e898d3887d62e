// TEST INFRASTRUCTURE: C entry point around the reference's own k-means initialisation (init_centroids_by_sampling, a host
// function inside clustering/kmeans/kmeans.cu), compiled in place from the reference checkout together with
// clustering/kmeans/kmeans_utils.cu.  Four functions of other translation units that only the Lloyd iterations call (the flash-assign variant, a CUTLASS
// translation unit that does not build here, and the row-norm launcher) are stubbed: the initialisation never calls them.  Nothing of the product links this, and no
// GPU is used.
#include "clustering/kmeans/kmeans.cuh"
#include "clustering/flash_kmeans/flash_kmeans_assign.cuh"
#include "l2norm/l2norm.cuh"

#include <cstdlib>

namespace paraselect::clustering::kmeans {
void reserve_flash_kmeans_assign_scratch_workspace(FlashKMeansAssignWorkspace&, int, int, const FlashKMeansAssignConfig&) { std::abort(); }
void release_flash_kmeans_assign_workspace(FlashKMeansAssignWorkspace&) {}
FlashKMeansAssignResult flash_kmeans_assign_l2_precomputed_norms(const float*, const float*, const float*, const float*, int, int, int, idx_t*,
                                                                  float*, const FlashKMeansAssignConfig&, FlashKMeansAssignWorkspace&,
                                                                  cudaStream_t) { std::abort(); }
}  // namespace paraselect::clustering::kmeans
// the row-norm kernel launcher of another translation unit (Lloyd iterations only)
void compute_l2_squared_gpu(const float*, float*, int, int, L2NormVersion, cudaStream_t) { std::abort(); }

extern "C" {

// policy: 0 = by the reference's n * k threshold, 1 = random rows (partial Fisher-Yates), 2 = k-means++.
int psbref_kmeans_init(int n, int dim, int k, int seed, int policy, const float* data, float* out_centroids) {
    KMeansCase cfg{};
    cfg.n = n; cfg.dim = dim; cfg.k = k; cfg.iters = 1; cfg.minibatch_iters = 1; cfg.seed = seed; cfg.dist = L2_DISTANCE;
    cfg.init_policy = policy == 1 ? KMEANS_INIT_FORCE_RANDOM : policy == 2 ? KMEANS_INIT_FORCE_KMEANSPP : KMEANS_INIT_AUTO_THRESHOLD;
    init_centroids_by_sampling(cfg, data, out_centroids);
    return 0;
}

}  // extern "C"
