// Host-callable launchers of the CUDA kernels (all asynchronous on the given stream).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/psb.h"

namespace psb {

// ---- limits shared by host validation and kernels -----------------------------------------------
constexpr int kMaxProbe = 4096;       // nprobe and coarse top-k
constexpr int kMaxStage1 = 2048;      // candidates kept per query by the ADC stage
constexpr int kMaxTopk = 2048;
constexpr int kMaxRerankWidth = 4096; // candidates per query accepted by the rerank operator
constexpr int kPoolCapMax = 16384;    // per-query admission pool entries
constexpr int kScanChunkRows = 16384; // rows per scan work item
constexpr int kMaxCodebook = 256;

// Power of two (the selection kernel sorts the pool padded to a power of two in shared memory).
inline int pool_capacity(int stage1_k) {
    int c = 1024;
    while (c < 16 * stage1_k && c < kPoolCapMax) c <<= 1;
    return c;
}

// ---- coarse ---------------------------------------------------------------------------------------
// Exact fp32 distance matrix tile: dist[q][c] = sum_d (queries[q][d] - centroids[c][d])^2 evaluated as the
// sequential non-fused sum.  dist is [nq][nlist].
psb_status launch_coarse_dist_exact(const float* d_queries, int nq, const float* d_centroids, int nlist,
                                    int dim, float* d_dist, cudaStream_t s);
// Per query the k smallest (distance, id) pairs of a [nq][n] distance matrix, sorted ascending.
psb_status launch_select_rows(const float* d_dist, int nq, int n, int k, int* d_ids, float* d_out,
                              cudaStream_t s);

// ---- coarse, tensor-core filter (coarse_tc.cu) ----------------------------------------------------------------
struct CoarseTcIndex {
    const float* centroids;  // [nlist][dim] fp32 (exact re-scoring)
    const void* cb;          // [nlist][dimp] bf16, centred on mu
    const float* cn2;        // [tiles * 256] |c'|^2 (+inf padding)
    const float* mu;         // [dim] mean centroid
    float cmax;              // max |c'|
    int nlist, dim;
};
struct CoarseTcWorkspace {
    void* qb;        // [nq][dimp] bf16
    float* qnorm;    // [nq]
    float* gmin;     // [nq][groups]
    float* seltop;   // [nq][nprobe]
    int* selids;     // [nq][nprobe]
    int* cand_cnt;   // [nq]
    int* cand;       // [nq][mask words]: pass 2's candidate bit mask, one bit per (padded) centroid
    int* fail_list;  // [nq]
    int* n_fail;     // [2]: count, cursor
    int* status;     // [1]
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // optional: begin/end of GEMM pass 1 and pass 2
    int test_wait_limit = 0, test_skip_loads = 0;              // test hooks of the time-out path (0: off)
};
int coarse_tc_padded_dim(int dim);
int coarse_tc_tiles(int nlist);
int coarse_tc_cand_cap();
int coarse_tc_mask_words(int nlist);
int coarse_tc_group(int nlist, int nprobe);
bool coarse_tc_supported(int nq, int nlist, int dim, int nprobe);
// d_cb [nlist][dimp] bf16, d_cn2 [tiles*256], d_cnorm [nlist] out.
psb_status launch_tc_prep_centroids(const float* d_centroids, int nlist, int dim, const float* d_mu, void* d_cb,
                                    float* d_cn2, float* d_cnorm, cudaStream_t s);
psb_status launch_coarse_tc(const CoarseTcIndex& ix, const CoarseTcWorkspace& ws, const float* d_queries, int nq,
                            int nprobe, int* d_ids, float* d_dist, int sm_count, cudaStream_t s);

// Nearest centroid of every row with a previous assignment at hand (d_prev [nq]; may alias d_ids): the row's distance to its
// previous centroid bounds the nearest distance, so the filter GEMM runs once instead of twice.  Same results as
// launch_coarse_tc(..., nprobe = 1, ...).
psb_status launch_coarse_tc_assign(const CoarseTcIndex& ix, const CoarseTcWorkspace& ws, const float* d_rows, int nq, const int* d_prev,
                                   int* d_ids, float* d_dist, int sm_count, cudaStream_t s);

// ---- OPQ rotation --------------------------------------------------------------------------------------
// d_out [n][dim] = rows of d_in times the transpose of d_matrix (row-major [out][in]): out[r][o] = sum_i M[o][i] in[r][i], one
// in-order fp32 fma chain per element.  d_out must not alias d_in.
psb_status launch_rotate_rows(const float* d_in, const float* d_matrix, long long n, int dim, float* d_out, cudaStream_t s);

// ---- TurboQuant 1-bit residual codec (sign_codec.cu) ----------------------------------------------------------
int sign_padded_dim(int dim);   // 32, 64, 128 or 256; -1 above 256
psb_status launch_sign_scale(int padded_dim, float* d_out, cudaStream_t s);   // the device's rsqrtf(padded_dim)
// Any of d_rotated [n][padded], d_codes [n][padded / 32], d_norms [n], d_norm_sq [n] may be null.
psb_status launch_sign_rotate(const float* d_rows, long long n, int dim, int padded_dim, uint32_t seed, float* d_rotated,
                              uint32_t* d_codes, float* d_norms, float* d_norm_sq, int sm_count, cudaStream_t s);
// Rows [row_offset, row_offset + n) of a list-contiguous index; codes and scales are indexed by global row.
psb_status launch_sign_encode_database(const void* d_rows, int elem_bytes, long long n, const float* d_centroids,
                                       const long long* d_offsets, int nlist, int dim, int padded_dim, uint32_t seed,
                                       long long row_offset, uint32_t* d_codes, float* d_scales, int sm_count, cudaStream_t s);
psb_status launch_sign_encode_queries(const float* d_queries, const float* d_centroids, const int* d_probes, int nq, int nprobe,
                                      int nlist, int dim, int padded_dim, uint32_t seed, float* d_states, float* d_norm_sq,
                                      uint32_t* d_state_codes, float* d_norms, int sm_count, cudaStream_t s);
// mode 0: float states + norm_sq against reconstruction scales; mode 1: sign-coded states + norms against row norms.
psb_status launch_sign_candidates(int mode, const float* d_states, const float* d_norm_sq, const uint32_t* d_state_codes,
                                  const float* d_norms, const uint32_t* d_codes, const float* d_row_params,
                                  const long long* d_offsets, int nlist, const int* d_probes, int nq, int nprobe, int padded_dim,
                                  int candidate_count, int* d_rows_out, float* d_dist_out, int sm_count, cudaStream_t s);

// ---- PQ lookup tables --------------------------------------------------------------------------------
psb_status launch_build_lut(const float* d_queries, int nq, int dim, const float* d_codebook, int m, int k,
                            float* d_lut, cudaStream_t s);

// ---- schedule + scan -----------------------------------------------------------------------------------
struct ScanWorkspace {
    // per list
    int* vis_count;      // [nlist]
    int* vis_off;        // [nlist + 1]
    int* vis_cursor;     // [nlist]
    long long* item_off; // [nlist + 1]
    // per (query, probe)
    int* visitors;       // [max_batch * nprobe]
    // per query
    long long* q_rows;   // [max_batch] rows this query scans
    float* thr;          // [max_batch] admission cutoff
    int* pool_cnt;       // [max_batch]
    uint64_t* pool;      // [max_batch][pool_cap]
    int* fail_list;      // [max_batch]
    // scalars (device)
    int* n_fail;         // [1]
    int* fail_cursor;    // [1]
    unsigned long long* work_cursor; // [1]
    unsigned long long* counters;    // [4]: scanned rows, admitted, fallback queries, survivors of the tensor-core filter
    // tensor-core pre-filter scan (scan_tc.cu)
    long long* item_off_tc = nullptr;            // [nlist + 1] work items of the lists the tensor-core kernel takes
    unsigned long long* work_cursor_tc = nullptr;
    int* tc_status = nullptr;                    // [1] != 0 after a bounded wait of the tensor-core kernel gave up
    int tc_min_visitors = 0;                     // lists with at least this many visiting queries go to the tensor-core kernel (0 = 1)
    int tc_wait_limit = 0, tc_skip_mma = 0;      // test hooks of the time-out path
    int pool_cap;
    void* lut_h = nullptr;       // [tables][m*k] fp16 tables (tables = max_batch, x nprobe in residual mode) for the half pre-filter scan (null = fp32 scan only)
    float* lut_scale = nullptr;  // [tables]
    int scan_mode = 0;           // 0 = auto: tensor-core pre-filter when the call has the queries and the shape fits, else the
                                 //     SIMT half pre-filter, else the fp32 scan; 1 = fp32 SIMT scan only; 2 = SIMT scans only;
                                 //     3 = tensor-core pre-filter required
    uint64_t* fallback_partial = nullptr;  // [fallback_partial_bytes(stage1_k)]: partial top lists of the split exact fallback
    bool half_tables_ready = false;  // lut_h / lut_scale already hold this call's tables (launch_build_tables_residual)
    float seed_sigma = 0.f;      // margin of the sampled cutoff in standard deviations (0 = default)
    int cap_queries = 0;         // queries the per-query buffers above hold (launch_scan refuses more)
    long long cap_tables = 0;    // tables lut_h / lut_scale hold
    int reserve_ctas = 0;        // CTAs left out of the scan's persistent grid, so that kernels of another stream that
                                 // cannot share an SM with a scan CTA (a collective's) still find a free SM
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;  // optional: bracket the scan kernel
    // Sharded search: the cutoff of a query is placed on the rows of ALL shards.  Phase 1 (schedule + sampling) leaves each
    // query's smallest sample keys in seed_export; the caller exchanges these records between the shards; phase 2 places the
    // cutoff from every shard's records (seed_all) and runs the scan and the selection, which then no longer asks for
    // stage1_k rows of this shard alone.
    int phase = 0;                         // 0 = the whole scan, 1 = schedule + sampling only, 2 = cutoff from seed_all + scan + selection
    uint32_t* seed_export = nullptr;       // phase 1: [nq][seed_words]
    const uint32_t* seed_all = nullptr;    // phase 2: [seed_shards][nq][seed_words]
    int seed_shards = 0;
    int seed_keys = 0;                     // keys per record; a record is seed_keys + kSeedTail words
    long long* rows_global = nullptr;      // phase 2, optional: [nq] rows the query scans on all shards together
};
constexpr int kSeedTail = 4;               // words after the keys of a sample record: stride, key count, rows scanned (low, high)
// Keys per sample record of launch_scan's phase 1 for a candidate count and margin (a multiple of 32).
int seed_record_keys(int stage1_k, float sigma);

struct ScanIndex {
    const uint8_t* codes;      // device, shard rows only
    const long long* offsets;  // device [nlist + 1], global rows
    long long row_base;        // global row of codes[0]
    const long long* row_delta = nullptr;  // device [nlist] or null: reported row = scanned row + row_delta[list]
    int nlist;
    int list_begin, list_end;  // shard
    int m, k;
    // Residual ADC mode: codes encode x - centroid[list], so every (query, probe) pair has its own table.
    // d_lut then holds [nq * nprobe][m*k] tables (pair order) and the visitor lists carry pair indices.
    bool residual = false;
    // for the tensor-core pre-filter scan and the re-scoring selection
    const float* centroids = nullptr;  // device [nlist][dim]
    const float* codebook = nullptr;   // device [m][k][dim / m]
    const void* row_aug = nullptr;     // device [shard rows] x 8 bytes (launch_row_aug), null: no tensor-core scan
    const float* row_bias = nullptr;   // residual mode: device [shard rows] per-row correction as fp32 (launch_row_bias), or
    const uint16_t* row_bias_u16 = nullptr;  // the caller's affine u16 form of it (value = rc_offset + rc_scale * u16)
    float rc_scale = 0.f, rc_offset = 0.f;
    int dim = 0;
};

// ---- tensor-core pre-filter scan (scan_tc.cu) ------------------------------------------------------------------
// Whether the tensor-core scan supports the shape (dsub 2, 4 or 8, dim a multiple of 8, m of 4, operands within shared memory).
bool scan_tc_supported(int dim, int m, int k);
// Per-row terms of the tensor-core scan, computed once per index: d_out [rows] of 8 bytes (the extra K slots of each code row).
// Residual mode: value[row] = |recon(row)|^2 + 2 <centroid[list(row)], recon(row)> for every row of the shard: the per-row
// correction of the reference's shared-table form (src/common/row_correction.h:37-45).
psb_status launch_row_bias(const uint8_t* d_codes, const long long* d_offsets, long long row_base, int list_begin, int list_end,
                           int dim, int m, int k, const float* d_codebook, const float* d_centroids, float* d_out, cudaStream_t s);
psb_status launch_row_aug(const uint8_t* d_codes, long long rows, int dim, int m, int k, const float* d_codebook, void* d_out,
                          cudaStream_t s);
struct ScanTcLaunch {
    const float* queries; const float* centroids; const float* codebook; const int* probes;
    const void* row_aug;
    const uint8_t* codes; const long long* offsets; long long row_base;
    int nlist, dim, m, k, lut_div; bool residual;
    const int* vis_count; const int* vis_off; const int* visitors; const long long* item_off;
    const float* thr; int* pool_cnt; uint64_t* pool; int pool_cap;
    unsigned long long* work_cursor; unsigned long long* counters; int* status;
    int chunk_rows, reserve_ctas, sm_count, wait_limit, skip_mma;
};
psb_status launch_scan_tc(const ScanTcLaunch& L, cudaStream_t s);
// Selection over pools that may hold unscored survivors of the tensor-core filter (re-scored exactly here).
struct SelectRescoreLaunch {
    const uint64_t* pool; const int* pool_cnt; int pool_cap; const long long* q_rows; const float* thr; int stage1_k;
    const float* lut; const float* queries; const float* centroids; const float* codebook; const int* probes;
    int nprobe, dim, nlist; const uint8_t* codes; long long row_base; const long long* row_delta;
    int m, k; bool residual, tree;
    int* out_rows; float* out_dist; int* out_count; int* fail_list; int* n_fail; unsigned long long* counters;
    bool shared_cut = false;
};
psb_status launch_select_rescore(const SelectRescoreLaunch& L, int nq, cudaStream_t s);

// Tables of the residual mode: table (q, p) is built on queries[q] - centroids[probes[q][p]] (pairs whose probe is
// outside [0, nlist) are left untouched).  d_lut [nq * nprobe][m*k].
psb_status launch_build_lut_residual(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe,
                                     const float* d_centroids, int nlist, const float* d_codebook, int m, int k,
                                     float* d_lut, cudaStream_t s);

// Affine u8 quantisation of `tables` fp32 tables [m][k]: d_q8 [tables][m][k], d_scales [tables][m], d_lo_sum / d_inflation [tables].
psb_status launch_lut_to_u8(const float* d_lut, long long tables, int m, int k, int residual, uint8_t* d_q8, float* d_scales,
                            float* d_lo_sum, float* d_inflation, cudaStream_t s);

// d_cb_maxnorm [m]: per sub-quantiser the largest codeword norm (bounds a table's entries without a pass over them).
// Residual tables, fp32 and fp16 (ws.lut_h, ws.lut_scale) in one kernel, when residual_tables_fused(); the following
// launch_scan takes ws.half_tables_ready = true and skips its own conversion.
size_t fallback_partial_bytes(int stage1_k);
bool residual_tables_fused(const ScanWorkspace& ws, int m, int k);
psb_status launch_build_tables_residual(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe,
                                        const float* d_centroids, int nlist, const float* d_codebook, int m, int k,
                                        const float* d_cb_maxnorm, float* d_lut, const ScanWorkspace& ws, cudaStream_t s);

// d_queries [nq][dim] may be null: the tensor-core pre-filter then stays out and the SIMT scans take every list.
psb_status launch_scan(const ScanIndex& ix, const ScanWorkspace& ws, const float* d_lut, int nq,
                       const int* d_probes, int nprobe, int stage1_k, int* d_rows, float* d_dist,
                       int* d_count, int sm_count, cudaStream_t s, const float* d_queries = nullptr);

// ---- IVF-Flat fine scan (flat.cu) ------------------------------------------------------------------------------
// Exact fp32 distances of every query to the rows of its probed lists (device-resident rows, list-contiguous) and the topk
// nearest by (distance, row).  d_out_rows [nq][topk] list-contiguous rows (-1 pad), d_out_dist (FLT_MAX pad).
psb_status launch_flat_scan(const float* d_queries, int nq, int dim, const int* d_probes, int nprobe, const long long* d_offsets,
                            int nlist, const float* d_rows, long long row_base, int topk, int* d_out_rows, float* d_out_dist,
                            unsigned long long* d_counters, cudaStream_t s);

// ---- rerank ------------------------------------------------------------------------------------------------
// Which rows of the index-wide (list-contiguous) numbering a session's exact store and id table hold.
//   global_begin == nullptr: rows [base, base + count), stored in that order.
//   otherwise (striped shard): for every list l the rows [global_begin[l], global_begin[l] + len_l), stored at local
//   rows [local_offsets[l], local_offsets[l + 1]).
struct RowMap {
    const long long* global_begin = nullptr;   // device [nlist]
    const long long* local_offsets = nullptr;  // device [nlist + 1]
    int nlist = 0;
    long long base = 0;
    long long count = 0;
};
// Copies the candidate rows held here (fp32 or u8, elem_bytes 4 or 1) from src (device-visible: mapped host or
// device) to stage [nq][candidate_count][dim].  Candidates are global rows.  compact_ctas > 0: the kernel runs beside a scan
// on another stream as that many lean CTAs; owned_sms > 0 (takes precedence): as that many CTAs that each keep an SM to
// themselves.
psb_status launch_gather_rows(const void* src, const RowMap& mp, int dim, int elem_bytes, const int* d_candidates,
                              int nq, int candidate_count, int candidate_stride, const int* d_counts,
                              void* d_stage, cudaStream_t s, int sm_count, int compact_ctas = 0, int owned_sms = 0);
// d_out_dist [nq][candidate_count]: exact distance of each staged candidate, +inf for rows not held here.
psb_status launch_rerank_score(const void* d_stage, const RowMap& mp, int dim, int elem_bytes, const void* d_queries,
                               const int* d_candidates, int nq, int candidate_count, int candidate_stride,
                               const int* d_counts, float* d_out_dist, cudaStream_t s);
// Per query the topk (distance,row) pairs without duplicates from d_dist [nq][candidate_count].
psb_status launch_topk_select(const float* d_dist, const int* d_candidates, int nq, int candidate_count,
                              int candidate_stride, const int* d_counts, int topk, int* d_out_rows,
                              float* d_out_dist, cudaStream_t s);
psb_status launch_map_ids(const int* d_rows, long long n, const long long* d_reordered, const RowMap& mp,
                          long long* d_out, cudaStream_t s);
psb_status launch_merge(const int* d_rows, const float* d_dist, int parts, int nq, int k, int* d_out_rows,
                        float* d_out_dist, cudaStream_t s);
psb_status launch_offset_rows(int* d_rows, long long n, int delta, cudaStream_t s);
psb_status launch_widen_ids(const int* d_in, long long n, long long* d_out, cudaStream_t s);

// ---- training ------------------------------------------------------------------------------------------------
psb_status launch_pq_encode(const float* d_data, long long n, int dim, const float* d_codebook, int m, int k,
                            uint8_t* d_codes, cudaStream_t s);
// Nearest codeword per sub-vector for the Lloyd iterations of PQ training (|c|^2 - 2 x.c with fused multiply-adds; the exact
// encoder's arithmetic is launch_pq_encode).  Falls back to launch_pq_encode for sub-vector lengths other than 2, 4, 8.
psb_status launch_pq_assign_train(const float* d_data, long long n, int dim, const float* d_codebook, int m, int k,
                                  uint8_t* d_codes, cudaStream_t s);
psb_status launch_pq_accumulate(const float* d_data, long long n, int dim, const uint8_t* d_codes, int m, int k,
                                double* d_sums, int* d_counts, cudaStream_t s);
psb_status launch_pq_update(const double* d_sums, const int* d_counts, int m, int k, int dsub, float* d_codebook,
                            cudaStream_t s);
// Initial codewords taken from given data rows: d_rows [m][k] (row of the data for codeword c of subspace sub).
psb_status launch_pq_init_rows(const float* d_data, int dim, int m, int k, const long long* d_rows, float* d_codebook, cudaStream_t s);
psb_status launch_pq_init(const float* d_data, long long n, int dim, int m, int k, uint64_t seed,
                          float* d_codebook, cudaStream_t s);
// Workspace of the k-means accumulation: rows grouped by centroid (order [n], offsets [k + 1], cursor [k], all int32).
struct KmeansAccumWs { int* order = nullptr; int* offsets = nullptr; int* cursor = nullptr; };
// d_counts [k] and *d_obj zeroed by the caller; d_sums [k][dim] is written whole (zeros for a centroid without rows).
psb_status launch_kmeans_accumulate(const float* d_data, long long n, int dim, const int* d_assign, const float* d_best, int k,
                                    double* d_sums, int* d_counts, double* d_obj, const KmeansAccumWs& ws, cudaStream_t s);
psb_status launch_residual_rows(const float* d_data, long long n, int dim, const float* d_centroids, const int* d_assign,
                                float* d_out, cudaStream_t s);
psb_status launch_kmeans_update(const double* d_sums, const int* d_counts, int k, int dim, float* d_centroids,
                                cudaStream_t s);

// ---- synthetic data --------------------------------------------------------------------------------------------
psb_status launch_gen_mixture(const float* d_centres, const long long* d_offsets, int ncomp, int dim, float sigma,
                              uint64_t seed, long long row_begin, long long n, float* d_out, cudaStream_t s);
psb_status launch_gen_normal(uint64_t seed, long long first, long long n, float scale, float* d_out,
                             cudaStream_t s);

// What the group layer (group.cu) needs to know of a session.
struct SessionShape {
    int dim = 0, m = 0, k = 0, nlist = 0, n_rerank = 0, exact_elem = 0, device = 0;
    bool residual = false, flat = false;
    cudaStream_t stream = nullptr;
};
}  // namespace psb
struct psb_session;
namespace psb {
SessionShape session_shape(const psb_session* s);

}  // namespace psb
