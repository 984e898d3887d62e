/*
 * psb.h - C ABI of the B200 (sm_100a) IVF-PQ search path.
 *
 * Drop-in boundary for ParaSelect's IVF search hot path: the structs below mirror the reference's
 * caller-owned "views" (same fields, same order, same types) and the functions are what a binding of the
 * reference's entry points for this path would call.  Each declaration names the reference interface it
 * replaces as path:line inside the ParaSelect source tree.
 *
 * Conventions
 *   - Every function returns a psb_status; nothing aborts, throws or resets the device (the reference's
 *     CUDA_CHECK prints, resets the device and aborts: src/utils/check_cuda_error.cuh:64-82).
 *     psb_last_error() gives the message of the calling thread's last failure.
 *   - Pointers named h_* / in *_view structs are HOST pointers owned by the caller; pointers named d_*
 *     are DEVICE pointers on the session's device.  The library never frees caller memory.
 *   - Distances are squared L2.  Missing results are id -1 / distance FLT_MAX
 *     (src/search/ivf_common/ivf_exact_topk.h:87-90).
 *   - A session serves one caller thread at a time (src/search/ivfrespq/ivfrespq_search.cuh:118-119).
 *   - There is no CPU fallback: every compute entry point fails with PSB_NO_DEVICE when no sm_100 GPU
 *     is usable.
 */
#ifndef PSB_H
#define PSB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int psb_status;
enum {
    PSB_OK = 0,
    PSB_INVALID_ARGUMENT = 1,   /* std::invalid_argument in the reference (src/search/ivfpq/ivfpq_index.cu:52-93) */
    PSB_UNSUPPORTED_SHAPE = 2,  /* shape outside the kernels' supported ranges */
    PSB_CUDA_ERROR = 3,         /* a CUDA call failed; the message holds cudaGetErrorString */
    PSB_OUT_OF_MEMORY = 4,
    PSB_NO_DEVICE = 5,          /* no usable sm_100 device */
    PSB_INTERNAL = 6,           /* device status word reported an inconsistency (bad list id, row overflow) */
    PSB_TIMEOUT = 7             /* a bounded device-side wait gave up */
};

/* ---- views of caller-owned host memory ------------------------------------------------------- */

/* IVFCoarseIndexView, src/search/ivf_common/ivf_search_types.h:41-45 */
typedef struct psb_coarse_index_view {
    const float* centroids; /* [nlist][dim] row-major */
    int nlist;
    int dim;
} psb_coarse_index_view;

/* IVFListLayoutView, src/search/ivf_common/ivf_list_layout.h:12-17 (validated as in :19-45) */
typedef struct psb_list_layout_view {
    const int64_t* offsets;       /* [nlist + 1], offsets[0] == 0, monotone, offsets[nlist] == n_vectors */
    const int64_t* reordered_ids; /* [n_vectors] list-contiguous row -> original id */
    int nlist;
    int64_t n_vectors;
} psb_list_layout_view;

/* IVFPQCodeStorageView, src/search/ivf_common/ivf_storage.h:17-23 */
typedef struct psb_pq_code_storage_view {
    const uint8_t* codes;     /* [n_vectors][subvectors] list-contiguous */
    const void* code_storage; /* reference's optional paged CPU view; must be NULL here */
    const float* codebook;    /* [subvectors][codebook_size][dim / subvectors] */
    int subvectors;
    int codebook_size;
} psb_pq_code_storage_view;

/* IVFHostStorageView, src/search/ivf_common/ivf_host_storage.h:5-12 (exact rows for the rerank) */
typedef struct psb_host_storage_view {
    const float* fp32;      /* [count][dim] in list-contiguous order, or NULL */
    const uint8_t* u8;      /* [count][dim], or NULL */
    int64_t count;
    int dim;
    const int* source_rows; /* must be NULL (physical row == IVF row) */
} psb_host_storage_view;

/* IVFQueryBatchView, src/search/ivf_common/ivf_search_types.h:47-55 */
typedef struct psb_query_batch_view {
    const float* fp32;    /* [count][dim] */
    const uint8_t* u8;    /* [count][dim], only for the u8 rerank */
    int count;
    int dim;
    const uint16_t* fp16; /* ignored: the coarse stage converts on the device */
} psb_query_batch_view;

/* IVFSearchParams, src/search/ivf_common/ivf_search_types.h:63-69 */
typedef struct psb_search_params {
    int nprobe;
    int topk;
    int batch_size;            /* queries per internal batch */
    int distance;              /* 0 = squared L2 (the only mode on this path) */
    unsigned char fp16_coarse; /* accepted and ignored: results are always the exact fp32 ones */
} psb_search_params;

/* IVFSearchOutputView, src/search/ivf_common/ivf_search_types.h:71-75 */
typedef struct psb_search_output_view {
    int64_t* indices;  /* [count][topk] original ids */
    float* distances;  /* [count][topk] */
    int* coarse_ids;   /* optional [count][nprobe] */
} psb_search_output_view;

/* IVFPQIndexView, src/search/ivfpq/ivfpq_search_context.h:19-29 */
typedef struct psb_index_view {
    psb_coarse_index_view coarse;
    psb_list_layout_view lists;
    psb_pq_code_storage_view pq;
    psb_host_storage_view exact; /* rerank rows; fp32 == u8 == NULL disables the rerank */
} psb_index_view;

/* How the exact rows reach the GPU during the rerank. */
enum {
    PSB_EXACT_HOST_MAPPED = 0, /* register (pin + map) the caller's host rows once; kernels gather rows over PCIe */
    PSB_EXACT_HOST_STAGED = 1, /* host threads gather rows into pinned rings, cudaMemcpyAsync overlaps the copies */
    PSB_EXACT_RESIDENT = 2,    /* exact.fp32 / exact.u8 is already a device pointer (IVFExactStorageKind::Resident,
                                  src/search/ivf_common/ivf_storage.h:25-30) */
    PSB_EXACT_HOST_CACHED = 3, /* the session copies the caller's host rows into device memory once at creation and reranks from
                                  there (refused with PSB_OUT_OF_MEMORY when they do not fit); no counterpart in the reference,
                                  whose rerank rows stay on the host */
    PSB_EXACT_HOST_HYBRID = 4  /* both host transports at once: the rows are registered and mapped as in HOST_MAPPED, and of every
                                  sub-batch psb_options.zero_copy_pct percent of the queries have their rows gathered by a kernel
                                  over PCIe - on reserve_sms SMs of its own (default 32), which the scan's grid leaves free -
                                  while host threads stage the others through the pinned rings; neither the host cores nor
                                  the kernel's reads fill the link alone */
};

/* IVFPQSearchOptions (src/search/ivfpq/ivfpq_search_context.h:31-45) reduced to what this path uses,
 * plus the placement options the reference has no counterpart for. */
typedef struct psb_options {
    int device;         /* CUDA device ordinal */
    int n_rerank;       /* candidates kept by the ADC stage for the exact rerank (<= topk disables it) */
    int exact_mode;     /* PSB_EXACT_* */
    int max_batch;      /* largest internal batch the workspaces are sized for (0 = 10000) */
    int list_begin;     /* shard: this session scans lists [list_begin, list_end); 0,0 = all lists */
    int list_end;
    void* stream;       /* cudaStream_t to run on; NULL = a stream owned by the session */
    const int64_t* list_global_begin; /* striped shard (multi-GPU): the index view holds, for every list l, a contiguous
                           slice of the list; HOST array [nlist], list_global_begin[l] = index-wide row of the slice's
                           first row.  Candidate rows reported and accepted by the stage calls are index-wide rows.
                           NULL = the view is the whole index. */
    int coarse_mode;    /* 0 = auto, 1 = exact SIMT kernel only, 2 = tensor-core filter + exact refinement */
    int time_kernels;   /* 1 = bracket the ADC scan kernel with CUDA events (read back by psb_session_counters) */
    int serial_pipeline;/* 1 = never overlap the rerank of one sub-batch with the scan of the next (diagnostics) */
    int scan_mode;      /* which ADC scan runs; all give identical results.  0 = auto: the tensor-core pre-filter (bf16 tcgen05
                           GEMM of visiting queries against code rows decoded on the fly, survivors re-scored exactly in fp32)
                           when the shape fits, else the SIMT fp16 pre-filter scan, else the fp32 scan; 1 = fp32 SIMT scan only;
                           2 = SIMT scans only; 3 = tensor-core pre-filter required (PSB_UNSUPPORTED_SHAPE when it cannot run) */
    int adc_mode;       /* PQAdcDistanceMode (src/search/kernels/fine/fine_search_strategy.h:21-24): 0 = Plain (codes
                           encode the row), 1 = Residual (codes encode row - centroid[list]).  Residual mode follows
                           cpu_fine_kernel_pq_resid_cpu_lut_timed (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:594-735):
                           one table per (query, probe) on q - centroid, candidate width max(n_rerank, topk, 512), and
                           the exact rerank always runs (exact rows are required). */
    int reserve_sms;    /* SMs the ADC scan's persistent grid leaves free (0..64).  A multi-GPU caller that runs NCCL
                           collectives on a second stream while the scan is in flight sets a few: a collective's CTA
                           cannot share an SM with a scan CTA and would otherwise wait for the scan kernel to end. */
    /* Tuning, all optional (0 = the default): */
    float seed_sigma;   /* margin of the sampled admission cutoff in standard deviations (default 4; accepted 2..10).  Results do
                           not depend on it: a too-tight cutoff only sends more queries to the exact fallback. */
    int pipeline_parts; /* sub-batches per batch of the overlapped pipeline (default 4; accepted 2..32) */
    int even_cuts;      /* staged transport: 0 = a short first sub-batch (10/30/30/30 %: the transfer, the longer half, starts early),
                           1 = equal sub-batches, 2 = a short last sub-batch (32/32/26/10 %) */
    int gather_ctas;    /* 128-thread CTAs of the PCIe row-gather kernel when it runs beside a scan (default: two per SM) */
    int tc_min_visitors;/* lists with fewer visiting queries than this stay with the SIMT scan (default 1: none do) */
    /* Test hooks of the time-out paths of the tensor-core kernels (leave 0): test_wait_limit = polls before a device-side wait
       gives up; test_skip_mma bit 0 makes the scan's issuing warp skip its tcgen05.mma, bit 1 makes the coarse kernel's producer
       skip its loads - with nothing left in flight every waiting role then runs into the limit, the kernel frees its tensor
       memory and returns, and the call reports PSB_TIMEOUT. */
    int test_wait_limit;
    int test_skip_mma;
    int zero_copy_pct;  /* PSB_EXACT_HOST_HYBRID: share of each sub-batch gathered by the kernel, 1..100 (0 = 45) */
    /* Residual mode, optional: the per-row correction asset of the index, value[row] = |recon(row)|^2 + 2 <centroid[list(row)],
       recon(row)> (src/common/row_correction.h:37-45), as HOST arrays over the rows of the view - either fp32 or the affine u16
       form (value = rc_offset + rc_scale * u16, src/common/row_correction.h:7-20).  The residual cutoff estimate reads it;
       without it the session computes the fp32 values itself at creation.  Results never depend on it. */
    const float* row_correction_fp32;
    const uint16_t* row_correction_u16;
    float rc_scale, rc_offset;
    /* Plain mode, optional: the OPQ rotation of the index (IVFPQTransformKind::OPQ), HOST row-major [dim][dim] as [out][in].
       The PQ side of a search (tables, code scan) then works on R q while the coarse stage and the exact re-ranking keep the
       caller's q, as src/search/ivfpq/ivfpq_index.cu:205-217 and stage/ivfpq_fine_cpu_lut.cpp:29-31 do. */
    const float* opq_matrix;
    int host_threads;   /* gather threads of the staged / hybrid transport, 1..64 (0 = all hardware threads): several sessions in
                           one host - one per GPU - should share the cores between them */
} psb_options;

/* Counters and stage times of the last psb_session_search call; names follow the reference's
 * IVFSearchStatsCollector fields (src/search/ivfpq/pipeline/ivfpq_pipeline.cu:41-71,84-103). */
typedef struct psb_stats {
    double total_ms;
    double coarse_search_ms;
    double pq_lut_build_ms;
    double pq_adc_scan_ms;     /* schedule + seed + scan + selection */
    double pq_rerank_ms;
    double pq_map_ids_ms;
    double h2d_ms;
    double d2h_ms;
    long long pq_scanned_codes;    /* sum over (query, probe) of the list's row count */
    long long pq_adc_lookups;      /* pq_scanned_codes * subvectors */
    long long threshold_candidates;/* rows admitted into the candidate pools */
    long long fallback_queries;    /* queries re-scanned by the exact fallback */
    long long h2d_bytes;
    long long d2h_bytes;
    long long kernel_launches;
    double scan_kernel_ms;          /* device time of the ADC scan kernel alone (options.time_kernels) */
    long long scan_kernel_launches;
    double coarse_gemm_ms;          /* device time of the tensor-core coarse GEMM passes (options.time_kernels) */
    long long coarse_gemm_launches; /* two per coarse call */
    int batches;
    int coarse_fallback_queries;    /* queries the tensor-core coarse filter handed to the exact per-query kernel */
    long long prefilter_survivors;  /* (row, query) pairs the tensor-core scan filter let through to the exact re-scoring */
    /* Diagnostics of the tensor-core scan (psb_session_counters only): SM cycles its MMA-issuing threads spent waiting, summed
       over CTAs - for the next work item and its query tile, for decoded code rows, for a free accumulator - and the tiles
       (128 visitors x 128 rows) they issued. */
    long long tc_wait_item_cycles, tc_wait_rows_cycles, tc_wait_acc_cycles, tc_tiles;
    /* Staged rerank transport (psb_session_counters only): host time spent gathering exact rows into the pinned rings and the
       bytes gathered, since the last reset. */
    double staged_gather_ms;
    long long staged_gather_bytes;
    int reserved[4];
} psb_stats;

typedef struct psb_session psb_session;

/* ---- library ------------------------------------------------------------------------------------ */

/* Message of the calling thread's last failure ("" if none). */
const char* psb_last_error(void);
/* Number of usable sm_100 devices (0 when there is no GPU or no driver). */
int psb_device_count(void);
/* sizeof of a struct of this header as the library was built with it (0 psb_options, 1 psb_stats, 2 psb_index_view,
 * 3 psb_flat_index_view, 4 psb_row_correction_u16_header, 5 psb_search_params): lets a binding in another language check its
 * own declaration of the struct before it passes one. */
size_t psb_sizeof(int which);
const char* psb_version(void);

/* ---- session: prepare once, search many ----------------------------------------------------------- */

/* Uploads centroids, list offsets, ids, codes and codebook, maps the exact rows and sizes the
 * workspaces.  Replaces ivfpq_prepare_index + ivfpq_prepare (src/search/ivfpq/stage/ivfpq_prepare.cu:91-136,
 * declared src/search/ivfpq/stage/ivfpq_stages.cuh:8-9) and the IVFResPQSession constructor
 * (src/search/ivfrespq/ivfrespq_search.cuh:120-133).  Borrowed host assets must outlive the session. */
psb_status psb_session_create(const psb_index_view* index, const psb_options* options, psb_session** out);

/* ivfpq_release, src/search/ivfpq/stage/ivfpq_stages.cuh:10 */
psb_status psb_session_destroy(psb_session* session);

/* Whole search with HOST queries and HOST outputs: batches of params->batch_size through
 * coarse -> LUT -> scan -> rerank -> id map, results written at the global query offset.
 * Replaces IVFPQIndex::search (src/search/ivfpq/ivfpq_index.h:73-77), ivfpq_run_pipeline
 * (src/search/ivfpq/pipeline/ivfpq_pipeline.cu:8-116) and ivfrespq_search / IVFResPQSession::search
 * (src/search/ivfrespq/ivfrespq_search.cuh:114-133).  Returns after the results are in caller memory. */
psb_status psb_session_search(psb_session* session, const psb_query_batch_view* queries,
                              const psb_search_params* params, const psb_search_output_view* output,
                              psb_stats* stats);

/* The same search with DEVICE queries and DEVICE outputs, asynchronous on the session's stream (nq <= max_batch):
 * what psb_session_search runs per batch between its host copies.  When the rerank reads mapped or resident exact
 * rows the batch is processed in sub-batches and the PCIe gather + exact scoring of one overlaps the scan of the
 * next on a second stream (the GPU/CPU overlap of ivfrespq_pipeline_chunk_overlap,
 * src/search/ivfrespq/pipeline/ivfrespq_pipeline_cpu.cu:543-708, done with two CUDA streams).
 * d_queries_u8 only for a u8 rerank; d_coarse_ids optional [nq][nprobe]. */
psb_status psb_session_search_device(psb_session* session, const float* d_queries, const uint8_t* d_queries_u8, int nq,
                                     const psb_search_params* params, int64_t* d_indices, float* d_distances,
                                     int* d_coarse_ids);

/* Blocks until all work queued on the session's stream is done. */
psb_status psb_session_sync(psb_session* session);

/* Redirects the stage-level calls below to another stream (stream = NULL: back to the stream the session was created
 * with).  background != 0 marks the stream as the second stream of a caller-side pipeline: the PCIe row gather of the
 * rerank then runs on a small grid so that a scan queued on the first stream keeps the SMs.  The caller orders the two
 * streams with events; stage calls that share a workspace (two scans, two reranks) must not overlap.  No counterpart
 * in the reference (its overlap executor owns its streams, src/search/ivfrespq/pipeline/ivfrespq_pipeline_cpu.cu:433-527). */
psb_status psb_session_set_stream(psb_session* session, void* stream, int background);

/* ---- stage level, DEVICE pointers, asynchronous on the session's stream --------------------------- */
/* These mirror the reference's stage functions ivfpq_coarse / ivfpq_fine_* / ivfpq_rerank_cpu /
 * ivfpq_map_ids (src/search/ivfpq/stage/ivfpq_stages.cuh:11-19) with device buffers in place of the
 * context's host vectors.  nq must not exceed the session's max_batch. */

/* Coarse stage: per query the nprobe nearest centroids by exact fp32 squared L2, nearest first, ties by
 * list id.  Replaces coarse::search (src/search/kernels/coarse/coarse.h:18-60,
 * src/search/kernels/coarse/runtime/coarse_runtime.cu:340) and the CPU loop src/cpu/search/cpu_search.h:261-271.
 * d_ids [nq][nprobe] int32, d_dist [nq][nprobe] fp32 (may be NULL). */
psb_status psb_stage_coarse(psb_session* session, const float* d_queries, int nq, int nprobe,
                            int* d_ids, float* d_dist);

/* OPQ rotation of rows on the device: d_out[r][o] = sum_i matrix[o][i] d_in[r][i] (matrix row-major [out][in]), each element one
 * in-order fp32 fma chain.  Replaces OPQTransform::apply_device (src/transform/opq_transform.cu:73-78,124-163), which runs a
 * cuBLAS SGEMM whose summation order is unspecified; results agree to rounding.  d_out must not alias d_in. */
psb_status psb_rotate_rows(const float* d_in, const float* d_matrix, int64_t n, int dim, float* d_out, int device, void* stream);
/* The same with the session's own rotation (psb_options.opq_matrix): what a stage-by-stage caller feeds to
 * psb_stage_build_lut and psb_stage_scan_queries. */
psb_status psb_stage_rotate_queries(psb_session* session, const float* d_queries, int nq, float* d_rotated);

/* Per-query PQ lookup tables lut[q][m][c] = sum_d (q[m*dsub+d] - codebook[m][c][d])^2, built once per
 * query and shared by every probed list.  Replaces pq_build_query_lut_gpu
 * (src/search/kernels/fine/gpu_fine/pq_adc/pq_query_lut.cu:14-35) and
 * src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:51-63.  d_lut [nq][subvectors][codebook_size]. */
psb_status psb_stage_build_lut(psb_session* session, const float* d_queries, int nq, float* d_lut);

/* Residual mode tables: lut[q][p][m][c] = sum_d ((q - centroid[probes[q][p]])[m*dsub+d] - codebook[m][c][d])^2, one
 * table per (query, probe) pair.  Replaces build_query_residual + build_lut of the reference's CPU residual path
 * (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:87-130,440-451) and has the layout of its precomputed-LUT
 * argument (src/search/ivfrespq/stage/ivfrespq_query_scheduler.h:226-228).  d_probes [nq][nprobe] int32 (entries
 * outside [0, nlist) leave their table untouched), d_lut [nq][nprobe][subvectors][codebook_size].  A session created
 * with adc_mode = 1 expects this layout in psb_stage_scan. */
psb_status psb_stage_build_lut_residual(psb_session* session, const float* d_queries, int nq, const int* d_probes,
                                        int nprobe, float* d_lut);

/* Affine u8 quantisation of fp32 tables, per sub-quantiser: scale = max((hi - lo) / 255, 1e-6), u8 = clamp(rint((v - lo) /
 * scale), 0, 255), lo_sum = sum of lo, inflation = sum of scale * (0.5 plain, 1 residual) - the amount by which a cutoff on
 * u8 scores must be raised so that no true candidate is lost.  Replaces quantize_query_codeword_dot_lut_u8_kernel
 * (src/search/kernels/fine/gpu_fine/pq_adc/pq_query_lut.cu:37-97).  d_lut [tables][M][K] (tables = nq, or nq * nprobe in
 * residual mode), d_q8 the same shape in u8, d_scales [tables][M], d_lo_sum / d_inflation [tables].  This library's own scan
 * does not use u8 scores (its fp16 pre-filter is followed by exact fp32 re-scoring); the operator exists for callers
 * that keep the reference's u8 scoring elsewhere. */
psb_status psb_stage_quantize_lut_u8(psb_session* session, const float* d_lut, int64_t tables, uint8_t* d_q8, float* d_scales,
                                     float* d_lo_sum, float* d_inflation);

/* ADC scan of the probed lists with per-query selection of the stage1_k smallest distances
 * (ties by row).  Replaces ivfpq_fine_cpu_lut (src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:69-117) and
 * pq_query_lut_threshold_search_gpu + pq_candidate_cap_select
 * (src/search/kernels/fine/gpu_fine/pq_adc/pq_adc_gpu.cuh:98-112,
 *  src/search/kernels/fine/gpu_fine/pq_adc/pq_candidate_cap_select.cuh:13-33).
 * d_probes [nq][nprobe] int32 list ids (ids outside [0,nlist) are skipped);
 * d_rows [nq][stage1_k] list-contiguous row (-1 pad), d_dist same shape (FLT_MAX pad, may be NULL),
 * d_count [nq] (may be NULL). */
psb_status psb_stage_scan(psb_session* session, const float* d_lut, int nq, const int* d_probes, int nprobe,
                          int stage1_k, int* d_rows, float* d_dist, int* d_count);
/* The same stage with the queries at hand (d_queries [nq][dim]): lets the scan take the tensor-core pre-filter, which
 * needs the query vectors besides their tables.  Same results as psb_stage_scan.  In residual mode d_lut may be NULL when
 * the tensor-core scan takes every list (scan_mode 0 or 3 on a supported shape): no per-(query, probe) table is then
 * materialised at all - the scan works on q - centroid directly, and the cutoff, re-scoring and fallback kernels compute
 * the table entries they need from the query, the centroid and the codebook. */
psb_status psb_stage_scan_queries(psb_session* session, const float* d_queries, const float* d_lut, int nq,
                                  const int* d_probes, int nprobe, int stage1_k, int* d_rows, float* d_dist, int* d_count);

/* Sharded search (one session per shard of the index, e.g. one per GPU): the stage in two calls, so that the admission cutoff of
 * a query is placed on the rows of ALL shards instead of every shard looking for stage1_k rows of its own - with N shards the
 * shards then admit about 1/N of the rows each instead of as many as an unsharded search admits in all.
 *   1. psb_stage_scan_sample: schedule + sampling.  d_samples [nq][psb_scan_sample_words(session, stage1_k)] uint32 receives, per
 *      query, the smallest sample keys of this shard with their sampling stride and the rows the query scans here.
 *   2. the caller gathers the records of all shards: d_all_samples [shards][nq][words] (any shard order, the same on every shard
 *      is not required).
 *   3. psb_stage_scan_shared: cutoff from all records, scan, selection.  Outputs as psb_stage_scan_queries, except that a query
 *      may come back with fewer than stage1_k rows of this shard (d_count; -1 / FLT_MAX pad).  d_cutoff [nq] (optional) receives
 *      the cutoff (+inf: every row was admitted), d_rows_scanned [nq] (optional) the rows the query scans on all shards.
 * The caller must verify the outcome: after merging the shards' candidates, a query with a finite cutoff and fewer than
 * min(stage1_k, rows scanned) candidates had its cutoff placed too low (probability ~1e-9 per query at the default margin) and
 * must be searched again with psb_stage_scan_queries on every shard.  Both calls work on the session's scan workspace: no other
 * scan of this session may run between them. */
int psb_scan_sample_words(const psb_session* session, int stage1_k);
psb_status psb_stage_scan_sample(psb_session* session, const float* d_queries, const float* d_lut, int nq, const int* d_probes,
                                 int nprobe, int stage1_k, uint32_t* d_samples);
psb_status psb_stage_scan_shared(psb_session* session, const float* d_queries, const float* d_lut, int nq, const int* d_probes,
                                 int nprobe, int stage1_k, const uint32_t* d_all_samples, int shards, int* d_rows, float* d_dist,
                                 int* d_count, float* d_cutoff, int64_t* d_rows_scanned);

/* Exact rerank: drops candidates outside [0,count) and duplicates, recomputes fp32 squared L2 against the
 * exact rows and keeps the topk by (distance, row).  Replaces ivfpq_rerank_cpu -> ivf_rerank_host
 * (src/search/ivfpq/stage/ivfpq_rerank_cpu.cpp:14-66, src/search/ivf_common/ivf_host_rerank.h:7-27).
 * d_candidates [nq][candidate_stride] rows, first candidate_count (or d_counts[q]) used;
 * d_out_rows [nq][topk] int32, d_out_dist [nq][topk]. */
psb_status psb_stage_rerank(psb_session* session, const float* d_queries, int nq, const int* d_candidates,
                            int candidate_count, int candidate_stride, const int* d_counts, int topk,
                            int* d_out_rows, float* d_out_dist);

/* Multi-GPU halves of the rerank (no counterpart in the reference, whose search is single-GPU).
 * psb_stage_rerank_partial: d_dist [nq][candidate_count] = exact distance of every candidate whose row this
 * session holds, +inf for the others; the caller combines shards with an elementwise minimum.
 * psb_stage_select_topk: the topk (distance,row) pairs without duplicates from such a combined d_dist. */
psb_status psb_stage_rerank_partial(psb_session* session, const float* d_queries, int nq, const int* d_candidates,
                                    int candidate_count, int candidate_stride, const int* d_counts, float* d_dist);
psb_status psb_stage_select_topk(psb_session* session, const float* d_dist, const int* d_candidates, int nq,
                                 int candidate_count, int candidate_stride, const int* d_counts, int topk,
                                 int* d_out_rows, float* d_out_dist);

/* indices[i] = original id of row rows[i] when this session holds the row (always, for a whole index), else -1;
 * rows[i] < 0 gives -1.  Replaces ivfpq_map_ids
 * (src/search/ivfpq/stage/ivfpq_map_ids.cpp:4-15). */
psb_status psb_stage_map_ids(psb_session* session, const int* d_rows, int64_t n, int64_t* d_indices);

/* Merge of per-shard candidate lists (multi-GPU): d_rows/d_dist [parts][nq][k] -> the k smallest by
 * (distance, row) per query.  No counterpart in the reference (its search is single-GPU). */
psb_status psb_stage_merge(psb_session* session, const int* d_rows, const float* d_dist, int parts, int nq,
                           int k, int* d_out_rows, float* d_out_dist);

/* Counters gathered by the stage calls since the last reset (device-side counters are read back here). */
psb_status psb_session_counters(psb_session* session, psb_stats* stats, int reset);

/* ---- operator level with HOST pointers (one-shot; allocate, run, free) ------------------------------ */

/* ivf_rerank_host, src/search/ivf_common/ivf_host_rerank.h:7-27: same argument meaning; fp32 rows when
 * storage->fp32 is set, else u8 rows with u8 queries.  PSB_INVALID_ARGUMENT where the reference throws
 * std::invalid_argument. */
psb_status psb_rerank_host(const psb_host_storage_view* storage, const uint8_t* h_queries_u8,
                           const float* h_queries_fp32, const int* h_candidates, int batch_n,
                           int candidate_count, int candidate_stride, int topk, int* h_output_ids,
                           float* h_output_distances, const int* h_candidate_counts, int device);

/* Coarse stage on host arrays (device copies made internally). */
psb_status psb_coarse_host(const float* h_queries, int nq, const float* h_centroids, int nlist, int dim,
                           int nprobe, int coarse_mode, int64_t* h_ids, float* h_dist, int device);

/* Coarse stage that allocates nothing (no counterpart in the reference).  For callers that cannot call
 * cudaMalloc when they search - a fixed memory budget handed out at start-up, a host application that forbids
 * allocation after initialisation, a latency-critical thread that must not take the allocator's device
 * synchronisation or its late out-of-memory failure.  Inputs and outputs are DEVICE pointers owned by the
 * caller on the CURRENT device; the [nq][nlist] distance tile lives in a 16 MiB array built into the
 * library (each GPU that loads the library holds it until the process exits), so nq * nlist must not exceed
 * 4,194,304 (PSB_UNSUPPORTED_SHAPE otherwise).  Results are those of psb_stage_coarse bit for bit.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first call
 * before starting any stream capture.  All calls share the one array and it keeps the previous call's
 * contents (every element a call reads is first written by that call, so nothing needs clearing); two calls
 * whose kernels overlap on the GPU - different streams, different threads - race on it and must be serialised
 * by the caller.  d_ids [nq][nprobe] int32, d_dist [nq][nprobe] fp32 (may be NULL), asynchronous on stream. */
psb_status psb_coarse_search_static(const float* d_queries, int nq, const float* d_centroids, int nlist, int dim,
                                    int nprobe, int* d_ids, float* d_dist, void* stream);

/* Exact brute-force k nearest rows of d_base [n][dim] for each query (sequential fp32 squared L2, ties by
 * row): ground truth for recall.  The reference's counterpart is its brute-force scan helper
 * (src/search/kernels/brute_force/brute_force_scan.cu).  d_rows [nq][k] int32, d_dist [nq][k]; k <= 4096. */
psb_status psb_knn_exact(const float* d_queries, int nq, const float* d_base, int64_t n, int dim, int k,
                         int* d_rows, float* d_dist, int device, void* stream);

/* ---- IVF-Flat: exact fine scan over device-resident rows -------------------------------------------------- */

/* IVFFlatIndexView with row-major fp32 storage (src/search/ivfflat/ivfflat_search.cuh:11-29): caller-owned HOST memory. */
typedef struct psb_flat_index_view {
    psb_coarse_index_view coarse;
    psb_list_layout_view lists;
    const float* rowmajor_fp32; /* [n_vectors][dim] in list-contiguous order */
} psb_flat_index_view;

typedef struct psb_session psb_flat_session;

/* Uploads centroids, list layout, ids and the rows (they stay resident in device memory: the reference's GPU-resident fine
 * kind, IVFFlatFineKind, src/search/ivfflat/ivfflat_search.cuh:31-38).  options: device, max_batch, stream, coarse_mode. */
psb_status psb_flat_session_create(const psb_flat_index_view* index, const psb_options* options, psb_flat_session** out);
/* ivfflat_search (src/search/ivfflat/ivfflat_search.cuh:41-51): coarse top-nprobe, then the exact fp32 squared L2 distance to
 * every row of the probed lists and the topk nearest, ties by row; HOST queries and outputs, batches of params->batch_size.
 * Results equal the reference's CPU path cpu_ivf_search (src/cpu/search/cpu_search.h:226-332). */
psb_status psb_flat_session_search(psb_flat_session* session, const psb_query_batch_view* queries, const psb_search_params* params,
                                   const psb_search_output_view* output, psb_stats* stats);
/* The same with DEVICE queries and outputs, asynchronous on the session's stream (nq <= max_batch). */
psb_status psb_flat_session_search_device(psb_flat_session* session, const float* d_queries, int nq, const psb_search_params* params,
                                          int64_t* d_indices, float* d_distances);
psb_status psb_flat_session_destroy(psb_flat_session* session);

/* ---- sharded search: one rank of a group of sessions (multi-GPU) ----------------------------------------------
 *
 * Every rank - one process or thread per GPU - holds a session over its shard of the index (psb_options.list_global_begin; any
 * exact-row mode; psb_options.reserve_sms > 0 leaves SMs to the exchange) and passes two NCCL communicators of its own over
 * the same ranks.  A search runs, per sub-batch and on two streams, the session's stage calls and the exchanges between the
 * ranks: sample records -> shared cutoffs -> scan | all-to-all of the candidates -> merge of this rank's query slice ->
 * all-gather of the merged rows -> exact scoring of the rows held here -> all-reduce MIN -> top-k -> ids, and one all-reduce
 * MAX of the ids.  Every rank passes the same queries and receives the full result; it equals the unsharded search's.
 * The reference has no counterpart (its search is single-GPU, src/search/ivfpq/pipeline/ivfpq_pipeline.cu:8-116).
 *
 * nccl_comm / nccl_comm_samples: ncclComm_t handles (the second carries the sample records beside the exchange of the
 * previous sub-batch; NULL = use the first for both, which serialises the two).  nccl_library: path or soname of the NCCL
 * library that created them (NULL = "libnccl.so.2"); the copy already loaded in the process is used.  The collectives of
 * both communicators are issued in the same order on every rank.  The session must not be used for other calls while a
 * group search is in flight, and must outlive the group. */
typedef struct psb_group psb_group;
psb_status psb_group_create(psb_session* session, void* nccl_comm, void* nccl_comm_samples, const char* nccl_library,
                            int max_batch, int nprobe, int topk, psb_group** out);
/* parts: sub-batches per batch (default 4); shared_cutoff: 0 = every rank places its cutoffs on its own rows only. */
psb_status psb_group_set(psb_group* group, int parts, int shared_cutoff);
/* d_queries [nq][dim] fp32 (the same on every rank), d_indices [nq][topk], d_distances [nq][topk], all DEVICE memory;
 * asynchronous on the session's stream except for one host read per batch (the verification word of the shared cutoffs). */
psb_status psb_group_search_device(psb_group* group, const float* d_queries, int nq, const psb_search_params* params,
                                   int64_t* d_indices, float* d_distances);
/* Batches that were searched a second time because a shared cutoff came out too low (expected: 0). */
long long psb_group_searched_again(const psb_group* group);
psb_status psb_group_destroy(psb_group* group);

/* ---- training and encoding ---------------------------------------------------------------------------- */

/* Lloyd k-means on DEVICE data: assign = argmin squared L2 (strict <, lowest index wins), update = mean,
 * empty cluster keeps its centroid.  Replaces gpu_kmeans_lloyd (src/clustering/kmeans/kmeans.cuh:47-59,
 * src/clustering/kmeans/kmeans.cu:296-688).  d_centroids [k][dim] in/out, d_assign [n] out (may be NULL),
 * h_objective [iters + 1] out (may be NULL). */
psb_status psb_kmeans_train(const float* d_data, int64_t n, int dim, float* d_centroids, int k, int iters,
                            int* d_assign, double* h_objective, int device, void* stream);

/* One Lloyd iteration in three calls, for data-parallel training over several GPUs: every rank assigns and accumulates
 * its own rows, the caller all-reduces d_sums / d_counts / d_objective (NCCL), and every rank applies the same update.
 * Replaces the per-GPU accumulation and host reduction of the reference's multi-GPU trainers
 * (src/clustering/kmeans/kmeans_multigpu_train.cu:49-139, src/quantization/pq/residual_pq_multigpu_trainer.cu:336-411).
 *   assign:     d_assign [n] int32, d_best [n] fp32 (exact squared distance to the assigned centroid)
 *   accumulate: d_sums [k][dim] fp64, d_counts [k] int32, d_objective [1] fp64 - zeroed, then this rank's contribution
 *   update:     centroid = sums / counts rounded once to fp32; an empty cluster keeps its centroid */
psb_status psb_kmeans_assign(const float* d_data, int64_t n, int dim, const float* d_centroids, int k, int* d_assign,
                             float* d_best, int device, void* stream);
/* psb_kmeans_assign with the previous iteration's assignment at hand: have_previous != 0 says d_assign holds, on entry, a valid
 * centroid id per row (any ids in 0..k-1 do; ids outside send the row to the exact per-row path).  Each row's distance to that
 * centroid bounds its nearest distance, and the tensor-core filter runs once instead of twice; the result is the same. */
psb_status psb_kmeans_assign_bounded(const float* d_data, int64_t n, int dim, const float* d_centroids, int k, int* d_assign,
                                     float* d_best, int have_previous, int device, void* stream);
psb_status psb_kmeans_accumulate(const float* d_data, int64_t n, int dim, const int* d_assign, const float* d_best, int k,
                                 double* d_sums, int* d_counts, double* d_objective, int device, void* stream);
psb_status psb_kmeans_update(const double* d_sums, const int* d_counts, int k, int dim, float* d_centroids, int device,
                             void* stream);

/* Residual rows out[i] = data[i] - centroids[assign[i]] (fp32 subtraction; d_out may alias d_data): the input of
 * psb_pq_train / psb_pq_encode for a residual-mode index.  Replaces the residual step of the reference's residual PQ
 * trainer (src/quantization/pq/residual_pq_trainer.cuh:467-830). */
psb_status psb_residual_rows(const float* d_data, int64_t n, int dim, const float* d_centroids, const int* d_assign,
                             float* d_out, int device, void* stream);

/* Initial centroids as the reference picks them (init_centroids_by_sampling, src/clustering/kmeans/kmeans.cu:716-862):
 * std::mt19937(seed); policy 0 = k-means++ seeding while n * k <= 2e7, else k distinct rows by a partial Fisher-Yates shuffle;
 * 1 = always the random rows; 2 = always k-means++.  HOST data [n][dim]; h_centroids [k][dim] out; h_rows [k] (may be NULL)
 * receives the rows picked.  The same draws as the reference, draw for draw. */
psb_status psb_kmeans_init(const float* h_data, int64_t n, int dim, int k, int seed, int policy, float* h_centroids, int64_t* h_rows);

/* PQ codebooks: one k-means (codebook_size codewords) per subspace; subspace s starts from the rows the reference's
 * initialisation picks with seed + s * 104729 on that subspace (the same initial codewords as the reference's trainer).  Replaces train_plain_pq_codebooks_gpu (src/quantization/pq/pq_trainer.cuh:9-26,
 * src/quantization/pq/pq_trainer.cu:30-95).  d_codebook [m][k][dim/m] out. */
psb_status psb_pq_train(const float* d_data, int64_t n, int dim, int subvectors, int codebook_size, int iters,
                        uint64_t seed, float* d_codebook, int device, void* stream);

/* PQ encode: per (row, m) the nearest codeword, ties to the smallest code.  Replaces PQEncoderGPU
 * (src/quantization/pq/pq_encoder.cuh:10-26, src/quantization/pq/pq_encode.cuh:8-79).
 * d_codes [n][subvectors] out. */
psb_status psb_pq_encode(const float* d_data, int64_t n, int dim, const float* d_codebook, int subvectors,
                         int codebook_size, uint8_t* d_codes, int device, void* stream);

/* ---- index-build glue (host side: layout only, no arithmetic) ------------------------------------------------ */

/* From a list assignment to the IVF list layout: h_offsets [nlist + 1] and h_reordered_ids [n], rows ordered by
 * (list, original id) - the reorder-by-cluster step of the reference's index build (the `reordered_indices` / offsets of
 * its cluster cache, consumed by src/search/ivfpq/ivfpq_build.cu:150-209).  h_assign [n] list of every row, in 0..nlist-1
 * (PSB_INVALID_ARGUMENT otherwise). */
psb_status psb_ivf_layout_from_assignment(const int* h_assign, int64_t n, int nlist, int64_t* h_offsets, int64_t* h_reordered_ids);
/* h_dst[local] = h_src[h_reordered_ids[local]] for rows of row_bytes bytes: materialize_reordered
 * (src/search/ivfpq/ivfpq_build.cu:61-93), with its check that the ids are a permutation of 0..n-1. */
psb_status psb_reorder_rows(const void* h_src, int64_t n, size_t row_bytes, const int64_t* h_reordered_ids, void* h_dst);

/* ---- per-row correction of residual-PQ indices (host side) ------------------------------------------------------ */

/* The 32-byte header of the reference's affine u16 payload "row_correction.u16a" (src/common/row_correction.h:7-20). */
typedef struct psb_row_correction_u16_header {
    char magic[8];          /* "ISRC16\0\0" */
    uint32_t version;       /* 2 */
    uint32_t header_bytes;  /* 32 */
    uint64_t count;
    float scale;
    float offset;
} psb_row_correction_u16_header;

/* value[row] = |recon(row)|^2 + 2 <centroid[list(row)], recon(row)>, accumulated in fp64 and rounded once to fp32 as the
 * reference's builder does (src/index/row_correction/row_correction.cpp:143-169).  h_offsets [nlist + 1], h_codes [n][m]. */
psb_status psb_row_correction_compute(const float* h_centroids, const int64_t* h_offsets, int nlist, int dim, const uint8_t* h_codes,
                                      const float* h_codebook, int m, int k, float* h_values);
/* Affine u16 form of the values: offset = floor(min), scale = nextafter((max - offset) / 65534, +inf), u16 = ceil((v - offset) /
 * scale) - rounded UP, so a decoded value never undercuts the exact one (src/index/row_correction/row_correction.cpp:171-193).
 * Fills the header and h_u16 [n]. */
psb_status psb_row_correction_quantize_u16(const float* h_values, int64_t n, psb_row_correction_u16_header* header, uint16_t* h_u16);
/* The fixed-model form: a range that holds for EVERY code combination of the model, so rows encoded later (other pages, other
 * shards) share one scale / offset (src/quantization/row_correction/u16.h:28-91).  encode: u16 = ceil((v - offset) / scale),
 * refusing non-finite values and values outside the range (:17-24); decoding is fma(scale, u16, offset). */
psb_status psb_row_correction_model_u16(const float* h_centroids, int nlist, const float* h_codebook, int m, int k, int dsub,
                                        float* scale, float* offset);
psb_status psb_row_correction_encode_u16(const float* h_values, int64_t n, float scale, float offset, uint16_t* h_u16);
/* Writes / reads the payload file (header + u16 array) in the reference's layout.  read: h_u16 may be NULL to fetch the
 * header only; capacity = entries h_u16 can hold. */
psb_status psb_row_correction_write_u16(const char* path, const psb_row_correction_u16_header* header, const uint16_t* h_u16);
psb_status psb_row_correction_read_u16(const char* path, psb_row_correction_u16_header* header, uint16_t* h_u16, int64_t capacity);

/* ---- TurboQuant 1-bit residual codec -----------------------------------------------------------------------------
 * A row is stored as the signs of its rotated residual against its list's centroid (one bit per rotated dimension) and one
 * reconstruction scale; the rotation is a seeded sign flip followed by a Walsh-Hadamard transform of padded_dim (the next
 * power of two >= dim, 32..256) scaled by rsqrt(padded_dim).  These operators replace the reference's encoder
 * (src/quantization/turboquant/turboquant_1bit_encode.cuh:12-83, turboquant_1bit_encode.cu) and the candidate search of
 * its IVFResTurboQuant index (src/search/ivf_res_turboquant/ivf_res_turboquant_search.cuh:65-89,
 * src/quantization/turboquant/turboquant_1bit_scan.cuh:63-74).  All pointers are device pointers. */
#define PSB_SIGN_ROTATION_SEED 17u   /* src/search/ivf_res_turboquant/ivf_res_turboquant_search.cuh:41 */
#define PSB_SIGN_FLOAT_STATES 0      /* TurboQuant1BitScoreMode::MseFloatQuery */
#define PSB_SIGN_CODED_STATES 1      /* TurboQuant1BitScoreMode::BinaryQuery */
#define PSB_SIGN_MAX_CANDIDATES 8192 /* the reference takes up to 16,384 (ivf_res_turboquant_search.cuh:16) */

/* padded_dimension (ivf_res_turboquant_search.cu:24-29): 32, 64, 128 or 256; -1 when dim > 256 or dim <= 0. */
int psb_sign_padded_dim(int dim);
/* The rotation's scale as the device computes it, rsqrtf(padded_dim), for a checker that restates the rotation on the host. */
psb_status psb_sign_rotation_scale(int padded_dim, float* h_scale, int device, void* stream);
/* turboquant_1bit_encode_gpu: rotated rows [n][padded_dim], sign words [n][padded_dim / 32] (bit d % 32 of word d / 32 is set
 * when rotated[d] >= 0), sqrt of and the sum of squares of each input row.  Any output may be NULL. */
psb_status psb_sign_rotate(const float* d_rows, int64_t n, int dim, int padded_dim, uint32_t seed, float* d_rotated,
                           uint32_t* d_codes, float* d_norms, float* d_norm_sq, int device, void* stream);
/* ivf_res_turboquant_encode_database_u8_gpu: rows [row_offset, row_offset + n) of a list-contiguous index, u8 (elem_bytes 1,
 * the reference's input) or fp32 (elem_bytes 4); d_codes [total rows][padded_dim / 32] and d_scales [total rows] are written
 * at the global rows.  The scale is the mean magnitude of the rotated residual.  Encoding in chunks gives the same bits as
 * encoding at once. */
psb_status psb_sign_encode_database(const void* d_rows, int elem_bytes, int64_t n, const float* d_centroids,
                                    const int64_t* d_list_offsets, int nlist, int dim, int padded_dim, uint32_t seed,
                                    int64_t row_offset, uint32_t* d_codes, float* d_scales, int device, void* stream);
/* ivf_res_turboquant_encode_queries_gpu: one state per (query, probe), the rotated residual of the query against the probed
 * centroid: d_states [nq * nprobe][padded_dim] and d_norm_sq [nq * nprobe] (float states), d_state_codes
 * [nq * nprobe][padded_dim / 32] and d_norms [nq * nprobe] (sign-coded states); any may be NULL.  d_probes [nq][nprobe] int32 as
 * psb_stage_coarse writes them; a probe outside [0, nlist) gives a zero state. */
psb_status psb_sign_encode_queries(const float* d_queries, const float* d_centroids, const int* d_probes, int nq, int nprobe,
                                   int nlist, int dim, int padded_dim, uint32_t seed, float* d_states, float* d_norm_sq,
                                   uint32_t* d_state_codes, float* d_norms, int device, void* stream);
/* SearchWorkspace::search_candidates: every row of every probed list is scored against the state of its (query, probe) -
 * float states: norm_sq + dim s^2 - 2 s sum_d(+-state[d]) with s = d_row_params[row]; sign-coded states:
 * qn^2 + dn^2 - 2 qn dn (dim - 2 hamming) / dim with dn = d_row_params[row] - and the candidate_count smallest by (score, row)
 * come out in ascending order: d_rows_out [nq][candidate_count] int32 (global rows, -1 when fewer rows were scanned),
 * d_dist_out the scores (FLT_MAX there; may be NULL).  Probes outside [0, nlist) are skipped.  candidate_count <=
 * PSB_SIGN_MAX_CANDIDATES; at most 65,535 probes per query; the index holds fewer than 2^31 rows (rows come out as int32, as in
 * the reference); d_codes must be 16-byte aligned. */
psb_status psb_sign_search_candidates(int mode, const float* d_states, const float* d_norm_sq, const uint32_t* d_state_codes,
                                      const float* d_norms, const uint32_t* d_codes, const float* d_row_params,
                                      const int64_t* d_list_offsets, int nlist, const int* d_probes, int nq, int nprobe,
                                      int padded_dim, int candidate_count, int* d_rows_out, float* d_dist_out, int device,
                                      void* stream);

/* ---- synthetic data (bench and tests): counter-based generator, identical for any launch shape -------- */

/* rows [row_begin, row_begin + n) of a Gaussian mixture in component-contiguous order:
 * x = centre[component(row)] + sigma * N(0,1), component from d_offsets [ncomp + 1].
 * d_out [n][dim]. */
psb_status psb_gen_mixture_rows(const float* d_centres, const int64_t* d_offsets, int ncomp, int dim,
                                float sigma, uint64_t seed, int64_t row_begin, int64_t n, float* d_out,
                                int device, void* stream);
/* d_out [n][dim] = scale * N(0,1), element e of the stream seeded by (seed, first_elem + e). */
psb_status psb_gen_normal(uint64_t seed, int64_t first_elem, int64_t n_elems, float scale, float* d_out,
                          int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PSB_H */
