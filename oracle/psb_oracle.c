/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * CPU restatement of the reference's IVF search path, in plain C, used only as
 * the checker by the tests, the smoke entry and the bench's cpu_baseline leg.
 * The shipped library never links or calls anything in this file.
 *
 * Parity status: PINNED.  Every function here is checked (tests/test_oracle.py) against the reference's own CPU code compiled in place
 * (oracle/_ref, built by oracle/Makefile) and against the known-answer
 * constructions of the reference's unit tests.
 *
 * Arithmetic conventions restated (reference file:line):
 *   - coarse distance: sequential fp32 sum of (q-c)^2, no FMA
 *       src/cpu/utils/cpu_distance.h:74-81, src/cpu/search/cpu_search.h:261-271
 *   - PQ LUT entry: sequential fp32 sum of (q-cb)^2 over dsub, no FMA
 *       src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:51-63
 *   - ADC distance: dist = 0; for m = 0..M-1: dist += lut[m][code[m]]
 *       src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:76-80
 *   - exact rerank distance: the AVX-512 kernel's accumulation order (four
 *     16-lane FMA accumulators, pairwise combine, halving tree), emulated in scalar
 *       src/cpu/distance/fp32_l2_avx512.h:16-53
 *   - exact top-k order: (distance, id) ascending, pad id -1 / FLT_MAX
 *       src/search/ivf_common/ivf_exact_topk.h:12-22,87-90
 *   - candidate hygiene: ids outside [0,count) dropped, duplicates dropped
 *       src/search/ivf_common/ivf_host_rerank.cpp:152-177
 *   - id mapping: src/search/ivfpq/stage/ivfpq_map_ids.cpp:4-15
 * Where the reference leaves tie order unspecified (coarse partial_sort, the
 * stage-1 heap) this restatement fixes it to (distance, index) ascending.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <omp.h>

typedef struct { float d; int64_t i; } pair_t;

static int pair_cmp(const void* a, const void* b) {
    const pair_t* x = (const pair_t*)a; const pair_t* y = (const pair_t*)b;
    if (x->d < y->d) return -1;
    if (x->d > y->d) return 1;
    if (x->i < y->i) return -1;
    if (x->i > y->i) return 1;
    return 0;
}
static int pair_less(pair_t a, pair_t b) { return a.d < b.d || (a.d == b.d && a.i < b.i); }

/* Keep the k smallest (by (d,i)) of n pairs in buf[0..k), sorted ascending.
 * Max-heap of size k over the stream, then a sort: O(n log k). */
static void heap_sift_down(pair_t* h, int n, int pos) {
    for (;;) {
        int l = 2 * pos + 1, r = l + 1, big = pos;
        if (l < n && pair_less(h[big], h[l])) big = l;
        if (r < n && pair_less(h[big], h[r])) big = r;
        if (big == pos) return;
        pair_t t = h[pos]; h[pos] = h[big]; h[big] = t; pos = big;
    }
}
typedef struct { pair_t* h; int k; int n; } topk_t;
static void topk_init(topk_t* t, pair_t* storage, int k) { t->h = storage; t->k = k; t->n = 0; }
static void topk_push(topk_t* t, float d, int64_t i) {
    pair_t p = {d, i};
    if (t->n < t->k) {
        int pos = t->n++;
        t->h[pos] = p;
        while (pos > 0) {
            int par = (pos - 1) >> 1;
            if (!pair_less(t->h[par], t->h[pos])) break;
            pair_t x = t->h[par]; t->h[par] = t->h[pos]; t->h[pos] = x; pos = par;
        }
    } else if (t->k > 0 && pair_less(p, t->h[0])) {
        t->h[0] = p;
        heap_sift_down(t->h, t->n, 0);
    }
}
static void topk_finish(topk_t* t) { qsort(t->h, (size_t)t->n, sizeof(pair_t), pair_cmp); }

/* ---- distances ---------------------------------------------------------- */

/* src/cpu/utils/cpu_distance.h:74-81 */
static float l2_seq(const float* a, const float* b, int dim) {
    float sum = 0.0f;
    for (int i = 0; i < dim; ++i) { float diff = a[i] - b[i]; sum += diff * diff; }
    return sum;
}

/* Scalar emulation of src/cpu/distance/fp32_l2_avx512.h:16-53, including the
 * compiler's halving tree for the 16-lane horizontal add. */
float psbo_l2_exact(const float* q, const float* v, int dim) {
    float acc[4][16];
    memset(acc, 0, sizeof(acc));
    int i = 0;
    for (; i + 64 <= dim; i += 64)
        for (int a = 0; a < 4; ++a)
            for (int j = 0; j < 16; ++j) {
                float d = q[i + 16 * a + j] - v[i + 16 * a + j];
                acc[a][j] = fmaf(d, d, acc[a][j]);
            }
    for (; i + 16 <= dim; i += 16)
        for (int j = 0; j < 16; ++j) {
            float d = q[i + j] - v[i + j];
            acc[0][j] = fmaf(d, d, acc[0][j]);
        }
    float s[16], t3[8], t6[4];
    for (int j = 0; j < 16; ++j) s[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
    for (int j = 0; j < 8; ++j) t3[j] = s[j + 8] + s[j];
    for (int j = 0; j < 4; ++j) t6[j] = t3[j + 4] + t3[j];
    float out = (t6[0] + t6[2]) + (t6[1] + t6[3]);
    for (; i < dim; ++i) { float d = q[i] - v[i]; out = fmaf(d, d, out); }
    return out;
}

/* ---- coarse --------------------------------------------------------------- */

/* src/cpu/search/cpu_search.h:261-271.  out_ids [nq][nprobe] sorted nearest first. */
int psbo_coarse(const float* queries, int nq, const float* centroids, int nlist, int dim,
                int nprobe, int64_t* out_ids, float* out_dist) {
    if (!queries || !centroids || !out_ids || nprobe <= 0 || nprobe > nlist) return 1;
#pragma omp parallel
    {
        pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)nprobe);
#pragma omp for schedule(static)
        for (int q = 0; q < nq; ++q) {
            topk_t t; topk_init(&t, heap, nprobe);
            for (int c = 0; c < nlist; ++c)
                topk_push(&t, l2_seq(queries + (size_t)q * dim, centroids + (size_t)c * dim, dim), c);
            topk_finish(&t);
            for (int p = 0; p < nprobe; ++p) {
                out_ids[(size_t)q * nprobe + p] = heap[p].i;
                if (out_dist) out_dist[(size_t)q * nprobe + p] = heap[p].d;
            }
        }
        free(heap);
    }
    return 0;
}

/* ---- PQ lookup table ------------------------------------------------------- */

/* src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:51-63.  lut [M][K]. */
void psbo_pq_lut(const float* query, const float* codebook, int pq_m, int pq_k, int dsub, float* lut) {
    for (int m = 0; m < pq_m; ++m)
        for (int c = 0; c < pq_k; ++c) {
            const float* center = codebook + ((size_t)m * pq_k + c) * dsub;
            float dist = 0.0f;
            for (int d = 0; d < dsub; ++d) { float diff = query[m * dsub + d] - center[d]; dist += diff * diff; }
            lut[(size_t)m * pq_k + c] = dist;
        }
}

int psbo_pq_lut_batch(const float* queries, int nq, int dim, const float* codebook, int pq_m, int pq_k, float* luts) {
    if (pq_m <= 0 || dim % pq_m) return 1;
#pragma omp parallel for schedule(static)
    for (int q = 0; q < nq; ++q)
        psbo_pq_lut(queries + (size_t)q * dim, codebook, pq_m, pq_k, dim / pq_m, luts + (size_t)q * pq_m * pq_k);
    return 0;
}

/* Affine u8 quantisation of one query's LUT, per sub-quantiser:
 * src/search/kernels/fine/gpu_fine/pq_adc/pq_query_lut.cu:37-97.
 * scale = max((hi-lo)/255, 1e-6); u8 = clamp(rn((v-lo)/scale)); lo_sum = sum lo;
 * inflation = sum scale * (0.5 plain | 1.0 residual). */
void psbo_pq_lut_u8(const float* lut, int pq_m, int pq_k, int residual,
                    uint8_t* q8, float* scales, float* lo_sum, float* inflation) {
    float ls = 0.0f, inf = 0.0f;
    for (int m = 0; m < pq_m; ++m) {
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (int c = 0; c < pq_k; ++c) {
            float v = lut[(size_t)m * pq_k + c];
            if (v < lo) lo = v;
            if (v > hi) hi = v;
        }
        float scale = (hi - lo) / 255.0f;
        if (scale < 1e-6f) scale = 1e-6f;
        for (int c = 0; c < pq_k; ++c) {
            float r = rintf((lut[(size_t)m * pq_k + c] - lo) / scale);
            if (r < 0.0f) r = 0.0f;
            if (r > 255.0f) r = 255.0f;
            q8[(size_t)m * pq_k + c] = (uint8_t)r;
        }
        scales[m] = scale;
        ls += lo;
        inf += scale * (residual ? 1.0f : 0.5f);
    }
    *lo_sum = ls; *inflation = inf;
}

/* ---- ADC scan + stage-1 selection ------------------------------------------ */

/* src/search/ivfpq/stage/ivfpq_fine_cpu_lut.cpp:69-98.
 * probes [nq][nprobe] (invalid list ids skipped), out_rows/out_dist [nq][stage1_k]
 * (list-contiguous row index, -1 / FLT_MAX padded), out_count [nq].
 * Ties are resolved by (distance, row) ascending. */
int psbo_pq_scan(const float* queries, int nq, int dim, const int64_t* probes, int nprobe,
                 const int64_t* offsets, int nlist, const uint8_t* codes, const float* codebook,
                 int pq_m, int pq_k, int stage1_k, int* out_rows, float* out_dist, int* out_count,
                 long long* scanned_rows) {
    if (pq_m <= 0 || dim % pq_m || stage1_k <= 0) return 1;
    const int dsub = dim / pq_m;
    long long scanned_total = 0;
#pragma omp parallel reduction(+ : scanned_total)
    {
        float* lut = (float*)malloc(sizeof(float) * (size_t)pq_m * pq_k);
        pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)stage1_k);
#pragma omp for schedule(dynamic, 1)
        for (int q = 0; q < nq; ++q) {
            psbo_pq_lut(queries + (size_t)q * dim, codebook, pq_m, pq_k, dsub, lut);
            topk_t t; topk_init(&t, heap, stage1_k);
            for (int p = 0; p < nprobe; ++p) {
                int64_t list = probes[(size_t)q * nprobe + p];
                if (list < 0 || list >= nlist) continue;
                for (int64_t row = offsets[list]; row < offsets[list + 1]; ++row) {
                    const uint8_t* code = codes + (size_t)row * pq_m;
                    float dist = 0.0f;
                    for (int m = 0; m < pq_m; ++m) dist += lut[(size_t)m * pq_k + code[m]];
                    topk_push(&t, dist, row);
                    ++scanned_total;
                }
            }
            topk_finish(&t);
            for (int i = 0; i < stage1_k; ++i) {
                out_rows[(size_t)q * stage1_k + i] = i < t.n ? (int)heap[i].i : -1;
                if (out_dist) out_dist[(size_t)q * stage1_k + i] = i < t.n ? heap[i].d : FLT_MAX;
            }
            if (out_count) out_count[q] = t.n;
        }
        free(lut); free(heap);
    }
    if (scanned_rows) *scanned_rows = scanned_total;
    return 0;
}

/* ---- exact rerank ------------------------------------------------------------ */

/* src/search/ivf_common/ivf_host_rerank.cpp:55-316 (fp32 rows or u8 rows).
 * candidates [batch][stride]; counts optional (else candidate_count each).
 * out_ids (row index) / out_dist [batch][topk]. */
int psbo_rerank(const float* base_fp32, const uint8_t* base_u8, int64_t count, int dim,
                const float* queries_fp32, const uint8_t* queries_u8,
                const int* candidates, int batch_n, int candidate_count, int candidate_stride,
                int topk, const int* candidate_counts, int* out_ids, float* out_dist) {
    if (!candidates || !out_ids || !out_dist || batch_n <= 0 || candidate_count <= 0 ||
        candidate_stride < candidate_count || topk <= 0 || count <= 0 || dim <= 0) return 1;
    const int use_float = base_fp32 != NULL;
    if ((use_float && !queries_fp32) || (!use_float && (!base_u8 || !queries_u8))) return 1;
    if (candidate_counts)
        for (int q = 0; q < batch_n; ++q)
            if (candidate_counts[q] < 0 || candidate_counts[q] > candidate_count) return 1;
#pragma omp parallel
    {
        pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)topk);
        int* uniq = (int*)malloc(sizeof(int) * (size_t)candidate_count);
        pair_t* sorted = (pair_t*)malloc(sizeof(pair_t) * (size_t)candidate_count);
#pragma omp for schedule(dynamic, 4)
        for (int q = 0; q < batch_n; ++q) {
            const int* cand = candidates + (size_t)q * candidate_stride;
            const int n = candidate_counts ? candidate_counts[q] : candidate_count;
            /* hygiene + de-duplication (first occurrence wins; order is irrelevant to the result) */
            int nv = 0;
            for (int i = 0; i < n; ++i) if (cand[i] >= 0 && cand[i] < count) { sorted[nv].d = 0; sorted[nv].i = cand[i]; ++nv; }
            qsort(sorted, (size_t)nv, sizeof(pair_t), pair_cmp);
            int nu = 0;
            for (int i = 0; i < nv; ++i) if (i == 0 || sorted[i].i != sorted[i - 1].i) uniq[nu++] = (int)sorted[i].i;
            topk_t t; topk_init(&t, heap, topk);
            for (int i = 0; i < nu; ++i) {
                float d;
                if (use_float) d = psbo_l2_exact(queries_fp32 + (size_t)q * dim, base_fp32 + (size_t)uniq[i] * dim, dim);
                else {
                    int32_t s = 0;
                    for (int j = 0; j < dim; ++j) {
                        int x = (int)queries_u8[(size_t)q * dim + j] - (int)base_u8[(size_t)uniq[i] * dim + j];
                        s += x * x;
                    }
                    d = (float)s;
                }
                topk_push(&t, d, uniq[i]);
            }
            topk_finish(&t);
            for (int i = 0; i < topk; ++i) {
                out_ids[(size_t)q * topk + i] = i < t.n ? (int)heap[i].i : -1;
                out_dist[(size_t)q * topk + i] = i < t.n ? heap[i].d : FLT_MAX;
            }
        }
        free(heap); free(uniq); free(sorted);
    }
    return 0;
}

/* src/search/ivfpq/stage/ivfpq_map_ids.cpp:4-15 */
void psbo_map_ids(const int* local, int64_t n, const int64_t* reordered_ids, int64_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = local[i] >= 0 ? reordered_ids[local[i]] : (int64_t)-1;
}

/* ---- whole plain IVF-PQ search ------------------------------------------------ */

/* Two-stage semantics of src/search/ivfpq/stage/ivfpq_prepare.cu:108-118:
 * stage1_k = min(n_rerank, n_vectors) when rerank rows are given and n_rerank > topk, else topk;
 * without rerank the output distances are the ADC distances. */
int psbo_ivfpq_search(const float* centroids, int nlist, int dim,
                      const int64_t* offsets, const int64_t* reordered_ids, int64_t n_vectors,
                      const uint8_t* codes, const float* codebook, int pq_m, int pq_k,
                      const float* rerank_fp32, const float* queries, int nq,
                      int nprobe, int topk, int n_rerank,
                      int64_t* out_indices, float* out_distances, int64_t* out_coarse,
                      int* out_stage1, long long* scanned_rows) {
    if (nprobe <= 0 || nprobe > nlist || topk <= 0 || nq < 0) return 1;
    if (nq == 0) return 0;
    const int rerank = rerank_fp32 != NULL && n_rerank > topk;
    const int stage1_k = rerank ? (int)(n_rerank < n_vectors ? n_rerank : n_vectors) : topk;
    int64_t* probes = (int64_t*)malloc(sizeof(int64_t) * (size_t)nq * nprobe);
    int* rows = (int*)malloc(sizeof(int) * (size_t)nq * stage1_k);
    float* adc = (float*)malloc(sizeof(float) * (size_t)nq * stage1_k);
    int* local = (int*)malloc(sizeof(int) * (size_t)nq * topk);
    int rc = psbo_coarse(queries, nq, centroids, nlist, dim, nprobe, probes, NULL);
    if (!rc) rc = psbo_pq_scan(queries, nq, dim, probes, nprobe, offsets, nlist, codes, codebook, pq_m, pq_k,
                               stage1_k, rows, adc, NULL, scanned_rows);
    if (!rc) {
        if (rerank) {
            rc = psbo_rerank(rerank_fp32, NULL, n_vectors, dim, queries, NULL, rows, nq, stage1_k, stage1_k,
                             topk, NULL, local, out_distances);
        } else {
            for (int q = 0; q < nq; ++q)
                for (int i = 0; i < topk; ++i) {
                    local[(size_t)q * topk + i] = rows[(size_t)q * stage1_k + i];
                    out_distances[(size_t)q * topk + i] = adc[(size_t)q * stage1_k + i];
                }
        }
    }
    if (!rc) psbo_map_ids(local, (int64_t)nq * topk, reordered_ids, out_indices);
    if (!rc && out_coarse) memcpy(out_coarse, probes, sizeof(int64_t) * (size_t)nq * nprobe);
    if (!rc && out_stage1) memcpy(out_stage1, rows, sizeof(int) * (size_t)nq * stage1_k);
    free(probes); free(rows); free(adc); free(local);
    return rc;
}

/* ---- residual IVF-PQ (codes encode x - centroid[list]) ------------------------- */

/* ADC sum in the order of src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:
 *   M == 16, K == 256 (:226-242) and M == 8, K == 256 (:250-259): balanced pairwise tree,
 *   every other shape (:203-217): sequential. */
static float resid_adc(const float* lut, const uint8_t* code, int pq_m, int pq_k) {
    if (pq_k == 256 && (pq_m == 16 || pq_m == 8)) {
        float s[16];
        for (int j = 0; j < pq_m; ++j) s[j] = lut[(size_t)j * 256 + code[j]];
        for (int n = pq_m; n > 1; n >>= 1)
            for (int j = 0; j < n / 2; ++j) s[j] = s[2 * j] + s[2 * j + 1];
        return s[0];
    }
    float d = 0.0f;
    for (int j = 0; j < pq_m; ++j) d += lut[(size_t)j * pq_k + code[j]];
    return d;
}

/* Stage 1 of the residual mode: per (query, probe) table on q - centroid[list]
 * (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:440-451 residual, :113-128 table entries:
 * sequential fp32 sum, no FMA; src/search/ivfrespq/stage/ivfrespq_query_scheduler.h:142-254 probe loop),
 * the stage1_k smallest ADC distances per query.  luts_out (optional) [nq][nprobe][M][K].
 * Ties by (distance, row) ascending. */
int psbo_pq_scan_residual(const float* queries, int nq, int dim, const int64_t* probes, int nprobe,
                          const float* centroids, const int64_t* offsets, int nlist, const uint8_t* codes,
                          const float* codebook, int pq_m, int pq_k, int stage1_k, int* out_rows, float* out_dist,
                          int* out_count, float* luts_out, long long* scanned_rows) {
    if (pq_m <= 0 || dim % pq_m || stage1_k <= 0) return 1;
    const int dsub = dim / pq_m;
    long long scanned_total = 0;
#pragma omp parallel reduction(+ : scanned_total)
    {
        float* lut = (float*)malloc(sizeof(float) * (size_t)pq_m * pq_k);
        float* resid = (float*)malloc(sizeof(float) * (size_t)dim);
        pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)stage1_k);
#pragma omp for schedule(dynamic, 1)
        for (int q = 0; q < nq; ++q) {
            topk_t t; topk_init(&t, heap, stage1_k);
            for (int p = 0; p < nprobe; ++p) {
                int64_t list = probes[(size_t)q * nprobe + p];
                if (list < 0 || list >= nlist) continue;
                if (offsets[list + 1] <= offsets[list] && !luts_out) continue;
                for (int d = 0; d < dim; ++d) resid[d] = queries[(size_t)q * dim + d] - centroids[(size_t)list * dim + d];
                psbo_pq_lut(resid, codebook, pq_m, pq_k, dsub, lut);
                if (luts_out) memcpy(luts_out + ((size_t)q * nprobe + p) * pq_m * pq_k, lut, sizeof(float) * (size_t)pq_m * pq_k);
                for (int64_t row = offsets[list]; row < offsets[list + 1]; ++row) {
                    topk_push(&t, resid_adc(lut, codes + (size_t)row * pq_m, pq_m, pq_k), row);
                    ++scanned_total;
                }
            }
            topk_finish(&t);
            for (int i = 0; i < stage1_k; ++i) {
                out_rows[(size_t)q * stage1_k + i] = i < t.n ? (int)heap[i].i : -1;
                if (out_dist) out_dist[(size_t)q * stage1_k + i] = i < t.n ? heap[i].d : FLT_MAX;
            }
            if (out_count) out_count[q] = t.n;
        }
        free(lut); free(resid); free(heap);
    }
    if (scanned_rows) *scanned_rows = scanned_total;
    return 0;
}

/* Candidate width of the residual mode: max(n_rerank, topk, 512)
 * (src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:623-625). */
int psbo_residual_stage1_width(int topk, int n_rerank) {
    int w = n_rerank < topk ? topk : n_rerank;
    return w < 512 ? 512 : w;
}

/* Whole residual search: coarse, stage 1 above, exact rerank of the candidates (always, with their counts:
 * src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:722-730), id map.  out_stage1 [nq][width] (optional). */
int psbo_ivfrespq_search(const float* centroids, int nlist, int dim,
                         const int64_t* offsets, const int64_t* reordered_ids, int64_t n_vectors,
                         const uint8_t* codes, const float* codebook, int pq_m, int pq_k,
                         const float* rerank_fp32, const float* queries, int nq,
                         int nprobe, int topk, int n_rerank,
                         int64_t* out_indices, float* out_distances, int64_t* out_coarse,
                         int* out_stage1, int* out_stage1_count, long long* scanned_rows) {
    if (nprobe <= 0 || nprobe > nlist || topk <= 0 || nq < 0 || !rerank_fp32) return 1;
    if (nq == 0) return 0;
    const int width = psbo_residual_stage1_width(topk, n_rerank);
    int64_t* probes = (int64_t*)malloc(sizeof(int64_t) * (size_t)nq * nprobe);
    int* rows = (int*)malloc(sizeof(int) * (size_t)nq * width);
    int* counts = (int*)malloc(sizeof(int) * (size_t)nq);
    int* local = (int*)malloc(sizeof(int) * (size_t)nq * topk);
    int rc = psbo_coarse(queries, nq, centroids, nlist, dim, nprobe, probes, NULL);
    if (!rc) rc = psbo_pq_scan_residual(queries, nq, dim, probes, nprobe, centroids, offsets, nlist, codes, codebook,
                                        pq_m, pq_k, width, rows, NULL, counts, NULL, scanned_rows);
    if (!rc) rc = psbo_rerank(rerank_fp32, NULL, n_vectors, dim, queries, NULL, rows, nq, width, width, topk, counts,
                              local, out_distances);
    if (!rc) psbo_map_ids(local, (int64_t)nq * topk, reordered_ids, out_indices);
    if (!rc && out_coarse) memcpy(out_coarse, probes, sizeof(int64_t) * (size_t)nq * nprobe);
    if (!rc && out_stage1) memcpy(out_stage1, rows, sizeof(int) * (size_t)nq * width);
    if (!rc && out_stage1_count) memcpy(out_stage1_count, counts, sizeof(int) * (size_t)nq);
    free(probes); free(rows); free(counts); free(local);
    return rc;
}

/* ---- IVF-Flat (exact fp32 fine scan) ------------------------------------------ */

/* src/cpu/search/cpu_search.h:226-332: coarse as above, every row of each probed
 * list scored with the sequential fp32 sum, top-k, ids through reordered_ids. */
int psbo_ivfflat_search(const float* centroids, int nlist, int dim, const int64_t* offsets,
                        const int64_t* reordered_ids, const float* base, const float* queries, int nq,
                        int nprobe, int topk, int64_t* out_indices, float* out_distances) {
    if (nprobe <= 0 || nprobe > nlist || topk <= 0) return 1;
    int64_t* probes = (int64_t*)malloc(sizeof(int64_t) * (size_t)nq * nprobe);
    int rc = psbo_coarse(queries, nq, centroids, nlist, dim, nprobe, probes, NULL);
    if (!rc) {
#pragma omp parallel
        {
            pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)topk);
#pragma omp for schedule(dynamic, 1)
            for (int q = 0; q < nq; ++q) {
                topk_t t; topk_init(&t, heap, topk);
                for (int p = 0; p < nprobe; ++p) {
                    int64_t list = probes[(size_t)q * nprobe + p];
                    for (int64_t row = offsets[list]; row < offsets[list + 1]; ++row)
                        topk_push(&t, l2_seq(queries + (size_t)q * dim, base + (size_t)row * dim, dim), row);
                }
                topk_finish(&t);
                for (int i = 0; i < topk; ++i) {
                    out_indices[(size_t)q * topk + i] =
                        i < t.n ? (reordered_ids ? reordered_ids[heap[i].i] : heap[i].i) : (int64_t)-1;
                    out_distances[(size_t)q * topk + i] = i < t.n ? heap[i].d : FLT_MAX;
                }
            }
            free(heap);
        }
    }
    free(probes);
    return rc;
}

/* ---- training: Lloyd k-means, PQ codebooks, PQ encoding ------------------------ */

/* Lloyd k-means in the reference's CPU form (src/cpu/clustering/cpu_kmeans.h:27-143): assign = argmin
 * of the sequential squared L2 (strict <, lowest index wins), update = mean of members, an empty
 * cluster keeps its centroid.  The reference sums members in fp32 in a thread-dependent order, so its
 * own test compares objectives and centroid RMSE, not bits (tests/unit/clustering/test_kmeans.cu:395-405);
 * this restatement sums in fp64 so that it is order independent. */

/* Assignment with the GPU trainer's rule (src/clustering/kmeans/kmeans_utils.cu:359-413):
 * strict '<', lowest centroid index wins ties.  Distances here are the exact sequential
 * squared L2 (the GPU trainer recomputes the winner exactly, src/clustering/kmeans/kmeans.cu:59-101). */
void psbo_kmeans_assign(const float* data, int64_t n, int dim, const float* centroids, int k,
                        int* assign, float* dist) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float best = FLT_MAX; int bi = 0;
        for (int c = 0; c < k; ++c) {
            float d = l2_seq(data + (size_t)i * dim, centroids + (size_t)c * dim, dim);
            if (d < best) { best = d; bi = c; }
        }
        assign[i] = bi;
        if (dist) dist[i] = best;
    }
}

/* Update: mean of members (sums in fp64 for order independence, rounded once to fp32);
 * empty cluster keeps its old centroid (src/clustering/kmeans/kmeans_utils.cu:267-284). */
void psbo_kmeans_update(const float* data, int64_t n, int dim, const int* assign, float* centroids, int k,
                        int* counts_out) {
    double* sums = (double*)calloc((size_t)k * dim, sizeof(double));
    int64_t* cnt = (int64_t*)calloc((size_t)k, sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i) {
        int c = assign[i];
        cnt[c]++;
        for (int d = 0; d < dim; ++d) sums[(size_t)c * dim + d] += data[(size_t)i * dim + d];
    }
    for (int c = 0; c < k; ++c) {
        if (cnt[c] > 0)
            for (int d = 0; d < dim; ++d) centroids[(size_t)c * dim + d] = (float)(sums[(size_t)c * dim + d] / (double)cnt[c]);
        if (counts_out) counts_out[c] = (int)cnt[c];
    }
    free(sums); free(cnt);
}

/* iters Lloyd iterations from caller-supplied initial centroids; returns the objective
 * (sum of squared distances under the final centroids' preceding assignment) per iteration. */
int psbo_kmeans_lloyd(const float* data, int64_t n, int dim, float* centroids, int k, int iters,
                      int* assign_out, double* objective_out) {
    int* assign = (int*)malloc(sizeof(int) * (size_t)n);
    float* dist = (float*)malloc(sizeof(float) * (size_t)n);
    for (int it = 0; it < iters; ++it) {
        psbo_kmeans_assign(data, n, dim, centroids, k, assign, dist);
        double obj = 0.0;
        for (int64_t i = 0; i < n; ++i) obj += dist[i];
        if (objective_out) objective_out[it] = obj;
        psbo_kmeans_update(data, n, dim, assign, centroids, k, NULL);
    }
    psbo_kmeans_assign(data, n, dim, centroids, k, assign, dist);
    if (objective_out) { double obj = 0.0; for (int64_t i = 0; i < n; ++i) obj += dist[i]; objective_out[iters] = obj; }
    if (assign_out) memcpy(assign_out, assign, sizeof(int) * (size_t)n);
    free(assign); free(dist);
    return 0;
}

/* PQ encode: per (row, m) argmin over the K codewords of the sequential squared L2, ties ->
 * smallest code (src/quantization/pq/pq_encode.cuh:24-40,69-77). */
int psbo_pq_encode(const float* data, int64_t n, int dim, const float* codebook, int pq_m, int pq_k,
                   uint8_t* codes) {
    if (pq_m <= 0 || dim % pq_m || pq_k > 256) return 1;
    const int dsub = dim / pq_m;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i)
        for (int m = 0; m < pq_m; ++m) {
            float best = FLT_MAX; int bc = 0;
            for (int c = 0; c < pq_k; ++c) {
                float d = l2_seq(data + (size_t)i * dim + (size_t)m * dsub, codebook + ((size_t)m * pq_k + c) * dsub, dsub);
                if (d < best) { best = d; bc = c; }
            }
            codes[(size_t)i * pq_m + m] = (uint8_t)bc;
        }
    return 0;
}

/* Recall by id-set intersection (definition of src/benchmark/recall_method.h:3-8, idx_intersection). */
double psbo_recall(const int64_t* got, const int64_t* truth, int nq, int k) {
    long long hit = 0, tot = 0;
    for (int q = 0; q < nq; ++q)
        for (int i = 0; i < k; ++i) {
            int64_t t = truth[(size_t)q * k + i];
            if (t < 0) continue;
            ++tot;
            for (int j = 0; j < k; ++j) if (got[(size_t)q * k + j] == t) { ++hit; break; }
        }
    return tot ? (double)hit / (double)tot : 1.0;
}

/* ---------------------------------------------------------------------------------------------------------------
 * OPQ rotation of rows: out[r][o] = sum_i matrix[o][i] in[r][i], matrix row-major [out][in].  The reference runs this as
 * one cuBLAS SGEMM (src/transform/opq_transform.cu:124-163), whose summation order is not specified, and its own test
 * compares against an in-order host loop with a tolerance (tests/unit/transform/test_opq_transform.cu:22-39).  The chain is
 * pinned here as fp32 fma in input order - the order the GPU kernel of the product uses. */
int psbo_rotate_rows(const float* in, const float* matrix, int64_t n, int dim, float* out) {
    if (!in || !matrix || !out || n < 0 || dim <= 0) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r)
        for (int o = 0; o < dim; ++o) {
            float acc = 0.0f;
            for (int i = 0; i < dim; ++i) acc = fmaf(matrix[(size_t)o * dim + i], in[(size_t)r * dim + i], acc);
            out[(size_t)r * dim + o] = acc;
        }
    return 0;
}
