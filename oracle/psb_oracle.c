/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * CPU restatement of the reference's IVF search path, in plain C, used only as
 * the checker by the tests, the smoke entry and the bench's cpu_baseline leg.
 * The shipped library never links or calls anything in this file.
 *
 * Parity status: PINNED, with one exception stated at the block it concerns (the TurboQuant 1-bit codec at the end of the
 * file: partly pinned).  Every other function here is checked (tests/test_oracle.py) against the reference's own CPU code
 * compiled in place (oracle/_ref, built by oracle/Makefile) and against the known-answer
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

/* ---------------------------------------------------------------------------------------------------------------
 * TurboQuant 1-bit residual codec: random sign flips + Walsh-Hadamard rotation, one sign bit per rotated dimension and
 * one scale per row; candidates are the rows of the probed lists with the smallest reconstructed distance.
 *
 * Parity status of this block: PARTLY PINNED.  The reference's encoder and scan are GPU kernels that cannot run
 * where this file is tested; what it has as host code - the bit layout, the Hamming count and the unfused distance
 * formulas of src/quantization/turboquant/turboquant_1bit_format.h:14-117 - is compiled in place and compared bit for
 * bit (psbo_sign_pack, psbo_sign_hamming, psbo_sign_scale_l2, psbo_sign_binary_l2), with the known answers of
 * tests/unit/turboquant/test_turboquant_1bit_format.cpp:15-47.  The rotation, the scales and the fused scores restate
 * the kernels' arithmetic order from their source and are unpinned:
 *   - sign flip of lane d when the low bit of mix(seed ^ d) is set, butterflies of widths 1,2,4,... writing
 *     (lhs+rhs, lhs-rhs), then every value times `scale` (src/quantization/turboquant/turboquant_1bit_encode.cu:13-19,
 *     44-72).  The kernel takes scale = rsqrtf(padded_dim) on the device; here the caller passes it.
 *   - per-row statistic: a 32-lane shuffle-down tree per group of 32 values, then the same tree over the group sums
 *     (turboquant_1bit_encode.cu:86-108): L1 scale = sum|rotated| / padded_dim for database rows, sum original^2
 *     for query states.
 *   - score of a row against a float state: one chain over d = 0..dim-1 of +-state[d], then
 *     norm_sq + dim*s*s - 2*s*dot (src/quantization/turboquant/turboquant_1bit_score.cuh:54-72), taken here with the
 *     two products fused into the sums: fma(-(2s), dot, fma(dim*s, s, norm_sq)).
 *   - order of candidates: (distance, row) ascending, pad -1 / FLT_MAX (turboquant_1bit_score.cuh:8-14,
 *     turboquant_1bit_grouped_scan.cu:66,155-156). */
static uint32_t sign_mix(uint32_t v) {
    v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu;
    return v ^ (v >> 16);
}

/* What lane 0 holds after `for delta = 16..1: v += shfl_down(v, delta)` over 32 lanes. */
static float sign_tree32(const float* in) {
    float v[32];
    memcpy(v, in, sizeof(v));
    for (int delta = 16; delta > 0; delta >>= 1)
        for (int l = 0; l + delta < 32; ++l) v[l] = v[l] + v[l + delta];
    return v[0];
}

static float sign_block_sum(const float* per_lane, int padded) {
    float groups[32];
    for (int g = 0; g < 32; ++g) groups[g] = 0.0f;
    for (int g = 0; g < padded / 32; ++g) groups[g] = sign_tree32(per_lane + 32 * g);
    return sign_tree32(groups);
}

int psbo_sign_padded_dim(int dim) {
    int p = 32;
    while (p < dim) p <<= 1;
    return (dim <= 0 || p > 256) ? -1 : p;
}

static int sign_shape_ok(int dim, int padded) {
    return dim > 0 && dim <= padded && padded >= 32 && padded <= 256 && (padded & (padded - 1)) == 0;
}

/* values[0..padded) hold the (zero padded) original row on entry and the rotated row on return. */
static void sign_rotate_inplace(float* values, int padded, uint32_t seed, float scale) {
    for (int d = 0; d < padded; ++d)
        if (sign_mix(seed ^ (uint32_t)d) & 1u) values[d] = -values[d];
    for (int width = 1; width < padded; width <<= 1)
        for (int t = 0; t < padded / 2; ++t) {
            const int group = t / width, off = t - group * width;
            const int left = group * (width << 1) + off, right = left + width;
            const float lhs = values[left], rhs = values[right];
            values[left] = lhs + rhs;
            values[right] = lhs - rhs;
        }
    for (int d = 0; d < padded; ++d) values[d] = values[d] * scale;
}

void psbo_sign_pack(const float* values, int dim, uint32_t* words) {
    for (int w = 0; w < (dim + 31) / 32; ++w) words[w] = 0;
    for (int d = 0; d < dim; ++d)
        if (values[d] >= 0.0f) words[d / 32] |= 1u << (d % 32);
}

int psbo_sign_hamming(const uint32_t* a, const uint32_t* b, int dim) {
    int h = 0;
    for (int w = 0; w < dim / 32; ++w) h += __builtin_popcount(a[w] ^ b[w]);
    if (dim % 32) h += __builtin_popcount((a[dim / 32] ^ b[dim / 32]) & ((1u << (dim % 32)) - 1u));
    return h;
}

static float sign_dot(const float* state, const uint32_t* code, int dim) {
    float dot = 0.0f;
    for (int d = 0; d < dim; ++d) dot += ((code[d / 32] >> (d % 32)) & 1u) ? state[d] : -state[d];
    return dot;
}

/* The host formula (turboquant_1bit_format.h:86-103): sequential sums, no fused operations. */
float psbo_sign_scale_l2(const float* query, const uint32_t* code, int dim, float s) {
    float norm = 0.0f;
    for (int d = 0; d < dim; ++d) norm += query[d] * query[d];
    const float dot = sign_dot(query, code, dim);
    return norm + (float)dim * s * s - 2.0f * s * dot;
}

float psbo_sign_binary_l2(const uint32_t* qcode, const uint32_t* code, int dim, float qn, float dn) {
    if (dim == 0) return 0.0f;
    const int h = psbo_sign_hamming(qcode, code, dim);
    const float cosine = ((float)dim - 2.0f * (float)h) / (float)dim;
    return qn * qn + dn * dn - 2.0f * qn * dn * cosine;
}

/* The scan kernel's scores (fused). */
float psbo_sign_score_mse(const float* state, float norm_sq, const uint32_t* code, int dim, float s) {
    const float dot = sign_dot(state, code, dim);
    return fmaf(-(2.0f * s), dot, fmaf((float)dim * s, s, norm_sq));
}

float psbo_sign_score_binary(const uint32_t* qcode, const uint32_t* code, int dim, float qn, float dn) {
    const int h = psbo_sign_hamming(qcode, code, dim);
    const float cosine = ((float)dim - 2.0f * (float)h) / (float)dim;
    return fmaf(-(2.0f * qn * dn), cosine, fmaf(dn, dn, qn * qn));
}

/* turboquant_1bit_encode_gpu (turboquant_1bit_encode.cu:113-172): rotated rows, sign words, sqrt and sum of squares of the
 * original row.  Any output may be null. */
int psbo_sign_rotate(const float* rows, int64_t n, int dim, int padded, uint32_t seed, float scale,
                     float* rotated, uint32_t* codes, float* norms, float* norm_sq) {
    if (!rows || n < 0 || !sign_shape_ok(dim, padded)) return 1;
    const int words = padded / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        float v[256], sq[256];
        for (int d = 0; d < padded; ++d) {
            const float x = d < dim ? rows[(size_t)r * dim + d] : 0.0f;
            v[d] = x; sq[d] = d < dim ? x * x : 0.0f;
        }
        sign_rotate_inplace(v, padded, seed, scale);
        if (rotated) memcpy(rotated + (size_t)r * padded, v, sizeof(float) * (size_t)padded);
        if (codes) psbo_sign_pack(v, padded, codes + (size_t)r * words);
        const float sum = sign_block_sum(sq, padded);
        if (norm_sq) norm_sq[r] = sum;
        if (norms) norms[r] = sqrtf(sum);
    }
    return 0;
}

static int sign_row_list(int64_t row, const int64_t* offsets, int nlist) {
    int lo = 0, hi = nlist;
    while (lo + 1 < hi) {
        const int mid = lo + (hi - lo) / 2;
        if (offsets[mid] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

/* ivf_res_turboquant_encode_database_u8_gpu (turboquant_1bit_encode.cu:188-206): residual of row (row_offset + r)
 * against the centroid of its list, rotated; sign words and L1 scale land at the global row.  elem_bytes 1 = u8 rows (the
 * reference's input), 4 = fp32 rows. */
int psbo_sign_encode_database(const void* rows, int elem_bytes, int64_t n, const float* centroids, const int64_t* offsets,
                              int nlist, int dim, int padded, uint32_t seed, float scale, int64_t row_offset,
                              uint32_t* codes, float* scales) {
    if (!rows || !centroids || !offsets || !codes || n < 0 || nlist <= 0 || !sign_shape_ok(dim, padded)) return 1;
    if (elem_bytes != 1 && elem_bytes != 4) return 1;
    const int words = padded / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const int64_t g = r + row_offset;
        const int list = sign_row_list(g, offsets, nlist);
        float v[256], mag[256];
        for (int d = 0; d < padded; ++d) {
            float x = 0.0f;
            if (d < dim) {
                const float raw = elem_bytes == 1 ? (float)((const uint8_t*)rows)[(size_t)r * dim + d]
                                                  : ((const float*)rows)[(size_t)r * dim + d];
                x = raw - centroids[(size_t)list * dim + d];
            }
            v[d] = x;
        }
        sign_rotate_inplace(v, padded, seed, scale);
        psbo_sign_pack(v, padded, codes + (size_t)g * words);
        for (int d = 0; d < padded; ++d) mag[d] = fabsf(v[d]);
        if (scales) scales[g] = sign_block_sum(mag, padded) / (float)padded;
    }
    return 0;
}

/* ivf_res_turboquant_encode_queries_gpu (turboquant_1bit_encode.cu:208-228): one state per (query, probe): the rotated
 * residual against the probed centroid, its sign words, and sqrt / sum of squares of the residual.  A probe outside
 * [0, nlist) yields a zero state. */
int psbo_sign_encode_queries(const float* queries, const float* centroids, const int* probes, int nq, int nprobe,
                             int nlist, int dim, int padded, uint32_t seed, float scale, float* states, float* norm_sq,
                             uint32_t* state_codes, float* norms) {
    if (!queries || !centroids || !probes || nq < 0 || nprobe <= 0 || !sign_shape_ok(dim, padded)) return 1;
    const int words = padded / 32;
#pragma omp parallel for schedule(static)
    for (int64_t st = 0; st < (int64_t)nq * nprobe; ++st) {
        const int q = (int)(st / nprobe), list = probes[st];
        float v[256], sq[256];
        const int ok = list >= 0 && list < nlist;
        for (int d = 0; d < padded; ++d) {
            const float x = (ok && d < dim) ? queries[(size_t)q * dim + d] - centroids[(size_t)list * dim + d] : 0.0f;
            v[d] = x; sq[d] = x * x;
        }
        sign_rotate_inplace(v, padded, seed, scale);
        if (states) memcpy(states + (size_t)st * padded, v, sizeof(float) * (size_t)padded);
        if (state_codes) psbo_sign_pack(v, padded, state_codes + (size_t)st * words);
        const float sum = sign_block_sum(sq, padded);
        if (norm_sq) norm_sq[st] = sum;
        if (norms) norms[st] = sqrtf(sum);
    }
    return 0;
}

/* SearchWorkspace::search_candidates (src/search/ivf_res_turboquant/ivf_res_turboquant_search.cu:226-343): every row of
 * every valid probed list scored against the state of its (query, probe), the candidate_count smallest by (score, row).
 * mode 0 = float states (MseFloatQuery), 1 = sign-coded states (BinaryQuery). */
int psbo_sign_candidates(int mode, const float* states, const float* norm_sq, const uint32_t* state_codes,
                         const float* norms, const uint32_t* codes, const float* row_params, const int64_t* offsets,
                         int nlist, const int* probes, int nq, int nprobe, int padded, int candidate_count,
                         int* rows_out, float* dist_out) {
    if (!codes || !row_params || !offsets || !probes || !rows_out || nq < 0 || nprobe <= 0 || candidate_count <= 0) return 1;
    if (mode == 0 ? (!states || !norm_sq) : (!state_codes || !norms)) return 1;
    if (!sign_shape_ok(padded, padded)) return 1;
    const int words = padded / 32;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int q = 0; q < nq; ++q) {
        pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)candidate_count);
        if (!heap) { bad = 1; continue; }
        topk_t t;
        topk_init(&t, heap, candidate_count);
        for (int p = 0; p < nprobe; ++p) {
            const int64_t st = (int64_t)q * nprobe + p;
            const int list = probes[st];
            if (list < 0 || list >= nlist) continue;
            for (int64_t r = offsets[list]; r < offsets[list + 1]; ++r) {
                const uint32_t* code = codes + (size_t)r * words;
                const float d = mode == 0
                    ? psbo_sign_score_mse(states + (size_t)st * padded, norm_sq[st], code, padded, row_params[r])
                    : psbo_sign_score_binary(state_codes + (size_t)st * words, code, padded, norms[st], row_params[r]);
                topk_push(&t, d, r);
            }
        }
        topk_finish(&t);
        for (int i = 0; i < candidate_count; ++i) {
            rows_out[(size_t)q * candidate_count + i] = i < t.n ? (int)t.h[i].i : -1;
            if (dist_out) dist_out[(size_t)q * candidate_count + i] = i < t.n ? t.h[i].d : FLT_MAX;
        }
        free(heap);
    }
    return bad;
}
