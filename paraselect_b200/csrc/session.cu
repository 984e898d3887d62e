// Host side of the C ABI: sessions (device copies of the index, workspaces, the batch pipeline), the
// stage-level and one-shot operator entry points, training drivers and the synthetic-data entry points.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <climits>
#include <cmath>
#include <cstring>
#include <limits>
#include <random>
#include <memory>
#include <new>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace psb {

// ---- status plumbing ------------------------------------------------------------------------------
std::string& last_error_ref() {
    thread_local std::string e;
    return e;
}
psb_status fail(psb_status code, const std::string& message) {
    last_error_ref() = message;
    return code;
}
psb_status cuda_fail(cudaError_t err, const char* what, const char* file, int line) {
    const char* base = std::strrchr(file, '/');
    last_error_ref() = std::string(cudaGetErrorString(err)) + " in " + what + " (" + (base ? base + 1 : file) + ":" +
                       std::to_string(line) + ")";
    if (err == cudaErrorMemoryAllocation) { cudaGetLastError(); return PSB_OUT_OF_MEMORY; }
    return PSB_CUDA_ERROR;
}
static std::atomic<long long> g_launches{0};
void count_launch(long long n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches_total() { return g_launches.load(std::memory_order_relaxed); }

namespace {

// Device buffer that grows on demand (contents are not preserved).
struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    ~DevBuf() { release(); }
    void release() { if (p) cudaFree(p); p = nullptr; bytes = 0; }
    psb_status reserve(size_t need) {
        if (need <= bytes) return PSB_OK;
        release();
        PSB_CUDA(cudaMalloc(&p, need ? need : 1));
        bytes = need;
        return PSB_OK;
    }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

psb_status check_device(int device, cudaDeviceProp* prop_out = nullptr) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fail(PSB_NO_DEVICE, "no CUDA device is usable; this library has no CPU path");
    }
    if (device < 0 || device >= n) return fail(PSB_INVALID_ARGUMENT, "device ordinal out of range");
    cudaDeviceProp prop;
    PSB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(PSB_NO_DEVICE, "device is not sm_100 (kernels are built for sm_100a only)");
    if (prop_out) *prop_out = prop;
    PSB_CUDA(cudaSetDevice(device));
    return PSB_OK;
}

// The same check for operators called once per batch: attribute queries (microseconds) instead of the full property
// block (milliseconds), and the SM count remembered per device.
psb_status check_device_quick(int device, int* sm_count) {
    static int known_sms[64] = {0};
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fail(PSB_NO_DEVICE, "no CUDA device is usable; this library has no CPU path");
    }
    if (device < 0 || device >= n) return fail(PSB_INVALID_ARGUMENT, "device ordinal out of range");
    if (device >= 64 || known_sms[device] == 0) {
        int major = 0, sms = 0;
        PSB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        PSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        if (major != 10) return fail(PSB_NO_DEVICE, "device is not sm_100 (kernels are built for sm_100a only)");
        if (device < 64) known_sms[device] = sms;
        if (sm_count) *sm_count = sms;
    } else if (sm_count) {
        *sm_count = known_sms[device];
    }
    PSB_CUDA(cudaSetDevice(device));
    return PSB_OK;
}

// Persistent fork-join pool of host threads for the staged rerank transport (the reference keeps a persistent rerank pool
// too: src/search/ivf_common/ivf_host_rerank.cpp:42-51).  run(job) calls job(t) on every thread t and returns when all are done.
class HostPool {
public:
    explicit HostPool(int n) : n_(n) {
        for (int t = 0; t < n_; ++t) threads_.emplace_back([this, t] { loop(t); });
    }
    ~HostPool() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; ++gen_; }
        cv_.notify_all();
        for (auto& th : threads_) th.join();
    }
    int size() const { return n_; }
    template <typename F>
    void run(F&& job) {
        std::function<void(int)> f = std::forward<F>(job);
        { std::lock_guard<std::mutex> lk(mu_); job_ = &f; pending_ = n_; ++gen_; }
        cv_.notify_all();
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [this] { return pending_ == 0; });
        job_ = nullptr;
    }
private:
    void loop(int t) {
        unsigned long long seen = 0;
        for (;;) {
            const std::function<void(int)>* f = nullptr;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
                f = job_;
            }
            if (f) (*f)(t);
            { std::lock_guard<std::mutex> lk(mu_); if (--pending_ == 0) done_.notify_all(); }
        }
    }
    int n_;
    std::vector<std::thread> threads_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    const std::function<void(int)>* job_ = nullptr;
    unsigned long long gen_ = 0;
    int pending_ = 0;
    bool stop_ = false;
};

struct EventTimer {
    std::vector<cudaEvent_t> ev;
    ~EventTimer() { for (auto e : ev) cudaEventDestroy(e); }
    psb_status mark(cudaStream_t s) {
        cudaEvent_t e;
        PSB_CUDA(cudaEventCreate(&e));
        ev.push_back(e);
        PSB_CUDA(cudaEventRecord(e, s));
        return PSB_OK;
    }
    double ms(size_t a, size_t b) const {
        float t = 0.f;
        if (a < ev.size() && b < ev.size()) cudaEventElapsedTime(&t, ev[a], ev[b]);
        return t;
    }
};

// Centroid-side buffers of the tensor-core coarse filter (built once per index).
struct TcIndexBuffers {
    DevBuf cb, cn2, cnorm, mu;
    float cmax = 0.f;
    bool ready = false;
    psb_status prepare(const float* h_centroids, const float* d_centroids, int nlist, int dim, cudaStream_t st) {
        std::vector<double> acc((size_t)dim, 0.0);
        for (int c = 0; c < nlist; ++c)
            for (int d = 0; d < dim; ++d) acc[(size_t)d] += h_centroids[(size_t)c * dim + d];
        std::vector<float> mean((size_t)dim);
        for (int d = 0; d < dim; ++d) mean[(size_t)d] = (float)(acc[(size_t)d] / nlist);
        const int dimp = coarse_tc_padded_dim(dim);
        PSB_TRY(mu.reserve(sizeof(float) * (size_t)dim));
        PSB_TRY(cb.reserve((size_t)2 * nlist * dimp));
        PSB_TRY(cn2.reserve(sizeof(float) * (size_t)coarse_tc_tiles(nlist) * 256));
        PSB_TRY(cnorm.reserve(sizeof(float) * (size_t)nlist));
        PSB_CUDA(cudaMemcpyAsync(mu.p, mean.data(), sizeof(float) * (size_t)dim, cudaMemcpyHostToDevice, st));
        PSB_TRY(launch_tc_prep_centroids(d_centroids, nlist, dim, mu.as<float>(), cb.p, cn2.as<float>(), cnorm.as<float>(), st));
        std::vector<float> norms((size_t)nlist);
        PSB_CUDA(cudaMemcpyAsync(norms.data(), cnorm.p, sizeof(float) * (size_t)nlist, cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaStreamSynchronize(st));
        cmax = 0.f;
        for (float v : norms) cmax = std::max(cmax, v);
        ready = true;
        return PSB_OK;
    }
    CoarseTcIndex view(const float* d_centroids, int nlist, int dim) const {
        CoarseTcIndex ix;
        ix.centroids = d_centroids; ix.cb = cb.p; ix.cn2 = cn2.as<float>(); ix.mu = mu.as<float>(); ix.cmax = cmax;
        ix.nlist = nlist; ix.dim = dim;
        return ix;
    }
};

// Per-batch buffers of the tensor-core coarse filter.
struct TcWorkBuffers {
    DevBuf qb, qnorm, gmin, seltop, selids, cand_cnt, cand, fail_list, scalars;
    psb_status ensure(int nq, int nlist, int dim, int nprobe, cudaStream_t st) {
        const int dimp = coarse_tc_padded_dim(dim);
        const int groups = coarse_tc_tiles(nlist) * (256 / coarse_tc_group(nlist, nprobe));
        PSB_TRY(qb.reserve((size_t)2 * nq * dimp));
        PSB_TRY(qnorm.reserve(sizeof(float) * (size_t)nq));
        PSB_TRY(gmin.reserve(sizeof(float) * (size_t)nq * groups));
        PSB_TRY(seltop.reserve(sizeof(float) * (size_t)nq * nprobe));
        PSB_TRY(selids.reserve(sizeof(int) * (size_t)nq * nprobe));
        PSB_TRY(cand_cnt.reserve(sizeof(int) * (size_t)nq));
        PSB_TRY(cand.reserve(sizeof(int) * (size_t)nq * coarse_tc_mask_words(nlist)));
        PSB_TRY(fail_list.reserve(sizeof(int) * (size_t)nq));
        if (!scalars.p) {
            PSB_TRY(scalars.reserve(sizeof(int) * 4));
            PSB_CUDA(cudaMemsetAsync(scalars.p, 0, sizeof(int) * 4, st));
        }
        return PSB_OK;
    }
    CoarseTcWorkspace view() const {
        CoarseTcWorkspace w;
        w.qb = qb.p; w.qnorm = qnorm.as<float>(); w.gmin = gmin.as<float>(); w.seltop = seltop.as<float>();
        w.selids = selids.as<int>(); w.cand_cnt = cand_cnt.as<int>(); w.cand = cand.as<int>();
        w.fail_list = fail_list.as<int>(); w.n_fail = scalars.as<int>(); w.status = scalars.as<int>() + 2;
        return w;
    }
    // Reads the sticky time-out word (the stream must be idle).
    psb_status check_status() const {
        if (!scalars.p) return PSB_OK;
        int st = 0;
        PSB_CUDA(cudaMemcpy(&st, scalars.as<int>() + 2, sizeof(int), cudaMemcpyDeviceToHost));
        if (st) return fail(PSB_TIMEOUT, "a bounded wait in the tensor-core coarse kernel gave up");
        return PSB_OK;
    }
};

}  // namespace
}  // namespace psb

using namespace psb;

struct psb_session {
    TcIndexBuffers tc_index;
    TcWorkBuffers tc_work;
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaStream_t aux_stream = nullptr;  // second stream of the overlapped pipeline (created on first use)
    cudaStream_t zc_stream = nullptr;   // hybrid transport: the kernel gather runs here, beside the copies of aux_stream
    cudaEvent_t zc_ev_a = nullptr, zc_ev_b = nullptr;  // stage-level hybrid rerank: fork to and join from zc_stream

    cudaStream_t home_stream = nullptr; // the stream the session was created with (psb_session_set_stream(NULL) returns to it)
    bool background = false;            // stage calls currently run on a caller's second stream: small-grid gather
    psb_options opt{};
    // index shape
    int nlist = 0, dim = 0, m = 0, k = 0;
    long long n_vectors = 0;
    int list_begin = 0, list_end = 0;
    long long row_base = 0, shard_rows = 0;
    // device copies
    DevBuf centroids, offsets, reordered, codes, codebook, cb_maxnorm, global_begin, row_delta, exact_cache, row_aug, row_bias;
    bool striped = false;          // shard holds a slice of every list (options.list_global_begin)
    // exact rows
    int exact_elem = 0;            // 4 = fp32, 1 = u8, 0 = rerank disabled
    const void* exact_host = nullptr;
    const void* exact_dev = nullptr;  // device-visible pointer (mapped host or resident)
    bool registered = false;
    long long exact_count = 0;
    // staged mode
    void* pinned[2] = {nullptr, nullptr};
    size_t pinned_bytes = 0;
    cudaEvent_t pinned_ev[2] = {nullptr, nullptr};
    bool pinned_used[2] = {false, false};  // a copy out of the ring buffer may still be in flight (its event tells)
    int pinned_slot = 0;
    DevBuf opq, q_rot;                     // OPQ rotation [dim][dim] and the rotated queries of the batch in flight
    bool row_bias_is_u16 = false;          // row_bias holds the caller's affine u16 row correction
    bool flat = false;                     // IVF-Flat session: exact rows resident in flat_rows, no PQ parts
    DevBuf flat_rows;
    std::unique_ptr<HostPool> host_pool;   // gather threads of the staged transport (created on first use)
    double staged_gather_s = 0.0;          // host time spent gathering rows, and the bytes gathered (reported by the bench)
    long long staged_gather_bytes = 0;
    std::vector<int> h_cand;
    int* h_cand_pinned = nullptr;        // candidates of the whole batch on the host (overlapped staged transport)
    size_t h_cand_pinned_count = 0;
    std::vector<long long> h_global_begin, h_offsets;  // striped shards: host copies for the staged transport
    // workspaces
    DevBuf q, q_u8, dist_tile, probes, probe_dist, lut, vis_count, vis_off, vis_cursor, item_off, item_off_tc, visitors, q_rows, thr,
        pool_cnt, pool, fail_list, fallback_partial, scalars, lut_h, lut_scale, cand_rows, cand_dist, cand_count, stage, score, out_rows, out_dist, out_ids;
    int ws_scan_queries = 0;        // queries the scan workspace (visitors, pools, cutoffs) currently holds
    long long ws_scan_tables = 0;   // tables the fp16 table buffer currently holds
    int pool_cap = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> scan_events;  // pending (options.time_kernels)
    double scan_ms_total = 0.0;
    long long scan_launches_total = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> gemm_events;  // pending coarse GEMM passes (options.time_kernels)
    double gemm_ms_total = 0.0;
    long long gemm_launches_total = 0;

    psb_session() = default;
    psb_session(const psb_session&) = delete;
    psb_session& operator=(const psb_session&) = delete;
    // Releases what the session owns; runs for a partially built session too (every failure path of psb_session_create),
    // so the caller's rows never stay pinned after an error.
    ~psb_session() {
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (home_stream) {  // a redirected session: drain and return to the stream it was created with
            cudaStreamSynchronize(home_stream);
            stream = home_stream;
        }
        collect_scan_events();
        if (registered) cudaHostUnregister(const_cast<void*>(exact_host));
        for (int i = 0; i < 2; ++i) {
            if (pinned[i]) cudaFreeHost(pinned[i]);
            if (pinned_ev[i]) cudaEventDestroy(pinned_ev[i]);
        }
        if (h_cand_pinned) cudaFreeHost(h_cand_pinned);
        if (aux_stream) { cudaStreamSynchronize(aux_stream); cudaStreamDestroy(aux_stream); }
        if (zc_stream) { cudaStreamSynchronize(zc_stream); cudaStreamDestroy(zc_stream); }
        if (zc_ev_a) cudaEventDestroy(zc_ev_a);
        if (zc_ev_b) cudaEventDestroy(zc_ev_b);

        if (own_stream && stream) cudaStreamDestroy(stream);
        cudaGetLastError();
    }

    ScanIndex scan_index() const {
        ScanIndex ix;
        ix.codes = codes.as<uint8_t>(); ix.offsets = offsets.as<long long>(); ix.row_base = row_base;
        ix.nlist = nlist; ix.list_begin = list_begin; ix.list_end = list_end; ix.m = m; ix.k = k;
        ix.row_delta = striped ? row_delta.as<long long>() : nullptr;
        ix.residual = opt.adc_mode == 1;
        ix.centroids = centroids.as<float>(); ix.codebook = codebook.as<float>(); ix.dim = dim; ix.row_aug = row_aug.p; if (row_bias_is_u16) { ix.row_bias_u16 = row_bias.as<uint16_t>(); ix.rc_scale = opt.rc_scale; ix.rc_offset = opt.rc_offset; }
        else ix.row_bias = row_bias.as<float>();
        return ix;
    }
    // Which index-wide rows the exact store and the id table of this session hold.
    RowMap row_map() const {
        RowMap mp;
        if (striped) {
            mp.global_begin = global_begin.as<long long>(); mp.local_offsets = offsets.as<long long>(); mp.nlist = nlist;
        }
        mp.base = 0; mp.count = n_vectors;
        return mp;
    }
    // Reads (and clears) the time-out word of the tensor-core scan; the stream must be idle.
    psb_status check_scan_status() {
        if (!scalars.p) return PSB_OK;
        int st = 0;
        int* word = reinterpret_cast<int*>(scalars.as<unsigned long long>() + 12);
        PSB_CUDA(cudaMemcpy(&st, word, sizeof(int), cudaMemcpyDeviceToHost));
        if (st) {
            PSB_CUDA(cudaMemset(word, 0, sizeof(int)));
            return fail(PSB_TIMEOUT, "a bounded wait in the tensor-core scan kernel gave up");
        }
        return PSB_OK;
    }
    ScanWorkspace scan_ws() const {
        ScanWorkspace w;
        w.vis_count = vis_count.as<int>(); w.vis_off = vis_off.as<int>(); w.vis_cursor = vis_cursor.as<int>();
        w.item_off = item_off.as<long long>(); w.visitors = visitors.as<int>(); w.q_rows = q_rows.as<long long>();
        w.thr = thr.as<float>(); w.pool_cnt = pool_cnt.as<int>(); w.pool = pool.as<uint64_t>();
        w.fail_list = fail_list.as<int>();
        w.fallback_partial = fallback_partial.as<uint64_t>();
        unsigned long long* sc = scalars.as<unsigned long long>();
        w.counters = sc;                                   // [0..7]
        w.work_cursor = sc + 8;
        w.n_fail = reinterpret_cast<int*>(sc + 9);
        w.fail_cursor = reinterpret_cast<int*>(sc + 10);
        w.pool_cap = pool_cap;
        w.lut_h = lut_h.p; w.lut_scale = lut_scale.as<float>(); w.scan_mode = opt.scan_mode;
        w.reserve_ctas = opt.reserve_sms;
        w.seed_sigma = opt.seed_sigma;
        w.item_off_tc = item_off_tc.as<long long>(); w.work_cursor_tc = sc + 11; w.tc_status = reinterpret_cast<int*>(sc + 12);
        w.tc_min_visitors = opt.tc_min_visitors; w.tc_wait_limit = opt.test_wait_limit; w.tc_skip_mma = opt.test_skip_mma & 1;
        w.cap_queries = ws_scan_queries; w.cap_tables = ws_scan_tables;
        return w;
    }
    // Scan workspace with a fresh event pair when kernel timing is on.
    psb_status timed_scan_ws(ScanWorkspace* w) {
        *w = scan_ws();
        if (!opt.time_kernels) return PSB_OK;
        cudaEvent_t a, b;
        PSB_CUDA(cudaEventCreate(&a));
        PSB_CUDA(cudaEventCreate(&b));
        scan_events.emplace_back(a, b);
        w->ev_begin = a; w->ev_end = b;
        return PSB_OK;
    }
    // Folds finished event pairs into the totals (call after a stream synchronisation).
    void collect_scan_events() {
        for (auto& pr : scan_events) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) { scan_ms_total += t; ++scan_launches_total; }
            cudaEventDestroy(pr.first); cudaEventDestroy(pr.second);
        }
        scan_events.clear();
        for (auto& pr : gemm_events) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) { gemm_ms_total += t; ++gemm_launches_total; }
            cudaEventDestroy(pr.first); cudaEventDestroy(pr.second);
        }
        gemm_events.clear();
        cudaGetLastError();
    }
};

namespace {

// Plain mode: the rerank runs when exact rows exist and n_rerank > topk.  Residual mode: always (the rows are required).
bool rerank_enabled(const psb_session* s, int topk) {
    if (s->opt.adc_mode == 1) return true;
    return s->exact_elem != 0 && s->opt.n_rerank > topk;
}

int stage1_width(const psb_session* s, int topk) {
    if (s->opt.adc_mode == 1)  // src/search/ivfrespq/stage/ivfrespq_cpu_rerank.cpp:623-625
        return std::max(std::max(s->opt.n_rerank, topk), 512);
    if (!rerank_enabled(s, topk)) return topk;
    return (int)std::min<long long>(s->opt.n_rerank, s->n_vectors);
}

// Residual mode without tables: when the tensor-core scan takes every list, nothing reads a materialised per-(query, probe)
// table - the cutoff, the re-scoring selection and the fallback build entries from the query, the centroid and the codebook.
bool residual_table_free(const psb_session* s, int stage1_k) {
    return s->opt.adc_mode == 1 && s->row_aug.p != nullptr && s->row_bias.p != nullptr && (s->opt.scan_mode == 0 || s->opt.scan_mode == 3) &&
           s->opt.tc_min_visitors <= 1 && scan_tc_supported(s->dim, s->m, s->k) &&
           (size_t)pool_capacity(stage1_k) * 8 + (size_t)s->dim * 4 <= (size_t)226 * 1024;
}

// Tables one scan call needs for nq queries.
size_t table_count(const psb_session* s, int nq, int nprobe) {
    return s->opt.adc_mode == 1 ? (size_t)nq * nprobe : (size_t)nq;
}

// Queries per sub-batch of the pipeline: a quarter of the batch when the rerank overlaps the scan, and in residual mode
// few enough that the per-(query, probe) tables stay below ~16 GiB.
int sub_batch_rows(const psb_session* s, int n, int nprobe, bool overlap) {
    const int pipeline_parts = s->opt.pipeline_parts >= 2 && s->opt.pipeline_parts <= 32 ? s->opt.pipeline_parts : 4;
    int parts = overlap ? pipeline_parts : 1;
    if (s->opt.adc_mode == 1 && !residual_table_free(s, stage1_width(s, 1))) {
        const double bytes = (double)n * nprobe * s->m * s->k * sizeof(float);
        parts = std::max(parts, (int)std::ceil(bytes / (16.0 * 1024 * 1024 * 1024)));
    }
    parts = std::min(parts, std::max(n, 1));
    return (n + parts - 1) / parts;
}

// The staged transport (host gather threads + pinned rings), alone or with the kernel gather beside it.
bool staged_mode(const psb_session* s) { return s->opt.exact_mode == PSB_EXACT_HOST_STAGED || s->opt.exact_mode == PSB_EXACT_HOST_HYBRID; }

bool overlap_enabled(const psb_session* s, int n, bool rerank) {
    return rerank && !staged_mode(s) && n >= 2048 && !s->opt.serial_pipeline;
}

// Grows the scan workspace to hold nq queries (never shrinks; a growing buffer is freed first, which waits for the device).
psb_status ensure_scan_ws(psb_session* s, int nq, int nprobe, int stage1_k) {
    const size_t tables = table_count(s, nq, nprobe);
    s->ws_scan_queries = 0; s->ws_scan_tables = 0;  // set again below once every buffer has its size
    PSB_TRY(s->vis_count.reserve(sizeof(int) * (size_t)s->nlist));
    PSB_TRY(s->vis_off.reserve(sizeof(int) * ((size_t)s->nlist + 1)));
    PSB_TRY(s->vis_cursor.reserve(sizeof(int) * (size_t)s->nlist));
    PSB_TRY(s->item_off.reserve(sizeof(long long) * ((size_t)s->nlist + 1)));
    PSB_TRY(s->item_off_tc.reserve(sizeof(long long) * ((size_t)s->nlist + 1)));
    PSB_TRY(s->visitors.reserve(sizeof(int) * (size_t)nq * nprobe));
    PSB_TRY(s->q_rows.reserve(sizeof(long long) * (size_t)nq));
    PSB_TRY(s->thr.reserve(sizeof(float) * (size_t)nq));
    PSB_TRY(s->pool_cnt.reserve(sizeof(int) * (size_t)nq));
    const int cap = pool_capacity(stage1_k);
    PSB_TRY(s->pool.reserve(sizeof(uint64_t) * (size_t)nq * cap));
    s->pool_cap = cap;
    PSB_TRY(s->fail_list.reserve(sizeof(int) * (size_t)nq));
    PSB_TRY(s->fallback_partial.reserve(fallback_partial_bytes(stage1_k)));
    const bool half_tables = s->opt.scan_mode != 1 && !residual_table_free(s, stage1_k);
    if (half_tables) {
        PSB_TRY(s->lut_h.reserve(sizeof(unsigned short) * tables * s->m * s->k));
        PSB_TRY(s->lut_scale.reserve(sizeof(float) * tables));
    }
    if (!s->scalars.p) {
        PSB_TRY(s->scalars.reserve(sizeof(unsigned long long) * 16));
        PSB_CUDA(cudaMemsetAsync(s->scalars.p, 0, sizeof(unsigned long long) * 16, s->stream));
    }
    // what the buffers hold now (reserve() keeps a larger buffer from an earlier call)
    s->ws_scan_queries = (int)std::min<size_t>({s->q_rows.bytes / sizeof(long long), s->thr.bytes / sizeof(float),
                                                s->pool_cnt.bytes / sizeof(int), s->fail_list.bytes / sizeof(int),
                                                s->pool.bytes / (sizeof(uint64_t) * (size_t)cap),
                                                s->visitors.bytes / (sizeof(int) * (size_t)nprobe), (size_t)INT_MAX});
    s->ws_scan_tables = half_tables ? (long long)std::min(s->lut_h.bytes / (sizeof(unsigned short) * (size_t)s->m * s->k),
                                                                    s->lut_scale.bytes / sizeof(float))
                                              : (long long)tables;
    return PSB_OK;
}

psb_status ensure_pipeline_ws(psb_session* s, int nq, int nprobe, int topk, int stage1_k) {
    const int sb = sub_batch_rows(s, nq, nprobe, overlap_enabled(s, nq, rerank_enabled(s, topk)));
    PSB_TRY(s->q.reserve(sizeof(float) * (size_t)nq * s->dim));
    PSB_TRY(s->probes.reserve(sizeof(int) * (size_t)nq * nprobe));
    PSB_TRY(s->probe_dist.reserve(sizeof(float) * (size_t)nq * nprobe));
    if (!residual_table_free(s, stage1_k)) PSB_TRY(s->lut.reserve(sizeof(float) * table_count(s, sb, nprobe) * s->m * s->k));
    PSB_TRY(s->cand_rows.reserve(sizeof(int) * (size_t)nq * stage1_k));
    PSB_TRY(s->cand_dist.reserve(sizeof(float) * (size_t)nq * stage1_k));
    PSB_TRY(s->cand_count.reserve(sizeof(int) * (size_t)nq));
    PSB_TRY(s->out_rows.reserve(sizeof(int) * (size_t)nq * topk));
    PSB_TRY(s->out_dist.reserve(sizeof(float) * (size_t)nq * topk));
    PSB_TRY(s->out_ids.reserve(sizeof(long long) * (size_t)nq * topk));
    return ensure_scan_ws(s, sb, nprobe, stage1_k);  // the scan runs one sub-batch at a time
}

// Coarse stage on device queries: exact distance tiles + row selection, query-chunked so the distance tile
// stays below ~1 GiB.
psb_status coarse_exact(psb_session* s, const float* d_queries, int nq, int nprobe, int* d_ids, float* d_dist) {
    const int mode = s->opt.coarse_mode;
    const bool tc_ok = s->tc_index.ready && coarse_tc_supported(nq, s->nlist, s->dim, nprobe);
    if (mode == 2 && !tc_ok) return fail(PSB_UNSUPPORTED_SHAPE, "tensor-core coarse stage does not support this shape");
    if (mode != 1 && tc_ok) {
        PSB_TRY(s->tc_work.ensure(nq, s->nlist, s->dim, nprobe, s->stream));
        CoarseTcWorkspace tw = s->tc_work.view();
        tw.test_wait_limit = s->opt.test_wait_limit; tw.test_skip_loads = (s->opt.test_skip_mma & 2) ? 1 : 0;
        if (s->opt.time_kernels) {
            for (int i = 0; i < 4; ++i) PSB_CUDA(cudaEventCreate(&tw.ev[i]));
            s->gemm_events.emplace_back(tw.ev[0], tw.ev[1]);
            s->gemm_events.emplace_back(tw.ev[2], tw.ev[3]);
        }
        return launch_coarse_tc(s->tc_index.view(s->centroids.as<float>(), s->nlist, s->dim), tw, d_queries,
                                nq, nprobe, d_ids, d_dist, s->sm_count, s->stream);
    }
    const size_t row_bytes = sizeof(float) * (size_t)s->nlist;
    int chunk = (int)std::max<size_t>(64, ((size_t)1 << 30) / row_bytes);
    chunk = std::min(chunk, nq);
    PSB_TRY(s->dist_tile.reserve(row_bytes * (size_t)chunk));
    for (int q0 = 0; q0 < nq; q0 += chunk) {
        const int n = std::min(chunk, nq - q0);
        PSB_TRY(launch_coarse_dist_exact(d_queries + (size_t)q0 * s->dim, n, s->centroids.as<float>(), s->nlist, s->dim,
                                         s->dist_tile.as<float>(), s->stream));
        PSB_TRY(launch_select_rows(s->dist_tile.as<float>(), n, s->nlist, nprobe, d_ids + (size_t)q0 * nprobe,
                                   d_dist ? d_dist + (size_t)q0 * nprobe : nullptr, s->stream));
    }
    return PSB_OK;
}

psb_status validate_index(const psb_index_view* ix) {
    if (!ix) return fail(PSB_INVALID_ARGUMENT, "index view is null");
    const auto& L = ix->lists;
    if (!L.offsets) return fail(PSB_INVALID_ARGUMENT, "IVF list offsets are null");
    if (L.nlist <= 0 || L.n_vectors < 0) return fail(PSB_INVALID_ARGUMENT, "invalid IVF list layout shape");
    if (L.n_vectors > 0 && !L.reordered_ids) return fail(PSB_INVALID_ARGUMENT, "IVF reordered IDs are null");
    if (L.offsets[0] != 0) return fail(PSB_INVALID_ARGUMENT, "IVF list offsets must start at zero");
    for (int l = 0; l < L.nlist; ++l) {
        const int64_t b = L.offsets[l], e = L.offsets[l + 1];
        if (e < b) return fail(PSB_INVALID_ARGUMENT, "IVF list offsets must be monotonic");
        if (e - b > INT_MAX) return fail(PSB_INVALID_ARGUMENT, "IVF list size exceeds int32 backend limit");
    }
    if (L.offsets[L.nlist] != L.n_vectors) return fail(PSB_INVALID_ARGUMENT, "IVF terminal offset does not match n_vectors");
    if (L.n_vectors > INT_MAX) return fail(PSB_INVALID_ARGUMENT, "n_vectors exceeds int32 row index limit");
    const auto& C = ix->coarse;
    if (!C.centroids || C.nlist != L.nlist || C.dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid IVF coarse index view");
    const auto& P = ix->pq;
    if (!P.codes && L.n_vectors > 0) return fail(PSB_INVALID_ARGUMENT, "PQ codes are null");
    if (P.code_storage) return fail(PSB_UNSUPPORTED_SHAPE, "paged CPU code storage is not supported; pass row-major codes");
    if (!P.codebook || P.subvectors <= 0 || C.dim % P.subvectors != 0)
        return fail(PSB_INVALID_ARGUMENT, "PQ subvectors must divide dim");
    if (P.codebook_size <= 0 || P.codebook_size > kMaxCodebook) return fail(PSB_INVALID_ARGUMENT, "PQ codebook_size must be in 1..256");
    const auto& E = ix->exact;
    if (E.fp32 || E.u8) {
        if (E.count != L.n_vectors || E.dim != C.dim) return fail(PSB_INVALID_ARGUMENT, "exact storage shape does not match the index");
        if (E.source_rows) return fail(PSB_UNSUPPORTED_SHAPE, "exact storage with a row permutation is not supported");
    }
    return PSB_OK;
}

psb_status validate_params(const psb_session* s, const psb_query_batch_view* qv, const psb_search_params* p,
                           const psb_search_output_view* out) {
    if (!qv || !p || !out) return fail(PSB_INVALID_ARGUMENT, "null query, params or output view");
    if (qv->count < 0 || qv->dim != s->dim) return fail(PSB_INVALID_ARGUMENT, "query dim does not match the index");
    if (qv->count > 0 && !qv->fp32) return fail(PSB_INVALID_ARGUMENT, "fp32 queries are required");
    if (p->nprobe <= 0 || p->nprobe > s->nlist) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist");
    if (p->topk <= 0) return fail(PSB_INVALID_ARGUMENT, "topk must be positive");
    if (p->batch_size <= 0) return fail(PSB_INVALID_ARGUMENT, "batch_size must be positive");
    if (p->distance != 0) return fail(PSB_UNSUPPORTED_SHAPE, "only squared L2 is supported on this path");
    if (p->nprobe > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 is not supported");
    if (p->topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "topk above 2048 is not supported");
    if (qv->count > 0 && (!out->indices || !out->distances)) return fail(PSB_INVALID_ARGUMENT, "output buffers are null");
    if (qv->count > 0 && s->exact_elem == 1 && rerank_enabled(s, p->topk) && !qv->u8) return fail(PSB_INVALID_ARGUMENT, "u8 rerank needs u8 queries");
    return PSB_OK;
}

// Host-side twin of the device row mapping (staged transport only).
long long host_local_row(const psb_session* s, long long r) {
    if (r < 0) return -1;
    if (!s->striped) return r < s->n_vectors ? r : -1;
    const auto& gb = s->h_global_begin;
    auto it = std::upper_bound(gb.begin(), gb.end(), r);
    if (it == gb.begin()) return -1;
    const size_t l = (size_t)(it - gb.begin()) - 1;
    const long long loc = s->h_offsets[l] + (r - gb[l]);
    return loc < s->h_offsets[l + 1] ? loc : -1;
}

// Staged rerank transport: candidate rows come back to the host, host threads gather the exact rows into two
// pinned buffers, and cudaMemcpyAsync moves each filled buffer while the other is being filled.
// h_cand: the candidates on the host; d_stage: destination [nq][width][row bytes]; copies are queued on `stream`.
psb_status staged_gather_host(psb_session* s, const int* h_cand, int nq, int width, int stride, void* d_stage, cudaStream_t stream) {
    const size_t row_bytes = (size_t)s->dim * s->exact_elem;
    const size_t chunk_q = std::max<size_t>(1, ((size_t)64 << 20) / std::max<size_t>(1, row_bytes * width));
    const size_t need = chunk_q * width * row_bytes;
    if (s->pinned_bytes < need) {
        for (int i = 0; i < 2; ++i) {
            if (s->pinned_used[i]) PSB_CUDA(cudaEventSynchronize(s->pinned_ev[i]));  // no copy may still read the old buffer
            s->pinned_used[i] = false;
            if (s->pinned[i]) cudaFreeHost(s->pinned[i]);
            s->pinned[i] = nullptr;
            PSB_CUDA(cudaHostAlloc(&s->pinned[i], need, cudaHostAllocDefault));
            if (!s->pinned_ev[i]) PSB_CUDA(cudaEventCreateWithFlags(&s->pinned_ev[i], cudaEventDisableTiming));
        }
        s->pinned_bytes = need;
    }
    if (!s->host_pool) {
        const unsigned hc = s->opt.host_threads > 0 ? (unsigned)s->opt.host_threads : std::max(1u, std::thread::hardware_concurrency());
        s->host_pool.reset(new HostPool((int)std::min<unsigned>(hc, 64)));
    }
    const int nthreads = s->host_pool->size();
    // The ring state outlives the call: the next call may start while this call's last copy is still in flight.
    for (size_t q0 = 0; q0 < (size_t)nq; q0 += chunk_q, s->pinned_slot ^= 1) {
        const int slot = s->pinned_slot;
        const size_t n = std::min(chunk_q, (size_t)nq - q0);
        if (s->pinned_used[slot]) PSB_CUDA(cudaEventSynchronize(s->pinned_ev[slot]));
        unsigned char* dst = static_cast<unsigned char*>(s->pinned[slot]);
        const unsigned char* src = static_cast<const unsigned char*>(s->exact_host);
        const size_t total = n * width;
        const auto t_begin = std::chrono::steady_clock::now();
        s->host_pool->run([&](int t) {
            // Rows sit at random places of a host array far larger than the caches: each copy would wait for DRAM.  The rows of
            // the next kAhead candidates are resolved and prefetched while the current one is copied, so a thread keeps
            // several misses in flight.
            constexpr int kAhead = 8;
            const size_t b = total * t / nthreads, e = total * (t + 1) / nthreads;
            long long rows[kAhead];
            auto resolve = [&](size_t i) -> long long {
                const size_t q = q0 + i / width, c = i % width;
                const long long row = host_local_row(s, h_cand[q * stride + c]);
                return (row >= 0 && row < s->exact_count) ? row : -1;
            };
            for (size_t i = b; i < std::min(e, b + kAhead); ++i) {
                rows[i % kAhead] = resolve(i);
                if (rows[i % kAhead] >= 0)
                    for (size_t off = 0; off < row_bytes; off += 64) __builtin_prefetch(src + (size_t)rows[i % kAhead] * row_bytes + off, 0, 0);
            }
            for (size_t i = b; i < e; ++i) {
                const long long row = rows[i % kAhead];
                if (i + kAhead < e) {
                    const long long nx = resolve(i + kAhead);
                    rows[i % kAhead] = nx;
                    if (nx >= 0)
                        for (size_t off = 0; off < row_bytes; off += 64) __builtin_prefetch(src + (size_t)nx * row_bytes + off, 0, 0);
                }
                if (row >= 0) std::memcpy(dst + i * row_bytes, src + (size_t)row * row_bytes, row_bytes);
            }
        });
        s->staged_gather_s += std::chrono::duration<double>(std::chrono::steady_clock::now() - t_begin).count();
        s->staged_gather_bytes += (long long)(total * row_bytes);
        PSB_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(d_stage) + q0 * width * row_bytes, dst, total * row_bytes,
                                 cudaMemcpyHostToDevice, stream));
        PSB_CUDA(cudaEventRecord(s->pinned_ev[slot], stream));
        s->pinned_used[slot] = true;
    }
    return PSB_OK;
}

psb_status staged_gather(psb_session* s, const int* d_cand, int nq, int width, int stride, const int* d_counts) {
    (void)d_counts;
    s->h_cand.resize((size_t)nq * stride);
    PSB_CUDA(cudaMemcpyAsync(s->h_cand.data(), d_cand, sizeof(int) * (size_t)nq * stride, cudaMemcpyDeviceToHost, s->stream));
    PSB_CUDA(cudaStreamSynchronize(s->stream));
    return staged_gather_host(s, s->h_cand.data(), nq, width, stride, s->stage.p, s->stream);
}

// The stream of the hybrid transport's gather kernel.  Highest priority: its few CTAs each need an SM to themselves and must be
// placed before the large grids of the scan stage that become runnable at the same moment.
psb_status ensure_zc_stream(psb_session* s) {
    if (s->zc_stream) return PSB_OK;
    int lo = 0, hi = 0;
    PSB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    PSB_CUDA(cudaStreamCreateWithPriority(&s->zc_stream, cudaStreamNonBlocking, hi));
    return PSB_OK;
}

psb_status rerank_impl(psb_session* s, const void* d_queries, int nq, const int* d_cand, int width, int stride,
                       const int* d_counts, int topk, int* d_out_rows, float* d_out_dist, float* d_score = nullptr) {
    if (!s->exact_elem) return fail(PSB_INVALID_ARGUMENT, "session has no exact rows for the rerank");
    if (width <= 0 || stride < width || topk <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid rerank request");
    if (width > kMaxRerankWidth || topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "rerank width above 4096 or topk above 2048");
    PSB_TRY(s->stage.reserve((size_t)nq * width * s->dim * s->exact_elem));
    const int zc_pct = s->opt.zero_copy_pct > 0 ? s->opt.zero_copy_pct : 45;
    const int mz = (int)((long long)nq * zc_pct / 100);
    if (s->opt.exact_mode == PSB_EXACT_HOST_HYBRID && s->exact_dev && mz > 0 && mz < nq && (long long)nq * width >= 65536) {
        // Both transports for one stage call (the sharded step's exchange half): the kernel gathers the rows of the last mz
        // queries on a stream of its own while this thread gathers the others through the pinned rings.  The call blocks for
        // the host gather; a caller that overlaps it with a scan queues that scan first.
        const int mh = nq - mz;
        const size_t row_bytes = (size_t)s->dim * s->exact_elem;
        const bool beside = s->background || (s->aux_stream != nullptr && s->stream == s->aux_stream);
        PSB_TRY(ensure_zc_stream(s));
        if (!s->zc_ev_a) PSB_CUDA(cudaEventCreateWithFlags(&s->zc_ev_a, cudaEventDisableTiming));
        if (!s->zc_ev_b) PSB_CUDA(cudaEventCreateWithFlags(&s->zc_ev_b, cudaEventDisableTiming));
        PSB_CUDA(cudaEventRecord(s->zc_ev_a, s->stream));
        PSB_CUDA(cudaStreamWaitEvent(s->zc_stream, s->zc_ev_a, 0));
        PSB_TRY(launch_gather_rows(s->exact_dev, s->row_map(), s->dim, s->exact_elem, d_cand + (size_t)mh * stride, mz, width, stride,
                                   d_counts ? d_counts + mh : nullptr, static_cast<unsigned char*>(s->stage.p) + (size_t)mh * width * row_bytes,
                                   s->zc_stream, s->sm_count, 0, beside && s->opt.gather_ctas == 0 ? (s->opt.reserve_sms > 0 ? s->opt.reserve_sms : 8) : 0));
        PSB_CUDA(cudaEventRecord(s->zc_ev_b, s->zc_stream));
        PSB_TRY(staged_gather(s, d_cand, mh, width, stride, d_counts));
        PSB_CUDA(cudaStreamWaitEvent(s->stream, s->zc_ev_b, 0));
    } else if (staged_mode(s) && !(s->opt.exact_mode == PSB_EXACT_HOST_HYBRID && s->exact_dev && mz >= nq)) {
        PSB_TRY(staged_gather(s, d_cand, nq, width, stride, d_counts));
    } else {
        // Beside a scan on the other stream the gather runs on SMs of its own: the ones the scan's persistent grid leaves free
        // (reserve_sms), or gather_ctas lean CTAs spread over all SMs when the caller asks for that.
        const bool beside = s->background || (s->aux_stream != nullptr && s->stream == s->aux_stream);
        const bool host_rows = s->opt.exact_mode == PSB_EXACT_HOST_MAPPED || s->opt.exact_mode == PSB_EXACT_HOST_HYBRID;
        const int owned = beside && host_rows && s->opt.gather_ctas == 0 ? (s->opt.reserve_sms > 0 ? s->opt.reserve_sms : 8) : 0;
        PSB_TRY(launch_gather_rows(s->exact_dev, s->row_map(), s->dim, s->exact_elem, d_cand, nq, width, stride, d_counts,
                                   s->stage.p, s->stream, s->sm_count,
                                   beside ? (s->opt.gather_ctas > 0 ? s->opt.gather_ctas : 2 * s->sm_count) : 0, owned));
    }
    float* score = d_score;
    if (!score) {
        PSB_TRY(s->score.reserve(sizeof(float) * (size_t)nq * width));
        score = s->score.as<float>();
    }
    PSB_TRY(launch_rerank_score(s->stage.p, s->row_map(), s->dim, s->exact_elem, d_queries, d_cand, nq, width, stride,
                                d_counts, score, s->stream));
    if (!d_out_rows) return PSB_OK;  // partial rerank: the caller combines the scores of all shards
    return launch_topk_select(score, d_cand, nq, width, stride, d_counts, topk, d_out_rows, d_out_dist, s->stream);
}

}  // namespace

namespace psb {
SessionShape session_shape(const psb_session* s) {
    SessionShape o;
    o.dim = s->dim; o.m = s->m; o.k = s->k; o.nlist = s->nlist; o.n_rerank = s->opt.n_rerank; o.exact_elem = s->exact_elem;
    o.device = s->device; o.residual = s->opt.adc_mode == 1; o.flat = s->flat; o.stream = s->stream;
    return o;
}
}  // namespace psb

extern "C" {

const char* psb_last_error(void) { return last_error_ref().c_str(); }
const char* psb_version(void) { return kNvtxCompiled ? "paraselect-b200 0.1 (sm_100a, nvtx)" : "paraselect-b200 0.1 (sm_100a)"; }

size_t psb_sizeof(int which) {
    switch (which) {
        case 0: return sizeof(psb_options);
        case 1: return sizeof(psb_stats);
        case 2: return sizeof(psb_index_view);
        case 3: return sizeof(psb_flat_index_view);
        case 4: return sizeof(psb_row_correction_u16_header);
        case 5: return sizeof(psb_search_params);
        default: return 0;
    }
}

int psb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess && p.major == 10) ++ok;
    }
    return ok;
}

psb_status psb_session_create(const psb_index_view* index, const psb_options* options, psb_session** out) {
    PSB_RANGE("ivfpq_prepare");
    if (!out) return fail(PSB_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    PSB_TRY(validate_index(index));
    psb_options opt{};
    if (options) opt = *options;
    if (opt.max_batch <= 0) opt.max_batch = 10000;
    if (opt.exact_mode < 0 || opt.exact_mode > PSB_EXACT_HOST_HYBRID) return fail(PSB_INVALID_ARGUMENT, "unknown exact_mode");
    const int nlist = index->lists.nlist;
    int lb = opt.list_begin, le = opt.list_end;
    if (lb == 0 && le == 0) le = nlist;
    if (lb < 0 || le > nlist || lb > le) return fail(PSB_INVALID_ARGUMENT, "invalid list shard range");
    const int64_t* gb = opt.list_global_begin;
    if (gb) {
        if (lb != 0 || le != nlist) return fail(PSB_INVALID_ARGUMENT, "list_global_begin excludes a list range");
        for (int l = 0; l < nlist; ++l) {
            const int64_t len = index->lists.offsets[l + 1] - index->lists.offsets[l];
            if (gb[l] < 0 || gb[l] + len > INT_MAX || (l + 1 < nlist && gb[l] + len > gb[l + 1]))
                return fail(PSB_INVALID_ARGUMENT, "list_global_begin must give disjoint ascending row ranges below 2^31");
        }
    }
    if (opt.n_rerank > kMaxStage1) return fail(PSB_UNSUPPORTED_SHAPE, "n_rerank above 2048 is not supported");
    if (opt.adc_mode != 0 && opt.adc_mode != 1) return fail(PSB_INVALID_ARGUMENT, "unknown adc_mode");
    if (opt.reserve_sms < 0 || opt.reserve_sms > 64) return fail(PSB_INVALID_ARGUMENT, "reserve_sms must be in 0..64");
    if (opt.seed_sigma != 0.f && !(opt.seed_sigma >= 2.f && opt.seed_sigma <= 10.f)) return fail(PSB_INVALID_ARGUMENT, "seed_sigma must be 0 or in 2..10");
    if (opt.pipeline_parts != 0 && (opt.pipeline_parts < 2 || opt.pipeline_parts > 32)) return fail(PSB_INVALID_ARGUMENT, "pipeline_parts must be 0 or in 2..32");
    if (opt.scan_mode < 0 || opt.scan_mode > 3) return fail(PSB_INVALID_ARGUMENT, "scan_mode must be in 0..3");
    if (opt.tc_min_visitors < 0) return fail(PSB_INVALID_ARGUMENT, "tc_min_visitors must not be negative");
    if (opt.zero_copy_pct < 0 || opt.zero_copy_pct > 100) return fail(PSB_INVALID_ARGUMENT, "zero_copy_pct must be in 0..100");
    if (opt.host_threads < 0 || opt.host_threads > 64) return fail(PSB_INVALID_ARGUMENT, "host_threads must be in 0..64");
    // hybrid transport: the gather kernel runs beside the scan on SMs of its own, which the scan's grid has to leave free
    if (opt.exact_mode == PSB_EXACT_HOST_HYBRID && opt.reserve_sms == 0 && opt.gather_ctas == 0) opt.reserve_sms = 32;
    if (opt.gather_ctas < 0 || opt.gather_ctas > 1024) return fail(PSB_INVALID_ARGUMENT, "gather_ctas must be in 0..1024");
    if (opt.adc_mode == 1 && !index->exact.fp32 && !index->exact.u8)
        return fail(PSB_INVALID_ARGUMENT, "residual mode always reranks: exact rows are required");
    cudaDeviceProp prop;
    PSB_TRY(check_device(opt.device, &prop));
    std::unique_ptr<psb_session> s(new (std::nothrow) psb_session());
    if (!s) return fail(PSB_OUT_OF_MEMORY, "host allocation failed");
    s->device = opt.device; s->sm_count = prop.multiProcessorCount; s->opt = opt;
    s->nlist = nlist; s->dim = index->coarse.dim; s->m = index->pq.subvectors; s->k = index->pq.codebook_size;
    s->n_vectors = index->lists.n_vectors; s->list_begin = lb; s->list_end = le;
    s->row_base = index->lists.offsets[lb];
    s->shard_rows = index->lists.offsets[le] - s->row_base;
    if (opt.stream) s->stream = static_cast<cudaStream_t>(opt.stream);
    else { PSB_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking)); s->own_stream = true; }
    cudaStream_t st = s->stream;
    if (gb) {
        s->striped = true;
        s->h_global_begin.assign(gb, gb + nlist);
        s->h_offsets.assign(index->lists.offsets, index->lists.offsets + nlist + 1);
        std::vector<long long> delta((size_t)nlist);
        for (int l = 0; l < nlist; ++l) delta[(size_t)l] = gb[l] - index->lists.offsets[l];
        PSB_TRY(s->global_begin.reserve(sizeof(long long) * (size_t)nlist));
        PSB_TRY(s->row_delta.reserve(sizeof(long long) * (size_t)nlist));
        PSB_CUDA(cudaMemcpyAsync(s->global_begin.p, s->h_global_begin.data(), sizeof(long long) * (size_t)nlist, cudaMemcpyHostToDevice, st));
        PSB_CUDA(cudaMemcpy(s->row_delta.p, delta.data(), sizeof(long long) * (size_t)nlist, cudaMemcpyHostToDevice));
    }
    PSB_TRY(s->centroids.reserve(sizeof(float) * (size_t)nlist * s->dim));
    PSB_CUDA(cudaMemcpyAsync(s->centroids.p, index->coarse.centroids, sizeof(float) * (size_t)nlist * s->dim, cudaMemcpyHostToDevice, st));
    if (opt.coarse_mode != 1 && nlist >= 1024 && coarse_tc_padded_dim(s->dim) <= 128)
        PSB_TRY(s->tc_index.prepare(index->coarse.centroids, s->centroids.as<float>(), nlist, s->dim, st));
    PSB_TRY(s->offsets.reserve(sizeof(long long) * ((size_t)nlist + 1)));
    PSB_CUDA(cudaMemcpyAsync(s->offsets.p, index->lists.offsets, sizeof(long long) * ((size_t)nlist + 1), cudaMemcpyHostToDevice, st));
    PSB_TRY(s->reordered.reserve(sizeof(long long) * (size_t)std::max<long long>(1, s->n_vectors)));
    if (s->n_vectors > 0)
        PSB_CUDA(cudaMemcpyAsync(s->reordered.p, index->lists.reordered_ids, sizeof(long long) * (size_t)s->n_vectors, cudaMemcpyHostToDevice, st));
    PSB_TRY(s->codes.reserve((size_t)std::max<long long>(1, s->shard_rows) * s->m + 16));
    if (s->shard_rows > 0)
        PSB_CUDA(cudaMemcpyAsync(s->codes.p, index->pq.codes + (size_t)s->row_base * s->m, (size_t)s->shard_rows * s->m, cudaMemcpyHostToDevice, st));
    const size_t cb_bytes = sizeof(float) * (size_t)s->m * s->k * (s->dim / s->m);
    PSB_TRY(s->codebook.reserve(cb_bytes));
    PSB_CUDA(cudaMemcpyAsync(s->codebook.p, index->pq.codebook, cb_bytes, cudaMemcpyHostToDevice, st));
    if (opt.opq_matrix) {
        if (opt.adc_mode == 1) return fail(PSB_INVALID_ARGUMENT, "the OPQ rotation belongs to the plain ADC mode");
        PSB_TRY(s->opq.reserve(sizeof(float) * (size_t)s->dim * s->dim));
        PSB_CUDA(cudaMemcpyAsync(s->opq.p, opt.opq_matrix, sizeof(float) * (size_t)s->dim * s->dim, cudaMemcpyHostToDevice, st));
    }
    // per-row terms of the tensor-core scan (8 bytes per code row), once per index
    if ((opt.scan_mode == 0 || opt.scan_mode == 3) && s->shard_rows > 0 && scan_tc_supported(s->dim, s->m, s->k)) {
        PSB_TRY(s->row_aug.reserve((size_t)s->shard_rows * 8));
        PSB_TRY(launch_row_aug(s->codes.as<uint8_t>(), s->shard_rows, s->dim, s->m, s->k, s->codebook.as<float>(), s->row_aug.p, st));
        if (opt.adc_mode == 1 && opt.row_correction_u16) {  // the caller's row correction, affine u16
            if (!(opt.rc_scale > 0.f)) return fail(PSB_INVALID_ARGUMENT, "row_correction_u16 needs a positive rc_scale");
            PSB_TRY(s->row_bias.reserve(sizeof(uint16_t) * (size_t)s->shard_rows));
            PSB_CUDA(cudaMemcpyAsync(s->row_bias.p, opt.row_correction_u16 + s->row_base, sizeof(uint16_t) * (size_t)s->shard_rows, cudaMemcpyHostToDevice, st));
            s->row_bias_is_u16 = true;
        } else if (opt.adc_mode == 1 && opt.row_correction_fp32) {
            PSB_TRY(s->row_bias.reserve(sizeof(float) * (size_t)s->shard_rows));
            PSB_CUDA(cudaMemcpyAsync(s->row_bias.p, opt.row_correction_fp32 + s->row_base, sizeof(float) * (size_t)s->shard_rows, cudaMemcpyHostToDevice, st));
        } else if (opt.adc_mode == 1) {  // computed here: the per-row correction of the residual cutoff estimate
            PSB_TRY(s->row_bias.reserve(sizeof(float) * (size_t)s->shard_rows));
            PSB_TRY(launch_row_bias(s->codes.as<uint8_t>(), s->offsets.as<long long>(), s->row_base, lb, le, s->dim, s->m, s->k,
                                    s->codebook.as<float>(), s->centroids.as<float>(), s->row_bias.as<float>(), st));
        }
    }
    {   // per sub-quantiser the largest codeword norm (residual-mode table builder)
        const int dsub = s->dim / s->m;
        std::vector<float> mx((size_t)s->m, 0.0f);
        for (int j = 0; j < s->m; ++j)
            for (int c = 0; c < s->k; ++c) {
                double n2 = 0.0;
                for (int d = 0; d < dsub; ++d) { const double v = index->pq.codebook[((size_t)j * s->k + c) * dsub + d]; n2 += v * v; }
                mx[(size_t)j] = std::max(mx[(size_t)j], (float)(std::sqrt(n2) * 1.0001));
            }
        PSB_TRY(s->cb_maxnorm.reserve(sizeof(float) * (size_t)s->m));
        PSB_CUDA(cudaMemcpy(s->cb_maxnorm.p, mx.data(), sizeof(float) * (size_t)s->m, cudaMemcpyHostToDevice));
    }
    // exact rows
    const auto& E = index->exact;
    if (E.fp32 || E.u8) {
        s->exact_elem = E.fp32 ? 4 : 1;
        s->exact_host = E.fp32 ? static_cast<const void*>(E.fp32) : static_cast<const void*>(E.u8);
        s->exact_count = E.count;
        const size_t bytes = (size_t)E.count * E.dim * s->exact_elem;
        if (opt.exact_mode == PSB_EXACT_RESIDENT) {
            s->exact_dev = s->exact_host;
        } else if (opt.exact_mode == PSB_EXACT_HOST_CACHED && bytes > 0) {
            // the session's own copy of the rows in device memory (a B200 holds 180 GB: C4's 38.4 GB of rows fit beside the index)
            size_t free_b = 0, total_b = 0;
            PSB_CUDA(cudaMemGetInfo(&free_b, &total_b));
            if (bytes + ((size_t)8 << 30) > free_b)
                return fail(PSB_OUT_OF_MEMORY, "the exact rows do not fit in device memory beside the workspaces; use a host mode");
            PSB_TRY(s->exact_cache.reserve(bytes));
            const size_t chunk = (size_t)1 << 30;
            for (size_t off = 0; off < bytes; off += chunk)
                PSB_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(s->exact_cache.p) + off,
                                         static_cast<const unsigned char*>(s->exact_host) + off, std::min(chunk, bytes - off),
                                         cudaMemcpyHostToDevice, st));
            s->exact_dev = s->exact_cache.p;
        } else if ((opt.exact_mode == PSB_EXACT_HOST_MAPPED || opt.exact_mode == PSB_EXACT_HOST_HYBRID) && bytes > 0) {
            cudaError_t e = cudaHostRegister(const_cast<void*>(s->exact_host), bytes, cudaHostRegisterMapped | cudaHostRegisterReadOnly);
            if (e == cudaErrorHostMemoryAlreadyRegistered) { cudaGetLastError(); e = cudaSuccess; }
            else if (e != cudaSuccess) {
                cudaGetLastError();
                e = cudaHostRegister(const_cast<void*>(s->exact_host), bytes, cudaHostRegisterMapped);
                if (e == cudaSuccess) s->registered = true;
            } else s->registered = true;
            if (e != cudaSuccess) {
                cudaGetLastError();
                return fail(PSB_CUDA_ERROR, std::string("cannot map the exact rows into the device address space (") +
                                                cudaGetErrorString(e) + "); use PSB_EXACT_HOST_STAGED");
            }
            void* dp = nullptr;
            PSB_CUDA(cudaHostGetDevicePointer(&dp, const_cast<void*>(s->exact_host), 0));
            s->exact_dev = dp;
        }
    }
    PSB_CUDA(cudaStreamSynchronize(st));
    *out = s.release();
    return PSB_OK;
}

psb_status psb_session_destroy(psb_session* s) {
    delete s;  // the destructor releases everything the session owns (also a partially built one)
    return PSB_OK;
}

psb_status psb_session_sync(psb_session* s) {
    if (!s) return fail(PSB_INVALID_ARGUMENT, "session is null");
    PSB_CUDA(cudaStreamSynchronize(s->stream));
    PSB_TRY(s->tc_work.check_status());
    return s->check_scan_status();
}

psb_status psb_session_set_stream(psb_session* s, void* stream, int background) {
    if (!s) return fail(PSB_INVALID_ARGUMENT, "session is null");
    if (!s->home_stream) s->home_stream = s->stream;
    s->stream = stream ? static_cast<cudaStream_t>(stream) : s->home_stream;
    s->background = stream != nullptr && background != 0;
    return PSB_OK;
}

psb_status psb_stage_coarse(psb_session* s, const float* d_queries, int nq, int nprobe, int* d_ids, float* d_dist) {
    PSB_RANGE("coarse_search");
    if (!s || !d_queries || !d_ids) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nprobe <= 0 || nprobe > s->nlist) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist");
    if (nprobe > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 is not supported");
    PSB_CUDA(cudaSetDevice(s->device));
    return coarse_exact(s, d_queries, nq, nprobe, d_ids, d_dist);
}

psb_status psb_rotate_rows(const float* d_in, const float* d_matrix, int64_t n, int dim, float* d_out, int device, void* stream) {
    if (!d_in || !d_matrix || !d_out || n < 0 || dim <= 0 || d_in == d_out) return fail(PSB_INVALID_ARGUMENT, "invalid rotation request");
    PSB_TRY(check_device(device));
    return launch_rotate_rows(d_in, d_matrix, n, dim, d_out, static_cast<cudaStream_t>(stream));
}

int psb_sign_padded_dim(int dim) { return sign_padded_dim(dim); }

psb_status psb_sign_rotation_scale(int padded_dim, float* h_scale, int device, void* stream) {
    if (!h_scale || sign_padded_dim(padded_dim) != padded_dim) return fail(PSB_INVALID_ARGUMENT, "padded_dim must be 32, 64, 128 or 256");
    PSB_TRY(check_device(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* d = nullptr;
    PSB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d), sizeof(float)));
    psb_status rc = launch_sign_scale(padded_dim, d, st);
    cudaError_t e = rc == PSB_OK ? cudaMemcpyAsync(h_scale, d, sizeof(float), cudaMemcpyDeviceToHost, st) : cudaSuccess;
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d);
    if (rc == PSB_OK && e != cudaSuccess) rc = cuda_fail(e, "psb_sign_rotation_scale", __FILE__, __LINE__);
    return rc;
}

psb_status psb_sign_rotate(const float* d_rows, int64_t n, int dim, int padded_dim, uint32_t seed, float* d_rotated,
                           uint32_t* d_codes, float* d_norms, float* d_norm_sq, int device, void* stream) {
    if (!d_rows || n < 0 || (!d_rotated && !d_codes && !d_norms && !d_norm_sq)) return fail(PSB_INVALID_ARGUMENT, "invalid sign rotation request");
    int sms = 0;
    PSB_TRY(check_device_quick(device, &sms));
    return launch_sign_rotate(d_rows, n, dim, padded_dim, seed, d_rotated, d_codes, d_norms, d_norm_sq, sms,
                              static_cast<cudaStream_t>(stream));
}

psb_status psb_sign_encode_database(const void* d_rows, int elem_bytes, int64_t n, const float* d_centroids,
                                    const int64_t* d_list_offsets, int nlist, int dim, int padded_dim, uint32_t seed,
                                    int64_t row_offset, uint32_t* d_codes, float* d_scales, int device, void* stream) {
    if (!d_rows || !d_centroids || !d_list_offsets || !d_codes || n < 0 || nlist <= 0 || row_offset < 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid sign database encoding request");
    if (elem_bytes != 1 && elem_bytes != 4) return fail(PSB_INVALID_ARGUMENT, "rows must be u8 (1) or fp32 (4)");
    int sms = 0;
    PSB_TRY(check_device_quick(device, &sms));
    return launch_sign_encode_database(d_rows, elem_bytes, n, d_centroids, reinterpret_cast<const long long*>(d_list_offsets), nlist,
                                       dim, padded_dim, seed, row_offset, d_codes, d_scales, sms,
                                       static_cast<cudaStream_t>(stream));
}

psb_status psb_sign_encode_queries(const float* d_queries, const float* d_centroids, const int* d_probes, int nq, int nprobe,
                                   int nlist, int dim, int padded_dim, uint32_t seed, float* d_states, float* d_norm_sq,
                                   uint32_t* d_state_codes, float* d_norms, int device, void* stream) {
    if (!d_queries || !d_centroids || !d_probes || nq < 0 || nprobe <= 0 || nlist <= 0 || (!d_states && !d_state_codes))
        return fail(PSB_INVALID_ARGUMENT, "invalid sign query encoding request");
    int sms = 0;
    PSB_TRY(check_device_quick(device, &sms));
    return launch_sign_encode_queries(d_queries, d_centroids, d_probes, nq, nprobe, nlist, dim, padded_dim, seed, d_states, d_norm_sq,
                                      d_state_codes, d_norms, sms, static_cast<cudaStream_t>(stream));
}

psb_status psb_sign_search_candidates(int mode, const float* d_states, const float* d_norm_sq, const uint32_t* d_state_codes,
                                      const float* d_norms, const uint32_t* d_codes, const float* d_row_params,
                                      const int64_t* d_list_offsets, int nlist, const int* d_probes, int nq, int nprobe,
                                      int padded_dim, int candidate_count, int* d_rows_out, float* d_dist_out, int device,
                                      void* stream) {
    PSB_RANGE("sign_candidates");
    if (mode != PSB_SIGN_FLOAT_STATES && mode != PSB_SIGN_CODED_STATES) return fail(PSB_INVALID_ARGUMENT, "unknown sign score mode");
    if (mode == PSB_SIGN_FLOAT_STATES ? (!d_states || !d_norm_sq) : (!d_state_codes || !d_norms))
        return fail(PSB_INVALID_ARGUMENT, "the states of the chosen score mode are missing");
    if (!d_codes || !d_row_params || !d_list_offsets || !d_probes || !d_rows_out || nq < 0 || nprobe <= 0 || nlist <= 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid sign candidate search request");
    int sms = 0;
    PSB_TRY(check_device_quick(device, &sms));
    return launch_sign_candidates(mode, d_states, d_norm_sq, d_state_codes, d_norms, d_codes, d_row_params,
                                  reinterpret_cast<const long long*>(d_list_offsets), nlist, d_probes, nq, nprobe, padded_dim,
                                  candidate_count, d_rows_out, d_dist_out, sms, static_cast<cudaStream_t>(stream));
}

psb_status psb_stage_rotate_queries(psb_session* s, const float* d_queries, int nq, float* d_rotated) {
    if (!s || !d_queries || !d_rotated || nq < 0 || d_queries == d_rotated) return fail(PSB_INVALID_ARGUMENT, "invalid rotation request");
    if (!s->opq.p) return fail(PSB_INVALID_ARGUMENT, "the session has no OPQ rotation");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_rotate_rows(d_queries, s->opq.as<float>(), nq, s->dim, d_rotated, s->stream);
}

psb_status psb_stage_build_lut(psb_session* s, const float* d_queries, int nq, float* d_lut) {
    PSB_RANGE("pq_lut_build");
    if (!s || !d_queries || !d_lut) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_build_lut(d_queries, nq, s->dim, s->codebook.as<float>(), s->m, s->k, d_lut, s->stream);
}

psb_status psb_stage_build_lut_residual(psb_session* s, const float* d_queries, int nq, const int* d_probes, int nprobe,
                                        float* d_lut) {
    PSB_RANGE("pq_lut_build");
    if (!s || !d_queries || !d_probes || !d_lut) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nprobe <= 0 || nprobe > kMaxProbe) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..4096");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_build_lut_residual(d_queries, nq, s->dim, d_probes, nprobe, s->centroids.as<float>(), s->nlist,
                                     s->codebook.as<float>(), s->m, s->k, d_lut, s->stream);
}

psb_status psb_stage_quantize_lut_u8(psb_session* s, const float* d_lut, int64_t tables, uint8_t* d_q8, float* d_scales,
                                     float* d_lo_sum, float* d_inflation) {
    if (!s || !d_lut || !d_q8 || !d_scales || !d_lo_sum || !d_inflation || tables < 0) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_lut_to_u8(d_lut, tables, s->m, s->k, s->opt.adc_mode == 1 ? 1 : 0, d_q8, d_scales, d_lo_sum, d_inflation, s->stream);
}

psb_status psb_stage_scan(psb_session* s, const float* d_lut, int nq, const int* d_probes, int nprobe,
                          int stage1_k, int* d_rows, float* d_dist, int* d_count) {
    return psb_stage_scan_queries(s, nullptr, d_lut, nq, d_probes, nprobe, stage1_k, d_rows, d_dist, d_count);
}

psb_status psb_stage_scan_queries(psb_session* s, const float* d_queries, const float* d_lut, int nq, const int* d_probes,
                                  int nprobe, int stage1_k, int* d_rows, float* d_dist, int* d_count) {
    PSB_RANGE("pq_adc_scan");
    if (!s || !d_probes || !d_rows) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nprobe <= 0 || stage1_k <= 0) return fail(PSB_INVALID_ARGUMENT, "nprobe and stage1_k must be positive");
    if (nprobe > kMaxProbe || stage1_k > kMaxStage1) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 or stage1_k above 2048");
    PSB_CUDA(cudaSetDevice(s->device));
    PSB_TRY(ensure_scan_ws(s, nq, nprobe, stage1_k));
    ScanWorkspace ws;
    PSB_TRY(s->timed_scan_ws(&ws));
    return launch_scan(s->scan_index(), ws, d_lut, nq, d_probes, nprobe, stage1_k, d_rows, d_dist, d_count,
                       s->sm_count, s->stream, d_queries);
}

int psb_scan_sample_words(const psb_session* s, int stage1_k) {
    if (!s || stage1_k <= 0) return 0;
    return seed_record_keys(stage1_k, s->opt.seed_sigma) + kSeedTail;
}

namespace {
psb_status check_scan_stage(psb_session* s, const int* d_probes, int nprobe, int stage1_k) {
    if (!s || !d_probes) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nprobe <= 0 || stage1_k <= 0) return fail(PSB_INVALID_ARGUMENT, "nprobe and stage1_k must be positive");
    if (nprobe > kMaxProbe || stage1_k > kMaxStage1) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 or stage1_k above 2048");
    return PSB_OK;
}
}  // namespace

psb_status psb_stage_scan_sample(psb_session* s, const float* d_queries, const float* d_lut, int nq, const int* d_probes,
                                 int nprobe, int stage1_k, uint32_t* d_samples) {
    PSB_RANGE("pq_adc_scan_sample");
    PSB_TRY(check_scan_stage(s, d_probes, nprobe, stage1_k));
    if (!d_samples) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    PSB_TRY(ensure_scan_ws(s, nq, nprobe, stage1_k));
    ScanWorkspace ws;
    PSB_TRY(s->timed_scan_ws(&ws));
    ws.phase = 1; ws.seed_export = d_samples; ws.seed_keys = seed_record_keys(stage1_k, s->opt.seed_sigma);
    return launch_scan(s->scan_index(), ws, d_lut, nq, d_probes, nprobe, stage1_k, nullptr, nullptr, nullptr, s->sm_count, s->stream, d_queries);
}

psb_status psb_stage_scan_shared(psb_session* s, const float* d_queries, const float* d_lut, int nq, const int* d_probes,
                                 int nprobe, int stage1_k, const uint32_t* d_all_samples, int shards, int* d_rows, float* d_dist,
                                 int* d_count, float* d_cutoff, int64_t* d_rows_scanned) {
    PSB_RANGE("pq_adc_scan");
    PSB_TRY(check_scan_stage(s, d_probes, nprobe, stage1_k));
    if (!d_all_samples || !d_rows || shards <= 0) return fail(PSB_INVALID_ARGUMENT, "null argument or no shards");
    PSB_CUDA(cudaSetDevice(s->device));
    if (nq > s->ws_scan_queries) return fail(PSB_INVALID_ARGUMENT, "psb_stage_scan_shared follows psb_stage_scan_sample of the same queries");
    ScanWorkspace ws;
    PSB_TRY(s->timed_scan_ws(&ws));
    ws.phase = 2; ws.seed_all = d_all_samples; ws.seed_shards = shards; ws.seed_keys = seed_record_keys(stage1_k, s->opt.seed_sigma);
    ws.rows_global = reinterpret_cast<long long*>(d_rows_scanned);
    PSB_TRY(launch_scan(s->scan_index(), ws, d_lut, nq, d_probes, nprobe, stage1_k, d_rows, d_dist, d_count, s->sm_count, s->stream, d_queries));
    if (d_cutoff) PSB_CUDA(cudaMemcpyAsync(d_cutoff, ws.thr, sizeof(float) * (size_t)nq, cudaMemcpyDeviceToDevice, s->stream));
    return PSB_OK;
}

psb_status psb_stage_rerank(psb_session* s, const float* d_queries, int nq, const int* d_candidates,
                            int candidate_count, int candidate_stride, const int* d_counts, int topk,
                            int* d_out_rows, float* d_out_dist) {
    PSB_RANGE("pq_rerank");
    if (!s || !d_queries || !d_candidates || !d_out_rows || !d_out_dist) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    return rerank_impl(s, d_queries, nq, d_candidates, candidate_count, candidate_stride, d_counts, topk, d_out_rows, d_out_dist);
}

psb_status psb_stage_rerank_partial(psb_session* s, const float* d_queries, int nq, const int* d_candidates,
                                    int candidate_count, int candidate_stride, const int* d_counts, float* d_dist) {
    PSB_RANGE("pq_rerank");
    if (!s || !d_queries || !d_candidates || !d_dist) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    return rerank_impl(s, d_queries, nq, d_candidates, candidate_count, candidate_stride, d_counts, 1, nullptr, nullptr, d_dist);
}

psb_status psb_stage_select_topk(psb_session* s, const float* d_dist, const int* d_candidates, int nq,
                                 int candidate_count, int candidate_stride, const int* d_counts, int topk,
                                 int* d_out_rows, float* d_out_dist) {
    if (!s || !d_dist || !d_candidates || !d_out_rows || !d_out_dist) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (candidate_count <= 0 || candidate_stride < candidate_count || topk <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid selection request");
    if (topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "topk above 2048 is not supported");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_topk_select(d_dist, d_candidates, nq, candidate_count, candidate_stride, d_counts, topk, d_out_rows,
                              d_out_dist, s->stream);
}

psb_status psb_stage_map_ids(psb_session* s, const int* d_rows, int64_t n, int64_t* d_indices) {
    PSB_RANGE("pq_map_ids");
    if (!s || !d_rows || !d_indices) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_map_ids(d_rows, n, s->reordered.as<long long>(), s->row_map(), reinterpret_cast<long long*>(d_indices), s->stream);
}

psb_status psb_stage_merge(psb_session* s, const int* d_rows, const float* d_dist, int parts, int nq, int k,
                           int* d_out_rows, float* d_out_dist) {
    if (!s || !d_rows || !d_dist || !d_out_rows || !d_out_dist || parts <= 0 || k <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid merge request");
    PSB_CUDA(cudaSetDevice(s->device));
    return launch_merge(d_rows, d_dist, parts, nq, k, d_out_rows, d_out_dist, s->stream);
}

psb_status psb_session_counters(psb_session* s, psb_stats* stats, int reset) {
    if (!s || !stats) return fail(PSB_INVALID_ARGUMENT, "null argument");
    PSB_CUDA(cudaSetDevice(s->device));
    unsigned long long h[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (s->scalars.p) {
        PSB_CUDA(cudaMemcpyAsync(h, s->scalars.p, sizeof(h), cudaMemcpyDeviceToHost, s->stream));
        if (reset) PSB_CUDA(cudaMemsetAsync(s->scalars.p, 0, sizeof(h), s->stream));
        PSB_CUDA(cudaStreamSynchronize(s->stream));
    }
    stats->pq_scanned_codes = (long long)h[0];
    stats->pq_adc_lookups = (long long)h[0] * s->m;
    stats->threshold_candidates = (long long)h[1];
    stats->fallback_queries = (long long)h[2];
    stats->prefilter_survivors = (long long)h[3];
    stats->tc_wait_item_cycles = (long long)h[4]; stats->tc_wait_rows_cycles = (long long)h[5];
    stats->tc_wait_acc_cycles = (long long)h[6]; stats->tc_tiles = (long long)h[7];
    stats->staged_gather_ms = s->staged_gather_s * 1e3; stats->staged_gather_bytes = s->staged_gather_bytes;
    if (reset) { s->staged_gather_s = 0.0; s->staged_gather_bytes = 0; }
    stats->kernel_launches = launches_total();
    if (!s->scalars.p) PSB_CUDA(cudaStreamSynchronize(s->stream));
    s->collect_scan_events();
    stats->scan_kernel_ms = s->scan_ms_total;
    stats->scan_kernel_launches = s->scan_launches_total;
    stats->coarse_gemm_ms = s->gemm_ms_total;
    stats->coarse_gemm_launches = s->gemm_launches_total;
    if (reset) { s->gemm_ms_total = 0.0; s->gemm_launches_total = 0; }
    stats->coarse_fallback_queries = 0;
    if (s->tc_work.scalars.p) {
        int v = 0;
        PSB_CUDA(cudaMemcpy(&v, s->tc_work.scalars.as<int>() + 3, sizeof(int), cudaMemcpyDeviceToHost));
        stats->coarse_fallback_queries = v;
        if (reset) PSB_CUDA(cudaMemset(s->tc_work.scalars.as<int>() + 3, 0, sizeof(int)));
    }
    if (reset) { s->scan_ms_total = 0.0; s->scan_launches_total = 0; }
    return PSB_OK;
}

namespace {

struct StageTimes { double coarse = 0, lut = 0, scan = 0, rerank = 0, map = 0; };

// One batch, device in / device out.  With a rerank from mapped or resident exact rows the batch is cut into
// sub-batches: coarse + LUT + scan of sub-batch i run on the session's stream while the PCIe gather, exact scoring,
// selection and id map of sub-batch i-1 run on a second stream, so the transfer hides behind the scan.
psb_status search_device(psb_session* s, const float* dq, const void* dq_exact, int n, int nprobe, int topk, int stage1_k,
                         bool rerank, long long* d_ids, float* d_dist, int* d_probes, StageTimes* times) {
    PSB_RANGE("ivfpq_batch");
    cudaStream_t st = s->stream;
    const bool overlap = overlap_enabled(s, n, rerank);
    // Staged transport, overlapped: a host worker thread takes each sub-batch's candidates as soon as its scan has finished,
    // gathers the rows with the host cores into the pinned rings and queues copies + exact scoring on the second stream,
    // while this thread goes on queueing the next sub-batch's scan.  No SM is spent on the transfer.
    const bool staged_overlap = rerank && staged_mode(s) && n >= 2048 && !s->opt.serial_pipeline;
    const int sb = sub_batch_rows(s, n, nprobe, overlap || staged_overlap);
    const bool residual = s->opt.adc_mode == 1;
    // Sub-batch boundaries.  Equal cuts, except with the overlapped staged transport.  There the transfer costs the scan
    // nothing and is the longer of the two (3.84 GB per 10,000-query batch at the host's ~30 GB/s of random row reads, against
    // ~60 ms of scanning), so it should start as early as possible: the first sub-batch is the small one (10/30/30/30 %).
    std::vector<int> cuts;
    const int plan = s->opt.even_cuts;
    if (staged_overlap && (!residual || residual_table_free(s, stage1_k)) && sb * 4 >= n && n >= 4096 && plan != 1) {
        if (plan == 2) cuts = {0, (int)(0.32 * n), (int)(0.64 * n), (int)(0.90 * n), n};  // short last sub-batch (scan-bound hosts)
        else cuts = {0, (int)(0.10 * n), (int)(0.40 * n), (int)(0.70 * n), n};
    } else {
        for (int p0 = 0; p0 < n; p0 += sb) cuts.push_back(p0);
        cuts.push_back(n);
    }
    int sb_max = 0;
    for (size_t ci = 0; ci + 1 < cuts.size(); ++ci) sb_max = std::max(sb_max, cuts[ci + 1] - cuts[ci]);
    // The sub-batch size depends on this batch's own n (a short tail batch may run in one piece where the full batch ran
    // in four), so the tables and the scan workspace are sized here, for the largest sub-batch of THIS batch.
    const bool table_free = residual_table_free(s, stage1_k);
    if (!table_free) PSB_TRY(s->lut.reserve(sizeof(float) * table_count(s, sb_max, nprobe) * s->m * s->k));
    PSB_TRY(ensure_scan_ws(s, sb_max, nprobe, stage1_k));
    if ((overlap || staged_overlap) && !s->aux_stream) {
        int lo = 0, hi = 0;  // lowest priority: the scan's CTAs get the SMs first, the transfer fills the gaps
        PSB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        PSB_CUDA(cudaStreamCreateWithPriority(&s->aux_stream, cudaStreamNonBlocking, lo));
    }
    cudaStream_t sx = (overlap || staged_overlap) ? s->aux_stream : st;
    struct EventList {  // destroyed on every way out of this function (an event may be destroyed once the waits on it are queued)
        std::vector<cudaEvent_t> v;
        ~EventList() { for (auto e : v) cudaEventDestroy(e); }
        void push_back(cudaEvent_t e) { v.push_back(e); }
    } deps;
    EventTimer tm_s, tm_x;
    if (overlap || staged_overlap) {  // the second stream starts after everything already queued on the main stream
        cudaEvent_t e0;
        PSB_CUDA(cudaEventCreateWithFlags(&e0, cudaEventDisableTiming));
        deps.push_back(e0);
        PSB_CUDA(cudaEventRecord(e0, st));
        PSB_CUDA(cudaStreamWaitEvent(sx, e0, 0));
    }
    psb_status rc = PSB_OK;
    struct Job { int p0, m; cudaEvent_t ready; int mz; cudaEvent_t gathered; };
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Job> jobs;
    bool done = false;
    psb_status worker_rc = PSB_OK;
    std::string worker_msg;
    std::thread worker;
    const bool hybrid = staged_overlap && s->opt.exact_mode == PSB_EXACT_HOST_HYBRID && s->exact_dev != nullptr;
    const int zc_pct = s->opt.zero_copy_pct > 0 ? s->opt.zero_copy_pct : 45;
    if (hybrid) PSB_TRY(ensure_zc_stream(s));
    if (staged_overlap) {
        const size_t cand_count = (size_t)n * stage1_k;
        if (s->h_cand_pinned_count < cand_count) {
            if (s->h_cand_pinned) cudaFreeHost(s->h_cand_pinned);
            s->h_cand_pinned = nullptr; s->h_cand_pinned_count = 0;
            PSB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&s->h_cand_pinned), sizeof(int) * cand_count, cudaHostAllocDefault));
            s->h_cand_pinned_count = cand_count;
        }
        // Hybrid transport: every sub-batch has a staging region of its own (the whole batch: nq * stage1_k rows of device
        // memory), so that the gather kernel of a sub-batch depends on nothing but that sub-batch's scan.
        PSB_TRY(s->stage.reserve((size_t)(hybrid ? n : sb_max) * stage1_k * s->dim * s->exact_elem));
        PSB_TRY(s->score.reserve(sizeof(float) * (size_t)sb_max * stage1_k));
        worker = std::thread([&]() {
            cudaSetDevice(s->device);
            auto process = [&](const Job& j) -> psb_status {
                PSB_RANGE("pq_rerank");
                PSB_CUDA(cudaEventSynchronize(j.ready));
                const int* cand_d = s->cand_rows.as<int>() + (size_t)j.p0 * stage1_k;
                const int* cnt_d = s->cand_count.as<int>() + j.p0;
                if (times) PSB_TRY(tm_x.mark(sx));
                // Hybrid transport: the rows of the last j.mz queries come through the gather kernel, which the main thread queued
                // right behind this sub-batch's scan (j.gathered marks its end); the host threads and the copy engine bring the
                // others; the scoring waits for both.
                const int mh = j.m - j.mz;
                unsigned char* region = static_cast<unsigned char*>(s->stage.p) +
                                        (hybrid ? (size_t)j.p0 * stage1_k * s->dim * s->exact_elem : 0);
                if (mh > 0) PSB_TRY(staged_gather_host(s, s->h_cand_pinned + (size_t)j.p0 * stage1_k, mh, stage1_k, stage1_k, region, sx));
                if (j.mz > 0) PSB_CUDA(cudaStreamWaitEvent(sx, j.gathered, 0));
                const unsigned char* qe = static_cast<const unsigned char*>(dq_exact) + (size_t)j.p0 * s->dim * s->exact_elem;
                PSB_TRY(launch_rerank_score(region, s->row_map(), s->dim, s->exact_elem, qe, cand_d, j.m, stage1_k, stage1_k,
                                            cnt_d, s->score.as<float>(), sx));
                PSB_TRY(launch_topk_select(s->score.as<float>(), cand_d, j.m, stage1_k, stage1_k, cnt_d, topk,
                                           s->out_rows.as<int>() + (size_t)j.p0 * topk, d_dist + (size_t)j.p0 * topk, sx));
                if (times) PSB_TRY(tm_x.mark(sx));
                PSB_TRY(launch_map_ids(s->out_rows.as<int>() + (size_t)j.p0 * topk, (long long)j.m * topk,
                                       s->reordered.as<long long>(), s->row_map(), d_ids + (size_t)j.p0 * topk, sx));
                if (times) PSB_TRY(tm_x.mark(sx));
                return PSB_OK;
            };
            for (;;) {
                Job j;
                {
                    std::unique_lock<std::mutex> lk(mu);
                    cv.wait(lk, [&] { return !jobs.empty() || done; });
                    if (jobs.empty()) return;
                    j = jobs.front();
                    jobs.pop_front();
                }
                if (worker_rc != PSB_OK) continue;  // drain
                const psb_status r = process(j);
                if (r != PSB_OK) { worker_rc = r; worker_msg = psb_last_error(); }
            }
        });
    }
    auto finish_worker = [&]() {
        if (!worker.joinable()) return;
        { std::lock_guard<std::mutex> lk(mu); done = true; }
        cv.notify_all();
        worker.join();
    };
    // Coarse stage for the whole batch first: one large GEMM is more efficient than four small ones, and the tensor-core
    // kernel (a full SM's shared and tensor memory per CTA) then never has to share SMs with the transfer stream.
    if (times) rc = tm_s.mark(st);
    if (rc == PSB_OK) { PSB_RANGE("coarse_search"); rc = coarse_exact(s, dq, n, nprobe, d_probes, nullptr); }
    // OPQ index: the PQ side works on the rotated queries (counted with the coarse stage's time)
    const float* dq_pq = dq;
    if (rc == PSB_OK && s->opq.p) {
        rc = s->q_rot.reserve(sizeof(float) * (size_t)n * s->dim);
        if (rc == PSB_OK) rc = launch_rotate_rows(dq, s->opq.as<float>(), n, s->dim, s->q_rot.as<float>(), st);
        dq_pq = s->q_rot.as<float>();
    }
    if (rc == PSB_OK && times) rc = tm_s.mark(st);
    for (size_t ci = 0; ci + 1 < cuts.size() && rc == PSB_OK; ++ci) {
        const int p0 = cuts[ci];
        const int m = cuts[ci + 1] - p0;
        const float* q = dq_pq + (size_t)p0 * s->dim;
        int* probes = d_probes + (size_t)p0 * nprobe;
        int* rows_out = rerank ? s->cand_rows.as<int>() + (size_t)p0 * stage1_k : s->out_rows.as<int>() + (size_t)p0 * topk;
        float* dist_out = rerank ? s->cand_dist.as<float>() + (size_t)p0 * stage1_k : d_dist + (size_t)p0 * topk;
        int* cnt_out = s->cand_count.as<int>() + p0;
        if (times) rc = tm_s.mark(st);
        ScanWorkspace sws;
        if (rc == PSB_OK) rc = s->timed_scan_ws(&sws);
        if (rc == PSB_OK && !table_free) {
            PSB_RANGE("pq_lut_build");
            if (residual && residual_tables_fused(sws, s->m, s->k)) {  // fp32 and fp16 tables in one kernel
                rc = launch_build_tables_residual(q, m, s->dim, probes, nprobe, s->centroids.as<float>(), s->nlist,
                                                  s->codebook.as<float>(), s->m, s->k, s->cb_maxnorm.as<float>(), s->lut.as<float>(),
                                                  sws, st);
                sws.half_tables_ready = true;
            } else if (residual) {
                rc = launch_build_lut_residual(q, m, s->dim, probes, nprobe, s->centroids.as<float>(), s->nlist,
                                               s->codebook.as<float>(), s->m, s->k, s->lut.as<float>(), st);
            } else {
                rc = launch_build_lut(q, m, s->dim, s->codebook.as<float>(), s->m, s->k, s->lut.as<float>(), st);
            }
        }
        if (rc == PSB_OK && times) rc = tm_s.mark(st);
        if (rc == PSB_OK) {
            PSB_RANGE("pq_adc_scan");
            rc = launch_scan(s->scan_index(), sws, table_free ? nullptr : s->lut.as<float>(), m, probes, nprobe, stage1_k,
                             rows_out, dist_out, cnt_out, s->sm_count, st, q);
        }
        if (rc == PSB_OK && times) rc = tm_s.mark(st);
        if (rc != PSB_OK) break;
        if (staged_overlap) {  // hand the sub-batch to the worker: candidates to the host, an event marks them ready
            cudaEvent_t e;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { rc = fail(PSB_CUDA_ERROR, "event creation failed"); break; }
            deps.push_back(e);
            const int mz = hybrid ? (int)((long long)m * zc_pct / 100) : 0;
            cudaEvent_t gathered = nullptr;
            if (mz > 0) {   // the kernel's share of the transfer, queued now: it starts the moment this sub-batch's scan stage ends
                cudaEvent_t scanned;
                if (cudaEventCreateWithFlags(&scanned, cudaEventDisableTiming) != cudaSuccess ||
                    cudaEventCreateWithFlags(&gathered, cudaEventDisableTiming) != cudaSuccess) { rc = fail(PSB_CUDA_ERROR, "event creation failed"); break; }
                deps.push_back(scanned);
                deps.push_back(gathered);
                cudaEventRecord(scanned, st);
                cudaStreamWaitEvent(s->zc_stream, scanned, 0);
                const int mh = m - mz;
                // on the SMs the scan's grid leaves free (reserve_sms), unless the caller asked for lean CTAs on all SMs
                rc = launch_gather_rows(s->exact_dev, s->row_map(), s->dim, s->exact_elem, rows_out + (size_t)mh * stage1_k, mz, stage1_k, stage1_k,
                                        cnt_out + mh,
                                        static_cast<unsigned char*>(s->stage.p) + (size_t)(p0 + mh) * stage1_k * s->dim * s->exact_elem,
                                        s->zc_stream, s->sm_count, s->opt.gather_ctas > 0 ? s->opt.gather_ctas : 2 * s->sm_count,
                                        s->opt.gather_ctas > 0 ? 0 : s->opt.reserve_sms);
                if (rc != PSB_OK) break;
                cudaEventRecord(gathered, s->zc_stream);
            }
            cudaMemcpyAsync(s->h_cand_pinned + (size_t)p0 * stage1_k, rows_out, sizeof(int) * (size_t)m * stage1_k, cudaMemcpyDeviceToHost, st);
            cudaEventRecord(e, st);
            { std::lock_guard<std::mutex> lk(mu); jobs.push_back(Job{p0, m, e, mz, gathered}); }
            cv.notify_all();
            continue;
        }
        if (overlap) {
            cudaEvent_t e;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { rc = fail(PSB_CUDA_ERROR, "event creation failed"); break; }
            deps.push_back(e);
            cudaEventRecord(e, st);
            cudaStreamWaitEvent(sx, e, 0);
        }
        // second half of the sub-batch (on the second stream when overlapping)
        cudaStream_t keep = s->stream;
        s->stream = sx;  // rerank_impl and the launchers below run on s->stream
        if (times) rc = tm_x.mark(sx);
        if (rc == PSB_OK && rerank) {
            PSB_RANGE("pq_rerank");
            const unsigned char* qe = static_cast<const unsigned char*>(dq_exact) + (size_t)p0 * s->dim * s->exact_elem;
            rc = rerank_impl(s, qe, m, rows_out, stage1_k, stage1_k, cnt_out, topk, s->out_rows.as<int>() + (size_t)p0 * topk,
                             d_dist + (size_t)p0 * topk);
        }
        if (rc == PSB_OK && times) rc = tm_x.mark(sx);
        if (rc == PSB_OK) {
            PSB_RANGE("pq_map_ids");
            rc = launch_map_ids(s->out_rows.as<int>() + (size_t)p0 * topk, (long long)m * topk, s->reordered.as<long long>(),
                                s->row_map(), d_ids + (size_t)p0 * topk, sx);
        }
        if (rc == PSB_OK && times) rc = tm_x.mark(sx);
        s->stream = keep;
    }
    finish_worker();
    if (worker_rc != PSB_OK && rc == PSB_OK) rc = fail(worker_rc, "rerank worker: " + worker_msg);
    if (overlap || staged_overlap) {  // the main stream continues only after the second stream has finished this batch
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess) {
            deps.push_back(e);
            cudaEventRecord(e, sx);
            cudaStreamWaitEvent(st, e, 0);
        } else if (rc == PSB_OK) rc = fail(PSB_CUDA_ERROR, "event creation failed");
    }
    if (times && rc == PSB_OK) {
        if (cudaStreamSynchronize(st) != cudaSuccess) rc = fail(PSB_CUDA_ERROR, "stream synchronisation failed");
        if (tm_s.ev.size() >= 2) times->coarse += tm_s.ms(0, 1);
        for (size_t i = 2; i + 2 < tm_s.ev.size() + 0 && rc == PSB_OK; i += 3) {
            times->lut += tm_s.ms(i, i + 1); times->scan += tm_s.ms(i + 1, i + 2);
        }
        for (size_t i = 0; i + 2 < tm_x.ev.size() + 0 && rc == PSB_OK; i += 3) {
            times->rerank += tm_x.ms(i, i + 1); times->map += tm_x.ms(i + 1, i + 2);
        }
    }
    return rc;
}

}  // namespace

psb_status psb_session_search_device(psb_session* s, const float* d_queries, const uint8_t* d_queries_u8, int nq,
                                     const psb_search_params* params, int64_t* d_indices, float* d_distances,
                                     int* d_coarse_ids) {
    if (!s || !params || !d_queries || !d_indices || !d_distances) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nq < 0 || nq > s->opt.max_batch) return fail(PSB_INVALID_ARGUMENT, "nq must be in 0..max_batch");
    if (params->nprobe <= 0 || params->nprobe > s->nlist || params->topk <= 0) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist and topk positive");
    if (params->nprobe > kMaxProbe || params->topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 or topk above 2048");
    if (params->distance != 0) return fail(PSB_UNSUPPORTED_SHAPE, "only squared L2 is supported on this path");
    if (nq == 0) return PSB_OK;
    PSB_CUDA(cudaSetDevice(s->device));
    const int topk = params->topk;
    const int stage1_k = stage1_width(s, topk);
    const bool rerank = rerank_enabled(s, topk);
    if (stage1_k > kMaxStage1) return fail(PSB_UNSUPPORTED_SHAPE, "candidate width above 2048 is not supported");
    if (rerank && s->exact_elem == 1 && !d_queries_u8) return fail(PSB_INVALID_ARGUMENT, "u8 rerank needs u8 queries");
    PSB_TRY(ensure_pipeline_ws(s, nq, params->nprobe, topk, stage1_k));
    int* probes = d_coarse_ids ? d_coarse_ids : s->probes.as<int>();
    const void* qe = s->exact_elem == 1 ? static_cast<const void*>(d_queries_u8) : static_cast<const void*>(d_queries);
    return search_device(s, d_queries, qe, nq, params->nprobe, topk, stage1_k, rerank, reinterpret_cast<long long*>(d_indices),
                         d_distances, probes, nullptr);
}

psb_status psb_session_search(psb_session* s, const psb_query_batch_view* queries, const psb_search_params* params,
                              const psb_search_output_view* output, psb_stats* stats) {
    PSB_RANGE("ivfpq_search");
    if (!s) return fail(PSB_INVALID_ARGUMENT, "session is null");
    PSB_TRY(validate_params(s, queries, params, output));
    PSB_CUDA(cudaSetDevice(s->device));
    if (stats) std::memset(stats, 0, sizeof(*stats));
    const int total = queries->count;
    if (total == 0) return PSB_OK;
    const int nprobe = params->nprobe, topk = params->topk;
    const int batch = std::min(std::min(params->batch_size, s->opt.max_batch), total);
    const int stage1_k = stage1_width(s, topk);
    const bool rerank = rerank_enabled(s, topk);
    if (stage1_k > kMaxStage1) return fail(PSB_UNSUPPORTED_SHAPE, "candidate width above 2048 is not supported");
    PSB_TRY(ensure_pipeline_ws(s, batch, nprobe, topk, stage1_k));
    if (rerank && s->exact_elem == 1) PSB_TRY(s->q_u8.reserve((size_t)batch * s->dim));
    cudaStream_t st = s->stream;
    const long long launches0 = launches_total();
    unsigned long long c0[4] = {0, 0, 0, 0};
    if (stats) {
        PSB_CUDA(cudaMemcpyAsync(c0, s->scalars.p, sizeof(c0), cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaStreamSynchronize(st));
    }
    s->collect_scan_events();
    const double scan_ms0 = s->scan_ms_total;
    const long long scan_n0 = s->scan_launches_total;
    StageTimes times;
    double t_h2d = 0, t_d2h = 0, t_total = 0;
    long long h2d = 0, d2h = 0;
    int nb = 0;
    for (int q0 = 0; q0 < total; q0 += batch, ++nb) {
        const int n = std::min(batch, total - q0);
        EventTimer tm;
        if (stats) PSB_TRY(tm.mark(st));
        PSB_CUDA(cudaMemcpyAsync(s->q.p, queries->fp32 + (size_t)q0 * s->dim, sizeof(float) * (size_t)n * s->dim, cudaMemcpyHostToDevice, st));
        h2d += (long long)sizeof(float) * n * s->dim;
        if (rerank && s->exact_elem == 1) {
            PSB_CUDA(cudaMemcpyAsync(s->q_u8.p, queries->u8 + (size_t)q0 * s->dim, (size_t)n * s->dim, cudaMemcpyHostToDevice, st));
            h2d += (long long)n * s->dim;
        }
        if (stats) PSB_TRY(tm.mark(st));
        const void* qe = s->exact_elem == 1 ? s->q_u8.p : s->q.p;
        PSB_TRY(search_device(s, s->q.as<float>(), qe, n, nprobe, topk, stage1_k, rerank, s->out_ids.as<long long>(),
                              s->out_dist.as<float>(), s->probes.as<int>(), stats ? &times : nullptr));
        if (stats) PSB_TRY(tm.mark(st));
        PSB_CUDA(cudaMemcpyAsync(output->indices + (size_t)q0 * topk, s->out_ids.p, sizeof(long long) * (size_t)n * topk, cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaMemcpyAsync(output->distances + (size_t)q0 * topk, s->out_dist.p, sizeof(float) * (size_t)n * topk, cudaMemcpyDeviceToHost, st));
        d2h += (long long)(sizeof(long long) + sizeof(float)) * n * topk;
        if (output->coarse_ids) {
            PSB_CUDA(cudaMemcpyAsync(output->coarse_ids + (size_t)q0 * nprobe, s->probes.p, sizeof(int) * (size_t)n * nprobe, cudaMemcpyDeviceToHost, st));
            d2h += (long long)sizeof(int) * n * nprobe;
        }
        if (stats) PSB_TRY(tm.mark(st));
        PSB_CUDA(cudaStreamSynchronize(st));
        if (stats) { t_h2d += tm.ms(0, 1); t_d2h += tm.ms(2, 3); t_total += tm.ms(0, 3); }
    }
    PSB_TRY(s->tc_work.check_status());
    PSB_TRY(s->check_scan_status());
    if (stats) {
        unsigned long long c1[4];
        PSB_CUDA(cudaMemcpyAsync(c1, s->scalars.p, sizeof(c1), cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaStreamSynchronize(st));
        stats->h2d_ms = t_h2d; stats->coarse_search_ms = times.coarse; stats->pq_lut_build_ms = times.lut;
        stats->pq_adc_scan_ms = times.scan; stats->pq_rerank_ms = times.rerank; stats->pq_map_ids_ms = times.map; stats->d2h_ms = t_d2h;
        stats->total_ms = t_total;  // stage times can overlap: their sum may exceed the total
        stats->pq_scanned_codes = (long long)(c1[0] - c0[0]);
        stats->pq_adc_lookups = stats->pq_scanned_codes * s->m;
        stats->threshold_candidates = (long long)(c1[1] - c0[1]);
        stats->fallback_queries = (long long)(c1[2] - c0[2]);
        stats->prefilter_survivors = (long long)(c1[3] - c0[3]);
        stats->h2d_bytes = h2d; stats->d2h_bytes = d2h;
        stats->kernel_launches = launches_total() - launches0;
        s->collect_scan_events();
        stats->scan_kernel_ms = s->scan_ms_total - scan_ms0;
        stats->scan_kernel_launches = s->scan_launches_total - scan_n0;
        stats->batches = nb;
    }
    return PSB_OK;
}

// ---- IVF-Flat ----------------------------------------------------------------------------------------------------

psb_status psb_flat_session_create(const psb_flat_index_view* index, const psb_options* options, psb_flat_session** out) {
    if (!out) return fail(PSB_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!index) return fail(PSB_INVALID_ARGUMENT, "index view is null");
    {   // the list layout rules of the PQ index (src/search/ivf_common/ivf_list_layout.h:19-45)
        psb_index_view probe{};
        probe.coarse = index->coarse; probe.lists = index->lists;
        static const float one_codeword = 0.0f;
        static const uint8_t no_codes = 0;
        probe.pq.codes = &no_codes; probe.pq.codebook = &one_codeword; probe.pq.subvectors = 1; probe.pq.codebook_size = 1;
        if (index->coarse.dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid IVF coarse index view");
        PSB_TRY(validate_index(&probe));
    }
    if (!index->rowmajor_fp32 && index->lists.n_vectors > 0) return fail(PSB_INVALID_ARGUMENT, "IVF-Flat rows are null");
    psb_options opt{};
    if (options) opt = *options;
    if (opt.max_batch <= 0) opt.max_batch = 10000;
    cudaDeviceProp prop;
    PSB_TRY(check_device(opt.device, &prop));
    std::unique_ptr<psb_session> s(new (std::nothrow) psb_session());
    if (!s) return fail(PSB_OUT_OF_MEMORY, "host allocation failed");
    s->flat = true;
    s->device = opt.device; s->sm_count = prop.multiProcessorCount; s->opt = opt;
    s->nlist = index->lists.nlist; s->dim = index->coarse.dim; s->n_vectors = index->lists.n_vectors;
    s->list_begin = 0; s->list_end = s->nlist; s->row_base = 0; s->shard_rows = s->n_vectors;
    if (opt.stream) s->stream = static_cast<cudaStream_t>(opt.stream);
    else { PSB_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking)); s->own_stream = true; }
    cudaStream_t st = s->stream;
    const size_t nl = (size_t)s->nlist, n = (size_t)std::max<long long>(1, s->n_vectors);
    PSB_TRY(s->centroids.reserve(sizeof(float) * nl * s->dim));
    PSB_CUDA(cudaMemcpyAsync(s->centroids.p, index->coarse.centroids, sizeof(float) * nl * s->dim, cudaMemcpyHostToDevice, st));
    if (opt.coarse_mode != 1 && s->nlist >= 1024 && coarse_tc_padded_dim(s->dim) <= 128)
        PSB_TRY(s->tc_index.prepare(index->coarse.centroids, s->centroids.as<float>(), s->nlist, s->dim, st));
    PSB_TRY(s->offsets.reserve(sizeof(long long) * (nl + 1)));
    PSB_CUDA(cudaMemcpyAsync(s->offsets.p, index->lists.offsets, sizeof(long long) * (nl + 1), cudaMemcpyHostToDevice, st));
    PSB_TRY(s->reordered.reserve(sizeof(long long) * n));
    PSB_TRY(s->flat_rows.reserve(sizeof(float) * n * s->dim));
    if (s->n_vectors > 0) {
        PSB_CUDA(cudaMemcpyAsync(s->reordered.p, index->lists.reordered_ids, sizeof(long long) * n, cudaMemcpyHostToDevice, st));
        PSB_CUDA(cudaMemcpyAsync(s->flat_rows.p, index->rowmajor_fp32, sizeof(float) * n * s->dim, cudaMemcpyHostToDevice, st));
    }
    PSB_TRY(s->scalars.reserve(sizeof(unsigned long long) * 16));
    PSB_CUDA(cudaMemsetAsync(s->scalars.p, 0, sizeof(unsigned long long) * 16, st));
    PSB_CUDA(cudaStreamSynchronize(st));
    *out = s.release();
    return PSB_OK;
}

psb_status psb_flat_session_destroy(psb_flat_session* s) {
    delete s;
    return PSB_OK;
}

namespace {
psb_status flat_search_device(psb_session* s, const float* dq, int n, int nprobe, int topk, long long* d_ids, float* d_dist) {
    PSB_TRY(s->probes.reserve(sizeof(int) * (size_t)n * nprobe));
    PSB_TRY(s->out_rows.reserve(sizeof(int) * (size_t)n * topk));
    PSB_TRY(coarse_exact(s, dq, n, nprobe, s->probes.as<int>(), nullptr));
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    if (s->opt.time_kernels) {  // bracket the fine-scan kernel (read back by psb_session_counters)
        PSB_CUDA(cudaEventCreate(&ev0));
        PSB_CUDA(cudaEventCreate(&ev1));
        s->scan_events.emplace_back(ev0, ev1);
        PSB_CUDA(cudaEventRecord(ev0, s->stream));
    }
    PSB_TRY(launch_flat_scan(dq, n, s->dim, s->probes.as<int>(), nprobe, s->offsets.as<long long>(), s->nlist, s->flat_rows.as<float>(),
                             0, topk, s->out_rows.as<int>(), d_dist, s->scalars.as<unsigned long long>(), s->stream));
    if (ev1) PSB_CUDA(cudaEventRecord(ev1, s->stream));
    return launch_map_ids(s->out_rows.as<int>(), (long long)n * topk, s->reordered.as<long long>(), s->row_map(), d_ids, s->stream);
}
psb_status flat_check(const psb_session* s, const psb_search_params* p) {
    if (!s || !s->flat) return fail(PSB_INVALID_ARGUMENT, "not an IVF-Flat session");
    if (!p) return fail(PSB_INVALID_ARGUMENT, "params are null");
    if (p->nprobe <= 0 || p->nprobe > s->nlist) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist");
    if (p->topk <= 0) return fail(PSB_INVALID_ARGUMENT, "topk must be positive");
    if (p->batch_size <= 0) return fail(PSB_INVALID_ARGUMENT, "batch_size must be positive");
    if (p->distance != 0) return fail(PSB_UNSUPPORTED_SHAPE, "only squared L2 is supported on this path");
    if (p->nprobe > kMaxProbe || p->topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 or topk above 2048");
    return PSB_OK;
}
}  // namespace

psb_status psb_flat_session_search_device(psb_flat_session* s, const float* d_queries, int nq, const psb_search_params* params,
                                          int64_t* d_indices, float* d_distances) {
    PSB_TRY(flat_check(s, params));
    if (!d_queries || !d_indices || !d_distances) return fail(PSB_INVALID_ARGUMENT, "null argument");
    if (nq < 0 || nq > s->opt.max_batch) return fail(PSB_INVALID_ARGUMENT, "nq must be in 0..max_batch");
    if (nq == 0) return PSB_OK;
    PSB_CUDA(cudaSetDevice(s->device));
    return flat_search_device(s, d_queries, nq, params->nprobe, params->topk, reinterpret_cast<long long*>(d_indices), d_distances);
}

psb_status psb_flat_session_search(psb_flat_session* s, const psb_query_batch_view* queries, const psb_search_params* params,
                                   const psb_search_output_view* output, psb_stats* stats) {
    PSB_RANGE("ivfflat_search");
    PSB_TRY(flat_check(s, params));
    if (!queries || !output) return fail(PSB_INVALID_ARGUMENT, "null query or output view");
    if (queries->count < 0 || queries->dim != s->dim) return fail(PSB_INVALID_ARGUMENT, "query dim does not match the index");
    if (queries->count > 0 && (!queries->fp32 || !output->indices || !output->distances)) return fail(PSB_INVALID_ARGUMENT, "null query or output buffers");
    PSB_CUDA(cudaSetDevice(s->device));
    if (stats) std::memset(stats, 0, sizeof(*stats));
    const int total = queries->count, nprobe = params->nprobe, topk = params->topk;
    if (total == 0) return PSB_OK;
    const int batch = std::min(std::min(params->batch_size, s->opt.max_batch), total);
    cudaStream_t st = s->stream;
    PSB_TRY(s->q.reserve(sizeof(float) * (size_t)batch * s->dim));
    PSB_TRY(s->out_ids.reserve(sizeof(long long) * (size_t)batch * topk));
    PSB_TRY(s->out_dist.reserve(sizeof(float) * (size_t)batch * topk));
    const long long launches0 = launches_total();
    unsigned long long c0 = 0, c1 = 0;
    PSB_CUDA(cudaMemcpyAsync(&c0, s->scalars.p, sizeof(c0), cudaMemcpyDeviceToHost, st));
    EventTimer tm;
    PSB_TRY(tm.mark(st));
    int nb = 0;
    for (int q0 = 0; q0 < total; q0 += batch, ++nb) {
        const int n = std::min(batch, total - q0);
        PSB_CUDA(cudaMemcpyAsync(s->q.p, queries->fp32 + (size_t)q0 * s->dim, sizeof(float) * (size_t)n * s->dim, cudaMemcpyHostToDevice, st));
        PSB_TRY(flat_search_device(s, s->q.as<float>(), n, nprobe, topk, s->out_ids.as<long long>(), s->out_dist.as<float>()));
        PSB_CUDA(cudaMemcpyAsync(output->indices + (size_t)q0 * topk, s->out_ids.p, sizeof(long long) * (size_t)n * topk, cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaMemcpyAsync(output->distances + (size_t)q0 * topk, s->out_dist.p, sizeof(float) * (size_t)n * topk, cudaMemcpyDeviceToHost, st));
        if (output->coarse_ids)
            PSB_CUDA(cudaMemcpyAsync(output->coarse_ids + (size_t)q0 * nprobe, s->probes.p, sizeof(int) * (size_t)n * nprobe, cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaStreamSynchronize(st));  // the batch buffers are reused
    }
    PSB_TRY(tm.mark(st));
    PSB_CUDA(cudaMemcpyAsync(&c1, s->scalars.p, sizeof(c1), cudaMemcpyDeviceToHost, st));
    PSB_CUDA(cudaStreamSynchronize(st));
    PSB_TRY(s->tc_work.check_status());
    if (stats) {
        stats->total_ms = tm.ms(0, 1);
        stats->pq_scanned_codes = (long long)(c1 - c0);  // rows scanned
        stats->h2d_bytes = (long long)sizeof(float) * total * s->dim;
        stats->d2h_bytes = (long long)(sizeof(long long) + sizeof(float)) * total * topk;
        stats->kernel_launches = launches_total() - launches0;
        stats->batches = nb;
    }
    return PSB_OK;
}

// ---- one-shot operators on host arrays ------------------------------------------------------------------

psb_status psb_rerank_host(const psb_host_storage_view* storage, const uint8_t* h_queries_u8,
                           const float* h_queries_fp32, const int* h_candidates, int batch_n,
                           int candidate_count, int candidate_stride, int topk, int* h_output_ids,
                           float* h_output_distances, const int* h_candidate_counts, int device) {
    if (!storage || !h_candidates || !h_output_ids || !h_output_distances || batch_n <= 0 || candidate_count <= 0 ||
        candidate_stride < candidate_count || topk <= 0 || storage->count <= 0 || storage->dim <= 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid host IVF rerank request");
    const bool use_float = storage->fp32 != nullptr;
    if ((use_float && !h_queries_fp32) || (!use_float && (!storage->u8 || !h_queries_u8)))
        return fail(PSB_INVALID_ARGUMENT, "host IVF rerank dtype does not match storage");
    if (storage->source_rows) return fail(PSB_UNSUPPORTED_SHAPE, "exact storage with a row permutation is not supported");
    if (h_candidate_counts)
        for (int q = 0; q < batch_n; ++q)
            if (h_candidate_counts[q] < 0 || h_candidate_counts[q] > candidate_count)
                return fail(PSB_INVALID_ARGUMENT, "host rerank candidate count exceeds row width");
    if (candidate_count > kMaxRerankWidth || topk > kMaxTopk) return fail(PSB_UNSUPPORTED_SHAPE, "rerank width above 4096 or topk above 2048");
    cudaDeviceProp prop;
    PSB_TRY(check_device(device, &prop));
    const int elem = use_float ? 4 : 1;
    const int dim = storage->dim;
    const size_t base_bytes = (size_t)storage->count * dim * elem;
    DevBuf base, q, cand, counts, stage, out_rows, out_dist;
    PSB_TRY(base.reserve(base_bytes)); PSB_TRY(q.reserve((size_t)batch_n * dim * elem));
    PSB_TRY(cand.reserve(sizeof(int) * (size_t)batch_n * candidate_stride));
    PSB_TRY(stage.reserve((size_t)batch_n * candidate_count * dim * elem));
    PSB_TRY(out_rows.reserve(sizeof(int) * (size_t)batch_n * topk)); PSB_TRY(out_dist.reserve(sizeof(float) * (size_t)batch_n * topk));
    cudaStream_t st = nullptr;
    PSB_CUDA(cudaMemcpy(base.p, use_float ? (const void*)storage->fp32 : (const void*)storage->u8, base_bytes, cudaMemcpyHostToDevice));
    PSB_CUDA(cudaMemcpy(q.p, use_float ? (const void*)h_queries_fp32 : (const void*)h_queries_u8, (size_t)batch_n * dim * elem, cudaMemcpyHostToDevice));
    PSB_CUDA(cudaMemcpy(cand.p, h_candidates, sizeof(int) * (size_t)batch_n * candidate_stride, cudaMemcpyHostToDevice));
    const int* d_counts = nullptr;
    if (h_candidate_counts) {
        PSB_TRY(counts.reserve(sizeof(int) * (size_t)batch_n));
        PSB_CUDA(cudaMemcpy(counts.p, h_candidate_counts, sizeof(int) * (size_t)batch_n, cudaMemcpyHostToDevice));
        d_counts = counts.as<int>();
    }
    RowMap mp;
    mp.count = storage->count;
    DevBuf score;
    PSB_TRY(score.reserve(sizeof(float) * (size_t)batch_n * candidate_count));
    PSB_TRY(launch_gather_rows(base.p, mp, dim, elem, cand.as<int>(), batch_n, candidate_count, candidate_stride,
                               d_counts, stage.p, st, prop.multiProcessorCount));
    PSB_TRY(launch_rerank_score(stage.p, mp, dim, elem, q.p, cand.as<int>(), batch_n, candidate_count, candidate_stride,
                                d_counts, score.as<float>(), st));
    PSB_TRY(launch_topk_select(score.as<float>(), cand.as<int>(), batch_n, candidate_count, candidate_stride, d_counts,
                               topk, out_rows.as<int>(), out_dist.as<float>(), st));
    PSB_CUDA(cudaMemcpy(h_output_ids, out_rows.p, sizeof(int) * (size_t)batch_n * topk, cudaMemcpyDeviceToHost));
    PSB_CUDA(cudaMemcpy(h_output_distances, out_dist.p, sizeof(float) * (size_t)batch_n * topk, cudaMemcpyDeviceToHost));
    return PSB_OK;
}

psb_status psb_coarse_host(const float* h_queries, int nq, const float* h_centroids, int nlist, int dim,
                           int nprobe, int coarse_mode, int64_t* h_ids, float* h_dist, int device) {
    if (!h_queries || !h_centroids || !h_ids || nq < 0 || nlist <= 0 || dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid coarse request");
    if (nprobe <= 0 || nprobe > nlist) return fail(PSB_INVALID_ARGUMENT, "nprobe must be in 1..nlist");
    if (nprobe > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "nprobe above 4096 is not supported");
    PSB_TRY(check_device(device));
    if (nq == 0) return PSB_OK;
    DevBuf q, c, tile, ids, ids64, dist;
    PSB_TRY(q.reserve(sizeof(float) * (size_t)nq * dim)); PSB_TRY(c.reserve(sizeof(float) * (size_t)nlist * dim));
    PSB_TRY(ids.reserve(sizeof(int) * (size_t)nq * nprobe)); PSB_TRY(ids64.reserve(sizeof(long long) * (size_t)nq * nprobe));
    PSB_TRY(dist.reserve(sizeof(float) * (size_t)nq * nprobe));
    PSB_CUDA(cudaMemcpy(q.p, h_queries, sizeof(float) * (size_t)nq * dim, cudaMemcpyHostToDevice));
    PSB_CUDA(cudaMemcpy(c.p, h_centroids, sizeof(float) * (size_t)nlist * dim, cudaMemcpyHostToDevice));
    const bool tc_ok = coarse_tc_supported(nq, nlist, dim, nprobe);
    if (coarse_mode == 2 && !tc_ok) return fail(PSB_UNSUPPORTED_SHAPE, "tensor-core coarse stage does not support this shape");
    if (coarse_mode != 1 && tc_ok) {
        cudaDeviceProp prop;
        PSB_CUDA(cudaGetDeviceProperties(&prop, device));
        TcIndexBuffers tix;
        TcWorkBuffers twk;
        PSB_TRY(tix.prepare(h_centroids, c.as<float>(), nlist, dim, nullptr));
        PSB_TRY(twk.ensure(nq, nlist, dim, nprobe, nullptr));
        PSB_TRY(launch_coarse_tc(tix.view(c.as<float>(), nlist, dim), twk.view(), q.as<float>(), nq, nprobe, ids.as<int>(),
                                 dist.as<float>(), prop.multiProcessorCount, nullptr));
        PSB_CUDA(cudaDeviceSynchronize());
        PSB_TRY(twk.check_status());
    } else {
        const size_t row_bytes = sizeof(float) * (size_t)nlist;
        int chunk = (int)std::max<size_t>(64, ((size_t)1 << 30) / row_bytes);
        chunk = std::min(chunk, nq);
        PSB_TRY(tile.reserve(row_bytes * (size_t)chunk));
        for (int q0 = 0; q0 < nq; q0 += chunk) {
            const int n = std::min(chunk, nq - q0);
            PSB_TRY(launch_coarse_dist_exact(q.as<float>() + (size_t)q0 * dim, n, c.as<float>(), nlist, dim, tile.as<float>(), nullptr));
            PSB_TRY(launch_select_rows(tile.as<float>(), n, nlist, nprobe, ids.as<int>() + (size_t)q0 * nprobe,
                                       dist.as<float>() + (size_t)q0 * nprobe, nullptr));
        }
    }
    PSB_TRY(launch_widen_ids(ids.as<int>(), (long long)nq * nprobe, ids64.as<long long>(), nullptr));
    PSB_CUDA(cudaMemcpy(h_ids, ids64.p, sizeof(long long) * (size_t)nq * nprobe, cudaMemcpyDeviceToHost));
    if (h_dist) PSB_CUDA(cudaMemcpy(h_dist, dist.p, sizeof(float) * (size_t)nq * nprobe, cudaMemcpyDeviceToHost));
    return PSB_OK;
}

psb_status psb_knn_exact(const float* d_queries, int nq, const float* d_base, int64_t n, int dim, int k,
                         int* d_rows, float* d_dist, int device, void* stream) {
    if (!d_queries || !d_base || !d_rows || !d_dist || nq <= 0 || n <= 0 || dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid knn request");
    if (k <= 0 || k > n) return fail(PSB_INVALID_ARGUMENT, "k must be in 1..n");
    if (k > kMaxProbe) return fail(PSB_UNSUPPORTED_SHAPE, "k above 4096 is not supported");
    if (n > INT_MAX) return fail(PSB_UNSUPPORTED_SHAPE, "more than 2^31-1 base rows");
    PSB_TRY(check_device(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // tiles of base rows, each at most 1 GiB of distances, then a merge of the per-tile winners.  A last tile with fewer
    // than k rows is folded into the tile before it, so every tile selects exactly k rows.
    long long tile = std::max<long long>(std::max<long long>(4096, k), ((long long)1 << 28) / nq);
    tile = std::min<long long>(tile, n);
    std::vector<std::pair<long long, int>> spans;  // (first row, rows)
    for (long long r0 = 0; r0 < n;) {
        long long rows = std::min<long long>(tile, n - r0);
        const long long rest = n - (r0 + rows);
        if (rest > 0 && rest < k) rows += rest;
        spans.emplace_back(r0, (int)rows);
        r0 += rows;
    }
    const int tiles = (int)spans.size();
    if ((long long)tiles * k > 16384) return fail(PSB_UNSUPPORTED_SHAPE, "knn: too many tiles for the merge; pass fewer base rows per call");
    DevBuf dist, trows, tdist;
    PSB_TRY(dist.reserve(sizeof(float) * (size_t)nq * (size_t)(tile + k)));
    PSB_TRY(trows.reserve(sizeof(int) * (size_t)tiles * nq * k));
    PSB_TRY(tdist.reserve(sizeof(float) * (size_t)tiles * nq * k));
    for (int t = 0; t < tiles; ++t) {
        const long long r0 = spans[(size_t)t].first;
        const int rows = spans[(size_t)t].second;  // >= k: k <= n, and no span is shorter than k unless it is the only one
        PSB_TRY(launch_coarse_dist_exact(d_queries, nq, d_base + (size_t)r0 * dim, rows, dim, dist.as<float>(), st));
        PSB_TRY(launch_select_rows(dist.as<float>(), nq, rows, k, trows.as<int>() + (size_t)t * nq * k,
                                   tdist.as<float>() + (size_t)t * nq * k, st));
        PSB_TRY(launch_offset_rows(trows.as<int>() + (size_t)t * nq * k, (long long)nq * k, (int)r0, st));
    }
    PSB_TRY(launch_merge(trows.as<int>(), tdist.as<float>(), tiles, nq, k, d_rows, d_dist, st));
    PSB_CUDA(cudaStreamSynchronize(st));
    return PSB_OK;
}

// ---- training ---------------------------------------------------------------------------------------------

psb_status psb_kmeans_train(const float* d_data, int64_t n, int dim, float* d_centroids, int k, int iters,
                            int* d_assign, double* h_objective, int device, void* stream) {
    if (!d_data || !d_centroids || n <= 0 || dim <= 0 || k <= 0 || iters < 0) return fail(PSB_INVALID_ARGUMENT, "invalid k-means request");
    cudaDeviceProp prop;
    PSB_TRY(check_device(device, &prop));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DevBuf tile, assign, best, sums, counts, obj;
    const size_t row_bytes = sizeof(float) * (size_t)k;
    long long chunk = (long long)std::max<size_t>(64, ((size_t)1 << 30) / row_bytes);
    chunk = std::min<long long>(chunk, n);
    // Assignment = nearest centroid = the coarse stage with nprobe 1.  Large problems take the tensor-core filter with
    // exact refinement (identical assignments and distances: ties go to the lower centroid id on both paths); the bf16
    // centroid operand is rebuilt from the current centroids at the start of every iteration.
    const long long chunk_tc = std::min<long long>(n, 262144);
    const bool tc = coarse_tc_supported((int)chunk_tc, k, dim, 1);
    TcIndexBuffers tci;
    TcWorkBuffers tcw;
    std::vector<float> h_centroids;
    if (tc) { chunk = chunk_tc; h_centroids.resize((size_t)k * dim); }
    else PSB_TRY(tile.reserve(row_bytes * (size_t)chunk));
    PSB_TRY(best.reserve(sizeof(float) * (size_t)n));
    int* d_as = d_assign;
    if (!d_as) { PSB_TRY(assign.reserve(sizeof(int) * (size_t)n)); d_as = assign.as<int>(); }
    PSB_TRY(sums.reserve(sizeof(double) * (size_t)k * dim)); PSB_TRY(counts.reserve(sizeof(int) * (size_t)k));
    PSB_TRY(obj.reserve(sizeof(double) * ((size_t)iters + 1)));
    DevBuf acc_order, acc_offsets, acc_cursor;   // rows grouped by centroid for the accumulation
    PSB_TRY(acc_order.reserve(sizeof(int) * (size_t)n));
    PSB_TRY(acc_offsets.reserve(sizeof(int) * ((size_t)k + 1)));
    PSB_TRY(acc_cursor.reserve(sizeof(int) * (size_t)k));
    KmeansAccumWs acc_ws;
    acc_ws.order = acc_order.as<int>(); acc_ws.offsets = acc_offsets.as<int>(); acc_ws.cursor = acc_cursor.as<int>();
    PSB_CUDA(cudaMemsetAsync(obj.p, 0, sizeof(double) * ((size_t)iters + 1), st));
    for (int it = 0; it <= iters; ++it) {
        if (tc) {
            PSB_CUDA(cudaMemcpyAsync(h_centroids.data(), d_centroids, sizeof(float) * (size_t)k * dim, cudaMemcpyDeviceToHost, st));
            PSB_CUDA(cudaStreamSynchronize(st));
            PSB_TRY(tci.prepare(h_centroids.data(), d_centroids, k, dim, st));
        }
        for (long long r0 = 0; r0 < n; r0 += chunk) {
            const int nn = (int)std::min<long long>(chunk, n - r0);
            if (tc && coarse_tc_supported(nn, k, dim, 1)) {
                PSB_TRY(tcw.ensure(nn, k, dim, 1, st));
                // After the first iteration every row brings a bound along - its distance to the centroid it had, where that
                // centroid is now - and the filter GEMM runs once instead of twice.
                if (it > 0)
                    PSB_TRY(launch_coarse_tc_assign(tci.view(d_centroids, k, dim), tcw.view(), d_data + (size_t)r0 * dim, nn, d_as + r0,
                                                    d_as + r0, best.as<float>() + r0, prop.multiProcessorCount, st));
                else
                    PSB_TRY(launch_coarse_tc(tci.view(d_centroids, k, dim), tcw.view(), d_data + (size_t)r0 * dim, nn, 1,
                                             d_as + r0, best.as<float>() + r0, prop.multiProcessorCount, st));
            } else {
                PSB_TRY(tile.reserve(row_bytes * (size_t)nn));
                PSB_TRY(launch_coarse_dist_exact(d_data + (size_t)r0 * dim, nn, d_centroids, k, dim, tile.as<float>(), st));
                PSB_TRY(launch_select_rows(tile.as<float>(), nn, k, 1, d_as + r0, best.as<float>() + r0, st));
            }
        }
        PSB_CUDA(cudaMemsetAsync(counts.p, 0, sizeof(int) * (size_t)k, st));
        PSB_TRY(launch_kmeans_accumulate(d_data, n, dim, d_as, best.as<float>(), k, sums.as<double>(), counts.as<int>(),
                                         obj.as<double>() + it, acc_ws, st));
        if (it < iters) PSB_TRY(launch_kmeans_update(sums.as<double>(), counts.as<int>(), k, dim, d_centroids, st));
    }
    if (h_objective) PSB_CUDA(cudaMemcpyAsync(h_objective, obj.p, sizeof(double) * ((size_t)iters + 1), cudaMemcpyDeviceToHost, st));
    PSB_CUDA(cudaStreamSynchronize(st));
    if (tc) PSB_TRY(tcw.check_status());
    return PSB_OK;
}

// ---- one Lloyd iteration in three calls (data-parallel training: the caller all-reduces sums and counts in between) ----

psb_status psb_kmeans_assign(const float* d_data, int64_t n, int dim, const float* d_centroids, int k, int* d_assign,
                             float* d_best, int device, void* stream) {
    return psb_kmeans_assign_bounded(d_data, n, dim, d_centroids, k, d_assign, d_best, 0, device, stream);
}

psb_status psb_kmeans_assign_bounded(const float* d_data, int64_t n, int dim, const float* d_centroids, int k, int* d_assign,
                                     float* d_best, int have_previous, int device, void* stream) {
    if (!d_data || !d_centroids || !d_assign || !d_best || n <= 0 || dim <= 0 || k <= 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid k-means assignment request");
    cudaDeviceProp prop;
    PSB_TRY(check_device(device, &prop));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t row_bytes = sizeof(float) * (size_t)k;
    long long chunk = std::min<long long>((long long)std::max<size_t>(64, ((size_t)1 << 30) / row_bytes), n);
    const long long chunk_tc = std::min<long long>(n, 262144);
    const bool tc = coarse_tc_supported((int)chunk_tc, k, dim, 1);
    TcIndexBuffers tci;
    TcWorkBuffers tcw;
    DevBuf tile;
    if (tc) {
        chunk = chunk_tc;
        std::vector<float> h_centroids((size_t)k * dim);
        PSB_CUDA(cudaMemcpyAsync(h_centroids.data(), d_centroids, sizeof(float) * (size_t)k * dim, cudaMemcpyDeviceToHost, st));
        PSB_CUDA(cudaStreamSynchronize(st));
        PSB_TRY(tci.prepare(h_centroids.data(), d_centroids, k, dim, st));
    }
    for (long long r0 = 0; r0 < n; r0 += chunk) {
        const int nn = (int)std::min<long long>(chunk, n - r0);
        if (tc && coarse_tc_supported(nn, k, dim, 1)) {
            PSB_TRY(tcw.ensure(nn, k, dim, 1, st));
            if (have_previous)
                PSB_TRY(launch_coarse_tc_assign(tci.view(d_centroids, k, dim), tcw.view(), d_data + (size_t)r0 * dim, nn, d_assign + r0,
                                                d_assign + r0, d_best + r0, prop.multiProcessorCount, st));
            else
                PSB_TRY(launch_coarse_tc(tci.view(d_centroids, k, dim), tcw.view(), d_data + (size_t)r0 * dim, nn, 1, d_assign + r0,
                                         d_best + r0, prop.multiProcessorCount, st));
        } else {
            PSB_TRY(tile.reserve(row_bytes * (size_t)nn));
            PSB_TRY(launch_coarse_dist_exact(d_data + (size_t)r0 * dim, nn, d_centroids, k, dim, tile.as<float>(), st));
            PSB_TRY(launch_select_rows(tile.as<float>(), nn, k, 1, d_assign + r0, d_best + r0, st));
        }
    }
    PSB_CUDA(cudaStreamSynchronize(st));  // the work buffers above are released on return
    if (tc) PSB_TRY(tcw.check_status());
    return PSB_OK;
}

psb_status psb_kmeans_accumulate(const float* d_data, int64_t n, int dim, const int* d_assign, const float* d_best, int k,
                                 double* d_sums, int* d_counts, double* d_objective, int device, void* stream) {
    if (!d_data || !d_assign || !d_best || !d_sums || !d_counts || !d_objective || n < 0 || dim <= 0 || k <= 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid k-means accumulation request");
    PSB_TRY(check_device(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PSB_CUDA(cudaMemsetAsync(d_counts, 0, sizeof(int) * (size_t)k, st));
    PSB_CUDA(cudaMemsetAsync(d_objective, 0, sizeof(double), st));
    DevBuf order, offsets, cursor;   // rows grouped by centroid: freed after the stream has drained below
    PSB_TRY(order.reserve(sizeof(int) * (size_t)std::max<int64_t>(n, 1)));
    PSB_TRY(offsets.reserve(sizeof(int) * ((size_t)k + 1)));
    PSB_TRY(cursor.reserve(sizeof(int) * (size_t)k));
    KmeansAccumWs ws;
    ws.order = order.as<int>(); ws.offsets = offsets.as<int>(); ws.cursor = cursor.as<int>();
    PSB_TRY(launch_kmeans_accumulate(d_data, n, dim, d_assign, d_best, k, d_sums, d_counts, d_objective, ws, st));
    PSB_CUDA(cudaStreamSynchronize(st));
    return PSB_OK;
}

psb_status psb_kmeans_update(const double* d_sums, const int* d_counts, int k, int dim, float* d_centroids, int device,
                             void* stream) {
    if (!d_sums || !d_counts || !d_centroids || k <= 0 || dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid k-means update request");
    PSB_TRY(check_device(device));
    return launch_kmeans_update(d_sums, d_counts, k, dim, d_centroids, static_cast<cudaStream_t>(stream));
}

psb_status psb_residual_rows(const float* d_data, int64_t n, int dim, const float* d_centroids, const int* d_assign,
                             float* d_out, int device, void* stream) {
    if (!d_data || !d_centroids || !d_assign || !d_out || n < 0 || dim <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid residual request");
    if ((long long)n * dim > 0x7fffffffLL * 256) return fail(PSB_UNSUPPORTED_SHAPE, "too many elements for one call");
    PSB_TRY(check_device(device));
    return launch_residual_rows(d_data, n, dim, d_centroids, d_assign, d_out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

namespace {

// The reference's choice of initial centroids (init_centroids_by_sampling, src/clustering/kmeans/kmeans.cu:716-862), as the
// data rows it picks: std::mt19937(seed); below n * k = 2e7 (policy 0) k-means++ seeding - first row uniform, every further
// row with probability proportional to its squared distance from the nearest row picked so far (fp32 sequential sums,
// fp64 running total) - above it k distinct rows by a partial Fisher-Yates shuffle.  The standard library's engine and
// distributions make the draws the same as the reference's, draw for draw.  row(i) must return row i's `dim` values.
template <typename RowFn>
void kmeans_init_rows(long long n, int dim, int k, int seed, int policy, RowFn row, std::vector<long long>& picked) {
    picked.assign((size_t)k, 0);
    if (n <= 0 || k <= 0) return;
    const int ni = (int)n;
    const int k_eff = std::min<long long>(k, n);
    std::mt19937 rng((unsigned)seed);
    const bool plusplus = policy == 2 || (policy == 0 && (long long)ni * k_eff <= 20000000LL);
    if (!plusplus) {
        std::vector<int> idx((size_t)ni);
        for (int i = 0; i < ni; ++i) idx[(size_t)i] = i;
        for (int i = 0; i < k_eff; ++i) {
            std::uniform_int_distribution<int> dist(i, ni - 1);
            std::swap(idx[(size_t)i], idx[(size_t)dist(rng)]);
        }
        for (int c = 0; c < k; ++c) picked[(size_t)c] = idx[(size_t)(c < k_eff ? c : 0)];
        return;
    }
    auto dist2 = [&](const float* x, const float* c) {
        float acc = 0.0f;
        for (int d = 0; d < dim; ++d) { const float diff = x[d] - c[d]; acc = acc + diff * diff; }
        return acc;
    };
    std::uniform_int_distribution<int> uni(0, ni - 1);
    picked[0] = uni(rng);
    std::vector<float> best((size_t)ni);
    for (int i = 0; i < ni; ++i) best[(size_t)i] = dist2(row(i), row(picked[0]));
    for (int c = 1; c < k_eff; ++c) {
        double total = 0.0;
        for (int i = 0; i < ni; ++i) total += (double)best[(size_t)i];
        int next = -1;
        if (total <= 0.0) {
            next = uni(rng);
        } else {
            std::uniform_real_distribution<double> urd(0.0, total);
            const double r = urd(rng);
            double cum = 0.0;
            for (int i = 0; i < ni; ++i) {
                cum += (double)best[(size_t)i];
                if (cum >= r) { next = i; break; }
            }
            if (next < 0) next = ni - 1;
        }
        picked[(size_t)c] = next;
        const float* cc = row(next);
        for (int i = 0; i < ni; ++i) {
            const float d2 = dist2(row(i), cc);
            if (d2 < best[(size_t)i]) best[(size_t)i] = d2;
        }
    }
    for (int c = k_eff; c < k; ++c) picked[(size_t)c] = picked[0];
}

}  // namespace

extern "C" {

psb_status psb_kmeans_init(const float* h_data, int64_t n, int dim, int k, int seed, int policy, float* h_centroids, int64_t* h_rows) {
    if (!h_data || !h_centroids || n <= 0 || n > INT_MAX || dim <= 0 || k <= 0 || policy < 0 || policy > 2)
        return fail(PSB_INVALID_ARGUMENT, "invalid k-means initialisation request");
    std::vector<long long> picked;
    kmeans_init_rows(n, dim, k, seed, policy, [&](long long i) { return h_data + (size_t)i * dim; }, picked);
    for (int c = 0; c < k; ++c) {
        std::memcpy(h_centroids + (size_t)c * dim, h_data + (size_t)picked[(size_t)c] * dim, sizeof(float) * (size_t)dim);
        if (h_rows) h_rows[c] = picked[(size_t)c];
    }
    return PSB_OK;
}

psb_status psb_pq_train(const float* d_data, int64_t n, int dim, int subvectors, int codebook_size, int iters,
                        uint64_t seed, float* d_codebook, int device, void* stream) {
    if (!d_data || !d_codebook || n <= 0 || dim <= 0 || subvectors <= 0 || dim % subvectors || codebook_size <= 0 ||
        codebook_size > kMaxCodebook || iters < 0)
        return fail(PSB_INVALID_ARGUMENT, "invalid PQ training request");
    PSB_TRY(check_device(device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int dsub = dim / subvectors;
    DevBuf codes, sums, counts;
    PSB_TRY(codes.reserve((size_t)n * subvectors));
    PSB_TRY(sums.reserve(sizeof(double) * (size_t)subvectors * codebook_size * dsub));
    PSB_TRY(counts.reserve(sizeof(int) * (size_t)subvectors * codebook_size));
    // Initial codewords as the reference's GPU trainer picks them (src/quantization/pq/pq_trainer.cu:30-95): subspace `sub`
    // runs the k-means initialisation with seed + sub * 104729 on its own sub-vectors.  The random-rows policy needs no data;
    // the k-means++ policy (small training sets only: n * K <= 2e7) works on a host copy of the subspace.
    if (n > INT_MAX) return fail(PSB_UNSUPPORTED_SHAPE, "PQ training on more than 2^31-1 rows");
    {
        std::vector<long long> rows((size_t)subvectors * codebook_size), picked;
        const bool plusplus = (long long)n * std::min<long long>(codebook_size, n) <= 20000000LL;
        std::vector<float> sub_host;
        if (plusplus) sub_host.resize((size_t)n * dsub);
        for (int sub = 0; sub < subvectors; ++sub) {
            const int sub_seed = (int)((unsigned)seed + (unsigned)sub * 104729u);
            if (plusplus) {
                PSB_CUDA(cudaMemcpy2DAsync(sub_host.data(), sizeof(float) * (size_t)dsub, d_data + (size_t)sub * dsub, sizeof(float) * (size_t)dim,
                                           sizeof(float) * (size_t)dsub, (size_t)n, cudaMemcpyDeviceToHost, st));
                PSB_CUDA(cudaStreamSynchronize(st));
            }
            kmeans_init_rows(n, dsub, codebook_size, sub_seed, 0, [&](long long i) { return sub_host.data() + (size_t)i * dsub; }, picked);
            std::copy(picked.begin(), picked.end(), rows.begin() + (size_t)sub * codebook_size);
        }
        DevBuf d_rows;
        PSB_TRY(d_rows.reserve(sizeof(long long) * rows.size()));
        PSB_CUDA(cudaMemcpyAsync(d_rows.p, rows.data(), sizeof(long long) * rows.size(), cudaMemcpyHostToDevice, st));
        PSB_TRY(launch_pq_init_rows(d_data, dim, subvectors, codebook_size, d_rows.as<long long>(), d_codebook, st));
        PSB_CUDA(cudaStreamSynchronize(st));   // rows and d_rows go out of scope
    }
    for (int it = 0; it < iters; ++it) {
        PSB_TRY(launch_pq_assign_train(d_data, n, dim, d_codebook, subvectors, codebook_size, codes.as<uint8_t>(), st));
        PSB_CUDA(cudaMemsetAsync(sums.p, 0, sums.bytes, st));
        PSB_CUDA(cudaMemsetAsync(counts.p, 0, counts.bytes, st));
        PSB_TRY(launch_pq_accumulate(d_data, n, dim, codes.as<uint8_t>(), subvectors, codebook_size, sums.as<double>(), counts.as<int>(), st));
        PSB_TRY(launch_pq_update(sums.as<double>(), counts.as<int>(), subvectors, codebook_size, dsub, d_codebook, st));
    }
    PSB_CUDA(cudaStreamSynchronize(st));
    return PSB_OK;
}

psb_status psb_pq_encode(const float* d_data, int64_t n, int dim, const float* d_codebook, int subvectors,
                         int codebook_size, uint8_t* d_codes, int device, void* stream) {
    if (!d_data || !d_codebook || !d_codes || n < 0 || dim <= 0 || subvectors <= 0 || dim % subvectors ||
        codebook_size <= 0 || codebook_size > kMaxCodebook)
        return fail(PSB_INVALID_ARGUMENT, "invalid PQ encode request");
    PSB_TRY(check_device(device));
    return launch_pq_encode(d_data, n, dim, d_codebook, subvectors, codebook_size, d_codes, static_cast<cudaStream_t>(stream));
}

// ---- index-build glue (host) ---------------------------------------------------------------------------------

psb_status psb_ivf_layout_from_assignment(const int* h_assign, int64_t n, int nlist, int64_t* h_offsets, int64_t* h_reordered_ids) {
    if (!h_assign || !h_offsets || !h_reordered_ids || n < 0 || nlist <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid layout request");
    std::fill(h_offsets, h_offsets + nlist + 1, (int64_t)0);
    for (int64_t i = 0; i < n; ++i) {
        const int l = h_assign[i];
        if (l < 0 || l >= nlist) return fail(PSB_INVALID_ARGUMENT, "list assignment outside 0..nlist-1 at row " + std::to_string(i));
        ++h_offsets[l + 1];
    }
    for (int l = 0; l < nlist; ++l) h_offsets[l + 1] += h_offsets[l];
    std::vector<int64_t> cursor(h_offsets, h_offsets + nlist);
    for (int64_t i = 0; i < n; ++i) h_reordered_ids[cursor[(size_t)h_assign[i]]++] = i;  // stable: ascending id within a list
    return PSB_OK;
}

psb_status psb_reorder_rows(const void* h_src, int64_t n, size_t row_bytes, const int64_t* h_reordered_ids, void* h_dst) {
    if (!h_src || !h_dst || !h_reordered_ids || n < 0 || row_bytes == 0) return fail(PSB_INVALID_ARGUMENT, "invalid reorder request");
    std::vector<bool> seen((size_t)n, false);
    for (int64_t local = 0; local < n; ++local) {
        const int64_t id = h_reordered_ids[local];
        if (id < 0 || id >= n || seen[(size_t)id]) return fail(PSB_INVALID_ARGUMENT, "invalid IVF reordered IDs");
        seen[(size_t)id] = true;
    }
    const unsigned char* src = static_cast<const unsigned char*>(h_src);
    unsigned char* dst = static_cast<unsigned char*>(h_dst);
    const int threads = (int)std::min<unsigned>(std::max(1u, std::thread::hardware_concurrency()), 32u);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([=]() {
            for (int64_t local = n * t / threads; local < n * (t + 1) / threads; ++local)
                std::memcpy(dst + (size_t)local * row_bytes, src + (size_t)h_reordered_ids[local] * row_bytes, row_bytes);
        });
    for (auto& th : pool) th.join();
    return PSB_OK;
}

// ---- per-row correction of residual-PQ indices (host) ---------------------------------------------------------------

psb_status psb_row_correction_compute(const float* h_centroids, const int64_t* h_offsets, int nlist, int dim, const uint8_t* h_codes,
                                      const float* h_codebook, int m, int k, float* h_values) {
    if (!h_centroids || !h_offsets || !h_codes || !h_codebook || !h_values || nlist <= 0 || dim <= 0 || m <= 0 || k <= 0 || dim % m)
        return fail(PSB_INVALID_ARGUMENT, "row-correction builder input is incomplete");
    for (int l = 0; l < nlist; ++l)
        if (h_offsets[l] < 0 || h_offsets[l + 1] < h_offsets[l]) return fail(PSB_INVALID_ARGUMENT, "row-correction cluster offsets are invalid");
    const int dsub = dim / m;
    const int threads = (int)std::min<unsigned>(std::max(1u, std::thread::hardware_concurrency()), 64u);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([=]() {
            for (int l = t; l < nlist; l += threads) {
                const float* cen = h_centroids + (size_t)l * dim;
                for (int64_t row = h_offsets[l]; row < h_offsets[l + 1]; ++row) {
                    const uint8_t* code = h_codes + (size_t)row * m;
                    double corr = 0.0;
                    for (int sub = 0; sub < m; ++sub) {
                        const float* cw = h_codebook + ((size_t)sub * k + code[sub]) * dsub;
                        const float* cs = cen + sub * dsub;
                        for (int d = 0; d < dsub; ++d) corr += (double)cw[d] * cw[d] + 2.0 * (double)cs[d] * cw[d];
                    }
                    h_values[row] = (float)corr;
                }
            }
        });
    for (auto& th : pool) th.join();
    return PSB_OK;
}

psb_status psb_row_correction_quantize_u16(const float* h_values, int64_t n, psb_row_correction_u16_header* header, uint16_t* h_u16) {
    if (!h_values || !header || !h_u16 || n <= 0) return fail(PSB_INVALID_ARGUMENT, "invalid row-correction quantisation request");
    float lo = h_values[0], hi = h_values[0];
    for (int64_t i = 0; i < n; ++i) {
        if (!std::isfinite(h_values[i])) return fail(PSB_INVALID_ARGUMENT, "row-correction values contain non-finite data");
        lo = std::min(lo, h_values[i]); hi = std::max(hi, h_values[i]);
    }
    const float offset = std::floor(lo);
    const float range = hi - offset;
    const float scale = range > 0.0f ? std::nextafter(range / 65534.0f, std::numeric_limits<float>::infinity()) : 1.0f;
    if (!(scale > 0.0f) || !std::isfinite(scale)) return fail(PSB_INVALID_ARGUMENT, "row-correction range cannot be quantized");
    for (int64_t i = 0; i < n; ++i) {
        const double qv = std::ceil(((double)h_values[i] - offset) / scale);
        if (qv < 0.0 || qv > 65534.0) return fail(PSB_INTERNAL, "row-correction quantization overflow");
        h_u16[i] = (uint16_t)qv;
    }
    std::memset(header, 0, sizeof(*header));
    static const char magic[8] = {0x49, 0x53, 0x52, 0x43, 0x31, 0x36, 0x00, 0x00};
    std::memcpy(header->magic, magic, 8);
    header->version = 2; header->header_bytes = 32; header->count = (uint64_t)n; header->scale = scale; header->offset = offset;
    return PSB_OK;
}

psb_status psb_row_correction_model_u16(const float* h_centroids, int nlist, const float* h_codebook, int m, int k, int dsub,
                                        float* scale, float* offset) {
    if (!h_centroids || !h_codebook || !scale || !offset || nlist <= 0 || m <= 0 || k <= 0 || k > 256 || dsub <= 0)
        return fail(PSB_INVALID_ARGUMENT, "row correction: invalid PQ model");
    const int64_t dim = (int64_t)m * dsub;
    // slack for an fp32 producer's 2 dim + 8 roundings, relative to the magnitude, plus an absolute term for underflow
    const long double ops = 2.L * dim + 8;
    const long double err = ops * std::numeric_limits<float>::epsilon();
    if (err >= 0.25L) return fail(PSB_INVALID_ARGUMENT, "row correction: PQ dimension exceeds the error-bound contract");
    const long double gamma = err / (1 - err);
    const long double inf_ld = std::numeric_limits<long double>::infinity();
    long double lower = inf_ld, upper = -inf_ld;
    for (int c = 0; c < nlist; ++c) {
        long double lo = 0, hi = 0, mag = 0;
        for (int sub = 0; sub < m; ++sub) {
            long double s_lo = inf_ld, s_hi = -inf_ld, s_abs = 0;
            for (int code = 0; code < k; ++code) {
                long double score = 0, absolute = 0;
                for (int j = 0; j < dsub; ++j) {
                    const long double w = h_codebook[((size_t)sub * k + code) * dsub + j];
                    const long double cv = h_centroids[(size_t)c * dim + sub * dsub + j];
                    if (!std::isfinite(w) || !std::isfinite(cv)) return fail(PSB_INVALID_ARGUMENT, "row correction: non-finite PQ model");
                    score += w * w + 2 * cv * w;
                    absolute += w * w + 2 * std::abs(cv * w);
                }
                s_lo = std::min(s_lo, score); s_hi = std::max(s_hi, score); s_abs = std::max(s_abs, absolute);
            }
            lo += s_lo; hi += s_hi; mag += s_abs;
        }
        if (mag * (1 + gamma) >= std::numeric_limits<float>::max()) return fail(PSB_INVALID_ARGUMENT, "row correction: the model can overflow an fp32 producer");
        const long double pad = gamma * mag + ops * std::numeric_limits<float>::min();
        lower = std::min(lower, lo - pad); upper = std::max(upper, hi + pad);
    }
    const float inf = std::numeric_limits<float>::infinity();
    const float off = std::nextafter((float)lower, -inf);
    const float high = std::nextafter((float)upper, inf);
    const float sc = std::nextafter((float)(((double)high - off) / 65534.), inf);
    if (!std::isfinite(off) || !std::isfinite(high) || !std::isfinite(sc) || !(sc > 0.f) || !std::isfinite(std::fma(sc, 65534.f, off)))
        return fail(PSB_INVALID_ARGUMENT, "row correction: the model has no finite u16 encoding");
    *scale = sc; *offset = off;
    return PSB_OK;
}

psb_status psb_row_correction_encode_u16(const float* h_values, int64_t n, float scale, float offset, uint16_t* h_u16) {
    if (!h_values || !h_u16 || n < 0 || !(scale > 0.f) || !std::isfinite(scale) || !std::isfinite(offset))
        return fail(PSB_INVALID_ARGUMENT, "row correction: invalid u16 scale or offset");
    for (int64_t i = 0; i < n; ++i) {
        const float v = h_values[i];
        if (!std::isfinite(v)) return fail(PSB_INVALID_ARGUMENT, "row correction: non-finite value");
        const double code = std::ceil(((double)v - (double)offset) / (double)scale);
        if (v < offset || !(code >= 0 && code <= 65534)) return fail(PSB_INVALID_ARGUMENT, "row correction: value outside the fixed u16 range");
        h_u16[i] = (uint16_t)code;
    }
    return PSB_OK;
}

psb_status psb_row_correction_write_u16(const char* path, const psb_row_correction_u16_header* header, const uint16_t* h_u16) {
    if (!path || !header || !h_u16) return fail(PSB_INVALID_ARGUMENT, "null argument");
    FILE* f = std::fopen(path, "wb");
    if (!f) return fail(PSB_INVALID_ARGUMENT, std::string("failed to create row-correction payload ") + path);
    const bool ok = std::fwrite(header, sizeof(*header), 1, f) == 1 &&
                    std::fwrite(h_u16, sizeof(uint16_t), (size_t)header->count, f) == (size_t)header->count;
    if (std::fclose(f) != 0 || !ok) return fail(PSB_INTERNAL, "failed to write row-correction payload");
    return PSB_OK;
}

psb_status psb_row_correction_read_u16(const char* path, psb_row_correction_u16_header* header, uint16_t* h_u16, int64_t capacity) {
    if (!path || !header) return fail(PSB_INVALID_ARGUMENT, "null argument");
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(PSB_INVALID_ARGUMENT, std::string("cannot open row-correction payload ") + path);
    psb_status st = PSB_OK;
    static const char magic[8] = {0x49, 0x53, 0x52, 0x43, 0x31, 0x36, 0x00, 0x00};
    if (std::fread(header, sizeof(*header), 1, f) != 1 || std::memcmp(header->magic, magic, 8) != 0 || header->version != 2 ||
        header->header_bytes != 32 || !std::isfinite(header->scale) || !(header->scale > 0.0f) || !std::isfinite(header->offset))
        st = fail(PSB_INVALID_ARGUMENT, "not a row-correction u16 payload (magic, version, header size, scale or offset)");
    else if (h_u16) {
        if ((int64_t)header->count > capacity) st = fail(PSB_INVALID_ARGUMENT, "row-correction payload holds more rows than the buffer");
        else if (std::fread(h_u16, sizeof(uint16_t), (size_t)header->count, f) != (size_t)header->count)
            st = fail(PSB_INVALID_ARGUMENT, "row-correction payload is truncated");
    }
    std::fclose(f);
    return st;
}

// ---- synthetic data -------------------------------------------------------------------------------------------

psb_status psb_gen_mixture_rows(const float* d_centres, const int64_t* d_offsets, int ncomp, int dim,
                                float sigma, uint64_t seed, int64_t row_begin, int64_t n, float* d_out,
                                int device, void* stream) {
    if (!d_centres || !d_offsets || !d_out || ncomp <= 0 || dim <= 0 || n < 0) return fail(PSB_INVALID_ARGUMENT, "invalid generator request");
    PSB_TRY(check_device(device));
    const long long step = ((long long)1 << 31) / dim;  // rows per launch
    for (long long r = 0; r < n; r += step)
        PSB_TRY(launch_gen_mixture(d_centres, reinterpret_cast<const long long*>(d_offsets), ncomp, dim, sigma, seed,
                                   row_begin + r, std::min<long long>(step, n - r), d_out + (size_t)r * dim,
                                   static_cast<cudaStream_t>(stream)));
    return PSB_OK;
}

psb_status psb_gen_normal(uint64_t seed, int64_t first_elem, int64_t n_elems, float scale, float* d_out,
                          int device, void* stream) {
    if (!d_out || n_elems < 0) return fail(PSB_INVALID_ARGUMENT, "invalid generator request");
    PSB_TRY(check_device(device));
    const long long step = (long long)1 << 31;
    for (long long r = 0; r < n_elems; r += step)
        PSB_TRY(launch_gen_normal(seed, first_elem + r, std::min<long long>(step, n_elems - r), scale, d_out + r,
                                  static_cast<cudaStream_t>(stream)));
    return PSB_OK;
}

}  // extern "C"
