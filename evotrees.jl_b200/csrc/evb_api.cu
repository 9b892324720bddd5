// C ABI of libevotrees_b200.so (declarations and per-function contracts: include/evb.h).
#include "evb_internal.cuh"
#include <chrono>
#include <stdarg.h>
#include <string.h>
#include <stdlib.h>
#include <new>
#include <algorithm>
#include <nvtx3/nvToolsExt.h>

static const char *const g_timer_names[EVB_NTIMERS] = {"evb:grads", "evb:rows_init", "evb:hist", "evb:hist_reduce", "evb:allreduce", "evb:scan",
                                                        "evb:partition", "evb:plan", "evb:finalize", "evb:d2h", "evb:h2d", "evb:tree"};

int32_t evb_launch_check_bins(evb_handle *h);
int32_t evb_launch_init_state(evb_handle *h, const float *w_dev, const float *pred0_dev, const float *mu_dev);
int32_t evb_launch_root_plan(evb_handle *h);
int32_t evb_hist_geometry(const evb_handle *h, int F, HistGeom *g);
int32_t evb_nccl_check(evb_handle *h);

static thread_local char g_err[512] = "";
void evb_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
extern "C" const char *evb_last_error(void) { return g_err; }
int evb_hist_mode_env() {
    const char *e = getenv("EVB_HIST_MODE");
#ifdef EVB_DIAG
    return e ? atoi(e) : 1;
#else
    return e ? (atoi(e) & 1) : 1;
#endif
}
extern "C" int32_t evb_version(void) { return EVB_VERSION; }

// ---- timing -----------------------------------------------------------------------------------------
// tic/toc bracket one kernel class (brackets do not nest); the events are read after the stream is
// synchronised at the end of evb_grow_tree.
void evb_tic(evb_handle *h, int cls) {
    if (!h->timing) return;
    nvtxRangePushA(g_timer_names[cls]); // with EVB_FLAG_TIMING every kernel class is also an NVTX range on the host timeline
    while (h->ev_used + 2 > h->ev.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) { h->timing = false; return; }
        h->ev.push_back(e);
    }
    cudaEventRecord(h->ev[h->ev_used], h->st);
}
void evb_toc(evb_handle *h, int cls) {
    h->tm.launches[cls] += 1;
    if (!h->timing) return;
    nvtxRangePop();
    cudaEventRecord(h->ev[h->ev_used + 1], h->st);
    h->ev_class.push_back(cls);
    h->ev_used += 2;
}
static void resolve_timing(evb_handle *h) {
    if (!h->timing) return;
    for (size_t i = 0; i < h->ev_used; i += 2) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, h->ev[i], h->ev[i + 1]) == cudaSuccess) h->tm.ms[h->ev_class[i / 2]] += ms;
    }
    float ms = 0.f;
    if (h->ev_tot[0] && cudaEventElapsedTime(&ms, h->ev_tot[0], h->ev_tot[1]) == cudaSuccess) h->tm.ms[EVB_T_TREE_TOTAL] += ms;
    h->ev_used = 0;
    h->ev_class.clear();
}

// stream on which dalloc() clears the blocks it hands out: the stream of the handle the calling thread works on
static thread_local cudaStream_t g_alloc_stream = nullptr;

struct BusyGuard {
    evb_handle *h;
    bool ok;
    explicit BusyGuard(evb_handle *hh) : h(hh) { ok = __sync_bool_compare_and_swap(&h->busy, 0, 1); }
    ~BusyGuard() { if (ok) __sync_lock_release(&h->busy); }
};
#define EVB_ENTER(h)                                                                   \
    if (!(h)) { evb_set_error("null handle"); return EVB_ERR_ARG; }                    \
    BusyGuard _guard(h);                                                               \
    if (!_guard.ok) { evb_set_error("handle is in use by another thread"); return EVB_ERR_BUSY; } \
    EVB_CUDA(cudaSetDevice((h)->dev));                                                 \
    g_alloc_stream = (h)->st

// Failure injection for the tests of the error paths: EVB_TEST_FAIL_ALLOC=k makes the k-th device allocation of the
// next evb_create* of this thread fail as if the device were out of memory (nothing is allocated, nothing faults).
static thread_local int g_alloc_countdown = 0;
// Blocks may come from the library's cache with the previous owner's contents.  Everything below 256 MB is cleared on
// the creating handle's stream (the large buffers -- bins, gradients, row lists -- are written in full before use).
template <typename T>
static cudaError_t dalloc(T **p, size_t count) {
    if (g_alloc_countdown > 0 && --g_alloc_countdown == 0) { *p = nullptr; return cudaErrorMemoryAllocation; }
    const size_t bytes = (count ? count : 1) * sizeof(T);
    cudaError_t e = evb_dev_alloc((void **)p, bytes);
    if (e == cudaSuccess && bytes < ((size_t)256 << 20)) e = cudaMemsetAsync(*p, 0, bytes, g_alloc_stream);
    return e;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Device block that travels to the host once per tree: [plan][err][eval sums][feat][gain][w][pred][packed][bin][split]
struct TreeBlockLayout {
    size_t plan, err, evsum, feat, gain, w, pred, packed, bin, split, total;
};
static TreeBlockLayout tree_block_layout(int D, int nn, int K) {
    TreeBlockLayout l;
    size_t o = 0;
    l.plan = o; o += align_up(sizeof(LevelPlan) * (D + 2), 16);
    l.err = o; o += 16;
    l.evsum = o; o += 16;
    l.feat = o; o += align_up(sizeof(int32_t) * nn, 16);
    l.gain = o; o += align_up(sizeof(float) * nn, 16);
    l.w = o; o += align_up(sizeof(float) * nn, 16);
    l.pred = o; o += align_up(sizeof(float) * nn * K, 16);
    l.packed = o; o += align_up(sizeof(uint32_t) * nn, 16);
    l.bin = o; o += align_up((size_t)nn, 16);
    l.split = o; o += align_up((size_t)nn, 16);
    l.total = o;
    return l;
}

static void drop_graphs(evb_handle *h);
static void free_eval(evb_handle *h) {
    void *ptrs[] = {h->ev_xT, h->ev_y, h->ev_w, h->ev_pred, h->ev_part};
    for (void *p : ptrs) evb_dev_free(p);
    h->ev_xT = nullptr; h->ev_y = nullptr; h->ev_w = nullptr; h->ev_pred = nullptr; h->ev_part = nullptr;
    h->ev_n = 0;
}
static void free_handle(evb_handle *h) {
    if (!h) return;
    cudaSetDevice(h->dev);
    if (h->st) cudaStreamSynchronize(h->st);
    static const bool trace = getenv("EVB_INIT_TRACE") != nullptr;
    auto t_last = std::chrono::steady_clock::now();
    auto phase = [&](const char *name) {
        if (!trace) return;
        const auto now = std::chrono::steady_clock::now();
        fprintf(stderr, "[evb destroy] %-21s %8.2f ms\n", name, std::chrono::duration<double, std::milli>(now - t_last).count());
        t_last = now;
    };
    evb_nccl_destroy(h);
    for (int i = 0; i < h->n_ipc_opened; ++i) cudaIpcCloseMemHandle(h->ipc_opened[i]);
    // blocks that the other ranks mapped through CUDA IPC go back to the driver, not into the cache
    const bool exported = h->peer_cand[h->rank] != nullptr;
    evb_dev_free(h->peer_cand[h->rank], true);
    evb_dev_free(h->peer_flags[h->rank], true);
    evb_dev_free(h->d_barrier_seq);
    evb_dev_free(h->hsum);
    if (exported) { evb_dev_free(h->hcomp, true); h->hcomp = nullptr; }
    free_eval(h);
    void *ptrs[] = {h->xH, h->xE, h->hsum_q, h->hcnt_q, h->qs_cnt, h->qs_prefix, h->qs_rank, h->qs_gamma, h->gradq, h->d_gmax, h->d_qinv, h->xT, h->xC, h->grad, h->pred, h->y, h->nidx, h->rows[0], h->rows[1], h->mask_d, h->feattypes_d, h->mono_d,
                    h->js_d, h->seg_start, h->seg_cnt, h->gcnt, h->nleft, (h->gnleft != h->nleft) ? h->gnleft : nullptr, h->kind,
                    h->bslot, h->nsum, h->plan /* base of the tree block */, h->cum, h->slot_node, h->item_node, h->item_left,
                    h->item_lprefix, h->item_bits, h->scan_tmp, h->hist, h->hcomp, h->scratch, h->fbest_gain, h->fbest_bin, h->obl_gain, h->obl_best};
    phase("exchange buffers");
    for (void *p : ptrs) evb_dev_free(p);
    phase("device buffers");
    drop_graphs(h);
    phase("graphs");
    for (int q = 0; q < 2; ++q) {
        evb_host_free(h->h_tree[q]);
        evb_host_free(h->h_js[q]);
        evb_event_put(h->ev_done[q]);
    }
    for (cudaEvent_t e : h->ev) cudaEventDestroy(e);
    for (cudaEvent_t e : h->ev_tot) if (e) cudaEventDestroy(e);
    evb_stream_put(h->st); // synchronised at the top of this function
    phase("pinned, events, stream");
    delete h;
}

extern "C" void evb_destroy(evb_handle *h) { free_handle(h); }

// x_bin != NULL: the binned matrix; else the raw matrix x (x_dtype) with its edges, binarized on the device
static int32_t create_impl(evb_handle *h, const evb_params *p, int64_t nobs, int32_t nfeats, const uint8_t *x_bin, const void *x,
                           int32_t x_dtype, const void *edges, int32_t nedges, const void *y,
                           int32_t y_dtype, int32_t ycols, const float *w, const float *pred0, const float *mu,
                           const uint8_t *feattypes, const int32_t *monotone) {
    // EVB_INIT_TRACE=1: host-side milliseconds of the phases of evb_create / evb_create_x on stderr
    static const bool trace = getenv("EVB_INIT_TRACE") != nullptr;
    auto t_last = std::chrono::steady_clock::now();
    auto phase = [&](const char *name) {
        if (!trace) return;
        cudaStreamSynchronize(h->st);
        const auto now = std::chrono::steady_clock::now();
        fprintf(stderr, "[evb init] %-24s %8.2f ms\n", name, std::chrono::duration<double, std::milli>(now - t_last).count());
        t_last = now;
    };
    h->p = *p;
    h->K = p->K; h->C = 2 * p->K + 1; h->B = p->nbins; h->D = p->max_depth; h->nn = (1 << p->max_depth) - 1;
    h->Ce = (p->loss == EVB_MSE && !getenv("EVB_NO_ELISION")) ? p->K + 1 : h->C;
    h->nfeats = nfeats; h->RS = (nfeats + 31) / 32 * 32; h->GS = (h->Ce + 3) / 4 * 4; h->n = nobs;
    { const int nct = (h->Ce + 3) / 4; h->rec_nch = (h->Ce + nct - 1) / nct; }
    // mse with one target runs the fixed-point histogram kernel (EVB_HIST_Q=0: the float kernel)
    { const char *e = getenv("EVB_HIST_Q"); h->use_q = p->loss == EVB_MSE && p->K == 1 && h->Ce == 2 && !(e && atoi(e) == 0); }
    h->unit_w = w == nullptr;
    h->wscale = 1.0f; h->winv = 1.0;
    if (h->use_q && w) {
        float wmax = 0.0f;
        for (int64_t i = 0; i < nobs; ++i) wmax = w[i] > wmax ? w[i] : wmax;
        if (wmax > 0.0f && wmax < INFINITY) {
            int e;
            frexpf(wmax, &e);
            h->wscale = ldexpf(1.0f, 29 - e);
            h->winv = ldexp(1.0, e - 29);
        }
    }
    h->dev = p->device; h->y_dtype = y_dtype; h->ycols = ycols;
    h->timing = (p->flags & EVB_FLAG_TIMING) != 0;
    h->world = 1; h->rank = 0; h->F = nfeats;
    h->hist_mode = evb_hist_mode_env();
    int cc_major = 0, cc_minor = 0; // single attributes: cudaGetDeviceProperties queries everything and takes milliseconds
    EVB_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, h->dev));
    EVB_CUDA(cudaDeviceGetAttribute(&cc_minor, cudaDevAttrComputeCapabilityMinor, h->dev));
    if (cc_major < 10) {
        evb_set_error("device %d is sm_%d%d; this library is built for sm_100a only", h->dev, cc_major, cc_minor);
        return EVB_ERR_CUDA;
    }
    EVB_CUDA(cudaDeviceGetAttribute(&h->num_sms, cudaDevAttrMultiProcessorCount, h->dev));
    EVB_CUDA(evb_stream_get(&h->st));
    g_alloc_stream = h->st;
    const int64_t n = nobs;
    const int nids = h->nn + 2, C = h->C, K = h->K, D = h->D;

    EVB_CUDA(dalloc(&h->xT, (size_t)n * h->RS));
    EVB_CUDA(dalloc(&h->grad, (size_t)n * h->GS));
    if (p->loss == EVB_QUANTILE || p->loss == EVB_MULTIQUANTILE) {
        const size_t e = (size_t)2 * (h->nn + 1);
        EVB_CUDA(dalloc(&h->qs_cnt, e * 256)); EVB_CUDA(dalloc(&h->qs_prefix, e)); EVB_CUDA(dalloc(&h->qs_rank, e));
        EVB_CUDA(dalloc(&h->qs_gamma, (size_t)h->nn + 1));
        EVB_CUDA(cudaMemset(h->qs_cnt, 0, e * 256 * sizeof(uint32_t)));
    }
    // unit weights: the register-direct kernel (EVB_HIST_Q2=0: the staged fixed-point kernel)
    { const char *e = getenv("EVB_HIST_Q2"); h->use_q2 = h->use_q && h->unit_w && !(e && atoi(e) == 0) && evb_q2_configure(h) == EVB_OK; }
    if (h->use_q) {
        if (!h->use_q2) EVB_CUDA(dalloc(&h->gradq, (size_t)n * (h->unit_w ? 1 : 2)));
        EVB_CUDA(dalloc(&h->d_gmax, (size_t)1));
        EVB_CUDA(dalloc(&h->d_qinv, (size_t)2));
        EVB_CUDA(cudaMemset(h->d_gmax, 0, sizeof(unsigned)));
    }
    EVB_CUDA(dalloc(&h->pred, (size_t)n * K));
    EVB_CUDA(dalloc(&h->nidx, (size_t)n));
    EVB_CUDA(dalloc(&h->rows[0], (size_t)n));
    EVB_CUDA(dalloc(&h->rows[1], (size_t)n));
    EVB_CUDA(dalloc(&h->mask_d, (size_t)n));
    EVB_CUDA(dalloc(&h->feattypes_d, (size_t)nfeats));
    EVB_CUDA(dalloc(&h->mono_d, (size_t)nfeats));
    EVB_CUDA(dalloc(&h->js_d, (size_t)nfeats));
    EVB_CUDA(dalloc(&h->seg_start, (size_t)nids)); EVB_CUDA(dalloc(&h->seg_cnt, (size_t)nids));
    EVB_CUDA(dalloc(&h->gcnt, (size_t)nids)); EVB_CUDA(dalloc(&h->nleft, (size_t)nids));
    h->gnleft = h->nleft;
    EVB_CUDA(dalloc(&h->kind, (size_t)nids)); EVB_CUDA(dalloc(&h->bslot, (size_t)nids));
    EVB_CUDA(dalloc(&h->nsum, (size_t)nids * C));
    EVB_CUDA(cudaMemset(h->nleft, 0, sizeof(int32_t) * nids));

    const TreeBlockLayout L = tree_block_layout(D, h->nn, K);
    unsigned char *blk = nullptr;
    EVB_CUDA(dalloc(&blk, L.total));
    EVB_CUDA(cudaMemset(blk, 0, L.total));
    h->plan = (LevelPlan *)(blk + L.plan); h->d_err = (int *)(blk + L.err); h->d_evsum = (double *)(blk + L.evsum);
    h->t_feat = (int32_t *)(blk + L.feat); h->t_gain = (float *)(blk + L.gain); h->t_w = (float *)(blk + L.w);
    h->t_pred = (float *)(blk + L.pred); h->t_packed = (uint32_t *)(blk + L.packed); h->t_bin = blk + L.bin; h->t_split = blk + L.split;
    h->h_tree_bytes = L.total;
    for (int q = 0; q < 2; ++q) {
        EVB_CUDA(evb_host_alloc(&h->h_tree[q], L.total));
        EVB_CUDA(evb_host_alloc((void **)&h->h_js[q], sizeof(uint32_t) * nfeats));
        EVB_CUDA(evb_event_get(&h->ev_done[q]));
    }
    { const char *e = getenv("EVB_GRAPH"); h->use_graphs = e ? atoi(e) != 0 : true; }
    h->graph_mask_cond = -1;

    h->maxslots = evb_level_slots(D > 1 ? D - 1 : 1);
    EVB_CUDA(dalloc(&h->cum, (size_t)h->maxslots + 1)); EVB_CUDA(dalloc(&h->slot_node, (size_t)h->maxslots));
    h->max_items = (int)(n / EVB_PART_CHUNK) + (1 << (D > 1 ? D - 1 : 0)) + 2;
    EVB_CUDA(dalloc(&h->item_node, (size_t)(1 << D) + 2));
    EVB_CUDA(dalloc(&h->item_left, (size_t)h->max_items)); EVB_CUDA(dalloc(&h->item_lprefix, (size_t)h->max_items));
    EVB_CUDA(dalloc(&h->item_bits, (size_t)h->max_items * (EVB_PART_CHUNK / 32)));
    EVB_CUDA(dalloc(&h->scan_tmp, (size_t)(n / 2048 + 2)));
    {
        const size_t lv = (size_t)evb_level_nodes(D > 1 ? D - 1 : 1) * nfeats;
        EVB_CUDA(dalloc(&h->fbest_gain, lv)); EVB_CUDA(dalloc(&h->fbest_bin, lv));
        if (p->tree_type == 1) {
            EVB_CUDA(dalloc(&h->obl_gain, ((size_t)evb_level_nodes(D > 1 ? D - 1 : 1) + 1) * nfeats * h->B));
            EVB_CUDA(dalloc(&h->obl_best, (size_t)2));
        }
    }

    const bool keep_all = (p->flags & EVB_FLAG_KEEP_ALL_HIST) != 0;
    h->hist_nodes = keep_all ? (1 << (D > 1 ? D - 1 : 0)) : (D >= 2 ? 1 << (D - 2) : 1);
    const size_t FCB = (size_t)nfeats * C * h->B;
    EVB_CUDA(dalloc(&h->hist, (size_t)h->hist_nodes * FCB));
    EVB_CUDA(dalloc(&h->hcomp, (size_t)h->maxslots * FCB));
    EVB_CHECK(evb_hist_configure(h));
    EVB_CUDA(dalloc(&h->scratch, h->scratch_floats));

    // ---- uploads: x_bin is kept feature-major (as given) for the row partition and transposed on the device to
    // observation-major rows for the histogram gathers and the tree traversal
    phase("allocations");
    EVB_CUDA(cudaMemsetAsync(h->xT, 0, (size_t)n * h->RS, h->st));
    EVB_CUDA(dalloc(&h->xC, (size_t)n * nfeats));
    phase("xC alloc + xT memset");
    if (x_bin) EVB_CHECK(evb_h2d_staged(h->xC, x_bin, (size_t)n * nfeats, h->st));
    else EVB_CHECK(evb_upload_binarize(h, x, x_dtype, edges, nedges));
    phase("upload (+ binarize)");
    EVB_CHECK(evb_launch_transpose(h, h->xC, n, n, 0, nfeats, h->xT, h->RS, h->st));
    phase("transpose to xT");
    if (h->use_q2) {
        const size_t acc = (size_t)h->maxslots * h->B * h->q2.SC;
        EVB_CUDA(dalloc(&h->xH, (size_t)(n + 1) * h->q2.RSH));
        EVB_CUDA(dalloc(&h->xE, (size_t)n + 1));
        EVB_CUDA(dalloc(&h->hsum_q, acc));
        EVB_CUDA(dalloc(&h->hcnt_q, acc));
        EVB_CUDA(cudaMemsetAsync(h->hsum_q, 0, acc * sizeof(unsigned long long), h->st));
        EVB_CUDA(cudaMemsetAsync(h->hcnt_q, 0, acc * sizeof(uint32_t), h->st));
        EVB_CHECK(evb_q2_build_layout(h));
        phase("chunk rows (xH, xE)");
    }
    {
        const size_t ybytes = (size_t)n * (y_dtype == EVB_U32 ? 4 : 4 * (size_t)ycols);
        EVB_CUDA(evb_dev_alloc(&h->y, ybytes ? ybytes : 1));
        EVB_CUDA(cudaMemcpyAsync(h->y, y, ybytes, cudaMemcpyHostToDevice, h->st));
        float *w_d = nullptr, *p0_d = nullptr, *mu_d = nullptr;
        if (w) { EVB_CUDA(dalloc(&w_d, (size_t)n)); EVB_CUDA(cudaMemcpyAsync(w_d, w, sizeof(float) * n, cudaMemcpyHostToDevice, h->st)); }
        if (pred0) { EVB_CUDA(dalloc(&p0_d, (size_t)n * K)); EVB_CUDA(cudaMemcpyAsync(p0_d, pred0, sizeof(float) * n * K, cudaMemcpyHostToDevice, h->st)); }
        else { EVB_CUDA(dalloc(&mu_d, (size_t)K)); EVB_CUDA(cudaMemcpyAsync(mu_d, mu, sizeof(float) * K, cudaMemcpyHostToDevice, h->st)); }
        int32_t rc = evb_launch_init_state(h, w_d, p0_d, mu_d);
        cudaStreamSynchronize(h->st);
        evb_dev_free(w_d);
        evb_dev_free(p0_d);
        evb_dev_free(mu_d);
        EVB_CHECK(rc);
    }
    {
        std::vector<uint8_t> ft(nfeats, 1);
        std::vector<int32_t> mo(nfeats, 0);
        if (feattypes) memcpy(ft.data(), feattypes, nfeats);
        if (monotone) memcpy(mo.data(), monotone, sizeof(int32_t) * nfeats);
        EVB_CUDA(cudaMemcpy(h->feattypes_d, ft.data(), nfeats, cudaMemcpyHostToDevice));
        EVB_CUDA(cudaMemcpy(h->mono_d, mo.data(), sizeof(int32_t) * nfeats, cudaMemcpyHostToDevice));
    }
    phase("targets + state");
    // bins made by the device binarize are 1 + (number of edges below the value): in range by construction
    if (x_bin) EVB_CHECK(evb_launch_check_bins(h));
    phase("bin range check");
    int err = 0;
    EVB_CUDA(cudaMemcpyAsync(&err, h->d_err, sizeof(int), cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    if (err == EVB_DERR_BIN_RANGE) {
        evb_set_error("x_bin holds values outside 1..nbins (%d)", h->B);
        return EVB_ERR_ARG;
    }
    if (err == EVB_DERR_NAN) {
        evb_set_error("the feature matrix holds NaN: missing values are not supported");
        return EVB_ERR_ARG;
    }
    return EVB_OK;
}

static int32_t create_common(evb_handle **out, const evb_params *p, int64_t nobs, int32_t nfeats, const uint8_t *x_bin, const void *x,
                             int32_t x_dtype, const void *edges, int32_t nedges, const void *y, int32_t y_dtype, int32_t ycols,
                             const float *w, const float *pred0, const float *mu, const uint8_t *feattypes, const int32_t *monotone) {
    if (!out) { evb_set_error("evb_create: out is null"); return EVB_ERR_ARG; }
    *out = nullptr;
    if (!p || (!x_bin && !x) || !y || (!pred0 && !mu)) { evb_set_error("evb_create: null argument"); return EVB_ERR_ARG; }
    if (x && (!edges || (x_dtype != EVB_F32 && x_dtype != EVB_F64) || nedges != p->nbins - 1)) {
        evb_set_error("evb_create_x: x needs EVB_F32 / EVB_F64 and nbins - 1 edges per feature");
        return EVB_ERR_ARG;
    }
    if (nobs < 1 || nobs > 2000000000ll || nfeats < 1 || nfeats > 65535) { evb_set_error("evb_create: nobs/nfeats out of range"); return EVB_ERR_ARG; }
    if (p->loss < 0 || p->loss > EVB_LOSS_LAST) { evb_set_error("evb_create: unknown loss %d", p->loss); return EVB_ERR_ARG; }
    if (p->K < 1 || p->K > 32) { evb_set_error("evb_create: K=%d outside 1..32", p->K); return EVB_ERR_ARG; }
    const bool mle = p->loss == EVB_GAUSSIAN_MLE || p->loss == EVB_LOGISTIC_MLE;
    if ((mle && (p->K % 2 != 0 || ycols != p->K / 2)) || (!mle && p->loss != EVB_MLOGLOSS && p->loss != EVB_MULTIQUANTILE && ycols != p->K) ||
        (p->loss == EVB_MULTIQUANTILE && (ycols != 1 || p->K > 8)) ||
        (p->loss == EVB_MLOGLOSS && p->K < 2)) {
        evb_set_error("evb_create: K=%d / ycols=%d inconsistent with the loss", p->K, ycols);
        return EVB_ERR_ARG;
    }
    if ((p->loss == EVB_MLOGLOSS) != (y_dtype == EVB_U32) || (y_dtype != EVB_U32 && y_dtype != EVB_F32)) {
        evb_set_error("evb_create: y_dtype must be EVB_U32 for mlogloss and EVB_F32 otherwise");
        return EVB_ERR_ARG;
    }
    if (p->nbins < 2 || p->nbins > 255) { evb_set_error("evb_create: nbins=%d outside 2..255", p->nbins); return EVB_ERR_ARG; }
    if (p->max_depth < 1 || p->max_depth > EVB_MAX_DEPTH) { evb_set_error("evb_create: max_depth=%d outside 1..%d", p->max_depth, EVB_MAX_DEPTH); return EVB_ERR_LIMIT; }
    if (p->loss == EVB_QUANTILE && (p->K != 1 || !(p->alpha > 0.0 && p->alpha < 1.0))) {
        evb_set_error("evb_create: the quantile loss needs K = 1 and 0 < alpha < 1 (alpha = %g)", p->alpha);
        return EVB_ERR_ARG;
    }
    if (p->loss == EVB_MULTIQUANTILE) {
        for (int k = 0; k < p->K; ++k)
            if (!(p->alphas[k] > 0.0 && p->alphas[k] < 1.0)) { evb_set_error("evb_create: alphas[%d] = %g outside (0, 1)", k, p->alphas[k]); return EVB_ERR_ARG; }
    }
    if (p->bagging_size < 1 || p->tree_type < 0 || p->tree_type > 1) { evb_set_error("evb_create: bagging_size must be >= 1 and tree_type 0 (binary) or 1 (oblivious)"); return EVB_ERR_ARG; }
    if (p->tree_type == 1 && !(p->gamma >= 0.0)) { evb_set_error("evb_create: oblivious trees need gamma >= 0"); return EVB_ERR_ARG; }
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) {
        evb_set_error("no CUDA device available (%s): this library has no CPU fallback", cudaGetErrorString(e));
        return EVB_ERR_CUDA;
    }
    if (p->device < 0 || p->device >= ndev) { evb_set_error("evb_create: device %d out of range", p->device); return EVB_ERR_ARG; }
    EVB_CUDA(cudaSetDevice(p->device));
    evb_handle *h = new (std::nothrow) evb_handle();
    if (!h) { evb_set_error("out of host memory"); return EVB_ERR_ARG; }
    memset(&h->tm, 0, sizeof(h->tm));
    { const char *e = getenv("EVB_TEST_FAIL_ALLOC"); g_alloc_countdown = e ? atoi(e) : 0; }
    int32_t rc = create_impl(h, p, nobs, nfeats, x_bin, x, x_dtype, edges, nedges, y, y_dtype, ycols, w, pred0, mu, feattypes, monotone);
    g_alloc_countdown = 0;
    if (rc != EVB_OK) { free_handle(h); return rc; }
    *out = h;
    return EVB_OK;
}

extern "C" int32_t evb_create(evb_handle **out, const evb_params *p, int64_t nobs, int32_t nfeats, const uint8_t *x_bin,
                              const void *y, int32_t y_dtype, int32_t ycols, const float *w, const float *pred0, const float *mu,
                              const uint8_t *feattypes, const int32_t *monotone) {
    if (!x_bin) { evb_set_error("evb_create: x_bin is null"); return EVB_ERR_ARG; }
    return create_common(out, p, nobs, nfeats, x_bin, nullptr, 0, nullptr, 0, y, y_dtype, ycols, w, pred0, mu, feattypes, monotone);
}

extern "C" int32_t evb_create_x(evb_handle **out, const evb_params *p, int64_t nobs, int32_t nfeats, const void *x, int32_t x_dtype,
                                const void *edges, int32_t nedges, const void *y, int32_t y_dtype, int32_t ycols, const float *w,
                                const float *pred0, const float *mu, const uint8_t *feattypes, const int32_t *monotone) {
    if (!x) { evb_set_error("evb_create_x: x is null"); return EVB_ERR_ARG; }
    return create_common(out, p, nobs, nfeats, nullptr, x, x_dtype, edges, nedges, y, y_dtype, ycols, w, pred0, mu, feattypes, monotone);
}

extern "C" int32_t evb_comm_unique_id(uint8_t id[128]) {
    if (!id) { evb_set_error("null id"); return EVB_ERR_ARG; }
    return evb_nccl_unique_id(id);
}

extern "C" int32_t evb_comm_init(evb_handle *h, const uint8_t id[128], int32_t rank, int32_t world) {
    EVB_ENTER(h);
    if (!id || world < 1 || rank < 0 || rank >= world) { evb_set_error("evb_comm_init: bad rank/world"); return EVB_ERR_ARG; }
    if (h->nccl_comm || h->nccl_pending) { evb_set_error("evb_comm_init: communicator already initialised"); return EVB_ERR_ARG; }
    if (world == 1) return EVB_OK;
    EVB_CHECK(evb_nccl_init(h, id, rank, world));
    return EVB_OK;
}

// Everything one tree launches, in stream order.  Runs either directly or under stream capture (then it is
// replayed as one CUDA graph per tree): it must not synchronise and must not touch pageable host memory.
static int32_t enqueue_tree(evb_handle *h, bool use_mask, uint8_t mask_cond, bool run_grads, bool quantize, bool fuse, int slot) {
    const int D = h->D;
    EVB_CUDA(cudaMemcpyAsync(h->js_d, h->h_js[slot], sizeof(uint32_t) * h->F, cudaMemcpyHostToDevice, h->st));
    if (run_grads) EVB_CHECK(evb_launch_grads(h));
    if (quantize) EVB_CHECK(h->use_q2 ? evb_launch_q2_quantize(h) : evb_launch_quantize(h)); // fixed-point histogram kernel: the gradients changed since the last tree
    EVB_CHECK(evb_launch_tree_reset(h));
    EVB_CHECK(evb_launch_rows_init(h, use_mask, mask_cond));
    EVB_CHECK(evb_launch_root_plan(h));
    const int last = D > 1 ? D - 1 : 1;
    const bool full_part = (h->p.flags & EVB_FLAG_FULL_PARTITION) != 0;
    for (int level = 1; level <= last; ++level) {
        if (h->use_q2) {
            EVB_CHECK(evb_launch_histq2(h, level));
            if (!evb_q2_direct(h)) EVB_CHECK(evb_launch_q2_reduce(h, level));
        } else {
            EVB_CHECK(evb_launch_hist(h, level));
            EVB_CHECK(evb_launch_hist_reduce(h, level));
        }
        if (h->world > 1 && !h->p2p) { // with peer access the ranks' histograms are summed inside the split scan instead
            evb_tic(h, EVB_T_ALLREDUCE);
            int32_t s = evb_nccl_allreduce_f64(h, h->hcomp, (size_t)evb_level_slots(level) * h->F * h->C * h->B);
            evb_toc(h, EVB_T_ALLREDUCE);
            EVB_CHECK(s);
        }
        EVB_CHECK(evb_launch_scan(h, level));
        if (evb_q2_direct(h)) EVB_CHECK(evb_launch_q2_clear(h, level));
        if (level < D - 1 || (full_part && level == D - 1)) EVB_CHECK(evb_launch_partition(h, level));
    }
    if (h->p.loss == EVB_QUANTILE || h->p.loss == EVB_MULTIQUANTILE) {
        // the leaf values need the leaf of every row first: leaf ids, per-leaf quantiles, then the usual update
        EVB_CHECK(evb_launch_finalize(h, false, 1));
        EVB_CHECK(evb_launch_quantile_leaves(h, use_mask, mask_cond));
        EVB_CHECK(evb_launch_finalize(h, fuse, 2));
    } else {
        EVB_CHECK(evb_launch_finalize(h, fuse, 0));
    }
    if (h->ev_n > 0) EVB_CHECK(evb_launch_eval(h, nullptr));
    EVB_CUDA(cudaMemcpyAsync(h->h_tree[slot], h->plan, h->h_tree_bytes, cudaMemcpyDeviceToHost, h->st));
    return EVB_OK;
}

static void drop_graphs(evb_handle *h) {
    for (auto &g : h->graph) { if (g) cudaGraphExecDestroy(g); g = nullptr; }
    for (auto &c : h->graph_calls) c = 0;
}

extern "C" int32_t evb_grow_tree_begin(evb_handle *h, const uint8_t *row_mask, uint8_t mask_cond, const uint32_t *js, int32_t njs,
                                       int32_t update_grads) {
    EVB_ENTER(h);
    if (!js || njs < 1 || njs > h->nfeats) { evb_set_error("evb_grow_tree: invalid argument"); return EVB_ERR_ARG; }
    if (h->pending >= 2 || (h->pending >= 1 && h->timing)) {
        evb_set_error("evb_grow_tree_begin: collect the previous tree with evb_grow_tree_end first");
        return EVB_ERR_BUSY;
    }
    const int slot = h->tree_seq & 1;
    for (int i = 0; i < njs; ++i) {
        if (js[i] < 1 || js[i] > (uint32_t)h->nfeats || (i > 0 && js[i] <= js[i - 1])) {
            evb_set_error("evb_grow_tree: js must be strictly ascending within 1..nfeats");
            return EVB_ERR_ARG;
        }
        h->h_js[slot][i] = js[i] - 1;
    }
    if (h->world > 1) EVB_CHECK(evb_nccl_check(h));
    if (njs != h->F && h->use_q2) { // this kernel always accumulates all features; the scan reads the sampled ones
        EVB_CUDA(cudaStreamSynchronize(h->st));
        h->F = njs;
        drop_graphs(h);
    }
    if (njs != h->F) {
        HistGeom g;
        EVB_CUDA(cudaStreamSynchronize(h->st));
        h->F = njs;
        EVB_CHECK(evb_hist_geometry(h, njs, &g));
        const size_t need = (size_t)g.NUG * g.PG * g.UB * g.img_floats;
        if (need > h->scratch_floats) {
            evb_dev_free(h->scratch);
            h->scratch = nullptr;
            EVB_CUDA(dalloc(&h->scratch, need));
            h->scratch_floats = need;
        }
        h->hg = g;
        h->q_active = g.q;
        drop_graphs(h);
    }
    if (update_grads) h->bag_idx = 0;
    const bool run_grads = update_grads && !h->grads_fresh;
    const bool fuse = h->bag_idx == h->p.bagging_size - 1;
    const bool use_mask = row_mask != nullptr;
    if (h->timing) {
        if (!h->ev_tot[0]) { EVB_CUDA(cudaEventCreate(&h->ev_tot[0])); EVB_CUDA(cudaEventCreate(&h->ev_tot[1])); }
        cudaEventRecord(h->ev_tot[0], h->st);
    }
    if (use_mask) {
        evb_tic(h, EVB_T_H2D);
        EVB_CUDA(cudaMemcpyAsync(h->mask_d, row_mask, (size_t)h->n, cudaMemcpyHostToDevice, h->st));
        evb_toc(h, EVB_T_H2D);
        h->tm.launches[EVB_T_H2D] -= 1; // a copy, not a kernel
    }
    // One CUDA graph per variant of the launch sequence, captured on the second call of a variant (the first
    // one runs directly: it also sets function attributes).  Per-kernel timing needs the direct path.
    if (update_grads) h->gradq_valid = false;
    const bool quantize = (h->q_active || h->use_q2) && !h->gradq_valid;
    if (quantize) h->gradq_valid = true;
    const int key = (use_mask ? 1 : 0) | (run_grads ? 2 : 0) | (fuse ? 4 : 0) | (slot ? 8 : 0) | (quantize ? 16 : 0);
    if (h->graph_mask_cond != (int)mask_cond) { drop_graphs(h); h->graph_mask_cond = mask_cond; }
    bool launched = false;
    // Sharded runs over NCCL stay on direct launches: a run that captured the NCCL collectives into the graph did not
    // complete on 2 GPUs, so collectives are never captured.  With peer access the exchange is made of this
    // library's own kernels (the barrier counts on the device), which replay like any other.
    // (The quantile losses add their leaves' digit counts with NCCL on every sharded path.)
    const bool quantile_leaves = h->p.loss == EVB_QUANTILE || h->p.loss == EVB_MULTIQUANTILE;
    if (h->use_graphs && !h->timing && (h->world == 1 || (h->p2p && !quantile_leaves))) {
        if (!h->graph[key] && h->tree_seq >= 1) { // the very first tree of a handle always runs directly
            int64_t before[EVB_NTIMERS];
            memcpy(before, h->tm.launches, sizeof(before));
            cudaGraph_t g = nullptr;
            cudaError_t e = cudaStreamBeginCapture(h->st, cudaStreamCaptureModeThreadLocal);
            int32_t rc = e == cudaSuccess ? enqueue_tree(h, use_mask, mask_cond, run_grads, quantize, fuse, slot) : EVB_ERR_CUDA;
            cudaError_t e2 = cudaStreamEndCapture(h->st, &g);
            for (int i = 0; i < EVB_NTIMERS; ++i) { h->graph_launches[key][i] = h->tm.launches[i] - before[i]; h->tm.launches[i] = before[i]; }
            if (rc == EVB_OK && e2 == cudaSuccess && g && cudaGraphInstantiate(&h->graph[key], g, 0) == cudaSuccess) {
                cudaGraphDestroy(g);
            } else {
                if (g) cudaGraphDestroy(g);
                h->graph[key] = nullptr;
                h->use_graphs = false; // capture is not possible here (e.g. an NCCL build without graph support): stay direct
                cudaGetLastError();
            }
        }
        if (h->graph[key]) {
            EVB_CUDA(cudaGraphLaunch(h->graph[key], h->st));
            for (int i = 0; i < EVB_NTIMERS; ++i) h->tm.launches[i] += h->graph_launches[key][i];
            launched = true;
        }
    }
    if (!launched) EVB_CHECK(enqueue_tree(h, use_mask, mask_cond, run_grads, quantize, fuse, slot));
    h->graph_calls[key] += 1;
    if (h->timing) cudaEventRecord(h->ev_tot[1], h->st);
    EVB_CUDA(cudaEventRecord(h->ev_done[slot], h->st));
    h->grads_fresh = fuse;
    h->bag_idx += 1;
    h->tree_seq += 1;
    h->pending += 1;
    return EVB_OK;
}

extern "C" int32_t evb_grow_tree_end(evb_handle *h, int64_t *feat, uint8_t *cond_bin, float *w_node, float *gain, float *leaf_pred,
                                     uint8_t *split) {
    EVB_ENTER(h);
    if (!feat || !cond_bin || !w_node || !gain || !leaf_pred || !split) { evb_set_error("evb_grow_tree_end: null output"); return EVB_ERR_ARG; }
    if (h->pending < 1) { evb_set_error("evb_grow_tree_end: no tree in flight"); return EVB_ERR_ARG; }
    const int slot = (h->tree_seq - h->pending) & 1;
    EVB_CUDA(cudaEventSynchronize(h->ev_done[slot]));
    h->pending -= 1;
    if (h->pending == 0) resolve_timing(h);
    const int D = h->D, last = D > 1 ? D - 1 : 1;
    const TreeBlockLayout L = tree_block_layout(D, h->nn, h->K);
    const unsigned char *hb = (const unsigned char *)h->h_tree[slot];
    const int derr = *(const int *)(hb + L.err);
    if (derr != EVB_DERR_NONE) {
        evb_set_error("device self-check failed (code %d: %s)", derr,
                      derr == EVB_DERR_WAIT_FULL ? "bounded wait for staged rows expired"
                      : derr == EVB_DERR_WAIT_EMPTY ? "bounded wait for a free stage expired"
                      : derr == EVB_DERR_PLAN ? "work list overflow"
                      : derr == EVB_DERR_PEER ? "bounded wait for the other ranks expired" : "unknown");
        cudaMemsetAsync(h->d_err, 0, sizeof(int), h->st);
        return EVB_ERR_DEVICE;
    }
    memcpy(h->last_eval, hb + L.evsum, sizeof(h->last_eval));
    const LevelPlan *hp = (const LevelPlan *)(hb + L.plan);
    if (hp[1].n_sel == 0 && h->world == 1) {
        evb_set_error("no subsample observation - choose larger rowsample");
        return EVB_ERR_EMPTY;
    }
    for (int level = 1; level <= last; ++level) { h->tm.hist_rows += hp[level].R; h->tm.hist_nodes += hp[level].nbuild; }
    h->tm.trees += 1;
    const int nn = h->nn;
    const int32_t *tf = (const int32_t *)(hb + L.feat);
    for (int i = 0; i < nn; ++i) feat[i] = tf[i];
    memcpy(gain, hb + L.gain, sizeof(float) * nn);
    memcpy(w_node, hb + L.w, sizeof(float) * nn);
    memcpy(leaf_pred, hb + L.pred, sizeof(float) * nn * h->K);
    memcpy(cond_bin, hb + L.bin, nn);
    memcpy(split, hb + L.split, nn);
    return EVB_OK;
}

extern "C" int32_t evb_grow_tree(evb_handle *h, const uint8_t *row_mask, uint8_t mask_cond, const uint32_t *js, int32_t njs,
                                 int32_t update_grads, int64_t *feat, uint8_t *cond_bin, float *w_node, float *gain,
                                 float *leaf_pred, uint8_t *split) {
    if (!feat || !cond_bin || !w_node || !gain || !leaf_pred || !split) { evb_set_error("evb_grow_tree: invalid argument"); return EVB_ERR_ARG; }
    if (h && h->pending > 0) { evb_set_error("evb_grow_tree: a tree started with evb_grow_tree_begin is still in flight"); return EVB_ERR_BUSY; }
    EVB_CHECK(evb_grow_tree_begin(h, row_mask, mask_cond, js, njs, update_grads));
    return evb_grow_tree_end(h, feat, cond_bin, w_node, gain, leaf_pred, split);
}

// ---- evaluation data on the device ---------------------------------------------------------------------------
static int32_t eval_attach_impl(evb_handle *h, int64_t nobs, const uint8_t *x_bin, const void *y, const float *w, const float *pred0,
                                const float *bias, int32_t metric, double sums[2]) {
    const int K = h->K;
    h->ev_metric = metric;
    h->ev_blocks = (int)std::min<int64_t>((nobs + 255) / 256, (int64_t)h->num_sms * 8);
    EVB_CUDA(dalloc(&h->ev_xT, (size_t)nobs * h->RS));
    EVB_CUDA(dalloc(&h->ev_pred, (size_t)nobs * K));
    EVB_CUDA(dalloc(&h->ev_part, (size_t)h->ev_blocks * 2));
    const size_t ybytes = (size_t)nobs * (h->y_dtype == EVB_U32 ? 4 : 4 * (size_t)h->ycols);
    EVB_CUDA(evb_dev_alloc(&h->ev_y, ybytes));
    EVB_CUDA(cudaMemcpyAsync(h->ev_y, y, ybytes, cudaMemcpyHostToDevice, h->st));
    if (w) {
        EVB_CUDA(dalloc(&h->ev_w, (size_t)nobs));
        EVB_CUDA(cudaMemcpyAsync(h->ev_w, w, sizeof(float) * nobs, cudaMemcpyHostToDevice, h->st));
    }
    if (pred0) EVB_CUDA(cudaMemcpyAsync(h->ev_pred, pred0, sizeof(float) * nobs * K, cudaMemcpyHostToDevice, h->st));
    else EVB_CUDA(cudaMemsetAsync(h->ev_pred, 0, sizeof(float) * nobs * K, h->st));
    // feature-major upload -> observation-major rows, column block by column block through a bounded staging buffer
    EVB_CUDA(cudaMemsetAsync(h->ev_xT, 0, (size_t)nobs * h->RS, h->st));
    uint8_t *stage = nullptr;
    float *leaf_d = nullptr;
    const int jb = (int)std::max<int64_t>(1, std::min<int64_t>(h->nfeats, ((int64_t)256 << 20) / nobs));
    EVB_CUDA(dalloc(&stage, (size_t)jb * nobs));
    int32_t rc = EVB_OK;
    for (int j0 = 0; j0 < h->nfeats && rc == EVB_OK; j0 += jb) {
        const int nj = std::min(jb, h->nfeats - j0);
        if (cudaMemcpyAsync(stage, x_bin + (size_t)j0 * nobs, (size_t)nj * nobs, cudaMemcpyHostToDevice, h->st) != cudaSuccess) rc = EVB_ERR_CUDA;
        if (rc == EVB_OK) rc = evb_launch_transpose(h, stage, nobs, nobs, j0, nj, h->ev_xT, h->RS, h->st);
    }
    h->ev_n = nobs;
    if (rc == EVB_OK) {
        // iteration 0: `cb(logger, 0, m.trees[end])` applies the bias tree (src/fit.jl:416); a model without one adds zeros
        std::vector<float> leaf(K, 0.0f);
        if (bias) memcpy(leaf.data(), bias, sizeof(float) * K);
        if (dalloc(&leaf_d, (size_t)K) != cudaSuccess || cudaMemcpyAsync(leaf_d, leaf.data(), sizeof(float) * K, cudaMemcpyHostToDevice, h->st) != cudaSuccess) rc = EVB_ERR_CUDA;
        if (rc == EVB_OK) rc = evb_launch_eval(h, leaf_d);
        if (rc == EVB_OK && cudaMemcpyAsync(h->last_eval, h->d_evsum, sizeof(h->last_eval), cudaMemcpyDeviceToHost, h->st) != cudaSuccess) rc = EVB_ERR_CUDA;
    }
    cudaError_t e = cudaStreamSynchronize(h->st);
    evb_dev_free(stage);
    evb_dev_free(leaf_d);
    if (rc == EVB_ERR_CUDA || e != cudaSuccess) {
        evb_set_error("evb_eval_attach: CUDA error %s", cudaGetErrorString(e != cudaSuccess ? e : cudaGetLastError()));
        return EVB_ERR_CUDA;
    }
    EVB_CHECK(rc);
    sums[0] = h->last_eval[0]; sums[1] = h->last_eval[1];
    return EVB_OK;
}

extern "C" int32_t evb_eval_attach(evb_handle *h, int64_t nobs, const uint8_t *x_bin, const void *y, const float *w, const float *pred0,
                                   const float *bias, int32_t metric, double sums[2]) {
    EVB_ENTER(h);
    if (!x_bin || !y || !sums || nobs < 1 || nobs > 2000000000ll) { evb_set_error("evb_eval_attach: invalid argument"); return EVB_ERR_ARG; }
    if (h->pending > 0) { evb_set_error("evb_eval_attach: a tree is still in flight"); return EVB_ERR_BUSY; }
    if (h->ev_n > 0) { evb_set_error("evb_eval_attach: evaluation data already attached (evb_eval_detach first)"); return EVB_ERR_ARG; }
    const int loss = h->p.loss;
    const bool ok = (loss == EVB_MLOGLOSS) ? metric == EVB_METRIC_MLOGLOSS
                    : (loss == EVB_GAUSSIAN_MLE || loss == EVB_LOGISTIC_MLE) ? (metric == EVB_METRIC_GAUSSIAN_MLE || metric == EVB_METRIC_LOGISTIC_MLE)
                    : (metric == EVB_METRIC_MSE || metric == EVB_METRIC_MAE || metric == EVB_METRIC_LOGLOSS ||
                       metric == EVB_METRIC_POISSON || metric == EVB_METRIC_GAMMA || metric == EVB_METRIC_TWEEDIE ||
                       metric == EVB_METRIC_QUANTILE || (metric == EVB_METRIC_MULTIQUANTILE && loss == EVB_MULTIQUANTILE));
    if (!ok) { evb_set_error("evb_eval_attach: metric %d is not defined for loss %d", metric, loss); return EVB_ERR_ARG; }
    drop_graphs(h); // the launch sequence of a tree changes
    int32_t rc = eval_attach_impl(h, nobs, x_bin, y, w, pred0, bias, metric, sums);
    if (rc != EVB_OK) free_eval(h);
    return rc;
}

extern "C" int32_t evb_eval_sums(evb_handle *h, double sums[2]) {
    EVB_ENTER(h);
    if (!sums) { evb_set_error("evb_eval_sums: null output"); return EVB_ERR_ARG; }
    if (h->ev_n == 0) { evb_set_error("evb_eval_sums: no evaluation data attached"); return EVB_ERR_ARG; }
    sums[0] = h->last_eval[0]; sums[1] = h->last_eval[1];
    return EVB_OK;
}

extern "C" int32_t evb_eval_get_pred(evb_handle *h, float *pred) {
    EVB_ENTER(h);
    if (!pred || h->ev_n == 0) { evb_set_error("evb_eval_get_pred: no evaluation data attached or null output"); return EVB_ERR_ARG; }
    EVB_CUDA(cudaMemcpyAsync(pred, h->ev_pred, sizeof(float) * h->ev_n * h->K, cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    return EVB_OK;
}

extern "C" int32_t evb_eval_detach(evb_handle *h) {
    EVB_ENTER(h);
    if (h->pending > 0) { evb_set_error("evb_eval_detach: a tree is still in flight"); return EVB_ERR_BUSY; }
    EVB_CUDA(cudaStreamSynchronize(h->st));
    drop_graphs(h);
    free_eval(h);
    return EVB_OK;
}

// ---- peer access between the ranks' processes (CUDA IPC) -----------------------------------------------------
struct IpcBlob { cudaIpcMemHandle_t hcomp, cand, flags; };
static_assert(sizeof(IpcBlob) <= 256, "blob size");

extern "C" int32_t evb_comm_ipc_export(evb_handle *h, uint8_t blob[256]) {
    EVB_ENTER(h);
    if (!blob) { evb_set_error("null blob"); return EVB_ERR_ARG; }
    if (h->world < 2 || h->world > 8) { evb_set_error("evb_comm_ipc_export: needs evb_comm_init with 2..8 ranks first"); return EVB_ERR_ARG; }
    if (h->p2p || h->peer_cand[h->rank]) { evb_set_error("evb_comm_ipc_export: already exported"); return EVB_ERR_ARG; }
    EVB_CUDA(cudaStreamSynchronize(h->st));
    const int D = h->D;
    // every scanned node keeps the summed histogram of the features this rank owns (children subtract from it)
    const int keep_nodes = 1 << (D > 1 ? D - 1 : 0);
    if (keep_nodes > h->hist_nodes) {
        evb_dev_free(h->hist);
        h->hist = nullptr;
        EVB_CUDA(dalloc(&h->hist, (size_t)keep_nodes * h->nfeats * h->C * h->B));
        h->hist_nodes = keep_nodes;
    }
    EVB_CUDA(dalloc(&h->hsum, (size_t)h->maxslots * h->nfeats * h->C * h->B));
    double *cand = nullptr;
    int *flags = nullptr;
    const size_t ncand = (size_t)keep_nodes * h->world * (3 + h->C);
    EVB_CUDA(dalloc(&cand, ncand));
    EVB_CUDA(cudaMemset(cand, 0, ncand * sizeof(double)));
    EVB_CUDA(dalloc(&flags, (size_t)8));
    EVB_CUDA(cudaMemset(flags, 0, 8 * sizeof(int)));
    h->peer_hcomp[h->rank] = h->hcomp; h->peer_cand[h->rank] = cand; h->peer_flags[h->rank] = flags;
    EVB_CUDA(dalloc(&h->d_barrier_seq, (size_t)1));
    EVB_CUDA(cudaMemset(h->d_barrier_seq, 0, sizeof(int)));
    IpcBlob b;
    memset(&b, 0, sizeof(b));
    EVB_CUDA(cudaIpcGetMemHandle(&b.hcomp, h->hcomp));
    EVB_CUDA(cudaIpcGetMemHandle(&b.cand, cand));
    EVB_CUDA(cudaIpcGetMemHandle(&b.flags, flags));
    memset(blob, 0, 256);
    memcpy(blob, &b, sizeof(b));
    return EVB_OK;
}

extern "C" int32_t evb_comm_ipc_import(evb_handle *h, const uint8_t *blobs) {
    EVB_ENTER(h);
    if (!blobs) { h->p2p = false; return EVB_OK; } // the ranks agreed not to use peer access: stay on the NCCL path
    if (!h->peer_cand[h->rank]) { evb_set_error("evb_comm_ipc_import: call evb_comm_ipc_export first"); return EVB_ERR_ARG; }
    for (int q = 0; q < h->world; ++q) {
        if (q == h->rank) continue;
        IpcBlob b;
        memcpy(&b, blobs + (size_t)q * 256, sizeof(b));
        void *p[3] = {nullptr, nullptr, nullptr};
        const cudaIpcMemHandle_t hs[3] = {b.hcomp, b.cand, b.flags};
        for (int k = 0; k < 3; ++k) {
            cudaError_t e = cudaIpcOpenMemHandle(&p[k], hs[k], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                evb_set_error("cannot map rank %d's buffers (%s): peer access between the GPUs is required", q, cudaGetErrorString(e));
                return EVB_ERR_CUDA;
            }
            h->ipc_opened[h->n_ipc_opened++] = p[k];
        }
        h->peer_hcomp[q] = (double *)p[0]; h->peer_cand[q] = (double *)p[1]; h->peer_flags[q] = (int *)p[2];
    }
    h->p2p = true;
    return EVB_OK;
}

extern "C" int32_t evb_test_peer_timeout(evb_handle *h, int32_t max_polls) {
    EVB_ENTER(h);
    if (max_polls < 1 || max_polls > 20000000) { evb_set_error("evb_test_peer_timeout: max_polls outside 1..20000000"); return EVB_ERR_ARG; }
    if (h->pending > 0) { evb_set_error("evb_test_peer_timeout: a tree is in flight"); return EVB_ERR_BUSY; }
    int *flags = nullptr;
    EVB_CUDA(cudaMalloc((void **)&flags, 16 * sizeof(int)));
    int derr = 0;
    cudaError_t e = cudaMemsetAsync(flags, 0, 16 * sizeof(int), h->st);
    int32_t rc = e == cudaSuccess ? evb_launch_lonely_barrier(h, flags, flags + 8, (unsigned)max_polls) : EVB_ERR_CUDA;
    if (rc == EVB_OK) e = cudaMemcpyAsync(&derr, h->d_err, sizeof(int), cudaMemcpyDeviceToHost, h->st);
    if (rc == EVB_OK && e == cudaSuccess) e = cudaStreamSynchronize(h->st);
    cudaMemsetAsync(h->d_err, 0, sizeof(int), h->st); // the handle stays usable
    cudaStreamSynchronize(h->st);
    cudaFree(flags);
    if (rc != EVB_OK || e != cudaSuccess) { evb_set_error("evb_test_peer_timeout: CUDA error %s", cudaGetErrorString(e)); return EVB_ERR_CUDA; }
    if (derr == EVB_DERR_PEER) { evb_set_error("device self-check failed (code %d: bounded wait for the other ranks expired)", derr); return EVB_ERR_DEVICE; }
    evb_set_error("evb_test_peer_timeout: the wait did not run out (error word %d)", derr);
    return EVB_ERR_ARG;
}

extern "C" int32_t evb_set_timing(evb_handle *h, int32_t on) {
    EVB_ENTER(h);
    if (h->pending > 0) { evb_set_error("evb_set_timing: a tree is in flight"); return EVB_ERR_BUSY; }
    h->timing = on != 0;
    return EVB_OK;
}

extern "C" int32_t evb_get_pred(evb_handle *h, float *pred) {
    EVB_ENTER(h);
    if (!pred) { evb_set_error("null output"); return EVB_ERR_ARG; }
    EVB_CUDA(cudaMemcpyAsync(pred, h->pred, sizeof(float) * h->n * h->K, cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    return EVB_OK;
}

extern "C" int32_t evb_get_grads(evb_handle *h, float *grad) {
    EVB_ENTER(h);
    if (!grad) { evb_set_error("null output"); return EVB_ERR_ARG; }
    // the device keeps padded records of GS floats (channel c at (c / NCH) * 4 + c % NCH); the reference
    // layout is [C x nobs]
    std::vector<float> tmp((size_t)h->n * h->GS);
    EVB_CUDA(cudaMemcpyAsync(tmp.data(), h->grad, sizeof(float) * tmp.size(), cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    const int NCH = h->rec_nch, C = h->C, GS = h->GS, K = h->K;
    const bool elided = h->Ce != h->C; // mse: records hold g_1..g_K, w; h_k = 2w
    for (int64_t i = 0; i < h->n; ++i) {
        const float *rec = tmp.data() + (size_t)i * GS;
        for (int c = 0; c < C; ++c) {
            float v;
            if (!elided) v = rec[(c / NCH) * 4 + (c % NCH)];
            else if (c < K) v = rec[(c / NCH) * 4 + (c % NCH)];
            else { const float w = rec[(K / NCH) * 4 + (K % NCH)]; v = c < 2 * K ? 2.0f * w : w; }
            grad[(size_t)i * C + c] = v;
        }
    }
    return EVB_OK;
}

extern "C" int32_t evb_get_nidx(evb_handle *h, uint32_t *nidx, int32_t from_partition) {
    EVB_ENTER(h);
    if (!nidx) { evb_set_error("null output"); return EVB_ERR_ARG; }
    if (from_partition) {
        if (!(h->p.flags & EVB_FLAG_FULL_PARTITION)) {
            evb_set_error("evb_get_nidx(from_partition=1) needs EVB_FLAG_FULL_PARTITION (the last level is otherwise not partitioned)");
            return EVB_ERR_ARG;
        }
        uint32_t *tmp = nullptr;
        EVB_CUDA(dalloc(&tmp, (size_t)h->n));
        int32_t rc = evb_launch_nidx_from_partition(h, tmp);
        if (rc == EVB_OK) {
            cudaError_t e = cudaMemcpyAsync(nidx, tmp, sizeof(uint32_t) * h->n, cudaMemcpyDeviceToHost, h->st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(h->st);
            if (e != cudaSuccess) { evb_set_error("CUDA error %s", cudaGetErrorString(e)); rc = EVB_ERR_CUDA; }
        }
        evb_dev_free(tmp);
        return rc;
    }
    EVB_CUDA(cudaMemcpyAsync(nidx, h->nidx, sizeof(uint32_t) * h->n, cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    return EVB_OK;
}

extern "C" int32_t evb_get_hist(evb_handle *h, int32_t node, double *hist) {
    EVB_ENTER(h);
    if (!hist || node < 1 || node >= h->hist_nodes) {
        evb_set_error("evb_get_hist: node %d is not retained (nodes 1..%d are)", node, h->hist_nodes - 1);
        return EVB_ERR_ARG;
    }
    const int F = h->F, C = h->C, B = h->B;
    const size_t FCB = (size_t)F * C * B;
    std::vector<double> tmp(FCB);
    EVB_CUDA(cudaMemcpyAsync(tmp.data(), h->hist + (size_t)node * FCB, sizeof(double) * FCB, cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    for (int f = 0; f < F; ++f)
        for (int c = 0; c < C; ++c)
            for (int b = 0; b < B; ++b) hist[c + (size_t)C * (b + (size_t)B * f)] = tmp[((size_t)f * C + c) * B + b];
    return EVB_OK;
}

extern "C" int32_t evb_get_node_sums(evb_handle *h, double *nsum) {
    EVB_ENTER(h);
    if (!nsum) { evb_set_error("null output"); return EVB_ERR_ARG; }
    EVB_CUDA(cudaMemcpyAsync(nsum, h->nsum + h->C, sizeof(double) * h->C * h->nn, cudaMemcpyDeviceToHost, h->st));
    EVB_CUDA(cudaStreamSynchronize(h->st));
    return EVB_OK;
}

extern "C" int32_t evb_get_stream(evb_handle *h, void **stream) {
    if (!h || !stream) { evb_set_error("null argument"); return EVB_ERR_ARG; }
    *stream = (void *)h->st;
    return EVB_OK;
}

extern "C" int32_t evb_get_timings(evb_handle *h, evb_timings *out) {
    EVB_ENTER(h);
    if (!out) { evb_set_error("null output"); return EVB_ERR_ARG; }
    *out = h->tm;
    return EVB_OK;
}

extern "C" int32_t evb_reset_timings(evb_handle *h) {
    EVB_ENTER(h);
    memset(&h->tm, 0, sizeof(h->tm));
    return EVB_OK;
}
