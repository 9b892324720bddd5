/*
 * evb.h -- C ABI of libevotrees_b200.so: the EvoTrees training / inference hot path as hand-written
 * sm_100a CUDA kernels.
 *
 * The library takes the place of the reference's GPU extension (ext/EvoTreesKernelAbstractionsExt/
 * behind ext/EvoTreesCUDAExt.jl).  Host glue (Julia through `ccall`, or the Python mirror shipped in
 * this repository) keeps everything that the reference keeps on the host: learner structs, the RNG
 * (row mask bytes, column samples), quantile edges, the initial bias and the `Tree` / `EvoTree`
 * containers.  The library owns all device memory behind an opaque handle.
 *
 * Conventions
 *   - every function returns 0 on success and a negative `evb_status` otherwise; a message for the
 *     last failure of the calling thread is available from evb_last_error();
 *   - host arrays are caller-owned and only touched during the call;
 *   - matrices use the reference's (Julia, column-major) layout; feature ids, node ids, class codes
 *     and bins are 1-based at this boundary exactly as in the reference's `Tree` fields;
 *   - one handle = one GPU = one shard of rows.  A handle must be used by one host thread at a time.
 *   - there is no CPU fallback: every entry point fails with EVB_ERR_CUDA when no sm_100 GPU is usable.
 */
#ifndef EVB_H
#define EVB_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EVB_API __attribute__((visibility("default")))
#else
#define EVB_API
#endif

typedef struct evb_handle evb_handle;

enum evb_status {
    EVB_OK = 0,
    EVB_ERR_ARG = -1,      /* invalid argument                                   */
    EVB_ERR_CUDA = -2,     /* CUDA runtime error (message has the CUDA string)   */
    EVB_ERR_NCCL = -3,     /* NCCL error or NCCL not loadable                    */
    EVB_ERR_EMPTY = -4,    /* row subsample selected no row (src/subsample.jl:36) */
    EVB_ERR_DEVICE = -5,   /* a kernel reported a failed self-check / bounded wait */
    EVB_ERR_BUSY = -6,     /* handle used concurrently                           */
    EVB_ERR_LIMIT = -7     /* size beyond a documented limit                     */
};

/* 0..3: the losses of the reference's GPU benchmark configurations; 4..7: the other gradient-regression and two-parameter
 * likelihood losses of src/loss.jl:65-84, 207-217 (poisson, gamma, tweedie with rho = 1.5: log link; logistic_mle);
 * 8..10: mae and the two credibility losses, whose split gain and leaf value are their own (src/split.jl:2-4, 119-145,
 * src/predict.jl:211-223, 250-262); 11: quantile (evb_params.alpha), the gain of mae and leaf values that are the
 * alpha-quantile of the residuals of the leaf's sampled rows (src/loss.jl:93-98, src/predict.jl:264-272) */
enum evb_loss { EVB_MSE = 0, EVB_LOGLOSS = 1, EVB_MLOGLOSS = 2, EVB_GAUSSIAN_MLE = 3,
                EVB_POISSON = 4, EVB_GAMMA = 5, EVB_TWEEDIE = 6, EVB_LOGISTIC_MLE = 7,
                EVB_MAE = 8, EVB_CRED_VAR = 9, EVB_CRED_STD = 10, EVB_QUANTILE = 11,
                EVB_MULTIQUANTILE = 12 /* one target, K = number of quantiles evb_params.alphas[0..K-1], K <= 8 (src/loss.jl:160-172) */ };
#define EVB_LOSS_LAST EVB_MULTIQUANTILE
enum evb_dtype { EVB_F32 = 0, EVB_U32 = 1, EVB_F64 = 2 };

/* flags of evb_params.flags */
#define EVB_FLAG_TIMING 1u         /* record a CUDA-event pair (and an NVTX range) around every kernel class (see evb_get_timings) */
#define EVB_FLAG_FULL_PARTITION 2u /* also partition the rows of the last split level (only evb_get_nidx(.., 1) reads that) */
#define EVB_FLAG_KEEP_ALL_HIST 4u  /* retain the histograms of the last split level too (for evb_get_hist)               */

/* Learner hyper-parameters needed on the device; filled by the glue from the reference's learner
 * struct (src/learners.jl:1-23).  K is the number of prediction rows (1 mse/logloss/poisson/gamma/tweedie, #classes for
 * mlogloss, 2 for gaussian_mle / logistic_mle); histogram channels are C = 2K+1 (g_1..g_K, h_1..h_K, w). */
typedef struct {
    int32_t loss;          /* enum evb_loss */
    int32_t K;
    int32_t nbins;         /* 2..255 */
    int32_t max_depth;     /* 1..15 */
    int32_t bagging_size;  /* >= 1 */
    int32_t tree_type;     /* 0 = binary, 1 = oblivious (one split per depth, src/fit.jl:147-263) */
    double eta, lambda, L2, gamma, min_weight;
    int32_t device;        /* CUDA device ordinal of this shard */
    uint32_t flags;
    double alpha;          /* quantile loss / metric: the target quantile in (0, 1) (src/learners.jl:44); else unused */
    double alphas[8];      /* multiquantile loss / metric: the K target quantiles (src/learners.jl:45); else unused */
} evb_params;

/* Accumulated device time per kernel class since the last evb_reset_timings (EVB_FLAG_TIMING). */
#define EVB_NTIMERS 12
enum evb_timer {
    EVB_T_GRADS = 0, EVB_T_ROWS_INIT = 1, EVB_T_HIST = 2, EVB_T_HIST_REDUCE = 3, EVB_T_ALLREDUCE = 4,
    EVB_T_SCAN = 5, EVB_T_PARTITION = 6, EVB_T_PLAN = 7, EVB_T_FINALIZE = 8, EVB_T_D2H = 9,
    EVB_T_H2D = 10, EVB_T_TREE_TOTAL = 11
};
typedef struct {
    double ms[EVB_NTIMERS];        /* summed kernel time, milliseconds                                    */
    int64_t launches[EVB_NTIMERS]; /* kernels launched in that class                                      */
    int64_t hist_rows;             /* rows streamed by the histogram kernel (sum over levels and trees)   */
    int64_t hist_nodes;            /* histograms built (build nodes, sum over levels and trees)           */
    int64_t trees;                 /* trees grown                                                         */
} evb_timings;

EVB_API const char *evb_last_error(void);
EVB_API int32_t evb_version(void);

/*
 * evb_create -- replaces `init_core(params, ::Type{<:GPU}, ...)` (ext/EvoTreesKernelAbstractionsExt/init.jl:1-151):
 * uploads the binned matrix, targets, weights and initial predictions of this shard and allocates all
 * training state.
 *   x_bin      host, uint8 [nobs x nfeats] column-major, values 1..nbins (binarize, src/fit-utils.jl:66-72)
 *   y          host; EVB_F32 [ycols x nobs] (ycols = 1 for a vector target) or EVB_U32 class codes 1..K
 *   w          host float [nobs], > 0, or NULL for ones       (src/init.jl:173-174)
 *   pred0      host float [K x nobs] initial predictions (mu + offset), or NULL with mu != NULL
 *   mu         host float [K] used when pred0 == NULL         (src/init.jl:168-170)
 *   feattypes  host uint8 [nfeats], 1 = numeric (<=), 0 = categorical (==); NULL = all numeric
 *   monotone   host int32 [nfeats] in {-1,0,1}; NULL = none   (src/init.jl:184-187)
 */
EVB_API int32_t evb_create(evb_handle **out, const evb_params *p, int64_t nobs, int32_t nfeats, const uint8_t *x_bin,
                   const void *y, int32_t y_dtype, int32_t ycols, const float *w, const float *pred0, const float *mu,
                   const uint8_t *feattypes, const int32_t *monotone);
/*
 * evb_create_x -- the same with `binarize` included, as `init_core` does it (ext/EvoTreesKernelAbstractionsExt/init.jl:3-12:
 * `get_edges` on the host, then `binarize(x_train; edges)`): the raw feature matrix is streamed to the device in blocks of
 * whole features and binarized there (`searchsortedfirst`, src/fit-utils.jl:66-72) straight into the training layouts; the
 * bins never visit the host.  A NaN in x fails the call (missing values are rejected, test/missings.jl).
 *   x       host, EVB_F32 / EVB_F64, column-major [nobs x nfeats]; ordinary (pageable) memory is fine: it is staged
 *           through pinned buffers by several host threads
 *   edges   host [nedges x nfeats] column-major, same dtype as x, ascending per feature; nedges = nbins - 1
 * All other arguments as evb_create.
 */
EVB_API int32_t evb_create_x(evb_handle **out, const evb_params *p, int64_t nobs, int32_t nfeats, const void *x, int32_t x_dtype,
                             const void *edges, int32_t nedges, const void *y, int32_t y_dtype, int32_t ycols, const float *w,
                             const float *pred0, const float *mu, const uint8_t *feattypes, const int32_t *monotone);
EVB_API void evb_destroy(evb_handle *h);
/*
 * Device memory released by evb_destroy and by the inference calls is kept by the library and reused by the next
 * evb_create* / evb_predict* of about the same size (cudaMalloc and cudaFree take driver-wide locks: a second `fit` of
 * the same shape then makes no allocator call).  The reference leaves this to CUDA.jl's memory pool and to
 * `post_fit_gc` (ext/EvoTreesCUDAExt.jl:7-12).  evb_trim_cache gives the kept blocks of one GPU back to the driver; the
 * library does so by itself when an allocation fails, and never keeps more than half of the device's memory
 * (EVB_CACHE_MAX_GB).  EVB_CACHE=0 in the environment turns the cache off.
 */
EVB_API int32_t evb_trim_cache(int32_t device);

/*
 * Row sharding over several GPUs (one handle per GPU, normally one process per GPU).  Rank 0 obtains an
 * id, the host distributes its 128 bytes (any channel), then every rank calls evb_comm_init.  After that
 * evb_grow_tree sums the per-level histograms over all ranks with NCCL, so every rank grows the identical tree.  The reference has no counterpart: it is single-GPU
 * (ext/EvoTreesCUDAExt.jl:7-12).  All ranks must call evb_grow_tree with the same js / update_grads.
 */
EVB_API int32_t evb_comm_unique_id(uint8_t id[128]);
EVB_API int32_t evb_comm_init(evb_handle *h, const uint8_t id[128], int32_t rank, int32_t world);
/*
 * Optional second step for ranks that are separate processes on one NVLink / NVSwitch node (2..8 ranks): every
 * rank exports a 256-byte blob (CUDA IPC handles of its per-level histogram buffer, candidate table and barrier
 * flags), the host gathers the blobs of all ranks in rank order, every rank imports them.  From then on the NCCL
 * all-reduce per level is replaced by peer loads inside the split scan: rank r scans the feature slots
 * f % world == r, summing the ranks' histograms straight from their memory in rank order, and writes its best
 * candidate per node into every rank's table; bounded flag barriers separate the phases.
 */
EVB_API int32_t evb_comm_ipc_export(evb_handle *h, uint8_t blob[256]);
EVB_API int32_t evb_comm_ipc_import(evb_handle *h, const uint8_t *blobs /* world x 256 bytes; NULL = do not use peer access */);

/*
 * evb_grow_tree -- replaces one bag iteration of `grow_evotree!(m, cache::CacheGPU, params)`
 * (ext/EvoTreesKernelAbstractionsExt/fit.jl:1-21): [update_grads!] + subsample + grow_tree! + predict!.
 *   row_mask     host uint8 [nobs] (the bytes of `rand!(rng, mask)`), rows with mask <= mask_cond are
 *                sampled (ext/.../subsample.jl:2-8); NULL = all rows
 *   js           host uint32 [njs], 1-based ascending sampled feature ids (ext/.../fit.jl:8-10)
 *   update_grads 1 on the first bag of a boosting round (`update_grads!`, ext/.../loss.jl)
 * Outputs, host, length nn = 2^max_depth - 1, laid out as the fields of `Tree{L,K}` (src/structs.jl:77-84):
 *   feat int64 (0 = none), cond_bin uint8 (0 = none), w float, gain float, leaf_pred float [K x nn], split uint8.
 */
EVB_API int32_t evb_grow_tree(evb_handle *h, const uint8_t *row_mask, uint8_t mask_cond, const uint32_t *js, int32_t njs,
                      int32_t update_grads, int64_t *feat, uint8_t *cond_bin, float *w_node, float *gain,
                      float *leaf_pred, uint8_t *split);

/*
 * The same call split in two, so that the host can enqueue tree t+1 while the GPU still works on tree t (the
 * reference's loop is strictly sequential: ext/.../fit.jl:296-300 reads the tree back before `predict!`).
 * evb_grow_tree_begin enqueues one tree and returns at once; evb_grow_tree_end waits for the oldest tree in
 * flight and writes its arrays.  At most two trees may be in flight.  After the first call of a given shape the
 * launch sequence of a tree is replayed as one CUDA graph (EVB_GRAPH=0 turns that off).
 */
EVB_API int32_t evb_grow_tree_begin(evb_handle *h, const uint8_t *row_mask, uint8_t mask_cond, const uint32_t *js, int32_t njs,
                                    int32_t update_grads);
EVB_API int32_t evb_grow_tree_end(evb_handle *h, int64_t *feat, uint8_t *cond_bin, float *w_node, float *gain, float *leaf_pred,
                                  uint8_t *split);
/*
 * Evaluation data tracked on the device -- replaces `CallBack(params, m, x_eval, y_eval, device; w_eval, offset_eval)`
 * and `(cb::CallBack)(logger, iter, tree)` (src/callback.jl:82-128) with the metric kernels of
 * ext/EvoTreesKernelAbstractionsExt/metrics.jl (`eval_metric_kernel!`, `eval_mlogloss_kernel!`, `eval_mle2p_kernel!`).
 * evb_eval_attach uploads one evaluation shard, sets its predictions to pred0 (or zeros), adds the bias leaf with
 * the clamps of `predict!` (src/predict.jl:1-62) and returns the metric sums of iteration 0.  From then on every
 * tree grown by the handle is also applied to the evaluation predictions and the metric is re-evaluated, inside the
 * same launch sequence; evb_eval_sums returns the sums that belong to the tree collected last.
 *   x_bin    host uint8 [nobs x nfeats] column-major, binarized with the model's edges (src/callback.jl:93)
 *   y        host, same dtype / ycols as the training target (class codes 1..K for mlogloss)
 *   w        host float [nobs] or NULL for ones
 *   pred0    host float [K x nobs] offsets in link space, or NULL for zeros (src/callback.jl:94, 110-118)
 *   bias     host float [K]: leaf of the bias tree (`m.trees[1].pred`), or NULL when the model has none
 *   sums     [0] = sum_i w_i * value_i in double, value_i the per-row metric of src/metrics.jl:1-110 rounded to
 *            float as there; [1] = sum_i w_i.  The metric is sums[0] / sums[1] (its square root for :rmse); a
 *            caller that shards the evaluation rows over several handles adds the sums first.
 * Metrics: mse / mae / logloss / poisson / gamma / tweedie for the regression losses (mse, logloss, poisson, gamma, tweedie),
 * mlogloss for mlogloss, gaussian_mle / logistic_mle for the two likelihood losses (src/learners.jl:75, 352).
 */
enum evb_metric { EVB_METRIC_MSE = 0, EVB_METRIC_MAE = 1, EVB_METRIC_LOGLOSS = 2, EVB_METRIC_MLOGLOSS = 3, EVB_METRIC_GAUSSIAN_MLE = 4,
                  EVB_METRIC_POISSON = 5, EVB_METRIC_GAMMA = 6, EVB_METRIC_TWEEDIE = 7, EVB_METRIC_LOGISTIC_MLE = 8,
                  EVB_METRIC_QUANTILE = 9 /* pinball loss at evb_params.alpha (`wmae`, src/metrics.jl:4-6) */,
                  EVB_METRIC_MULTIQUANTILE = 10 /* mean pinball loss over evb_params.alphas (src/metrics.jl:120-141) */ };
EVB_API int32_t evb_eval_attach(evb_handle *h, int64_t nobs, const uint8_t *x_bin, const void *y, const float *w, const float *pred0,
                                const float *bias, int32_t metric, double sums[2]);
EVB_API int32_t evb_eval_sums(evb_handle *h, double sums[2]);
EVB_API int32_t evb_eval_get_pred(evb_handle *h, float *pred /* [K x nobs_eval] */);
EVB_API int32_t evb_eval_detach(evb_handle *h);

/*
 * Diagnostic of the failure path of sharded runs (no counterpart in the reference, which is single-GPU): runs one flag
 * barrier of a two-rank world whose second rank does not exist, on the handle's own GPU.  The wait gives up after
 * max_polls polls of about 100 ns each and the call returns EVB_ERR_DEVICE with the message of the expired wait; the
 * handle stays usable.  Nothing hangs or faults: it exercises what a sharded run does when a peer stops answering.
 */
EVB_API int32_t evb_test_peer_timeout(evb_handle *h, int32_t max_polls);

/* Switches the per-kernel CUDA-event timing of EVB_FLAG_TIMING on or off (timed trees run without graphs); with it
 * on, every kernel class is also an NVTX range ("evb:hist", "evb:scan", ...). */
EVB_API int32_t evb_set_timing(evb_handle *h, int32_t on);

/* State read-back for parity checks (each synchronises the handle's stream). */
EVB_API int32_t evb_get_pred(evb_handle *h, float *pred /* [K x nobs] */);
EVB_API int32_t evb_get_grads(evb_handle *h, float *grad /* [C x nobs] as cache.∇, src/init.jl:173 */);
/* node of every row after the last evb_grow_tree: from_partition=1 reads the row lists produced by the
 * partition kernel (`split_set!`, src/fit-utils.jl:93-312; rows outside the sample get 0), 0 reads the
 * leaf found by the traversal in the training `predict!` (all rows). */
EVB_API int32_t evb_get_nidx(evb_handle *h, uint32_t *nidx /* [nobs] */, int32_t from_partition);
/* histogram of one node of the last tree, double [C x nbins x njs] with feature order = js; only nodes of
 * depth <= max_depth-2 are retained (deeper ones are consumed by the split scan and not stored). */
EVB_API int32_t evb_get_hist(evb_handle *h, int32_t node, double *hist);
EVB_API int32_t evb_get_node_sums(evb_handle *h, double *nsum /* [C x nn] */);

/* The CUDA stream (cudaStream_t) on which the handle enqueues all its work, so that a caller can record
 * its own events around a sequence of calls. */
EVB_API int32_t evb_get_stream(evb_handle *h, void **stream);
EVB_API int32_t evb_get_timings(evb_handle *h, evb_timings *out);
EVB_API int32_t evb_reset_timings(evb_handle *h);

/*
 * evb_predict -- replaces `_predict(m, data, ::Type{<:GPU}; ntree_limit)` and `_predict_leaf_indices`
 * (ext/EvoTreesKernelAbstractionsExt/predict.jl:115-158) after the host has binarized `data`.
 * Trees are passed packed: every tree padded to `nn` nodes (the one-node bias tree, src/structs.jl:86-95,
 * included), tree t at offset t*nn (leaf_pred at t*nn*K).
 *   out        host float [nobs x K] column-major as the reference returns it (link applied when apply_link)
 *   leaf_idx   host uint32 [nobs x ntrees] column-major, or NULL (predict_leaf_idx, src/predict.jl:173-185)
 */
EVB_API int32_t evb_predict(int32_t device, int32_t loss, int32_t K, int32_t ntrees, int32_t nn, const int64_t *feat,
                    const uint8_t *cond_bin, const uint8_t *split, const float *leaf_pred, const uint8_t *x_bin,
                    int64_t nobs, int32_t nfeats, const uint8_t *feattypes, int32_t apply_link, float *out,
                    uint32_t *leaf_idx);

/*
 * evb_predict_x -- the whole of `_predict(m, data, ::Type{<:GPU})` (ext/EvoTreesKernelAbstractionsExt/predict.jl:115-135),
 * `binarize` included: the raw feature matrix goes to the device block by block, is binarized there against the
 * model's edges (`searchsortedfirst`, src/fit-utils.jl:69) straight into observation-major bins, and the trees are
 * applied.  Same tree arguments and outputs as evb_predict.
 *   x            host, EVB_F32 / EVB_F64; column-major [nobs x nfeats] (x_row_major = 0, a Julia Matrix) or
 *                row-major (x_row_major = 1, a C-ordered array)
 *   edges        host [nedges x nfeats] column-major, same dtype as x
 *   kernel_ms    optional: receives the summed device time of the binarize + traversal kernels
 */
EVB_API int32_t evb_predict_x(int32_t device, int32_t loss, int32_t K, int32_t ntrees, int32_t nn, const int64_t *feat,
                              const uint8_t *cond_bin, const uint8_t *split, const float *leaf_pred, const void *x, int32_t x_dtype,
                              int32_t x_row_major, const void *edges, int32_t nedges, int64_t nobs, int32_t nfeats,
                              const uint8_t *feattypes, int32_t apply_link, float *out, uint32_t *leaf_idx, double *kernel_ms);

/*
 * evb_binarize -- `binarize(X; edges)` (src/fit-utils.jl:66-72) on the device: x_bin[i,j] =
 * searchsortedfirst(edges[j], x[i,j]).  x host column-major [nobs x nfeats] of dtype EVB_F32 / EVB_F64,
 * edges host [nedges x nfeats] column-major of the same dtype (ascending per feature), out host uint8.
 */
EVB_API int32_t evb_binarize(int32_t device, const void *x, int32_t dtype, int64_t nobs, int32_t nfeats, const void *edges,
                     int32_t nedges, uint8_t *x_bin);

/*
 * evb_hist_rows -- the histogram kernel on its own: `_hist!` for one node (src/fit-utils.jl:367-394; GPU
 * counterpart `hist_kernel!`, ext/EvoTreesKernelAbstractionsExt/fit-utils.jl:57-95) on buffers that already live
 * on the device.  out[f][c][b] = sum over the listed rows of grad[row][c], b = bin of feature f in that row.
 *   x_rows  device uint8 [nobs][row_stride], observation-major bins 1..nbins (row_stride >= nfeats, multiple of 16)
 *   grad    device float [nobs][4], channels c < nch are accumulated
 *   rows    device uint32 [nrows], 0-based row ids (ascending order gives the reference's summation order)
 *   out     device double [nfeats][nch][nbins]
 *   stream  cudaStream_t to run on (NULL = default stream); the call returns after the work has finished.
 * Work buffers are allocated and freed inside the call.
 */
EVB_API int32_t evb_hist_rows(int32_t device, void *stream, const uint8_t *x_rows, int64_t nobs, int32_t nfeats, int32_t row_stride,
                              int32_t nbins, const float *grad, int32_t nch, const uint32_t *rows, int64_t nrows, double *out);

/*
 * evb_hist_rows_noalloc -- same arguments and result as evb_hist_rows, for callers that are not allowed to allocate
 * device memory while they run: code executing between cudaMalloc-free phases of a real-time or long-running service,
 * plug-ins that work inside a host framework's memory pool, or anything that must not trigger the implicit
 * device synchronisation of cudaMalloc / cudaFree.  It has no counterpart in the reference.
 * It calls no allocator of any kind.  Its work memory is a fixed 8 MiB block that is part of the library image on
 * every GPU that loads the library (held until the process exits), so:
 *   - limits: nfeats <= 1024, nbins <= 255, nch <= 4, and two partial images (one per feature group of 32 features:
 *     32 x nbins x nch floats, per group) must fit in the 8 MiB; larger problems are rejected with EVB_ERR_LIMIT;
 *   - the first call on a device looks up the device addresses of that block (cudaGetSymbolAddress), under a lock, so
 *     two host threads may make it at once;
 *   - like evb_hist_rows the call waits for its work (it synchronises the stream to read the kernels' error word back),
 *     so it must never be made while the stream is being captured into a CUDA graph -- neither the first call nor a
 *     later one;
 *   - all calls on one GPU share the block and it keeps the previous call's contents: every value that is read is
 *     rewritten by the same call first, but two calls that overlap in time on the same GPU race with each other.
 *     Serialise them (one stream, or events).
 */
EVB_API int32_t evb_hist_rows_noalloc(int32_t device, void *stream, const uint8_t *x_rows, int64_t nobs, int32_t nfeats,
                                      int32_t row_stride, int32_t nbins, const float *grad, int32_t nch, const uint32_t *rows,
                                      int64_t nrows, double *out);

#ifdef __cplusplus
}
#endif
#endif /* EVB_H */
