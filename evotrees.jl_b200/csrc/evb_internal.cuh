// Internal declarations shared by the translation units of libevotrees_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>
#include "../../include/evb.h"

#define EVB_VERSION 1

// ---- error plumbing -------------------------------------------------------------------------------
void evb_set_error(const char *fmt, ...);
#define EVB_CUDA(call)                                                                                \
    do {                                                                                              \
        cudaError_t _e = (call);                                                                      \
        if (_e != cudaSuccess) {                                                                      \
            evb_set_error("CUDA error %s at %s:%d (%s)", cudaGetErrorString(_e), __FILE__, __LINE__, #call); \
            return EVB_ERR_CUDA;                                                                      \
        }                                                                                             \
    } while (0)
#define EVB_CHECK(call)                    \
    do {                                   \
        int32_t _s = (call);               \
        if (_s != EVB_OK) return _s;       \
    } while (0)

// device-side error codes written to evb_handle::d_err
enum { EVB_DERR_NONE = 0, EVB_DERR_WAIT_FULL = 1, EVB_DERR_WAIT_EMPTY = 2, EVB_DERR_BIN_RANGE = 3, EVB_DERR_PLAN = 4, EVB_DERR_PEER = 5, EVB_DERR_NAN = 6 };

// ---- geometry constants ---------------------------------------------------------------------------
constexpr int EVB_TILE_ROWS = 32;    // rows per staged tile (one per producer lane)
constexpr int EVB_PART_CHUNK = 2048; // rows per partition work item
constexpr int EVB_PART_THREADS = 256;
constexpr int EVB_MAX_UNITS_PER_BLOCK = 4;
constexpr int EVB_MAX_DEPTH = 15;

enum { EVB_KIND_NONE = 0, EVB_KIND_BUILD = 1, EVB_KIND_SUB = 2 };

// Per-level plan, device resident.  Written by the plan kernels, read by hist / reduce / scan.
struct LevelPlan {
    int32_t nbuild;   // build slots used at this level
    int32_t nitems;   // partition work items at this level
    int64_t R;        // rows (local) inside build nodes
    int32_t n_sel;    // rows selected by the row mask (root only)
    int32_t pad;
};

struct HistGeom {
    int BP;        // padded bins per image: 32/64/128/256
    int NCH;       // channels per unit image (<= 4)
    int FPL;       // feature slots per lane (1, 2 or 4): a unit covers 32 * FPL feature slots
    int NFG;       // feature groups of 32 * FPL slots
    int NCT;       // channel groups of 4
    int U;         // units = NFG*NCT
    int UB;        // units (consumer warps) per block
    int NUG;       // unit groups = ceil(U/UB)
    int stages;    // staged tiles in flight
    int G;         // row-range blocks (grid.x)
    bool q;        // geometry of the fixed-point kernel
    int PG;        // piece slots per unit group = G + max build slots
    size_t smem;   // dynamic shared memory per block
    size_t img_floats;   // floats per unit image in scratch: FPL*NCH*nbins*32
};

// geometry of the register-direct fixed-point histogram kernel (evb_histq2.cu)
struct Q2Geom {
    int NC;        // 16-byte chunks (16 features) per CTA group
    int ngroups;   // CTA groups (grid.y); xH rows hold ngroups * NC chunks
    int ntail;     // features kept beside the gradient word in xE (nfeats % 16 when that is 1..4, else 0)
    int nmain;     // features kept in xH
    int RSH;       // bytes per row of xH
    int SC;        // feature columns per bin of the accumulators
    int G;         // grid.x
    int TE;        // tiles of 32 rows between two flushes of a CTA's image
    int min_rows;  // rows per CTA below which fewer CTAs take part
    int QB;        // bits of the fixed-point gradient: |q| < 2^QB (26 or 24)
    size_t smem;
};

struct evb_handle {
    evb_params p;
    int K, C, B, D, nn;        // nn = 2^D-1
    int Ce;                    // channels actually accumulated: C, or K+1 for mse where h = 2w is rebuilt from w
    int rec_nch;               // channels per 16-byte group of the float gradient record (see gpos)
    int nfeats, RS, GS;        // RS: bytes per row of xT (multiple of 32); GS: floats per grad record (multiple of 4)
    int64_t n;                 // local rows
    int dev, num_sms;
    cudaStream_t st;
    int busy;

    // row data
    uint8_t *xT;       // [n][RS]  observation-major bins (1..B), zero padded
    uint8_t *xC;       // [nfeats][n] feature-major copy (the layout of the caller's x_bin) read by the row partition
    float *grad;       // [n][GS]  g_1..g_K,h_1..h_K,w,(pad)
    float *pred;       // [n][K]
    void *y;           // float [n][ycols] or uint32 [n]
    int y_dtype, ycols;
    uint32_t *nidx;    // [n] leaf of each row from the training traversal
    uint32_t *rows[2]; // [n] ping-pong row lists, segments ordered by node
    uint8_t *mask_d;   // [n]
    uint8_t *feattypes_d; // [nfeats]
    int32_t *mono_d;      // [nfeats]
    uint32_t *js_d;       // [nfeats] 0-based feature id per slot
    int F;                // njs of the current tree
    bool grads_fresh;     // gradients already computed for the next round (fused into finalize)
    int bag_idx;

    // node state, indexed by heap id 0..nn (0 unused); children of level D-1 nodes need ids < 2^D
    int32_t *seg_start, *seg_cnt; // local row segment of each node
    int32_t *gcnt;                // global (all ranks) row count
    int32_t *nleft, *gnleft;      // left-child row count of split nodes, local / global (gnleft == nleft when world == 1)
    uint8_t *kind;
    int32_t *bslot;
    double *nsum;                 // [nn+1][C]
    // tree arrays (device), heap id - 1
    int32_t *t_feat; uint8_t *t_bin; uint8_t *t_split; float *t_gain; float *t_w; float *t_pred;
    uint32_t *t_packed;           // per node: feat0 | bin<<16 | split<<24 | numeric<<25 (for traversal)

    // plans
    LevelPlan *plan;       // [D+1]
    int32_t *cum;          // [maxslots+1] exclusive prefix of build-node row counts (current level)
    int32_t *slot_node;    // [maxslots]
    int32_t *item_node, *item_chunk, *item_left, *item_lprefix; // partition items
    uint32_t *item_bits;   // [max_items][EVB_PART_CHUNK/32]
    int max_items, maxslots;
    int32_t *scan_tmp;     // block counts for the mask compaction
    double *fbest_gain;    // [nodes of a level][nfeats] per-feature best split of the scan
    int32_t *fbest_bin;
    double *obl_gain;      // oblivious trees: [nodes of a level + 1][nfeats * B] gain of every candidate, last row = level totals
    double *obl_best;      // [2] gain and candidate index (-1: none) of the level's shared split
    int *d_err;            // device error word
    int *h_err;            // pinned mirror

    // evaluation shard (evb_eval_attach): every grown tree is applied to ev_pred and the metric sums go to d_evsum
    int64_t ev_n;      // 0 = none attached
    uint8_t *ev_xT;    // [ev_n][RS]
    void *ev_y; float *ev_w; float *ev_pred;
    double *ev_part;   // [ev_blocks][2] per-block partial sums
    double *d_evsum;   // [2] inside the tree block: sum w*value, sum w
    int ev_metric, ev_blocks;
    double last_eval[2]; // sums of the tree collected last

    // fixed-point histogram variant (mse, one target): gradq holds the integer words of every row
    bool use_q, unit_w;   // unit_w: no weights were given, the w channel is a row count
    bool q_active;        // the current geometry is the fixed-point one (no column sample)
    bool gradq_valid;     // gradq holds the words of the current gradients
    int32_t *gradq;       // [n] fixed-point g, or [n][2] fixed-point g and w when weights were given
    unsigned *d_gmax;     // bits of max |g| over the rows, filled by the gradient kernels
    double *d_qinv;       // [2] 2^-s of the g words / of the w words
    float wscale; double winv;

    // register-direct variant (unit weights): rows as 16-byte chunks + {q, tail bins} per row, integer accumulators
    bool use_q2;
    Q2Geom q2;
    uint8_t *xH;                  // [n][q2.RSH]
    uint2 *xE;                    // [n] {fixed-point gradient, bins of the tail features}
    unsigned long long *hsum_q;   // [maxslots][B][q2.SC] sums of q per build slot
    uint32_t *hcnt_q;             // [maxslots][B][q2.SC] row counts

    // quantile loss: work memory of the per-leaf order-statistic selection
    uint32_t *qs_cnt, *qs_prefix, *qs_rank; float *qs_gamma;

    // histograms
    HistGeom hg;
    int hist_mode;    // EVB_HIST_MODE environment override (kernel variants / diagnostics)
    double *hist;     // [2^(D-2) nodes][F][C][B] retained for the subtraction trick
    int hist_nodes;   // nodes with id < hist_nodes are retained
    double *hcomp;    // [maxslots][F][C][B] freshly built histograms of the level (allreduce buffer)
    float *scratch;   // [NUG][PG][UB][NCH][B][32] per-piece partial images
    size_t scratch_floats;

    // pinned host staging, double buffered so that tree t+1 can be enqueued before tree t is collected
    void *h_tree[2]; size_t h_tree_bytes;
    uint32_t *h_js[2];
    cudaEvent_t ev_done[2];
    int tree_seq, pending;          // trees started / started but not yet collected
    // one CUDA graph per variant of the per-tree launch sequence (mask, gradients first, gradients fused, slot)
    bool use_graphs;
    cudaGraphExec_t graph[32];
    int graph_calls[32];
    int64_t graph_launches[32][EVB_NTIMERS];
    int graph_mask_cond;

    // multi-GPU
    void *nccl_comm; int rank, world;
    uint8_t nccl_id[128]; bool nccl_pending; // id recorded by evb_comm_init; the communicator is created by the first collective
    // peer access between the ranks' processes (CUDA IPC): histograms are summed by peer loads inside the split scan
    bool p2p;
    double *peer_hcomp[8]; double *peer_cand[8]; int *peer_flags[8];
    double *hsum; // sums over the ranks of the owned feature slots of hcomp
    void *ipc_opened[24]; int n_ipc_opened;
    int *d_barrier_seq; // device counter of the peer barriers passed

    // timing
    bool timing;
    std::vector<cudaEvent_t> ev; // pairs
    cudaEvent_t ev_tot[2];       // bracket of one whole evb_grow_tree
    std::vector<int> ev_class;
    size_t ev_used;
    evb_timings tm;
};

// ---- launchers (each enqueues on h->st and returns a status) ---------------------------------------
// evb_rows.cu
int32_t evb_launch_transpose(evb_handle *h, const uint8_t *xcol_dev, int64_t ld, int64_t nrows, int j0, int nj, uint8_t *xT, int RS, cudaStream_t st);
int32_t evb_launch_grads(evb_handle *h);
int32_t evb_launch_quantize(evb_handle *h);
int32_t evb_launch_rows_init(evb_handle *h, bool use_mask, uint8_t mask_cond);
int32_t evb_launch_finalize(evb_handle *h, bool compute_grads, int mode); // mode: see FinArgs in evb_rows.cu
int32_t evb_launch_quantile_leaves(evb_handle *h, bool use_mask, uint8_t mask_cond);
int32_t evb_launch_nidx_from_partition(evb_handle *h, uint32_t *out_dev);
int32_t evb_launch_eval(evb_handle *h, const float *fixed_leaf_dev);
int32_t evb_upload_binarize(evb_handle *h, const void *x, int32_t dtype, const void *edges, int32_t nedges); // raw host matrix -> h->xC
// evb_hist.cu
int32_t evb_hist_configure(evb_handle *h);   // fills h->hg from p / nfeats (uses max F = nfeats)
int32_t evb_launch_hist(evb_handle *h, int level);
int32_t evb_launch_hist_reduce(evb_handle *h, int level);
// evb_histq2.cu
int32_t evb_q2_configure(evb_handle *h);
int32_t evb_q2_build_layout(evb_handle *h);
int32_t evb_launch_q2_quantize(evb_handle *h);
int32_t evb_launch_histq2(evb_handle *h, int level);
int32_t evb_launch_q2_reduce(evb_handle *h, int level);
int32_t evb_launch_q2_clear(evb_handle *h, int level);
bool evb_q2_direct(const evb_handle *h);
// evb_tree.cu
int32_t evb_launch_tree_reset(evb_handle *h);
int32_t evb_launch_scan(evb_handle *h, int level);
int32_t evb_launch_partition(evb_handle *h, int level); // plan + flags + prefix (+allreduce) + level plan + scatter
int32_t evb_launch_lonely_barrier(evb_handle *h, int *flags, int *seq, unsigned max_polls);
// evb_nccl.cpp
int32_t evb_nccl_unique_id(uint8_t id[128]);
int32_t evb_nccl_init(evb_handle *h, const uint8_t id[128], int rank, int world);
int32_t evb_nccl_allreduce_f64(evb_handle *h, double *buf, size_t count);
int32_t evb_nccl_allreduce_i32(evb_handle *h, const int32_t *src, int32_t *dst, size_t count);
void evb_nccl_destroy(evb_handle *h);

// evb_stage.cu: pageable host memory -> device through a ring of pinned buffers filled by several host threads
// device memory through the library's block cache (evb_alloc.cu)
cudaError_t evb_dev_alloc(void **p, size_t bytes);
void evb_dev_free(void *p, bool really = false);
template <typename T> inline cudaError_t evb_dev_alloc(T **p, size_t bytes) { return evb_dev_alloc(reinterpret_cast<void **>(p), bytes); }
cudaError_t evb_host_alloc(void **p, size_t bytes);
void evb_host_free(void *p);
cudaError_t evb_stream_get(cudaStream_t *st);
void evb_stream_put(cudaStream_t st);
cudaError_t evb_event_get(cudaEvent_t *ev);
void evb_event_put(cudaEvent_t ev);

int32_t evb_h2d_staged(void *dst_dev, const void *src_host, size_t bytes, cudaStream_t st, bool drain = true);
int32_t evb_h2d_staged_strided(void *dst_dev, const void *src_host, size_t seg_bytes, size_t nseg, size_t stride, cudaStream_t st, bool drain = true);

// EVB_HIST_MODE of the environment, reduced to the documented values (0: TMA bulk staging, 1: cp.async staging)
int evb_hist_mode_env();
// timing helpers (evb_api.cu)
void evb_tic(evb_handle *h, int cls);
void evb_toc(evb_handle *h, int cls);

static inline int evb_level_nodes(int level) { return 1 << (level - 1); }            // nodes at depth `level`
static inline int evb_level_slots(int level) { return level <= 1 ? 1 : 1 << (level - 2); } // max build slots
