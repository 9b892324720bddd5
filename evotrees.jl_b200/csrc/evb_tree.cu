// Per-level tree growth on the device: sibling subtraction + split scan + split application
// (`subtract_hist!`, `get_best_split`/`_scan_node!`, `_child_sums!`, `pred_leaf_cpu!`: src/fit-utils.jl:321-332,
// 403-486, src/split.jl:1-117, src/predict.jl:198-247, src/fit.jl:85-137) and the stable row partition
// (`split_set!`, src/fit-utils.jl:93-312; GPU counterpart `update_nodes_idx_kernel!`,
// ext/EvoTreesKernelAbstractionsExt/fit-utils.jl:9-31).  Everything a level needs (active nodes, segment
// bounds, build/subtract choice, work lists) lives in device memory, so the host enqueues a fixed sequence of
// launches per level and never reads anything back until the tree is complete.
#include "evb_internal.cuh"
#include <float.h>

namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ double warp_incl_scan(double v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        double t = __shfl_up_sync(FULL, v, d);
        if (lane >= d) v += t;
    }
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(FULL, v, d);
    return v;
}
__device__ __forceinline__ int warp_incl_scan_i(int v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int t = __shfl_up_sync(FULL, v, d);
        if (lane >= d) v += t;
    }
    return v;
}
// exclusive scan over the threads of a block (blockDim.x <= 1024, multiple of 32); returns the exclusive
// prefix of v and writes the block total to *total.  `sm` is 33 ints of shared memory.
__device__ __forceinline__ int block_excl_scan(int v, int *sm, int *total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int incl = warp_incl_scan_i(v, lane);
    __syncthreads();
    if (lane == 31) sm[wid] = incl;
    __syncthreads();
    if (wid == 0) {
        int w = lane < nw ? sm[lane] : 0;
        int wi = warp_incl_scan_i(w, lane);
        sm[lane] = wi - w;
        if (lane == 31) sm[32] = wi;
    }
    __syncthreads();
    *total = sm[32];
    return incl - v + sm[wid];
}

// ------------------------------------------------------------------------------------------ reset / root
struct ResetArgs {
    int32_t *seg_start, *seg_cnt, *gcnt, *nleft, *gnleft, *bslot, *t_feat;
    uint8_t *kind, *t_bin, *t_split;
    float *t_gain, *t_w, *t_pred;
    uint32_t *t_packed;
    double *nsum;
    LevelPlan *plan;
    int nids, nn, K, C, D;
};
__global__ void k_tree_reset(ResetArgs a) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a.nids) {
        a.seg_start[i] = 0; a.seg_cnt[i] = 0; a.gcnt[i] = 0; a.kind[i] = 0; a.bslot[i] = 0;
        if (i > 0) { a.nleft[i] = 0; if (a.gnleft != a.nleft) a.gnleft[i] = 0; } // entry 0 carries the root count
        for (int c = 0; c < a.C; ++c) a.nsum[(size_t)i * a.C + c] = 0.0;
    }
    if (i < a.nn) {
        a.t_feat[i] = 0; a.t_bin[i] = 0; a.t_split[i] = 0; a.t_gain[i] = 0.f; a.t_w[i] = 0.f; a.t_packed[i] = 0u;
        for (int k = 0; k < a.K; ++k) a.t_pred[(size_t)i * a.K + k] = 0.f;
    }
    if (i >= 2 && i <= a.D) { a.plan[i].nbuild = 0; a.plan[i].nitems = 0; a.plan[i].R = 0; }
}

struct RootArgs {
    int32_t *seg_start, *seg_cnt, *gcnt, *bslot, *cum, *slot_node;
    const int32_t *nleft, *gnleft;
    uint8_t *kind;
    LevelPlan *plan;
};
__global__ void k_root_plan(RootArgs a) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int nsel = a.nleft[0];
        a.seg_start[1] = 0; a.seg_cnt[1] = nsel; a.gcnt[1] = a.gnleft[0];
        a.kind[1] = EVB_KIND_BUILD; a.bslot[1] = 0;
        a.cum[0] = 0; a.cum[1] = nsel; a.slot_node[0] = 1;
        a.plan[1].nbuild = 1; a.plan[1].R = nsel; a.plan[1].n_sel = nsel; a.plan[1].nitems = 0;
    }
}

// ------------------------------------------------------------------------------------------ split scan
constexpr int EVB_MAX_PEERS = 8;

struct ScanArgs {
    const double *hcomp;
    double *hist, *nsum;
    const uint8_t *kind;
    const int32_t *bslot;
    const uint32_t *js0;
    const uint8_t *feattypes;
    const int32_t *mono;
    int32_t *t_feat;
    uint8_t *t_bin, *t_split;
    float *t_gain, *t_w, *t_pred;
    uint32_t *t_packed;
    double *fbest_gain; // [nodes of the level][F] best gain of each feature
    int32_t *fbest_bin; // [nodes of the level][F] its bin (0-based) or -1
    // oblivious trees (null otherwise): [nodes of the level + 1][F * B] gain of every candidate (0: not eligible),
    // the last row receives the level totals; obl_best = {gain, candidate index or -1} of the shared split
    double *obl_gain, *obl_best;
    const LevelPlan *plan;
    const int32_t *slot_node;
    // Row-sharded runs with peer access: every rank scans the feature slots f with f % world == rank (`hcomp` then
    // points at the sums made by k_peer_reduce) and publishes one candidate per node to every rank.
    double *peer_cand[EVB_MAX_PEERS];
    const double *cand_local; // [nodes of the level][world][3 + C]: gain, feature slot, bin, left sums
    int world, rank;          // world == 1: no peers (single GPU, or histograms already summed by NCCL)
    int F, C, K, B, level, D, hist_nodes, loss;
    int elide_h;        // mse: the h channels equal twice the w channel and are rebuilt instead of read
    // non-null: the built histograms are read straight from the integer accumulators of the fixed-point kernel
    // ([slot][bin][SC] sums of q and row counts; g = sum * qinv[0], w = count, h = 2w) instead of from hcomp
    const unsigned long long *qsum;
    const uint32_t *qcnt;
    const double *qinv;
    int SC;
    double neb; // -eta / bagging_size
    double lambda, L2, gamma, min_weight;
};

__device__ __forceinline__ double term_gh(double g, double h, double w, double lambda, double L2) {
    return g * g / fmax(DBL_EPSILON, h + lambda * w + L2) / 2.0; // src/split.jl:1
}
// mae: |mean of the side - mean of the parent| * weight / (1 + lambda + L2 / w)   (src/split.jl:2, 119-130)
__device__ __forceinline__ double term_shift(double g, double w, double mu_p, double d) { return fabs(g / w - mu_p) * w / d; }
// credibility losses: Z * |m1| / (1 + L2 / w), Z from the ratio of variances or of standard deviations
// (src/split.jl:3-4, src/loss.jl:275-289)
__device__ __forceinline__ double term_cred(int loss, double m1, double m2, double w, double L2) {
    const double vhm = (m1 / w) * (m1 / w);
    const double evpv = fmax(DBL_EPSILON, m2 / w - vhm);
    const double z = loss == EVB_CRED_VAR ? vhm / (vhm + evpv) : sqrt(vhm) / (sqrt(vhm) + sqrt(evpv));
    return z * fabs(m1) / (1.0 + L2 / w);
}
__device__ __forceinline__ bool own_gain(int loss) { return loss >= EVB_MAE; }
// gain of one output row of a candidate split: left sums (gl, hl, w_l), parent sums (sg, sh, w_p)
__device__ __forceinline__ double side_gain(const ScanArgs &a, double gl, double hl, double w_l, double sg, double sh, double w_p) {
    const double w_r = w_p - w_l;
    if ((a.loss == EVB_MAE || a.loss == EVB_QUANTILE || a.loss == EVB_MULTIQUANTILE)) {
        const double d_l = fmax(DBL_EPSILON, 1.0 + a.lambda + a.L2 / w_l), d_r = fmax(DBL_EPSILON, 1.0 + a.lambda + a.L2 / w_r);
        const double mu_p = sg / w_p;
        return term_shift(gl, w_l, mu_p, d_l) + term_shift(sg - gl, w_r, mu_p, d_r);
    }
    return term_cred(a.loss, gl, hl, w_l, a.L2) + term_cred(a.loss, sg - gl, sh - hl, w_r, a.L2);
}
// pred_scalar of the three losses (src/predict.jl:219-222, 257-261): the sign is the gradient's, not minus it
__device__ __forceinline__ double own_scalar(const ScanArgs &a, double g, double w) {
    return -a.neb * g / ((a.loss == EVB_MAE || a.loss == EVB_QUANTILE || a.loss == EVB_MULTIQUANTILE) ? fmax(DBL_EPSILON, w + a.lambda * w + a.L2) : (w + a.L2));
}
// pred_leaf_cpu! for output row k (src/predict.jl:198-204, 224-234, 241-247; mae :250-257, cred :211-218)
__device__ __forceinline__ float leaf_value(const ScanArgs &a, const double *s, int k) {
    const int K = a.K, C = a.C;
    if (own_gain(a.loss)) return (float)own_scalar(a, s[k], s[C - 1]);
    double g, h;
    if (a.loss == EVB_GAUSSIAN_MLE || a.loss == EVB_LOGISTIC_MLE) {
        const int Y = K / 2, t = k >> 1, j = k & 1;
        g = s[2 * t + j];
        h = s[2 * Y + 2 * t + j];
    } else {
        g = s[k];
        h = s[K + k];
    }
    return (float)(a.neb * g / fmax(DBL_EPSILON, h + a.lambda * s[C - 1] + a.L2));
}

// Sharded with peer access: sums the ranks' freshly built histograms for the feature slots this rank owns, by
// loads from the peers' memory past the caches, in rank order (so the result does not depend on timing).  One CTA
// per (build slot, owned feature); at the root level feature slot 0 is summed on every rank (it gives the root sums).
struct PeerReduceArgs {
    const double *peer_hcomp[EVB_MAX_PEERS];
    double *hsum;
    const LevelPlan *plan;
    int world, rank, F, CB, level;
    int K, elided; // elided: mse, every rank's hessian channels are exactly 2 x its weight channel -- they are not fetched
};
__global__ void __launch_bounds__(256) k_peer_reduce(PeerReduceArgs a) {
    const int Fown = (a.F - a.rank + a.world - 1) / a.world;
    const int per = Fown + 1; // last index of a slot: feature slot 0 (root level only)
    const int s = blockIdx.x / per, fi = blockIdx.x % per;
    if (s >= a.plan->nbuild) return;
    int f;
    if (fi < Fown) f = fi * a.world + a.rank;
    else { if (a.level != 1 || a.rank == 0) return; f = 0; }
    const size_t base = ((size_t)s * a.F + f) * a.CB;
    const int B = a.CB / (2 * a.K + 1);
    for (int idx = threadIdx.x; idx < a.CB; idx += blockDim.x) {
        const int c = idx / B;
        if (a.elided && c >= a.K && c < 2 * a.K) continue;
        double v = 0.0;
#pragma unroll 8
        for (int q = 0; q < a.world; ++q) v += __ldcv(a.peer_hcomp[q] + base + idx);
        a.hsum[base + idx] = v;
        if (a.elided && c == 2 * a.K) // h_k = 2w (src/loss.jl:52): doubling commutes with the rounding of the sum
            for (int k = 0; k < a.K; ++k) a.hsum[base + (size_t)(a.K + k) * B + (idx - c * B)] = 2.0 * v;
    }
}

// Scan of one (node, feature): applies the sibling subtraction (`subtract_hist!`, fit-utils.jl:321-332) to the
// staged histogram `sm` of the build node, stores the node's histogram if its children will need it, scans the
// bins (`_scan_node!`, fit-utils.jl:403-436) and records the best split of this feature.
template <int MAXCHK, bool OWN, bool OBL, bool K1>
__device__ __forceinline__ void scan_one(const ScanArgs &a, int n, bool sub, int f, int slot, double *s_sum, int lane, bool first_owned) {
    // K1: one output with gradient, hessian and weight channels (C = 3), known at compile time: the loops over the
    // outputs and the channel tests fold away
    const int C = K1 ? 3 : a.C, K = K1 ? 1 : a.K, B = a.B, F = a.F;
    const uint32_t feat = a.js0[f];
    const double *__restrict__ sm = a.hcomp + ((size_t)slot * F + f) * C * B;
    const double qi = a.qsum ? a.qinv[0] : 0.0;
    // entry (channel c, bin b) of the histogram built for `slot` and feature slot f
    auto built = [&](int c, int b) -> double {
        if (a.qsum) {
            const size_t o = ((size_t)slot * B + b) * a.SC + feat;
            if (c < K) return (double)(long long)__ldg(a.qsum + o) * qi;
            const double w = (double)__ldg(a.qcnt + o);
            return c == C - 1 ? w : 2.0 * w;
        }
        return sm[c * B + b];
    };
    const int m = 1 << (a.level - 1);
    const size_t FCB = (size_t)F * C * B;
    const double *__restrict__ hp = a.hist + (size_t)(n >> 1) * FCB;
    const bool keep = n < a.hist_nodes;
    double *__restrict__ hn = a.hist + (size_t)n * FCB;
    if (n == 1) {
        // root sums = sum over the bins of feature slot 0 (every sampled row has exactly one bin there);
        // the reference sums the gradients of the sampled rows directly (src/fit.jl:66)
        for (int c = 0; c < C; ++c) {
            double v = 0.0;
            for (int b = lane; b < B; b += 32) v += built(c, b);
            v = warp_sum(v);
            if (lane == 0) { s_sum[c] = v; if (first_owned) a.nsum[(size_t)C + c] = v; }
        }
    } else {
        for (int c = lane; c < C; c += 32) s_sum[c] = a.nsum[(size_t)n * C + c];
    }
    __syncwarp();
    double gain_p = 0.0;
    const double w_p = s_sum[C - 1];
    if (!OWN) {
        for (int k = 0; k < K; ++k) gain_p += term_gh(s_sum[k], s_sum[K + k], w_p, a.lambda, a.L2); // node_gain, split.jl:58-66
    } else if (a.loss != EVB_MAE && a.loss != EVB_QUANTILE && a.loss != EVB_MULTIQUANTILE) {
        for (int k = 0; k < K; ++k) gain_p += term_cred(a.loss, s_sum[k], s_sum[K + k], w_p, a.L2);   // split.jl:70-78; mae: 0
    }

    // lane l holds the CH adjacent bins l * CH .. l * CH + CH - 1 (CH * 32 >= B): a running sum over the bins is a
    // running sum inside the lane plus ONE warp scan of the lanes' totals, whatever CH is
    constexpr int CH = MAXCHK;
    const int bin0 = lane * CH;
    const bool numeric = a.feattypes[feat] != 0;
    const int constraint = a.mono[feat];
    const int b_max = numeric ? B - 1 : B;
    const size_t fo = (size_t)f * C * B;
    const bool elide = a.elide_h != 0; // mse: every h entry is exactly twice the w entry (src/loss.jl:52), it is not read
    auto val = [&](int c, int b) -> double {
        const int o = c * B + b;
        double v = built(c, b);
        if (sub) v = __ldg(hp + fo + o) - v;
        if (keep) hn[fo + o] = v;
        return v;
    };
    auto running = [&](double (&v)[CH]) { // inclusive running sum over the bins (numeric features only)
        if (!numeric) return;
#pragma unroll
        for (int j = 1; j < CH; ++j) v[j] += v[j - 1];
        const double incl = warp_incl_scan(v[CH - 1], lane);
        double before = __shfl_up_sync(FULL, incl, 1);
        if (lane == 0) before = 0.0;
#pragma unroll
        for (int j = 0; j < CH; ++j) v[j] += before;
    };
    double lg = a.gamma; // get_best_split starts at gamma and takes strict improvements (fit-utils.jl:444-450)
    int lb = 0x7fffffff;
    if (a.level < a.D) {
        double wl[CH], gacc[CH];
        unsigned okmask = 0xffu;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            gacc[j] = 0.0;
            const int b = bin0 + j;
            wl[j] = b < B ? val(C - 1, b) : 0.0;
            if (elide && keep && b < B)
                for (int k = 0; k < K; ++k) hn[fo + (size_t)(K + k) * B + b] = 2.0 * wl[j];
        }
        running(wl);
        for (int k = 0; k < K; ++k) {
            const double sg = s_sum[k], sh = s_sum[K + k];
            double gl[CH], hl[CH];
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                const int b = bin0 + j;
                gl[j] = b < B ? val(k, b) : 0.0;
                if (!elide) hl[j] = b < B ? val(K + k, b) : 0.0;
            }
            running(gl);
            if (!elide) running(hl);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                if (elide) hl[j] = 2.0 * wl[j];
                const double w_l = wl[j], w_r = w_p - w_l;
                if (!OWN) gacc[j] += term_gh(gl[j], hl[j], w_l, a.lambda, a.L2) + term_gh(sg - gl[j], sh - hl[j], w_r, a.lambda, a.L2);
                else gacc[j] += side_gain(a, gl[j], hl[j], w_l, sg, sh, w_p);
                if (k == 0 && constraint != 0) {
                    // pred_scalar on left / right sums (src/predict.jl:205-208, 235-238)
                    const double pl = OWN ? own_scalar(a, gl[j], w_l) : a.neb * gl[j] / fmax(DBL_EPSILON, hl[j] + a.lambda * w_l + a.L2);
                    const double pr = OWN ? own_scalar(a, sg - gl[j], w_r)
                                          : a.neb * (sg - gl[j]) / fmax(DBL_EPSILON, (sh - hl[j]) + a.lambda * w_r + a.L2);
                    const bool ok = (constraint == -1 && pl > pr) || (constraint == 1 && pl < pr);
                    if (!ok) okmask &= ~(1u << j);
                }
            }
        }
        // candidate of this lane: lowest bin among its strict maxima
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int b = bin0 + j;
            const double w_l = wl[j], w_r = w_p - w_l;
            double g = 0.0;
            const bool elig = b < b_max && w_l > a.min_weight && w_r > a.min_weight && ((okmask >> j) & 1u);
            if (elig) {
                g = gacc[j] - gain_p;
                if (g > lg) { lg = g; lb = b; }
            }
            if (OBL && b < B) a.obl_gain[((size_t)(n - m) * F + f) * B + b] = g; // update_gains!, fit-utils.jl:457-463
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            const double og = __shfl_xor_sync(FULL, lg, d);
            const int ob = __shfl_xor_sync(FULL, lb, d);
            if (og > lg || (og == lg && ob < lb)) { lg = og; lb = ob; }
        }
    }
    if (lane == 0) {
        a.fbest_gain[(size_t)(n - m) * F + f] = lg;
        a.fbest_bin[(size_t)(n - m) * F + f] = lb == 0x7fffffff ? -1 : lb;
    }
    __syncwarp();
}

// Stage 1: one warp per (node, owned feature slot), lanes over bins.  The nodes of a level come in pairs sharing a
// build slot: the build node reads the slot's histogram, its sibling subtracts it from the parent's.  Warps are
// independent, so even the root level (one node) spreads over many SMs.
// OWN: the loss brings its own split gain (mae, credibility); OBL: oblivious trees, the gain of every candidate is
// stored as well.  The default instance carries neither code.
template <int MAXCHK, bool OWN, bool OBL, bool K1>
__global__ void __launch_bounds__(256, MAXCHK <= 2 ? (K1 ? 4 : 3) : 2) k_scan_feat(ScanArgs a) {
    __shared__ double s_sum_all[8][72];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int F = a.F;
    const int Fown = (F - a.rank + a.world - 1) / a.world;
    if (Fown <= 0) return;
    long long gw = (long long)blockIdx.x * wpb + wid;
    const int which = a.level > 1 ? (int)(gw & 1) : 0;
    if (a.level > 1) gw >>= 1;
    const int s = (int)(gw / Fown), fi = (int)(gw % Fown);
    if (s >= a.plan->nbuild) return;
    const int f = fi * a.world + a.rank;
    const int nb = a.slot_node[s];
    scan_one<MAXCHK, OWN, OBL, K1>(a, which ? nb ^ 1 : nb, which != 0, f, s, s_sum_all[wid], lane, fi == 0);
}

// Oblivious trees, stage 1b: one thread per candidate (feature slot, bin) adds the gains of the level's nodes in
// ascending node order and drops the candidate if any node holds no positive gain for it (src/fit.jl:196-211; at
// the root level the reference applies no mask, which changes nothing for gamma >= 0).  Sharded with peer access,
// every rank does this for its own feature slots; k_scan_node then publishes the rank's best split with each
// node's left sums and k_scan_final takes the best of the ranks (the same for every node: the gains are level totals).
__global__ void __launch_bounds__(128) k_obl_sum(ScanArgs a) {
    const int m = 1 << (a.level - 1);
    const size_t FB = (size_t)a.F * a.B;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= FB) return;
    double tot = 0.0;
    // sharded with peer access: only the feature slots this rank scans hold gains; the others never win here
    bool ok = (int)(e / a.B) % a.world == a.rank;
    for (int i = 0; ok && i < m; ++i) {
        const double g = a.obl_gain[(size_t)i * FB + e];
        tot += g;
        ok = ok && g > 0.0;
    }
    a.obl_gain[(size_t)m * FB + e] = ok ? tot : 0.0;
}

// Oblivious trees, stage 1c: first maximum of the level totals in (feature slot, bin) order (`findmax`,
// src/fit.jl:213-217); it is the level's split if it exceeds gamma.  One CTA.
__global__ void __launch_bounds__(1024) k_obl_pick(ScanArgs a) {
    __shared__ double s_g[32];
    __shared__ int s_e[32];
    const int m = 1 << (a.level - 1);
    const int FB = a.F * a.B;
    const double *tot = a.obl_gain + (size_t)m * FB;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    double bg = a.gamma;
    int be = 0x7fffffff;
    for (int e = threadIdx.x; e < FB; e += blockDim.x) {
        const double g = tot[e];
        if (g > bg) { bg = g; be = e; }
    }
    auto red = [&]() {
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            const double og = __shfl_xor_sync(FULL, bg, d);
            const int oe = __shfl_xor_sync(FULL, be, d);
            if (oe != 0x7fffffff && (og > bg || (og == bg && oe < be))) { bg = og; be = oe; }
        }
    };
    red();
    if (lane == 0) { s_g[wid] = bg; s_e[wid] = be; }
    __syncthreads();
    if (wid == 0) {
        bg = s_g[lane]; be = s_e[lane];
        red();
        if (lane == 0) { a.obl_best[0] = bg; a.obl_best[1] = be == 0x7fffffff ? -1.0 : (double)be; }
    }
}

// Writes everything that follows from the split decision of node n: child sums, tree arrays, leaf values
// (`_child_sums!` result, src/fit.jl:90-98, 120-121, 74-82, 131-135).  One warp; s_left holds the left sums.
__device__ __forceinline__ void apply_split(const ScanArgs &a, int n, bool has, double gain, int slot, int bin, const double *s_sum,
                                            double *s_left, double *s_right, int lane) {
    const int C = a.C, K = a.K;
    if (has) {
        const uint32_t feat = a.js0[slot];
        const bool numeric = a.feattypes[feat] != 0;
        for (int c = lane; c < C; c += 32) s_right[c] = s_sum[c] - s_left[c];
        __syncwarp();
        const int nl = n << 1, nr = nl + 1;
        for (int c = lane; c < C; c += 32) {
            a.nsum[(size_t)nl * C + c] = s_left[c];
            a.nsum[(size_t)nr * C + c] = s_right[c];
        }
        if (lane == 0) {
            a.t_w[n - 1] = (float)s_sum[C - 1];
            a.t_gain[n - 1] = (float)gain;
            a.t_bin[n - 1] = (uint8_t)(bin + 1);
            a.t_feat[n - 1] = (int32_t)feat + 1;
            a.t_split[n - 1] = 1;
            a.t_packed[n - 1] = feat | ((uint32_t)(bin + 1) << 16) | (1u << 24) | ((numeric ? 1u : 0u) << 25);
        }
        if (a.level + 1 == a.D) {
            // children sit at max depth: they are leaves (src/fit.jl:74-82)
            for (int k = lane; k < K; k += 32) {
                a.t_pred[(size_t)(nl - 1) * K + k] = leaf_value(a, s_left, k);
                a.t_pred[(size_t)(nr - 1) * K + k] = leaf_value(a, s_right, k);
            }
            if (lane == 0) { a.t_w[nl - 1] = (float)s_left[C - 1]; a.t_w[nr - 1] = (float)s_right[C - 1]; }
        }
    } else {
        if (lane == 0) a.t_w[n - 1] = (float)s_sum[C - 1];
        for (int k = lane; k < K; k += 32) a.t_pred[(size_t)(n - 1) * K + k] = leaf_value(a, s_sum, k);
    }
}

// Stage 2: one warp per node: first strict maximum over the (owned) features in ascending feature order and the
// left-child sums of the winner (`_child_sums!`, fit-utils.jl:472-486).  Single GPU: the split is applied at once.
// Sharded with peer access: the rank's candidate is written into every rank's candidate table instead.
template <bool K1>
__global__ void __launch_bounds__(256) k_scan_node(ScanArgs a) {
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = K1 ? 3 : a.C, B = a.B, F = a.F; // K1: one output, channels g, h, w known at compile time
    const int m = 1 << (a.level - 1);
    const int i = blockIdx.x * (blockDim.x >> 5) + wid;
    __shared__ double s_sum_all[8][72], s_left_all[8][72], s_right_all[8][72];
    double *s_sum = s_sum_all[wid], *s_left = s_left_all[wid], *s_right = s_right_all[wid];
    if (i >= m) return;
    const int n = m + i;
    // this kernel is a chain of dependent loads: everything that does not depend on the winner is requested up front
    const int kd = a.kind[n];
    const int slot_n = a.bslot[n];
    const int Fown = (F - a.rank + a.world - 1) / a.world;
    double fg[4];
    int fb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int fi = lane + 32 * u;
        fb[u] = -1; fg[u] = 0.0;
        if (fi < Fown && !a.obl_gain) {
            const int f = fi * a.world + a.rank;
            fg[u] = a.fbest_gain[(size_t)i * F + f];
            fb[u] = a.fbest_bin[(size_t)i * F + f];
        }
    }
    for (int c = lane; c < C; c += 32) s_sum[c] = a.nsum[(size_t)n * C + c];
    if (kd == EVB_KIND_NONE) return;
    const size_t FCB = (size_t)F * C * B;
    const double *hc = a.hcomp + (size_t)slot_n * FCB;
    const bool sub = kd == EVB_KIND_SUB;
    const double *hp = a.hist + (size_t)(n >> 1) * FCB;
    const double *hn = a.hist + (size_t)n * FCB;
    __syncwarp();

    double bg = a.gamma;
    int bs = 0x7fffffff, bb = -1;
    if (a.obl_gain) { // oblivious: every node of the level takes the split k_obl_pick chose (src/fit.jl:213-225)
        const double e = a.obl_best[1];
        if (e >= 0.0) { bg = a.obl_best[0]; bs = (int)e / B; bb = (int)e % B; }
    } else {
#pragma unroll
    for (int u = 0; u < 4; ++u)
        if (fb[u] >= 0 && fg[u] > bg) { bg = fg[u]; bs = (lane + 32 * u) * a.world + a.rank; bb = fb[u]; }
    for (int fi = lane + 128; fi < Fown; fi += 32) {
        const int f = fi * a.world + a.rank;
        const double g = a.fbest_gain[(size_t)i * F + f];
        const int b = a.fbest_bin[(size_t)i * F + f];
        if (b >= 0 && g > bg) { bg = g; bs = f; bb = b; }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const double og = __shfl_xor_sync(FULL, bg, d);
        const int os = __shfl_xor_sync(FULL, bs, d), ob = __shfl_xor_sync(FULL, bb, d);
        if (os != 0x7fffffff && (og > bg || (og == bg && os < bs))) { bg = og; bs = os; bb = ob; }
    }
    }
    const bool has = bs != 0x7fffffff;
    if (has) {
        const bool numeric = a.feattypes[a.js0[bs]] != 0;
        const size_t fo = (size_t)bs * C * B;
        const size_t qo = a.qsum ? (size_t)slot_n * B * a.SC + a.js0[bs] : 0;
        const double qi = a.qsum ? a.qinv[0] : 0.0;
        // entry (channel c, bin b) of the winner's histogram in this node
        auto entry = [&](int c, int b) -> double {
            const size_t o = fo + (size_t)c * B + b;
            if (a.world > 1) return hn[o]; // sharded: the summed histogram of every scanned node is retained locally for the owned features
            double built;
            if (a.qsum) {
                const size_t q = qo + (size_t)b * a.SC;
                built = c < a.K ? (double)(long long)a.qsum[q] * qi : (c == C - 1 ? 1.0 : 2.0) * (double)a.qcnt[q];
            } else {
                built = hc[o];
            }
            return sub ? hp[o] - built : built;
        };
        const int b0 = numeric ? lane : bb, b1 = bb;
        if (K1) { // the three channels side by side; the mse hessian is twice the weight, entry by entry
            double vg = 0.0, vh = 0.0, vw = 0.0;
            for (int b = b0; b <= b1; b += 32) {
                vg += entry(0, b);
                if (!a.elide_h) vh += entry(1, b);
                vw += entry(2, b);
                if (!numeric) break;
            }
            if (numeric) {
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) {
                    vg += __shfl_xor_sync(FULL, vg, d);
                    vh += __shfl_xor_sync(FULL, vh, d);
                    vw += __shfl_xor_sync(FULL, vw, d);
                }
            }
            if (a.elide_h) vh = 2.0 * vw;
            if (lane == 0) { s_left[0] = vg; s_left[1] = vh; s_left[2] = vw; }
        } else {
            for (int c = 0; c < C; ++c) {
                double v = 0.0;
                for (int b = b0; b <= b1; b += 32) {
                    v += entry(c, b);
                    if (!numeric) break;
                }
                if (numeric) v = warp_sum(v);
                if (lane == 0) s_left[c] = v;
            }
        }
        __syncwarp();
    }
    if (a.world == 1) {
        apply_split(a, n, has, bg, bs, bb, s_sum, s_left, s_right, lane);
        return;
    }
    const int RC = 3 + C;
    for (int q = 0; q < a.world; ++q) {
        double *rec = a.peer_cand[q] + ((size_t)i * a.world + a.rank) * RC;
        if (lane == 0) { rec[0] = bg; rec[1] = has ? (double)bs : -1.0; rec[2] = (double)bb; }
        if (has) for (int c = lane; c < C; c += 32) rec[3 + c] = s_left[c];
    }
}

// Stage 3 (sharded with peer access only): every rank picks, for every node, the best of the ranks' candidates
// (ties: lowest feature slot, as in the single-GPU order) and applies it.  All ranks read identical tables.
__global__ void __launch_bounds__(256) k_scan_final(ScanArgs a) {
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = a.C;
    const int m = 1 << (a.level - 1);
    const int i = blockIdx.x * (blockDim.x >> 5) + wid;
    __shared__ double s_sum_all[8][72], s_left_all[8][72], s_right_all[8][72];
    double *s_sum = s_sum_all[wid], *s_left = s_left_all[wid], *s_right = s_right_all[wid];
    if (i >= m) return;
    const int n = m + i;
    if (a.kind[n] == EVB_KIND_NONE) return;
    for (int c = lane; c < C; c += 32) s_sum[c] = a.nsum[(size_t)n * C + c];
    const int RC = 3 + C;
    double bg = a.gamma;
    int bs = 0x7fffffff, bb = -1, bq = -1;
    if (lane < a.world) {
        const double *rec = a.cand_local + ((size_t)i * a.world + lane) * RC;
        const double g = __ldcv(rec), sl = __ldcv(rec + 1), bn = __ldcv(rec + 2);
        if (sl >= 0.0 && g > bg) { bg = g; bs = (int)sl; bb = (int)bn; bq = lane; }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const double og = __shfl_xor_sync(FULL, bg, d);
        const int os = __shfl_xor_sync(FULL, bs, d), ob = __shfl_xor_sync(FULL, bb, d), oq = __shfl_xor_sync(FULL, bq, d);
        if (os != 0x7fffffff && (og > bg || (og == bg && os < bs))) { bg = og; bs = os; bb = ob; bq = oq; }
    }
    const bool has = bs != 0x7fffffff;
    if (has) {
        const double *rec = a.cand_local + ((size_t)i * a.world + bq) * RC;
        for (int c = lane; c < C; c += 32) s_left[c] = __ldcv(rec + 3 + c);
    }
    __syncwarp();
    apply_split(a, n, has, bg, bs, bb, s_sum, s_left, s_right, lane);
}

// Cross-GPU barrier for the peer-access path: every rank writes the sequence number into its slot of every
// rank's flag array and waits (bounded, ~2 s) until all slots of its own array have reached it.
struct BarrierArgs {
    int *peer_flags[EVB_MAX_PEERS];
    int *flags_local;
    int *err;
    int world, rank;
    int *seq_dev; // barriers passed so far: kept on the device so that a replayed CUDA graph keeps counting
    unsigned max_polls; // polls of ~100 ns before the wait gives up with EVB_DERR_PEER (20 M: about two seconds)
};
__global__ void k_peer_barrier(BarrierArgs a) {
    const int t = threadIdx.x;
    int seq = 0;
    if (t == 0) { seq = *a.seq_dev + 1; *a.seq_dev = seq; } // one warp, launched alone on the stream: no race
    seq = __shfl_sync(FULL, seq, 0);
    if (t >= a.world) return;
    __threadfence_system();
    *(volatile int *)(a.peer_flags[t] + a.rank) = seq;
    __threadfence_system();
    volatile int *mine = a.flags_local + t;
    for (unsigned it = 0; it < a.max_polls; ++it) {
        if (*mine - seq >= 0) { __threadfence_system(); return; }
        if ((it & 1023u) == 1023u && *(volatile int *)a.err != 0) return;
        __nanosleep(100);
    }
    atomicCAS(a.err, 0, EVB_DERR_PEER);
}

// ------------------------------------------------------------------------------------------ partition
struct PartArgs {
    const uint8_t *xC; // feature-major bins [nfeats][n]: the rows of a node ascend, so its reads of one feature are
                       // as dense as the node is (whole sectors near the root, one sector per row deep down)
    long long n;
    const uint32_t *rows_in;
    uint32_t *rows_out;
    const uint8_t *t_split;
    const uint32_t *t_packed;
    int32_t *seg_start, *seg_cnt, *gcnt, *nleft, *bslot, *cum, *slot_node;
    const int32_t *gnleft;
    uint8_t *kind;
    int32_t *ibase;       // [level nodes + 1] exclusive prefix of items per node
    int32_t *item_left, *item_lprefix; // left rows of every item; their running sum over all items of the level
    int32_t *nbase;       // [level nodes] value of the running sum at the node's first item
    uint32_t *item_bits;
    LevelPlan *plan;
    const double *nsum; // node sums [id][C]; channel C-1 is the sum of weights
    int C, by_weight;   // by_weight: sharded run, pick the build child by weight sum instead of row count
    int RS, level, D, max_items;
    int *err;
};

__global__ void __launch_bounds__(1024) k_part_plan(PartArgs a) {
    __shared__ int sm[33];
    const int lo = 1 << (a.level - 1), m = lo;
    int carry = 0;
    for (int base = 0; base < m; base += blockDim.x) {
        const int i = base + threadIdx.x;
        int cnt = 0;
        if (i < m && a.t_split[lo + i - 1]) cnt = (a.seg_cnt[lo + i] + EVB_PART_CHUNK - 1) / EVB_PART_CHUNK;
        int total;
        const int ex = block_excl_scan(cnt, sm, &total);
        if (i < m) a.ibase[i] = carry + ex;
        carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (carry > a.max_items) { atomicCAS(a.err, 0, EVB_DERR_PLAN); carry = 0; }
        a.ibase[m] = carry;
        a.plan[a.level].nitems = carry;
    }
}

__device__ __forceinline__ void item_lookup(const PartArgs &a, int item, int &n, int &chunk) {
    const int m = 1 << (a.level - 1);
    int l = 0, r = m - 1; // largest i with ibase[i] <= item
    while (l < r) { const int mid = (l + r + 1) >> 1; if (a.ibase[mid] <= item) l = mid; else r = mid - 1; }
    n = m + l;
    chunk = item - a.ibase[l];
}

__global__ void __launch_bounds__(EVB_PART_THREADS) k_part_flags(PartArgs a) {
    __shared__ int s_cnt[EVB_PART_THREADS / 32];
    const int nitems = a.plan[a.level].nitems;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        int n, chunk;
        item_lookup(a, item, n, chunk);
        const int start = a.seg_start[n] + chunk * EVB_PART_CHUNK;
        const int cnt = min(EVB_PART_CHUNK, a.seg_cnt[n] - chunk * EVB_PART_CHUNK);
        const uint32_t pk = a.t_packed[n - 1];
        const uint32_t feat = pk & 0xffffu, bin = (pk >> 16) & 0xffu;
        const bool numeric = (pk >> 25) & 1u;
        int local = 0;
        constexpr int NI = EVB_PART_CHUNK / EVB_PART_THREADS;
        // all row ids first, then all gathers: eight independent loads in flight per thread in each phase
        uint32_t row[NI], x[NI];
#pragma unroll
        for (int i8 = 0; i8 < NI; ++i8) {
            const int pos = i8 * EVB_PART_THREADS + threadIdx.x;
            row[i8] = pos < cnt ? __ldg(a.rows_in + start + pos) : 0xffffffffu;
        }
        const uint8_t *xf = a.xC + (size_t)feat * a.n;
#pragma unroll
        for (int i8 = 0; i8 < NI; ++i8) x[i8] = row[i8] != 0xffffffffu ? (uint32_t)__ldg(xf + row[i8]) : 0xffffu;
#pragma unroll
        for (int i8 = 0; i8 < NI; ++i8) {
            const bool left = x[i8] != 0xffffu && (numeric ? (x[i8] <= bin) : (x[i8] == bin)); // split_set! predicate (fit-utils.jl:173, 291)
            const unsigned bal = __ballot_sync(FULL, left);
            if (lane == 0) {
                a.item_bits[(size_t)item * (EVB_PART_CHUNK / 32) + i8 * (EVB_PART_THREADS / 32) + wid] = bal;
                local += __popc(bal);
            }
        }
        if (lane == 0) s_cnt[wid] = local;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < EVB_PART_THREADS / 32; ++w) t += s_cnt[w];
            a.item_left[item] = t;
        }
        __syncthreads();
    }
}

// Exclusive prefix of the left counts of every split node's work items and the node's left total.  Runs inside the
// single-CTA plan kernel.
__device__ void part_prefix(const PartArgs &a, int *sm) {
    const int lo = 1 << (a.level - 1), m = lo;
    const int nitems = a.ibase[m];
    // one running sum over the items of all nodes (they are ordered by node) ...
    int running = 0;
    for (int base = 0; base < nitems; base += blockDim.x) {
        const int idx = base + threadIdx.x;
        const int v = idx < nitems ? a.item_left[idx] : 0;
        int total;
        const int ex = block_excl_scan(v, sm, &total);
        if (idx < nitems) a.item_lprefix[idx] = running + ex;
        running += total;
        __syncthreads();
    }
    __threadfence_block();
    __syncthreads();
    // ... and per node the value it had at the node's first item: k_part_scatter subtracts it
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
        const int j0 = a.ibase[i], j1 = a.ibase[i + 1];
        const int p0 = j0 < nitems ? a.item_lprefix[j0] : running;
        const int p1 = j1 < nitems ? a.item_lprefix[j1] : running;
        a.nbase[i] = p0;
        a.nleft[lo + i] = p1 - p0; // a node that is not split has no items: 0
    }
    __threadfence_block();
    __syncthreads();
}

// children segments / counts, build-or-subtract choice (src/fit.jl:123-129: the child with fewer rows is
// built, ties build the left child), build slots and the histogram plan of the next level
__global__ void __launch_bounds__(1024) k_level_plan(PartArgs a) {
    __shared__ int sm[33];
    part_prefix(a, sm);
    const int lo = 1 << (a.level - 1), m = lo;
    const bool scan_children = a.level + 1 < a.D;
    int carry_slot = 0, carry_rows = 0;
    for (int base = 0; base < m; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const int n = lo + i;
        int sp = 0, cnt_build = 0, build_child = 0;
        if (i < m && a.t_split[n - 1]) {
            sp = 1;
            const int L = n << 1, Rn = L + 1;
            const int nl = a.nleft[n], gl = a.gnleft[n];
            const int s0 = a.seg_start[n], c0 = a.seg_cnt[n], g0 = a.gcnt[n];
            a.seg_start[L] = s0; a.seg_cnt[L] = nl; a.gcnt[L] = gl;
            a.seg_start[Rn] = s0 + nl; a.seg_cnt[Rn] = c0 - nl; a.gcnt[Rn] = g0 - gl;
            if (scan_children) {
                // The reference builds the child with fewer rows, ties build the left one (src/fit.jl:123-129).
                // With rows sharded over GPUs the global row counts would cost one more collective per level, so
                // there the child with the smaller weight sum is built: every rank knows the sums from the split
                // scan, and with unit weights it is the same rule.
                const bool build_left = a.by_weight
                    ? a.nsum[(size_t)Rn * a.C + a.C - 1] >= a.nsum[(size_t)L * a.C + a.C - 1]
                    : (g0 - gl) >= gl;
                a.kind[L] = build_left ? EVB_KIND_BUILD : EVB_KIND_SUB;
                a.kind[Rn] = build_left ? EVB_KIND_SUB : EVB_KIND_BUILD;
                build_child = build_left ? L : Rn;
                cnt_build = build_left ? nl : c0 - nl;
            }
        }
        int tot_s, tot_r;
        const int slot = carry_slot + block_excl_scan(scan_children ? sp : 0, sm, &tot_s);
        __syncthreads();
        const int cpre = carry_rows + block_excl_scan(cnt_build, sm, &tot_r);
        if (sp && scan_children) {
            a.bslot[n << 1] = slot; a.bslot[(n << 1) + 1] = slot;
            a.slot_node[slot] = build_child;
            a.cum[slot] = cpre;
        }
        carry_slot += tot_s; carry_rows += tot_r;
        __syncthreads();
    }
    if (threadIdx.x == 0 && a.level + 1 <= a.D) {
        a.cum[carry_slot] = carry_rows;
        a.plan[a.level + 1].nbuild = carry_slot;
        a.plan[a.level + 1].R = carry_rows;
    }
}

__global__ void __launch_bounds__(EVB_PART_THREADS) k_part_scatter(PartArgs a) {
    constexpr int NW = EVB_PART_CHUNK / 32;
    __shared__ uint32_t s_bits[NW];
    __shared__ int s_pref[NW];
    const int nitems = a.plan[a.level].nitems;
    const int lane = threadIdx.x & 31;
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        int n, chunk;
        item_lookup(a, item, n, chunk);
        const int start = a.seg_start[n] + chunk * EVB_PART_CHUNK;
        const int cnt = min(EVB_PART_CHUNK, a.seg_cnt[n] - chunk * EVB_PART_CHUNK);
        const int nL = a.nleft[n], lp = a.item_lprefix[item] - a.nbase[n - (1 << (a.level - 1))];
        if (threadIdx.x < NW) s_bits[threadIdx.x] = a.item_bits[(size_t)item * NW + threadIdx.x];
        __syncthreads();
        if (threadIdx.x < 32) { // NW == 64: two words per lane
            const int c0 = __popc(s_bits[2 * lane]), c1 = __popc(s_bits[2 * lane + 1]);
            const int incl = warp_incl_scan_i(c0 + c1, lane);
            s_pref[2 * lane] = incl - c0 - c1;
            s_pref[2 * lane + 1] = incl - c1;
        }
        __syncthreads();
        const int dstL = a.seg_start[n] + lp;
        const int dstR = a.seg_start[n] + nL + (chunk * EVB_PART_CHUNK - lp);
        constexpr int NI = EVB_PART_CHUNK / EVB_PART_THREADS;
        uint32_t row[NI];
#pragma unroll
        for (int i8 = 0; i8 < NI; ++i8) {
            const int pos = i8 * EVB_PART_THREADS + threadIdx.x;
            row[i8] = pos < cnt ? __ldg(a.rows_in + start + pos) : 0u;
        }
#pragma unroll
        for (int i8 = 0; i8 < NI; ++i8) {
            const int pos = i8 * EVB_PART_THREADS + threadIdx.x;
            if (pos < cnt) {
                const uint32_t word = s_bits[pos >> 5];
                const int before = s_pref[pos >> 5] + __popc(word & ((1u << lane) - 1u));
                if ((word >> lane) & 1u) a.rows_out[dstL + before] = row[i8];
                else a.rows_out[dstR + (pos - before)] = row[i8];
            }
        }
        __syncthreads();
    }
}

PartArgs make_part_args(evb_handle *h, int level) {
    PartArgs a;
    a.xC = h->xC; a.n = h->n; a.rows_in = h->rows[(level - 1) & 1]; a.rows_out = h->rows[level & 1];
    a.t_split = h->t_split; a.t_packed = h->t_packed;
    a.seg_start = h->seg_start; a.seg_cnt = h->seg_cnt; a.gcnt = h->gcnt; a.nleft = h->nleft; a.gnleft = h->gnleft;
    a.bslot = h->bslot; a.cum = h->cum; a.slot_node = h->slot_node; a.kind = h->kind;
    a.ibase = h->item_node; a.nbase = h->item_node + (1 << (h->D > 1 ? h->D - 1 : 0)) + 1; a.item_left = h->item_left; a.item_lprefix = h->item_lprefix; a.item_bits = h->item_bits;
    a.plan = h->plan; a.RS = h->RS; a.level = level; a.D = h->D; a.max_items = h->max_items; a.err = h->d_err;
    a.nsum = h->nsum; a.C = h->C; a.by_weight = h->world > 1 ? 1 : 0;
    return a;
}

} // namespace

static_assert(EVB_PART_CHUNK == 2048 && EVB_PART_THREADS == 256, "k_part_scatter assumes 64 ballot words per item");

int32_t evb_launch_tree_reset(evb_handle *h) {
    ResetArgs a;
    a.seg_start = h->seg_start; a.seg_cnt = h->seg_cnt; a.gcnt = h->gcnt; a.nleft = h->nleft; a.gnleft = h->gnleft;
    a.bslot = h->bslot; a.t_feat = h->t_feat; a.kind = h->kind; a.t_bin = h->t_bin; a.t_split = h->t_split;
    a.t_gain = h->t_gain; a.t_w = h->t_w; a.t_pred = h->t_pred; a.t_packed = h->t_packed; a.nsum = h->nsum;
    a.plan = h->plan; a.nids = h->nn + 2; a.nn = h->nn; a.K = h->K; a.C = h->C; a.D = h->D;
    const int threads = 256, blocks = (a.nids + threads - 1) / threads;
    evb_tic(h, EVB_T_PLAN);
    k_tree_reset<<<blocks, threads, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PLAN);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_root_plan(evb_handle *h) {
    RootArgs a;
    a.seg_start = h->seg_start; a.seg_cnt = h->seg_cnt; a.gcnt = h->gcnt; a.bslot = h->bslot; a.cum = h->cum;
    a.slot_node = h->slot_node; a.nleft = h->nleft; a.gnleft = h->gnleft; a.kind = h->kind; a.plan = h->plan;
    evb_tic(h, EVB_T_PLAN);
    k_root_plan<<<1, 32, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PLAN);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

static int32_t launch_peer_barrier(evb_handle *h) {
    BarrierArgs b;
    for (int q = 0; q < EVB_MAX_PEERS; ++q) b.peer_flags[q] = q < h->world ? h->peer_flags[q] : nullptr;
    b.flags_local = h->peer_flags[h->rank]; b.err = h->d_err; b.world = h->world; b.rank = h->rank; b.seq_dev = h->d_barrier_seq;
    b.max_polls = 20000000u;
    k_peer_barrier<<<1, 32, 0, h->st>>>(b);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// Diagnostic: one flag barrier of a two-rank world whose second rank does not exist, on the handle's own GPU: rank 1's
// flag is never written, so the wait runs out after `max_polls` polls and the kernel leaves EVB_DERR_PEER in the
// error word -- the path a sharded run takes when a peer stops answering, without a second GPU and without a hang.
int32_t evb_launch_lonely_barrier(evb_handle *h, int *flags, int *seq, unsigned max_polls) {
    BarrierArgs b;
    for (int q = 0; q < EVB_MAX_PEERS; ++q) b.peer_flags[q] = q < 2 ? flags : nullptr;
    b.flags_local = flags; b.err = h->d_err; b.world = 2; b.rank = 0; b.seq_dev = seq; b.max_polls = max_polls;
    k_peer_barrier<<<1, 32, 0, h->st>>>(b);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_scan(evb_handle *h, int level) {
    ScanArgs a;
    a.hcomp = h->hcomp; a.hist = h->hist; a.nsum = h->nsum; a.kind = h->kind; a.bslot = h->bslot; a.js0 = h->js_d;
    a.feattypes = h->feattypes_d; a.mono = h->mono_d; a.t_feat = h->t_feat; a.t_bin = h->t_bin; a.t_split = h->t_split;
    a.t_gain = h->t_gain; a.t_w = h->t_w; a.t_pred = h->t_pred; a.t_packed = h->t_packed;
    a.F = h->F; a.C = h->C; a.K = h->K; a.B = h->B; a.level = level; a.D = h->D; a.hist_nodes = h->hist_nodes;
    a.loss = h->p.loss; a.neb = -h->p.eta / (double)h->p.bagging_size;
    a.elide_h = h->Ce != h->C ? 1 : 0;
    const bool direct = evb_q2_direct(h);
    a.qsum = direct ? h->hsum_q : nullptr; a.qcnt = direct ? h->hcnt_q : nullptr; a.qinv = h->d_qinv; a.SC = h->q2.SC;
    a.lambda = h->p.lambda; a.L2 = h->p.L2; a.gamma = h->p.gamma; a.min_weight = h->p.min_weight;
    a.fbest_gain = h->fbest_gain; a.fbest_bin = h->fbest_bin;
    a.obl_gain = h->obl_gain; a.obl_best = h->obl_best;
    a.plan = h->plan + level; a.slot_node = h->slot_node;
    const bool p2p = h->p2p && h->world > 1;
    a.world = p2p ? h->world : 1; a.rank = p2p ? h->rank : 0;
    for (int q = 0; q < EVB_MAX_PEERS; ++q) a.peer_cand[q] = p2p && q < h->world ? h->peer_cand[q] : nullptr;
    a.cand_local = p2p ? h->peer_cand[h->rank] : nullptr;
    const int m = evb_level_nodes(level);
    const int slots = evb_level_slots(level);
    const int Fown = (h->F - a.rank + a.world - 1) / a.world;
    if (p2p) {
        // all ranks' histograms of this level are complete -> sum the owned feature slots from the peers' memory
        evb_tic(h, EVB_T_ALLREDUCE);
        int32_t rc = launch_peer_barrier(h);
        PeerReduceArgs r;
        for (int q = 0; q < EVB_MAX_PEERS; ++q) r.peer_hcomp[q] = q < h->world ? h->peer_hcomp[q] : nullptr;
        r.hsum = h->hsum; r.plan = h->plan + level; r.world = h->world; r.rank = h->rank; r.F = h->F; r.CB = h->C * h->B; r.level = level;
        r.K = h->K; r.elided = h->Ce != h->C ? 1 : 0;
        if (rc == EVB_OK) k_peer_reduce<<<slots * (Fown + 1), 256, 0, h->st>>>(r);
        evb_toc(h, EVB_T_ALLREDUCE);
        EVB_CHECK(rc);
        a.hcomp = h->hsum;
    }
    const long long warps = (long long)slots * Fown * (level > 1 ? 2 : 1);
    evb_tic(h, EVB_T_SCAN);
    if (warps > 0) {
        const unsigned grid = (unsigned)((warps + 7) / 8);
        const bool own = h->p.loss >= EVB_MAE;
        const bool obl = h->obl_gain != nullptr;
#define EVB_SCAN(M) do { \
            if (own && obl) k_scan_feat<M, true, true, false><<<grid, 256, 0, h->st>>>(a); \
            else if (own) k_scan_feat<M, true, false, false><<<grid, 256, 0, h->st>>>(a); \
            else if (obl) k_scan_feat<M, false, true, false><<<grid, 256, 0, h->st>>>(a); \
            else if (h->K == 1 && h->C == 3) k_scan_feat<M, false, false, true><<<grid, 256, 0, h->st>>>(a); \
            else k_scan_feat<M, false, false, false><<<grid, 256, 0, h->st>>>(a); } while (0)
        if (h->B <= 32) EVB_SCAN(1); else if (h->B <= 64) EVB_SCAN(2); else if (h->B <= 128) EVB_SCAN(4); else EVB_SCAN(8);
#undef EVB_SCAN
    }
    evb_toc(h, EVB_T_SCAN);
    if (h->obl_gain && level < h->D) {
        evb_tic(h, EVB_T_SCAN);
        k_obl_sum<<<(h->F * h->B + 127) / 128, 128, 0, h->st>>>(a);
        k_obl_pick<<<1, 1024, 0, h->st>>>(a);
        evb_toc(h, EVB_T_SCAN);
    }
    evb_tic(h, EVB_T_SCAN);
    if (h->K == 1 && h->C == 3) k_scan_node<true><<<(m + 7) / 8, 256, 0, h->st>>>(a);
    else k_scan_node<false><<<(m + 7) / 8, 256, 0, h->st>>>(a);
    evb_toc(h, EVB_T_SCAN);
    if (p2p) {
        evb_tic(h, EVB_T_ALLREDUCE); int32_t rc = launch_peer_barrier(h); evb_toc(h, EVB_T_ALLREDUCE); EVB_CHECK(rc);
        evb_tic(h, EVB_T_SCAN);
        k_scan_final<<<(m + 7) / 8, 256, 0, h->st>>>(a);
        evb_toc(h, EVB_T_SCAN);
    }
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_partition(evb_handle *h, int level) {
    PartArgs a = make_part_args(h, level);
    const int m = evb_level_nodes(level);
    int pgrid = h->num_sms * 8;
    if (pgrid > h->max_items) pgrid = h->max_items;
    if (pgrid < 1) pgrid = 1;
    evb_tic(h, EVB_T_PLAN);
    k_part_plan<<<1, 1024, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PLAN);
    evb_tic(h, EVB_T_PARTITION);
    k_part_flags<<<pgrid, EVB_PART_THREADS, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PARTITION);
    evb_tic(h, EVB_T_PLAN);
    k_level_plan<<<1, 1024, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PLAN);
    evb_tic(h, EVB_T_PARTITION);
    k_part_scatter<<<pgrid, EVB_PART_THREADS, 0, h->st>>>(a);
    evb_toc(h, EVB_T_PARTITION);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}
