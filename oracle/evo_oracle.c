/*
 * CPU oracle for the EvoTrees training / inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference's
 * CPU algorithm (EvoTrees.jl v0.19, `device=:cpu`).  It exists so that the CUDA
 * library can be checked against it; nothing in the shipped library calls it.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
 * load the shared object built from this file.
 *
 * PARITY PINNING.  The reference ships no golden vectors for histograms, gains
 * or tree structure and no Julia runtime was available when this was written, so
 * for those quantities this oracle is *unpinned*: it follows the reference source
 * line by line (citations below) but has not been diffed against a live run of the
 * reference.  What the reference's own tests do pin -- the scalar loss
 * gradients/hessians (test/metrics.jl:134-232), the softplus/invsoftplus round
 * trip, the inverse link (test/metrics.jl:199-204) and the traversal rule
 * `nid = nid<<1 + !cond` (test/predict-leaf-idx.jl:25-73) -- is checked against
 * this file in tests/test_oracle.py.
 *
 * Conventions: arrays use the reference's memory layout (Julia column-major):
 *   x_bin  [nobs x nfeats]  uint8, x_bin[i + nobs*j], values 1..nbins
 *   grad   [C x nobs]       float, grad[c + C*i], C = 2K+1, rows g_1..g_K,h_1..h_K,w
 *   pred   [K x nobs]       float
 *   hist   [C x nbins x nfeats x nnodes] double (as src/init.jl:204)
 * Row ids `is`, feature ids `js`, node ids and `cond_bin` are 1-based like the
 * reference; `feat[n]==0` / `cond_bin[n]==0` mean "no split".
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORC_MSE = 0, ORC_LOGLOSS = 1, ORC_MLOGLOSS = 2, ORC_GAUSSIAN_MLE = 3, ORC_POISSON = 4, ORC_GAMMA = 5, ORC_TWEEDIE = 6, ORC_LOGISTIC_MLE = 7,
       ORC_MAE = 8, ORC_CRED_VAR = 9, ORC_CRED_STD = 10, ORC_QUANTILE = 11, ORC_MULTIQUANTILE = 12 };
static inline int orc_is_mle(int loss) { return loss == ORC_GAUSSIAN_MLE || loss == ORC_LOGISTIC_MLE; }

typedef struct {
    int32_t loss, K, nbins, max_depth, bagging_size, tree_type;
    double eta, lambda, L2, gamma, min_weight;
    double alpha;     /* quantile loss */
    double alphas[8]; /* multiquantile loss: K values */
} orc_params;
static inline int orc_is_shift(int loss) { return loss == 8 || loss == 11 || loss == 12; } /* mae-type gain: MAE, Quantile, MultiQuantile (split.jl:68, 119) */

/* ---- scalar math: src/loss.jl:239-268 ------------------------------------------------ */
static inline float orc_sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }     /* loss.jl:249-251 */
static inline float orc_softplusf(float x) {                                       /* loss.jl:257-260 */
    float ax = fabsf(x);
    return fmaxf(x, 0.0f) + log1pf(expf(-ax));
}
float orc_sigmoid(float x) { return orc_sigmoidf(x); }
float orc_softplus(float x) { return orc_softplusf(x); }
double orc_softplus64(double x) { return fmax(x, 0.0) + log1p(exp(-fabs(x))); }
double orc_invsoftplus64(double x) { return x + log(-expm1(-x)); }                  /* loss.jl:266-268 */
double orc_sigmoid64(double x) { return 1.0 / (1.0 + exp(-x)); }

/* Gaussian MLE gradient / Fisher information in double, for the known-answer tests.
 * src/loss.jl:194-203 */
void orc_gaussian_grad_hess64(double loc, double scale_raw, double y, double out[4]) {
    double scale = orc_softplus64(scale_raw);
    double dscale = orc_sigmoid64(scale_raw);
    double resid = loc - y;
    out[0] = resid / (scale * scale);
    out[1] = (1.0 - resid * resid / (scale * scale)) * dscale / scale;
    out[2] = 1.0 / (scale * scale);
    out[3] = 2.0 * (dscale / scale) * (dscale / scale);
}
/* softmax gradient/hessian for one class in double.  src/loss.jl:95-98 */
void orc_mlogloss_grad_hess64(double pk, double isum, int is_target, double out[2]) {
    double prob = exp(pk) / isum;
    out[0] = is_target ? prob - 1.0 : prob;
    out[1] = prob * (1.0 - prob);
}

/* ---- update_grads!: src/loss.jl:100-128, 219-236 (Float32 arithmetic like the reference) */
void orc_update_grads(const orc_params *p, int64_t nobs, const float *pred, const void *yv, float *grad) {
    const int K = p->K, C = 2 * K + 1;
    if (p->loss == ORC_MSE || p->loss == ORC_LOGLOSS || p->loss == ORC_POISSON || p->loss == ORC_GAMMA || p->loss == ORC_TWEEDIE) {
        const float *y = (const float *)yv; /* [nobs] or [K x nobs] */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int k = 0; k < K; k++) {
                float pk = pred[k + K * i], yk = y[k + K * i];
                float g, h;
                if (p->loss == ORC_MSE) { g = 2.0f * (pk - yk); h = 2.0f; }          /* loss.jl:52 */
                else if (p->loss == ORC_LOGLOSS) { float s = orc_sigmoidf(pk); g = s - yk; h = s * (1.0f - s); } /* loss.jl:54-57 */
                else if (p->loss == ORC_POISSON) { float pr = expf(pk); g = pr - yk; h = pr; }                     /* loss.jl:59-62 */
                else if (p->loss == ORC_GAMMA) { float pr = expf(pk); g = 2.0f * (1.0f - yk / pr); h = 2.0f * yk / pr; } /* loss.jl:64-67 */
                else { /* tweedie, rho = 1.5: loss.jl:69-76 */
                    float rho = 1.5f, pr = expf(pk);
                    g = 2.0f * (powf(pr, 2.0f - rho) - yk * powf(pr, 1.0f - rho));
                    h = 2.0f * ((2.0f - rho) * powf(pr, 2.0f - rho) - (1.0f - rho) * yk * powf(pr, 1.0f - rho));
                }
                grad[k + C * i] = g * w;
                grad[K + k + C * i] = h * w;
            }
        }
    } else if (p->loss == ORC_MULTIQUANTILE) {
        const float *y = (const float *)yv; /* one target; update_grads! src/loss.jl:160-172 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int k = 0; k < K; k++) {
                float a = (float)p->alphas[k], d = y[i] - pred[k + K * i];
                grad[k + C * i] = (d > 0.0f ? a : a - 1.0f) * w;
                grad[K + k + C * i] = d;
            }
        }
    } else if (p->loss == ORC_QUANTILE) {
        const float *y = (const float *)yv; /* quantile_grad_diff: src/loss.jl:93-98, update_grads! :146-157 (diff is not weighted) */
        const float alpha = (float)p->alpha;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int k = 0; k < K; k++) {
                float d = y[k + K * i] - pred[k + K * i];
                grad[k + C * i] = (d > 0.0f ? alpha : alpha - 1.0f) * w;
                grad[K + k + C * i] = d;
            }
        }
    } else if (p->loss == ORC_MAE || p->loss == ORC_CRED_VAR || p->loss == ORC_CRED_STD) {
        const float *y = (const float *)yv; /* mae_grad_hess / cred_grad_hess: src/loss.jl:78-84 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int k = 0; k < K; k++) {
                float d = y[k + K * i] - pred[k + K * i];
                grad[k + C * i] = d * w;
                grad[K + k + C * i] = (p->loss == ORC_MAE ? 0.0f : d * d) * w;
            }
        }
    } else if (p->loss == ORC_MLOGLOSS) {
        const uint32_t *y = (const uint32_t *)yv; /* class codes 1..K */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float isum = 0.0f;
            for (int k = 0; k < K; k++) isum += expf(pred[k + K * i]);
            float w = grad[(C - 1) + C * i];
            for (int k = 0; k < K; k++) {
                float prob = expf(pred[k + K * i]) / isum;
                float g = ((uint32_t)(k + 1) == y[i]) ? prob - 1.0f : prob;
                float h = prob * (1.0f - prob);
                grad[k + C * i] = g * w;
                grad[K + k + C * i] = h * w;
            }
        }
    } else if (p->loss == ORC_LOGISTIC_MLE) { /* mle2p_grad_hess, loss.jl:207-217 */
        const float *y = (const float *)yv;
        const int Y = K / 2;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int t = 0; t < Y; t++) {
                int gb = 2 * t, hb = 2 * Y + 2 * t;
                float loc = pred[2 * t + K * i], sr = pred[2 * t + 1 + K * i];
                float scale = orc_softplusf(sr), ds = orc_sigmoidf(sr);
                float z = (y[t + Y * i] - loc) / scale, th = tanhf(z / 2.0f);
                grad[gb + C * i] = -th / scale * w;
                grad[gb + 1 + C * i] = (1.0f - z * th) * ds / scale * w;
                grad[hb + C * i] = 1.0f / (3.0f * scale * scale) * w;
                grad[hb + 1 + C * i] = (3.14159274f * 3.14159274f + 3.0f) / 9.0f * (ds / scale) * (ds / scale) * w;
            }
        }
    } else if (p->loss == ORC_GAUSSIAN_MLE) {
        const float *y = (const float *)yv; /* [Y x nobs], Y = K/2 */
        const int Y = K / 2;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nobs; i++) {
            float w = grad[(C - 1) + C * i];
            for (int t = 0; t < Y; t++) {
                int gb = 2 * t, hb = 2 * Y + 2 * t;
                float loc = pred[2 * t + K * i], sr = pred[2 * t + 1 + K * i];
                float scale = orc_softplusf(sr), ds = orc_sigmoidf(sr);
                float resid = loc - y[t + Y * i];
                float s2 = scale * scale;
                float g1 = resid / s2;
                float g2 = (1.0f - resid * resid / s2) * ds / scale;
                float h1 = 1.0f / s2;
                float h2 = 2.0f * (ds / scale) * (ds / scale);
                grad[gb + C * i] = g1 * w;
                grad[gb + 1 + C * i] = g2 * w;
                grad[hb + C * i] = h1 * w;
                grad[hb + 1 + C * i] = h2 * w;
            }
        }
    }
}

/* ---- gains: src/split.jl:1,58-66,108-117 ---------------------------------------------- */
static inline double term_gh(double g, double h, double w, double lambda, double L2, double eps) {
    return g * g / fmax(eps, h + lambda * w + L2) / 2.0;
}
/* _term_shift / _term_cred / _cred_Z: src/split.jl:2-4, src/loss.jl:275-289 */
static inline double term_shift(double g, double w, double mu_p, double d) { return fabs(g / w - mu_p) * w / d; }
static inline double term_cred(int loss, double m1, double m2, double w, double L2, double eps) {
    double vhm = (m1 / w) * (m1 / w);
    double evpv = fmax(eps, m2 / w - vhm);
    double z = loss == ORC_CRED_VAR ? vhm / (vhm + evpv) : sqrt(vhm) / (sqrt(vhm) + sqrt(evpv));
    return z * fabs(m1) / (1.0 + L2 / w);
}
static double node_gain(int loss, const double *s, int C, double lambda, double L2, double eps) {
    int K = (C - 1) / 2;
    double w = s[2 * K], gain = 0.0;
    if (orc_is_shift(loss)) return 0.0;                                                 /* split.jl:68 */
    if (loss == ORC_CRED_VAR || loss == ORC_CRED_STD) {                                 /* split.jl:70-78 */
        for (int k = 0; k < K; k++) gain += term_cred(loss, s[k], s[K + k], w, L2, eps);
        return gain;
    }
    for (int k = 0; k < K; k++) gain += term_gh(s[k], s[K + k], w, lambda, L2, eps);
    return gain;
}
static double split_gain(int loss, const double *s, const double *sl, int C, double w_l, double w_r, double lambda,
                         double L2, double eps) {
    int K = (C - 1) / 2;
    double gain = 0.0;
    if (orc_is_shift(loss)) {                                                           /* split.jl:119-130 */
        double w_p = s[2 * K];
        double d_l = fmax(eps, 1.0 + lambda + L2 / w_l), d_r = fmax(eps, 1.0 + lambda + L2 / w_r);
        for (int k = 0; k < K; k++) {
            double mu_p = s[k] / w_p;
            gain += term_shift(sl[k], w_l, mu_p, d_l) + term_shift(s[k] - sl[k], w_r, mu_p, d_r);
        }
        return gain;
    }
    if (loss == ORC_CRED_VAR || loss == ORC_CRED_STD) {                                 /* split.jl:132-141 */
        for (int k = 0; k < K; k++)
            gain += term_cred(loss, sl[k], sl[K + k], w_l, L2, eps) + term_cred(loss, s[k] - sl[k], s[K + k] - sl[K + k], w_r, L2, eps);
        return gain;
    }
    for (int k = 0; k < K; k++) {
        double g_l = sl[k], h_l = sl[K + k];
        gain += term_gh(g_l, h_l, w_l, lambda, L2, eps) + term_gh(s[k] - g_l, s[K + k] - h_l, w_r, lambda, L2, eps);
    }
    return gain;
}
/* pred_scalar: src/predict.jl:205-208 (gradient regression), :235-238 (MLE2P) */
static double pred_scalar(const double *s, const orc_params *p) {
    const double eps = DBL_EPSILON;
    if (orc_is_shift(p->loss)) /* src/predict.jl:259-262 (the reference defines none for Quantile; used for monotone tests only) */
        return p->eta / p->bagging_size * s[0] / fmax(eps, s[2] + p->lambda * s[2] + p->L2);
    if (p->loss == ORC_CRED_VAR || p->loss == ORC_CRED_STD)   /* src/predict.jl:220-222 */
        return p->eta / p->bagging_size * s[0] / (s[2] + p->L2);
    if (orc_is_mle(p->loss))
        return -p->eta / p->bagging_size * s[0] / fmax(eps, s[2] + p->lambda * s[4] + p->L2);
    return -p->eta / p->bagging_size * s[0] / fmax(eps, s[1] + p->lambda * s[2] + p->L2);
}
/* pred_leaf_cpu!: src/predict.jl:198-204, 224-234, 241-247 */
static void pred_leaf(float *tpred, int n0, const double *s, const orc_params *p) {
    const double eps = DBL_EPSILON;
    const int K = p->K, C = 2 * K + 1;
    if (p->loss == ORC_MAE) {          /* src/predict.jl:250-257 */
        double wv = s[C - 1], denom = fmax(eps, wv + p->lambda * wv + p->L2);
        for (int k = 0; k < K; k++) tpred[k + K * n0] = (float)(p->eta / p->bagging_size * s[k] / denom);
    } else if (p->loss == ORC_CRED_VAR || p->loss == ORC_CRED_STD) {   /* src/predict.jl:211-218 */
        for (int k = 0; k < K; k++) tpred[k + K * n0] = (float)(p->eta / p->bagging_size * s[k] / (s[C - 1] + p->L2));
    } else if (orc_is_mle(p->loss)) {
        int Y = K / 2;
        double wsum = s[C - 1];
        for (int t = 0; t < Y; t++) {
            int gb = 2 * t, hb = 2 * Y + 2 * t;
            tpred[2 * t + K * n0] = (float)(-p->eta / p->bagging_size * s[gb] / fmax(eps, s[hb] + p->lambda * wsum + p->L2));
            tpred[2 * t + 1 + K * n0] =
                (float)(-p->eta / p->bagging_size * s[gb + 1] / fmax(eps, s[hb + 1] + p->lambda * wsum + p->L2));
        }
    } else {
        for (int k = 0; k < K; k++)
            tpred[k + K * n0] = (float)(-p->eta / p->bagging_size * s[k] / fmax(eps, s[k + K] + p->lambda * s[C - 1] + p->L2));
    }
}

/* ---- grow_tree!: src/fit.jl:45-143 with its helpers from src/fit-utils.jl ------------- */
typedef struct { int64_t start, len; } seg_t;
int orc_num_threads(void);

/*
 * Grow one binary tree.  Returns 0, or a negative value on bad arguments.
 * Outputs (length nn = 2^max_depth - 1 unless noted, zero-initialised here):
 *   feat int64, cond_bin uint8, w float, gain float, tpred float [K x nn], split uint8
 *   nidx  uint32 [nobs]: final node id of each sampled row (0 for rows not in `is`)   (may be NULL)
 *   hist  double [C x nbins x nfeats x nn] working/returned histograms                 (may be NULL)
 *   nsum  double [C x nn] per-node sums                                                 (may be NULL)
 */
/* pred_leaf_cpu! of the quantile loss (src/predict.jl:264-272): Statistics.quantile (type 7) of the residuals kept
 * in the hessian slot, over the rows of the node */
static int cmp_float(const void *a, const void *b) { float x = *(const float *)a, y = *(const float *)b; return (x > y) - (x < y); }
static void pred_leaf_quantile(float *tpred, int n0, const double *s, const orc_params *p, const float *grad, const uint32_t *rows, int64_t len) {
    const int K = p->K, C = 2 * K + 1;
    float *v = (float *)malloc(sizeof(float) * (len > 0 ? len : 1));
    double denom = 1.0 + p->lambda + p->L2 / s[C - 1];
    if (p->loss == ORC_QUANTILE) denom = fmax(DBL_EPSILON, denom); /* :270 clamps, the multiquantile method (:279) does not */
    for (int k = 0; k < K; k++) {
        for (int64_t r = 0; r < len; r++) v[r] = grad[K + k + C * ((int64_t)rows[r] - 1)];
        qsort(v, (size_t)len, sizeof(float), cmp_float);
        double h = (double)(len - 1) * (p->loss == ORC_QUANTILE ? p->alpha : p->alphas[k]);
        int64_t lo = (int64_t)floor(h), hi = lo + 1 < len ? lo + 1 : lo;
        double q = len > 0 ? (double)v[lo] + (h - (double)lo) * ((double)v[hi] - (double)v[lo]) : 0.0;
        tpred[k + K * n0] = (float)(p->eta / p->bagging_size * q / denom);
    }
    free(v);
}

int orc_grow_tree(const orc_params *p, int64_t nobs, int32_t nfeats, const uint8_t *x_bin,
                  const uint8_t *x_bin_T /* optional [nfeats x nobs] observation-major copy, src/init.jl:155 */,
                  const float *grad,
                  const uint32_t *is_in, int64_t nis, const uint32_t *js, int32_t njs, const uint8_t *feattypes,
                  const int32_t *monotone, int64_t *feat, uint8_t *cond_bin, float *w, float *gain, float *tpred,
                  uint8_t *split, uint32_t *nidx, double *hist_out, double *nsum_out) {
    const int K = p->K, C = 2 * K + 1, B = p->nbins, D = p->max_depth;
    const int nn = (1 << D) - 1;
    if (nis <= 0 || njs <= 0 || D < 1) return -1;
    memset(feat, 0, sizeof(int64_t) * nn);
    memset(cond_bin, 0, nn);
    memset(w, 0, sizeof(float) * nn);
    memset(gain, 0, sizeof(float) * nn);
    memset(tpred, 0, sizeof(float) * K * nn);
    memset(split, 0, nn);
    if (nidx) memset(nidx, 0, sizeof(uint32_t) * nobs);

    const size_t hnode = (size_t)C * B * nfeats;
    double *hist = hist_out ? hist_out : (double *)calloc(hnode * nn, sizeof(double));
    if (hist_out) memset(hist, 0, sizeof(double) * hnode * nn);
    double *nsum = (double *)calloc((size_t)C * (nn + 1), sizeof(double)); /* indexed by node id (1-based) */
    seg_t *seg = (seg_t *)calloc(nn + 1, sizeof(seg_t));
    uint32_t *is = (uint32_t *)malloc(sizeof(uint32_t) * nis);
    uint32_t *tmp = (uint32_t *)malloc(sizeof(uint32_t) * nis);
    int *cur = (int *)malloc(sizeof(int) * (nn + 1));
    int *nxt = (int *)malloc(sizeof(int) * (nn + 1));
    memcpy(is, is_in, sizeof(uint32_t) * nis);
    const double eps = DBL_EPSILON;
    /* tree_type 1 = oblivious: gains of every node of the widest split level + the table they are added into */
    double *obl_gains = p->tree_type == 1 ? (double *)malloc(sizeof(double) * ((size_t)(nn + 1) / 2 + 1) * njs * B) : NULL;

    /* root sums: Float64 sequential sum of grad over `is`  (src/fit.jl:66) */
    seg[1].start = 0; seg[1].len = nis;
    for (int64_t r = 0; r < nis; r++) {
        int64_t i = (int64_t)is[r] - 1;
        for (int c = 0; c < C; c++) nsum[c + C * 1] += (double)grad[c + C * i];
    }
    int ncur = 1; cur[0] = 1;
    int depth = 1;
    while (ncur > 0 && depth <= D) {
        int nnext = 0;
        if (depth == D) { /* src/fit.jl:74-82 */
            for (int a = 0; a < ncur; a++) {
                int n = cur[a];
                w[n - 1] = (float)nsum[(C - 1) + C * n];
                if (p->loss == ORC_QUANTILE || p->loss == ORC_MULTIQUANTILE) pred_leaf_quantile(tpred, n - 1, &nsum[C * n], p, grad, is + seg[n].start, seg[n].len);
                else pred_leaf(tpred, n - 1, &nsum[C * n], p);
            }
        } else {
            /* build_nodes = n_current[1:2:end]; update_hist!  (src/fit.jl:85-86, fit-utils.jl:345-394) */
            int nbuild = (ncur + 1) / 2;
            /* tiles as in update_hist!: tile = cld(nj, max(1, cld(nthreads, n_build))) */
            int nth = orc_num_threads();
            int per = (nth + nbuild - 1) / nbuild; if (per < 1) per = 1;
            int tile = (njs + per - 1) / per;
            int ntiles = (njs + tile - 1) / tile;
#pragma omp parallel for schedule(dynamic)
            for (int t = 0; t < nbuild * ntiles; t++) {
                int bi = t / ntiles, ti = t % ntiles;
                int n = cur[2 * bi];
                int j0 = ti * tile, j1 = j0 + tile < njs ? j0 + tile : njs;
                double *hn = hist + hnode * (n - 1);
                for (int jj = j0; jj < j1; jj++) memset(hn + (size_t)C * B * ((int)js[jj] - 1), 0, sizeof(double) * C * B);
                const uint32_t *rows = is + seg[n].start;
                for (int64_t r = 0; r < seg[n].len; r++) {
                    int64_t i = (int64_t)rows[r] - 1;
                    const float *g = grad + C * i;
                    if (x_bin_T) {
                        const uint8_t *xr = x_bin_T + (size_t)nfeats * i;
                        if (r + 10 < seg[n].len) {
                            int64_t ip = (int64_t)rows[r + 10] - 1;
                            __builtin_prefetch(x_bin_T + (size_t)nfeats * ip);
                            if (nfeats > 64) __builtin_prefetch(x_bin_T + (size_t)nfeats * ip + 64);
                            __builtin_prefetch(grad + C * ip);
                        }
                        for (int jj = j0; jj < j1; jj++) {
                            int j = (int)js[jj] - 1;
                            int bin = xr[j];
                            if (bin < 1 || bin > B) continue;
                            double *hb = hn + (size_t)C * B * j + C * (bin - 1);
                            for (int c = 0; c < C; c++) hb[c] += (double)g[c];
                        }
                    } else {
                        for (int jj = j0; jj < j1; jj++) {
                            int j = (int)js[jj] - 1;
                            int bin = x_bin[i + (size_t)nobs * j];
                            if (bin < 1 || bin > B) continue;
                            double *hb = hn + (size_t)C * B * j + C * (bin - 1);
                            for (int c = 0; c < C; c++) hb[c] += (double)g[c];
                        }
                    }
                }
            }
            /* subtract_hist!: n_current[2:2:end]  (src/fit.jl:87, fit-utils.jl:321-332) */
#pragma omp parallel for schedule(dynamic)
            for (int a = 1; a < ncur; a += 2) {
                int n = cur[a], np = n >> 1, ns = n ^ 1;
                for (int jj = 0; jj < njs; jj++) {
                    int j = (int)js[jj] - 1;
                    double *h = hist + hnode * (n - 1) + (size_t)C * B * j;
                    const double *hp = hist + hnode * (np - 1) + (size_t)C * B * j;
                    const double *hs = hist + hnode * (ns - 1) + (size_t)C * B * j;
                    for (int e = 0; e < C * B; e++) h[e] = hp[e] - hs[e];
                }
            }
            /* sort!(n_current) (src/fit.jl:88) */
            for (int a = 1; a < ncur; a++) {
                int v = cur[a], b = a - 1;
                while (b >= 0 && cur[b] > v) { cur[b + 1] = cur[b]; b--; }
                cur[b + 1] = v;
            }
            /* get_best_split per node (src/fit.jl:89-98, fit-utils.jl:403-450) */
#pragma omp parallel for schedule(dynamic)
            for (int a = 0; a < ncur; a++) {
                int n = cur[a];
                const double *s = &nsum[C * n];
                w[n - 1] = (float)s[C - 1];
                double best_gain = p->gamma; int best_feat = 0, best_bin = 0;
                double sl[32], sr[32];
                double gain_p = node_gain(p->loss, s, C, p->lambda, p->L2, eps);
                double w_p = s[C - 1];
                /* oblivious: update_gains! keeps every eligible gain, 0 elsewhere (fit-utils.jl:457-463) */
                double *gn = obl_gains ? obl_gains + (size_t)a * njs * B : NULL;
                if (gn) memset(gn, 0, sizeof(double) * njs * B);
                for (int jj = 0; jj < njs; jj++) {
                    int j = (int)js[jj] - 1;
                    int constraint = monotone ? monotone[j] : 0;
                    int numeric = feattypes ? feattypes[j] != 0 : 1;
                    for (int c = 0; c < C; c++) sl[c] = 0.0;
                    int b_max = numeric ? B - 1 : B;
                    const double *h = hist + hnode * (n - 1) + (size_t)C * B * j;
                    for (int bin = 1; bin <= b_max; bin++) {
                        const double *hb = h + C * (bin - 1);
                        if (numeric) for (int c = 0; c < C; c++) sl[c] += hb[c];
                        else for (int c = 0; c < C; c++) sl[c] = hb[c];
                        double w_l = sl[C - 1], w_r = w_p - w_l;
                        if (w_l > p->min_weight && w_r > p->min_weight) {
                            int ok = 1;
                            if (constraint != 0) {
                                for (int c = 0; c < C; c++) sr[c] = s[c] - sl[c];
                                double pl = pred_scalar(sl, p), pr = pred_scalar(sr, p);
                                ok = (constraint == -1 && pl > pr) || (constraint == 1 && pl < pr);
                            }
                            if (ok) {
                                double g = split_gain(p->loss, s, sl, C, w_l, w_r, p->lambda, p->L2, eps) - gain_p;
                                if (gn) gn[(size_t)jj * B + (bin - 1)] = g;
                                else if (g > best_gain) { best_gain = g; best_feat = j + 1; best_bin = bin; }
                            }
                        }
                    }
                }
                if (best_bin != 0) {
                    gain[n - 1] = (float)best_gain;
                    cond_bin[n - 1] = (uint8_t)best_bin;
                    feat[n - 1] = best_feat;
                    split[n - 1] = 1;
                }
            }
            if (obl_gains) {
                /* one split for the whole depth (grow_otree!, src/fit.jl:196-225): the nodes' gains are added in
                   ascending node order into a zeroed table, a candidate that is not eligible (gain <= 0) in any
                   node is dropped, the first maximum in (feature, bin) order wins if it exceeds gamma */
                const size_t NG = (size_t)njs * B;
                double *tot = obl_gains + (size_t)ncur * NG;
                if (depth == 1) memcpy(tot, obl_gains, sizeof(double) * NG);
                else {
                    for (size_t e = 0; e < NG; e++) tot[e] = 0.0;
                    for (int a = 0; a < ncur; a++) for (size_t e = 0; e < NG; e++) tot[e] += obl_gains[(size_t)a * NG + e];
                    for (int a = 0; a < ncur; a++) for (size_t e = 0; e < NG; e++) tot[e] *= obl_gains[(size_t)a * NG + e] > 0.0 ? 1.0 : 0.0;
                }
                size_t be = 0;
                for (size_t e = 1; e < NG; e++) if (tot[e] > tot[be]) be = e;
                if (tot[be] > p->gamma) {
                    for (int a = 0; a < ncur; a++) {
                        int n = cur[a];
                        gain[n - 1] = (float)tot[be];
                        cond_bin[n - 1] = (uint8_t)(be % B + 1);
                        feat[n - 1] = (int64_t)js[be / B];
                        split[n - 1] = 1;
                    }
                }
            }
            /* split_set! / _child_sums! / next level (src/fit.jl:100-137, 226-253) */
            for (int a = 0; a < ncur; a++) {
                int n = cur[a];
                if (split[n - 1]) {
                    int bf = (int)feat[n - 1] - 1, bb = cond_bin[n - 1];
                    int numeric = feattypes ? feattypes[bf] != 0 : 1;
                    const uint8_t *xc = x_bin + (size_t)nobs * bf;
                    uint32_t *rows = is + seg[n].start;
                    int64_t len = seg[n].len, nl = 0, nr = 0;
                    /* stable partition (fit-utils.jl:277-312; the threaded variant gives the same order) */
                    for (int64_t r = 0; r < len; r++) {
                        uint32_t i = rows[r];
                        int c = numeric ? (xc[i - 1] <= bb) : (xc[i - 1] == bb);
                        if (c) rows[nl++] = i; else tmp[nr++] = i;
                    }
                    memcpy(rows + nl, tmp, sizeof(uint32_t) * nr);
                    int nL = n << 1, nR = nL + 1;
                    seg[nL].start = seg[n].start; seg[nL].len = nl;
                    seg[nR].start = seg[n].start + nl; seg[nR].len = nr;
                    /* _child_sums! (fit-utils.jl:472-486) */
                    double *sL = &nsum[C * nL], *sR = &nsum[C * nR];
                    const double *h = hist + hnode * (n - 1) + (size_t)C * B * bf;
                    for (int c = 0; c < C; c++) sL[c] = 0.0;
                    if (numeric) { for (int b = 1; b <= bb; b++) for (int c = 0; c < C; c++) sL[c] += h[c + C * (b - 1)]; }
                    else for (int c = 0; c < C; c++) sL[c] = h[c + C * (bb - 1)];
                    for (int c = 0; c < C; c++) sR[c] = nsum[c + C * n] - sL[c];
                    if (nr >= nl) { nxt[nnext++] = nL; nxt[nnext++] = nR; }
                    else { nxt[nnext++] = nR; nxt[nnext++] = nL; }
                } else {
                    if (p->loss == ORC_QUANTILE || p->loss == ORC_MULTIQUANTILE) pred_leaf_quantile(tpred, n - 1, &nsum[C * n], p, grad, is + seg[n].start, seg[n].len);
                else pred_leaf(tpred, n - 1, &nsum[C * n], p);
                }
            }
        }
        memcpy(cur, nxt, sizeof(int) * nnext);
        ncur = nnext;
        depth++;
    }
    /* final node of every sampled row: leaves are the nodes that own a segment and did not split */
    if (nidx) {
        for (int n = 1; n <= nn; n++) {
            if (seg[n].len > 0 && !split[n - 1]) {
                const uint32_t *rows = is + seg[n].start;
                for (int64_t r = 0; r < seg[n].len; r++) nidx[rows[r] - 1] = (uint32_t)n;
            }
        }
    }
    if (nsum_out) memcpy(nsum_out, nsum + C, sizeof(double) * C * nn);
    if (!hist_out) free(hist);
    free(nsum); free(seg); free(is); free(tmp); free(cur); free(nxt); free(obl_gains);
    return 0;
}

/* ---- predict! for one tree, all rows: src/predict.jl:1-84 ------------------------------ */
static inline int traverse(const int64_t *feat, const uint8_t *cond_bin, const uint8_t *split, const uint8_t *x_bin,
                           int64_t nobs, int64_t i, const uint8_t *feattypes) {
    int nid = 1;
    while (split[nid - 1]) {
        int f = (int)feat[nid - 1] - 1;
        uint8_t x = x_bin[i + nobs * f];
        int numeric = feattypes ? feattypes[f] != 0 : 1;
        int cond = numeric ? (x <= cond_bin[nid - 1]) : (x == cond_bin[nid - 1]);
        nid = (nid << 1) + !cond;
    }
    return nid;
}

void orc_predict_tree(int32_t loss, int32_t K, int64_t nobs, const uint8_t *x_bin, const uint8_t *feattypes,
                      const int64_t *feat, const uint8_t *cond_bin, const uint8_t *split, const float *tpred,
                      float *pred) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nobs; i++) {
        int nid = traverse(feat, cond_bin, split, x_bin, nobs, i, feattypes);
        float *pi = pred + K * i;
        const float *tp = tpred + K * (nid - 1);
        if (loss == ORC_LOGLOSS) {
            for (int k = 0; k < K; k++) { float v = pi[k] + tp[k]; pi[k] = fminf(fmaxf(v, -15.0f), 15.0f); }
        } else if (orc_is_mle(loss)) {
            for (int t = 0; t < K / 2; t++) {
                pi[2 * t] += tp[2 * t];
                pi[2 * t + 1] = fmaxf(-15.0f, pi[2 * t + 1] + tp[2 * t + 1]);
            }
        } else if (loss == ORC_MLOGLOSS) {
            float m = -INFINITY;
            for (int k = 0; k < K; k++) { pi[k] += tp[k]; m = fmaxf(m, pi[k]); }
            for (int k = 0; k < K; k++) pi[k] = fmaxf(-15.0f, pi[k] - m);
        } else {
            for (int k = 0; k < K; k++) pi[k] += tp[k];
        }
    }
}

/* predict_leaf_idx!: src/predict.jl:138-154 */
void orc_leaf_idx(int64_t nobs, const uint8_t *x_bin, const uint8_t *feattypes, const int64_t *feat,
                  const uint8_t *cond_bin, const uint8_t *split, uint32_t *leaf) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nobs; i++) leaf[i] = (uint32_t)traverse(feat, cond_bin, split, x_bin, nobs, i, feattypes);
}

/* apply_prediction_link!: src/predict.jl:105-116, softmax! :187-195 */
void orc_link(int32_t loss, int32_t K, int64_t nobs, float *pred) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nobs; i++) {
        float *pi = pred + K * i;
        if (loss == ORC_LOGLOSS) { for (int k = 0; k < K; k++) pi[k] = orc_sigmoidf(pi[k]); }
        else if (orc_is_mle(loss)) { for (int k = 1; k < K; k += 2) pi[k] = orc_softplusf(pi[k]); }
        else if (loss == ORC_POISSON || loss == ORC_GAMMA || loss == ORC_TWEEDIE) { for (int k = 0; k < K; k++) pi[k] = expf(pi[k]); }
        else if (loss == ORC_MLOGLOSS) {
            float s = 0.0f;
            for (int k = 0; k < K; k++) { pi[k] = expf(pi[k]); s += pi[k]; }
            for (int k = 0; k < K; k++) pi[k] /= s;
        }
    }
}

/* Evaluation metrics: `_eval_metric` (src/metrics.jl:31-49) for mse / mae / logloss, `mlogloss` (:60-76) and
 * `_eval_mle2p_metric` for gaussian_mle (:89-116).  eval[i] = w[i] * acc / K in float, then
 * sum(Float64, eval) / sum(Float64, w); out[0] and out[1] are the two sums (the caller divides; rmse takes the
 * square root of the mse ratio, :53-54).  Unpinned, like the rest of this file: the reference's own tests compare
 * the logged metric with a metric recomputed from `predict` (test/metrics.jl:71-123), which tests/ repeats. */
enum { ORC_METRIC_MSE = 0, ORC_METRIC_MAE = 1, ORC_METRIC_LOGLOSS = 2, ORC_METRIC_MLOGLOSS = 3, ORC_METRIC_GAUSSIAN_MLE = 4,
       ORC_METRIC_POISSON = 5, ORC_METRIC_GAMMA = 6, ORC_METRIC_TWEEDIE = 7, ORC_METRIC_LOGISTIC_MLE = 8, ORC_METRIC_QUANTILE = 9, ORC_METRIC_MULTIQUANTILE = 10 };
void orc_eval_metric(int32_t metric, int32_t K, int64_t nobs, const float *pred, const void *yv, int32_t ycols,
                     const float *w, float *eval, double out[2], double alpha_d, const double *alphas) {
    const float alpha = (float)alpha_d; /* `wmae` with the learner's alpha: src/metrics.jl:4-6, src/callback.jl:62 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nobs; i++) {
        const float *p = pred + (size_t)K * i;
        const float wi = w ? w[i] : 1.0f;
        if (metric == ORC_METRIC_MLOGLOSS) {
            const uint32_t yi = ((const uint32_t *)yv)[i];
            float isum = 0.0f;
            for (int k = 0; k < K; k++) isum += expf(p[k]);
            eval[i] = wi * (logf(isum) - p[yi - 1]);
        } else if (metric == ORC_METRIC_MULTIQUANTILE) { /* src/metrics.jl:120-141 */
            const float yi = ((const float *)yv)[i];
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                const float a = (float)alphas[k];
                acc += a * fmaxf(yi - p[k], 0.0f) + (1.0f - a) * fmaxf(p[k] - yi, 0.0f);
            }
            eval[i] = wi * acc / (float)K;
        } else if (metric == ORC_METRIC_GAUSSIAN_MLE || metric == ORC_METRIC_LOGISTIC_MLE) {
            const float *y = (const float *)yv + (size_t)ycols * i;
            const int Y = K / 2;
            float acc = 0.0f;
            for (int t = 0; t < Y; t++) {
                const float scale = orc_softplusf(p[2 * t + 1]);
                const float d = y[t] - p[2 * t];
                if (metric == ORC_METRIC_GAUSSIAN_MLE) acc += -(logf(scale) + d * d / (2.0f * scale * scale));
                else { const float az = fabsf(d / scale); acc += -logf(scale) - az - 2.0f * log1pf(expf(-az)); } /* metrics.jl:84-89 */
            }
            eval[i] = wi * acc / (float)Y;
        } else {
            const float *y = (const float *)yv + (size_t)ycols * i;
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                const float pk = p[k], yk = ycols == 1 ? y[0] : y[k]; /* _target(y, k, i), src/loss.jl:49-50 */
                if (metric == ORC_METRIC_MSE) acc += (pk - yk) * (pk - yk);
                else if (metric == ORC_METRIC_MAE) acc += fabsf(pk - yk);
                else if (metric == ORC_METRIC_QUANTILE) acc += alpha * fmaxf(yk - pk, 0.0f) + (1.0f - alpha) * fmaxf(pk - yk, 0.0f);
                else if (metric == ORC_METRIC_LOGLOSS) { const float s = orc_sigmoidf(pk); acc += -yk * logf(s) + (yk - 1.0f) * logf(1.0f - s); }
                else if (metric == ORC_METRIC_POISSON) { /* metrics.jl:13-17, eps(1f-7) = 2^-47 */
                    const float pr = expf(pk);
                    acc += 2.0f * (yk * logf(yk / pr + 7.1054274e-15f) + pr - yk);
                } else if (metric == ORC_METRIC_GAMMA) { const float pr = expf(pk); acc += 2.0f * (logf(pr / yk) + yk / pr - 1.0f); }
                else { /* tweedie, rho = 1.5: metrics.jl:24-28 */
                    const float rho = 1.5f, pr = expf(pk);
                    acc += 2.0f * (powf(yk, 2.0f - rho) / (1.0f - rho) / (2.0f - rho) - yk * powf(pr, 1.0f - rho) / (1.0f - rho) + powf(pr, 2.0f - rho) / (2.0f - rho));
                }
            }
            eval[i] = wi * acc / (float)K;
        }
    }
    double sv = 0.0, sw = 0.0;
    for (int64_t i = 0; i < nobs; i++) { sv += (double)eval[i]; sw += (double)(w ? w[i] : 1.0f); }
    out[0] = sv;
    out[1] = sw;
}

/* binarize: x_bin[i,j] = searchsortedfirst(edges[j], x[i,j])  (src/fit-utils.jl:66-72).
 * edges are passed flattened with a fixed count per feature (the Matrix method of get_edges never
 * de-duplicates, src/fit-utils.jl:16).  NaN is not handled: the reference rejects missings earlier. */
void orc_binarize_f32(int64_t nobs, int32_t nfeats, const float *x, const float *edges, int32_t nedges, uint8_t *x_bin) {
#pragma omp parallel for schedule(static)
    for (int32_t j = 0; j < nfeats; j++) {
        const float *e = edges + (size_t)nedges * j;
        for (int64_t i = 0; i < nobs; i++) {
            float v = x[i + nobs * j];
            int lo = 0, hi = nedges; /* first index with e[idx] >= v */
            while (lo < hi) { int mid = (lo + hi) >> 1; if (e[mid] < v) lo = mid + 1; else hi = mid; }
            x_bin[i + nobs * j] = (uint8_t)(lo + 1);
        }
    }
}
void orc_binarize_f64(int64_t nobs, int32_t nfeats, const double *x, const double *edges, int32_t nedges, uint8_t *x_bin) {
#pragma omp parallel for schedule(static)
    for (int32_t j = 0; j < nfeats; j++) {
        const double *e = edges + (size_t)nedges * j;
        for (int64_t i = 0; i < nobs; i++) {
            double v = x[i + nobs * j];
            int lo = 0, hi = nedges;
            while (lo < hi) { int mid = (lo + hi) >> 1; if (e[mid] < v) lo = mid + 1; else hi = mid; }
            x_bin[i + nobs * j] = (uint8_t)(lo + 1);
        }
    }
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the parallel loops, set explicitly: a launcher may export OMP_NUM_THREADS=1 to every rank
 * (torch.distributed.run does), which must not shrink the CPU baseline (the reference runs with
 * Threads.nthreads() = all host cores). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
