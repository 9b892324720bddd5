// Row-parallel kernels: layout conversion of the binned matrix, loss gradients (`update_grads!`,
// src/loss.jl:100-128, 219-236; GPU counterparts ext/EvoTreesKernelAbstractionsExt/loss.jl:106-191), row
// subsampling (`subsample`, src/subsample.jl:6-38), the training `predict!` (src/predict.jl:1-62) fused with
// the gradients of the next round, inference over all trees (`_predict`, src/predict.jl:118-136) and
// `binarize` (src/fit-utils.jl:66-72).
#include "evb_internal.cuh"
#include <float.h>
#include <algorithm>

namespace {

constexpr unsigned FULL = 0xffffffffu;

// ---------------------------------------------------------------------------------- scalar loss math
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }             // loss.jl:249-251
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); } // loss.jl:257-260

// Gradient record of one row.  Channel c (reference order g_1..g_K, h_1..h_K, w) lives at float
// (c / NCH) * 4 + c % NCH: the channels of one histogram unit start on a 16-byte boundary.
__device__ __forceinline__ int gpos(int c, int NCH) { return (c / NCH) * 4 + (c % NCH); }
#define REC(c) rec[gpos((c), NCH)]
// For mse the hessian channels are not stored (h = 2w is rebuilt when the histogram is reduced): the record is
// g_1..g_K, w, i.e. `elided` shifts w from channel 2K to channel K.
struct AlphaSet { float a[8]; }; // a[0]: alpha of the quantile loss; a[0..K-1]: alphas of the multiquantile loss
__device__ __forceinline__ void grad_row(int loss, int K, int NCH, bool elided, const float *p, const void *y, int ycols, long long i, float *rec,
                                         const AlphaSet &al) {
    const float alpha = al.a[0];
    const float w = REC(elided ? K : 2 * K);
    if (loss == EVB_MSE) {
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int k = 0; k < K; ++k) {
            REC(k) = 2.0f * (p[k] - yf[k]) * w;
            if (!elided) REC(K + k) = 2.0f * w;
        }
    } else if (loss == EVB_LOGLOSS) {
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int k = 0; k < K; ++k) {
            const float s = sigmoidf_(p[k]);
            REC(k) = (s - yf[k]) * w;
            REC(K + k) = s * (1.0f - s) * w;
        }
    } else if (loss == EVB_MLOGLOSS) {
        const uint32_t yi = ((const uint32_t *)y)[i];
        float isum = 0.0f;
        for (int k = 0; k < K; ++k) isum += expf(p[k]);
        for (int k = 0; k < K; ++k) {
            const float prob = expf(p[k]) / isum;
            REC(k) = (((uint32_t)(k + 1) == yi) ? prob - 1.0f : prob) * w;
            REC(K + k) = prob * (1.0f - prob) * w;
        }
    } else if (loss == EVB_MULTIQUANTILE) { // one target, one quantile per output row (src/loss.jl:160-172)
        const float yi = ((const float *)y)[i];
        for (int k = 0; k < K; ++k) {
            const float d = yi - p[k];
            REC(k) = (d > 0.0f ? al.a[k] : al.a[k] - 1.0f) * w;
            REC(K + k) = d;
        }
    } else if (loss == EVB_QUANTILE) { // quantile_grad_diff, src/loss.jl:93-98: the second slot keeps the raw residual
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int k = 0; k < K; ++k) {
            const float d = yf[k] - p[k];
            REC(k) = (d > 0.0f ? alpha : alpha - 1.0f) * w;
            REC(K + k) = d;
        }
    } else if (loss == EVB_MAE || loss == EVB_CRED_VAR || loss == EVB_CRED_STD) { // src/loss.jl:86-91
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int k = 0; k < K; ++k) {
            const float d = yf[k] - p[k];
            REC(k) = d * w;
            REC(K + k) = (loss == EVB_MAE ? 0.0f : d * d) * w;
        }
    } else if (loss == EVB_POISSON || loss == EVB_GAMMA || loss == EVB_TWEEDIE) { // src/loss.jl:65-84
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int k = 0; k < K; ++k) {
            const float pr = expf(p[k]), yk = yf[k];
            float g, h;
            if (loss == EVB_POISSON) { g = pr - yk; h = pr; }
            else if (loss == EVB_GAMMA) { g = 2.0f * (1.0f - yk / pr); h = 2.0f * yk / pr; }
            else { // rho = 1.5: pred^(2-rho) = sqrt(pred), pred^(1-rho) = 1 / sqrt(pred)
                const float a = sqrtf(pr), b = 1.0f / a;
                g = 2.0f * (a - yk * b);
                h = 2.0f * (0.5f * a + 0.5f * yk * b);
            }
            REC(k) = g * w;
            REC(K + k) = h * w;
        }
    } else if (loss == EVB_LOGISTIC_MLE) { // src/loss.jl:207-217
        const int Y = K / 2;
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int t = 0; t < Y; ++t) {
            const float loc = p[2 * t], sr = p[2 * t + 1];
            const float scale = softplusf_(sr), ds = sigmoidf_(sr);
            const float z = (yf[t] - loc) / scale, th = tanhf(z / 2.0f);
            REC(2 * t) = -th / scale * w;
            REC(2 * t + 1) = (1.0f - z * th) * ds / scale * w;
            REC(2 * Y + 2 * t) = 1.0f / (3.0f * scale * scale) * w;
            REC(2 * Y + 2 * t + 1) = (3.14159274f * 3.14159274f + 3.0f) / 9.0f * (ds / scale) * (ds / scale) * w;
        }
    } else { // EVB_GAUSSIAN_MLE
        const int Y = K / 2;
        const float *yf = (const float *)y + (size_t)i * ycols;
        for (int t = 0; t < Y; ++t) {
            const float loc = p[2 * t], sr = p[2 * t + 1];
            const float scale = softplusf_(sr), ds = sigmoidf_(sr);
            const float resid = loc - yf[t];
            const float s2 = scale * scale;
            REC(2 * t) = resid / s2 * w;
            REC(2 * t + 1) = (1.0f - resid * resid / s2) * ds / scale * w;
            REC(2 * Y + 2 * t) = 1.0f / s2 * w;
            REC(2 * Y + 2 * t + 1) = 2.0f * (ds / scale) * (ds / scale) * w;
        }
    }
}

// pred[:, i] += leaf with the loss-specific clamps of predict! (src/predict.jl:1-62)
__device__ __forceinline__ void pred_add(int loss, int K, float *p, const float *leaf) {
    if (loss == EVB_LOGLOSS) {
        for (int k = 0; k < K; ++k) p[k] = fminf(fmaxf(p[k] + leaf[k], -15.0f), 15.0f);
    } else if (loss == EVB_GAUSSIAN_MLE || loss == EVB_LOGISTIC_MLE) {
        for (int t = 0; t < K / 2; ++t) {
            p[2 * t] += leaf[2 * t];
            p[2 * t + 1] = fmaxf(-15.0f, p[2 * t + 1] + leaf[2 * t + 1]);
        }
    } else if (loss == EVB_MLOGLOSS) {
        float m = -INFINITY;
        for (int k = 0; k < K; ++k) { p[k] += leaf[k]; m = fmaxf(m, p[k]); }
        for (int k = 0; k < K; ++k) p[k] = fmaxf(-15.0f, p[k] - m);
    } else {
        for (int k = 0; k < K; ++k) p[k] += leaf[k];
    }
}

__device__ __forceinline__ int traverse(const uint32_t *packed, const uint8_t *xrow) {
    int nid = 1;
    uint32_t pk = packed[0];
    while ((pk >> 24) & 1u) {
        const uint32_t x = xrow[pk & 0xffffu], bin = (pk >> 16) & 0xffu;
        const bool cond = ((pk >> 25) & 1u) ? (x <= bin) : (x == bin);
        nid = (nid << 1) + (cond ? 0 : 1); // nid = nid << 1 + !cond (src/predict.jl:7)
        pk = packed[nid - 1];
    }
    return nid;
}

// ---------------------------------------------------------------------------------- layout
// xT[row][j] = xcol[j][row] for a block of columns; one thread = one row x 4 consecutive features
__global__ void k_transpose(const uint8_t *xcol, long long ld, long long nrows, int j0, int nj, uint8_t *xT, int RS) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int jj = blockIdx.y * 4;
    if (i >= nrows || jj >= nj) return;
    uint8_t v[4] = {0, 0, 0, 0};
#pragma unroll
    for (int q = 0; q < 4; ++q)
        if (jj + q < nj) v[q] = xcol[(size_t)(jj + q) * ld + i];
    uint8_t *dst = xT + (size_t)i * RS + j0 + jj;
    if (((j0 + jj) & 3) == 0 && jj + 4 <= nj) {
        *reinterpret_cast<uint32_t *>(dst) = (uint32_t)v[0] | ((uint32_t)v[1] << 8) | ((uint32_t)v[2] << 16) | ((uint32_t)v[3] << 24);
    } else {
        for (int q = 0; q < 4 && jj + q < nj; ++q) dst[q] = v[q];
    }
}

// range check of the binned matrix: counts values outside 1..nbins
__global__ void k_check_bins(const uint8_t *xT, long long n, int RS, int nfeats, int nbins, int *err) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    bool bad = false;
    for (int j = 0; j < nfeats; ++j) {
        const int v = xT[(size_t)i * RS + j];
        bad |= (v < 1 || v > nbins);
    }
    if (bad) atomicCAS(err, 0, EVB_DERR_BIN_RANGE);
}

#undef REC
__global__ void k_init_state(float *grad, float *pred, const float *w, const float *pred0, const float *mu, long long n, int K, int GS, int NCH, int wch) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float *rec = grad + (size_t)i * GS;
    for (int c = 0; c < GS; ++c) rec[c] = 0.0f;
    rec[gpos(wch, NCH)] = w ? w[i] : 1.0f; // ∇[end, :] .= w (src/init.jl:173-174)
    for (int k = 0; k < K; ++k) pred[(size_t)i * K + k] = pred0 ? pred0[(size_t)i * K + k] : mu[k];
}

// ---------------------------------------------------------------------------------- gradients
// max |g| over the rows of a 256-thread block -> global maximum (bit pattern of a non-negative float, which orders
// like an unsigned integer).  Every thread of the block must call it.
__device__ __forceinline__ void block_absmax(float v, unsigned *gmax) {
    __shared__ unsigned s_max[8];
    unsigned m = __reduce_max_sync(FULL, __float_as_uint(fabsf(v)));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int q = 1; q < 8; ++q) m = max(m, s_max[q]);
        if (m > *(volatile unsigned *)gmax) atomicMax(gmax, m);
    }
}
__global__ void __launch_bounds__(256) k_grads(int loss, int K, int GS, int NCH, int elided, int ycols, long long n, const float *pred, const void *y, float *grad, unsigned *gmax,
                                               AlphaSet alpha) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float g0 = 0.0f;
    if (i < n) {
        grad_row(loss, K, NCH, elided != 0, pred + (size_t)i * K, y, ycols, i, grad + (size_t)i * GS, alpha);
        g0 = grad[(size_t)i * GS];
    }
    if (gmax) block_absmax(g0, gmax);
}
// Fixed-point gradient of every row for the integer histogram kernel: q = rint(g * 2^s) with 2^s the largest power
// of two that keeps max |g| * 2^s below 2^qbits (26 when no weights were given and the kernel counts rows inside the
// low word, else 29); the weight likewise with its own scale.  2^-s goes to qinv for the reduce kernel.
__global__ void __launch_bounds__(256) k_quantize(const float *grad, int32_t *gradq, long long n, const unsigned *gmax, double *qinv,
                                                   float wscale, double winv, int unit_w) {
    const int qbits = unit_w ? 26 : 29;
    const float m = __uint_as_float(*gmax);
    float sc = 1.0f;
    double inv = 1.0;
    if (m > 0.0f && m < INFINITY) {
        int e;
        frexpf(m, &e); // m = f * 2^e, f in [0.5, 1)
        sc = ldexpf(1.0f, qbits - e);
        inv = ldexp(1.0, e - qbits);
    }
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) { qinv[0] = inv; qinv[1] = unit_w ? 1.0 : winv; }
    if (i >= n) return;
    const float2 gw = reinterpret_cast<const float2 *>(grad)[i * 2]; // record = g, w, pad, pad
    const int q = __float2int_rn(gw.x * sc);
    if (unit_w) gradq[i] = q;
    else reinterpret_cast<int2 *>(gradq)[i] = make_int2(q, __float2int_rn(gw.y * wscale));
}

// ---------------------------------------------------------------------------------- row sampling
__global__ void k_rows_identity(uint32_t *rows, long long n, int32_t *nleft0) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) rows[i] = (uint32_t)i;
    if (i == 0) nleft0[0] = (int32_t)n;
}
constexpr int SEL_CHUNK = 2048, SEL_THREADS = 256;
__global__ void __launch_bounds__(SEL_THREADS) k_sel_count(const uint8_t *mask, uint8_t cond, long long n, int32_t *bcnt) {
    __shared__ int s[SEL_THREADS / 32];
    const long long base = (long long)blockIdx.x * SEL_CHUNK;
    int c = 0;
    for (int i8 = 0; i8 < SEL_CHUNK / SEL_THREADS; ++i8) {
        const long long i = base + i8 * SEL_THREADS + threadIdx.x;
        const bool sel = i < n && mask[i] <= cond;
        c += __popc(__ballot_sync(FULL, sel));
    }
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < SEL_THREADS / 32; ++w) t += s[w];
        bcnt[blockIdx.x] = t;
    }
}
__global__ void __launch_bounds__(1024) k_sel_scan(int32_t *bcnt, int nblocks, int32_t *nleft0) {
    __shared__ int sm[33];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int carry = 0;
    for (int base = 0; base < nblocks; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < nblocks ? bcnt[i] : 0;
        int incl = v;
        for (int d = 1; d < 32; d <<= 1) { int t = __shfl_up_sync(FULL, incl, d); if (lane >= d) incl += t; }
        __syncthreads();
        if (lane == 31) sm[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            int w = sm[lane], wi = w;
            for (int d = 1; d < 32; d <<= 1) { int t = __shfl_up_sync(FULL, wi, d); if (lane >= d) wi += t; }
            sm[lane] = wi - w;
            if (lane == 31) sm[32] = wi;
        }
        __syncthreads();
        if (i < nblocks) bcnt[i] = carry + sm[wid] + incl - v;
        carry += sm[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) nleft0[0] = carry;
}
__global__ void __launch_bounds__(SEL_THREADS) k_sel_scatter(const uint8_t *mask, uint8_t cond, long long n, const int32_t *boff, uint32_t *rows) {
    constexpr int NW = SEL_CHUNK / 32;
    __shared__ uint32_t s_bits[NW];
    __shared__ int s_pref[NW];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long base = (long long)blockIdx.x * SEL_CHUNK;
    for (int i8 = 0; i8 < SEL_CHUNK / SEL_THREADS; ++i8) {
        const long long i = base + i8 * SEL_THREADS + threadIdx.x;
        const bool sel = i < n && mask[i] <= cond;
        const unsigned bal = __ballot_sync(FULL, sel);
        if (lane == 0) s_bits[i8 * (SEL_THREADS / 32) + wid] = bal;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int c0 = __popc(s_bits[2 * lane]), c1 = __popc(s_bits[2 * lane + 1]);
        int incl = c0 + c1;
        for (int d = 1; d < 32; d <<= 1) { int t = __shfl_up_sync(FULL, incl, d); if (lane >= d) incl += t; }
        s_pref[2 * lane] = incl - c0 - c1;
        s_pref[2 * lane + 1] = incl - c1;
    }
    __syncthreads();
    const int off = boff[blockIdx.x];
    for (int i8 = 0; i8 < SEL_CHUNK / SEL_THREADS; ++i8) {
        const int pos = i8 * SEL_THREADS + threadIdx.x;
        const uint32_t word = s_bits[pos >> 5];
        if ((word >> lane) & 1u) rows[off + s_pref[pos >> 5] + __popc(word & ((1u << lane) - 1u))] = (uint32_t)(base + pos);
    }
}
static_assert(SEL_CHUNK / 32 == 64, "k_sel_scatter assumes 64 ballot words");

// ---------------------------------------------------------------------------------- training predict (+ next gradients)
struct FinArgs {
    const uint8_t *xT;
    const uint32_t *t_packed;
    const float *t_pred;
    float *pred, *grad;
    const void *y;
    uint32_t *nidx;
    unsigned *gmax; // non-null: track max |g| of the gradients computed here (fixed-point histogram variant)
    long long n;
    int RS, K, GS, NCH, elided, loss, nn, ycols, compute_grads, packed_in_smem;
    AlphaSet alpha;
    int mode; // 0: traverse, add the leaf, next gradients; 1: traverse only (leaf ids); 2: leaf ids are in nidx, add + gradients
};
__global__ void __launch_bounds__(256) k_finalize(FinArgs a) {
    extern __shared__ uint32_t s_packed[];
    const uint32_t *packed = a.t_packed;
    if (a.packed_in_smem) {
        for (int i = threadIdx.x; i < a.nn; i += blockDim.x) s_packed[i] = a.t_packed[i];
        __syncthreads();
        packed = s_packed;
    }
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float g0 = 0.0f;
    if (i < a.n) {
        const int nid = a.mode == 2 ? (int)a.nidx[i] : traverse(packed, a.xT + (size_t)i * a.RS);
        a.nidx[i] = (uint32_t)nid;
        float *p = a.pred + (size_t)i * a.K;
        if (a.mode != 1) pred_add(a.loss, a.K, p, a.t_pred + (size_t)(nid - 1) * a.K);
        if (a.compute_grads && a.mode != 1) {
            grad_row(a.loss, a.K, a.NCH, a.elided != 0, p, a.y, a.ycols, i, a.grad + (size_t)i * a.GS, a.alpha);
            g0 = a.grad[(size_t)i * a.GS];
        }
    }
    if (a.gmax && a.compute_grads) block_absmax(g0, a.gmax);
}

// The same update with the rows of bins staged through shared memory: the CTA copies its 256 rows with fully
// coalesced 16-byte loads (one memory round trip instead of one per tree level and sector), then every thread walks
// the tree on its own row out of shared memory.  Rows are padded by one word so that equal byte offsets of different
// rows fall into different banks.  Used when a row is at most 256 bytes.
__global__ void __launch_bounds__(256) k_finalize_staged(FinArgs a) {
    extern __shared__ uint32_t s_fin[]; // [nn] packed tree, then [256][RS / 4 + 1] words of bins
    uint32_t *s_tree = s_fin;
    uint32_t *s_rows = s_fin + a.nn;
    const int rw = a.RS >> 2, rwp = rw + 1; // words per row, padded
    for (int i = threadIdx.x; i < a.nn; i += 256) s_tree[i] = a.t_packed[i];
    const long long row0 = (long long)blockIdx.x * 256;
    const int nr = (int)min((long long)256, a.n - row0);
    const uint4 *src = reinterpret_cast<const uint4 *>(a.xT + (size_t)row0 * a.RS);
    const int cpr = a.RS >> 4, nchunk = nr * cpr;
    for (int c = threadIdx.x; c < nchunk; c += 256) {
        const uint4 v = src[c];
        const int r = c / cpr, part = c - r * cpr;
        uint32_t *d = s_rows + r * rwp + part * 4;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    __syncthreads();
    const long long i = row0 + threadIdx.x;
    float g0 = 0.0f;
    if (i < a.n) {
        const int nid = traverse(s_tree, reinterpret_cast<const uint8_t *>(s_rows + threadIdx.x * rwp));
        a.nidx[i] = (uint32_t)nid;
        float *p = a.pred + (size_t)i * a.K;
        pred_add(a.loss, a.K, p, a.t_pred + (size_t)(nid - 1) * a.K);
        if (a.compute_grads) {
            grad_row(a.loss, a.K, a.NCH, a.elided != 0, p, a.y, a.ycols, i, a.grad + (size_t)i * a.GS, a.alpha);
            g0 = a.grad[(size_t)i * a.GS];
        }
    }
    if (a.gmax && a.compute_grads) block_absmax(g0, a.gmax);
}

// The same update as a pipeline: a few CTAs per SM stay resident and walk over tiles of 256 rows.  The tree (and, for
// one output, its leaf values) is loaded into shared memory once per CTA; the bins of tile t + 1 are copied into the
// other of two shared-memory buffers (`cp.async`, 16 bytes per copy; rows sit at an odd number of 16-byte chunks, so
// the same feature of 8 adjacent rows falls into different banks) while tile t is traversed, and the row's prediction
// and target are requested before the traversal starts, so that a tile costs one memory round trip, not three.
// Rows come from xT ([n][RS]) or, on the fixed-point histogram path, from the 16-byte chunk rows xH ([n][RSH], feature f
// at byte f) plus the word of tail features kept in xE: 104 instead of 128 bytes per row at 100 features.
struct FinPipeArgs {
    FinArgs f;
    const uint8_t *rowsA; // xT or xH
    const uint2 *xE;      // non-null: word y of xE[row] follows the row's bytes (tail features)
    int strideA;          // bytes between rows of rowsA
    int wordsA;           // words copied per row from rowsA
    int S;                // words per row in shared memory: a multiple of 4, an odd number of 16-byte chunks
    int ntiles, leaf_in_smem;
};
// MSE1: mse with one output and the record {g, w} (hessian rebuilt from w): loss, K and the record layout are
// compile-time constants
template <bool MSE1>
__global__ void __launch_bounds__(256) k_finalize_pipe(FinPipeArgs a) {
    // [nnp] packed tree, [nnp] leaf values (one output only), 2 x [256][S] words of bins; nnp = nn rounded up to four
    // words, so that the row buffers start on a 16-byte boundary (the copies into them are 16 bytes wide)
    extern __shared__ __align__(16) uint32_t s_fp[];
    const FinArgs &f = a.f;
    const int nnp = (f.nn + 3) & ~3;
    uint32_t *s_tree = s_fp;
    float *s_leaf = reinterpret_cast<float *>(s_fp + nnp);
    uint32_t *s_rows = s_fp + nnp + (a.leaf_in_smem ? nnp : 0);
    const int S = a.S, wA = a.wordsA;
    for (int i = threadIdx.x; i < f.nn; i += 256) {
        s_tree[i] = f.t_packed[i];
        if (a.leaf_in_smem) s_leaf[i] = f.t_pred[i];
    }
    const int cpr = wA >> 2;                     // 16-byte chunks per row
    const uint32_t magic = 65536u / (uint32_t)cpr + 1u; // (c * magic) >> 16 == c / cpr for c < 4096, cpr <= 16
    auto stage = [&](int tile, int buf) {
        if (tile < a.ntiles) {
            const long long row0 = (long long)tile * 256;
            const int nr = (int)min((long long)256, f.n - row0);
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_rows + (size_t)buf * 256 * S);
            const uint8_t *src = a.rowsA + (size_t)row0 * a.strideA;
            const int total = nr * cpr;
            for (int c = threadIdx.x; c < total; c += 256) {
                const int r = (int)(((uint32_t)c * magic) >> 16), part = c - r * cpr;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(r * S + part * 4) * 4u),
                             "l"(src + (size_t)r * a.strideA + part * 16) : "memory");
            }
            if (a.xE && (int)threadIdx.x < nr)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + (uint32_t)(threadIdx.x * S + wA) * 4u),
                             "l"(reinterpret_cast<const uint32_t *>(a.xE + row0 + threadIdx.x) + 1) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float gm = 0.0f;
    int buf = 0;
    stage(blockIdx.x, 0);
    for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x, buf ^= 1) {
        stage(tile + gridDim.x, buf ^ 1);
        const long long i = (long long)tile * 256 + threadIdx.x;
        const bool act = i < f.n;
        float *p = f.pred + (size_t)i * f.K;
        float p0 = 0.0f;
        if (act) {
            if (f.K == 1) p0 = *p;
            else asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
            if (f.compute_grads) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(f.y) + (size_t)i * 4 * (f.ycols > 0 ? f.ycols : 1)));
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads(); // tile `tile` (and, the first time, the tree) is in place
        if (act) {
            const int nid = traverse(s_tree, reinterpret_cast<const uint8_t *>(s_rows + ((size_t)buf * 256 + threadIdx.x) * S));
            f.nidx[i] = (uint32_t)nid;
            const int loss = MSE1 ? (int)EVB_MSE : f.loss, NCH = MSE1 ? 2 : f.NCH;
            if (f.K == 1) {
                float pl[1] = {p0};
                pred_add(loss, 1, pl, a.leaf_in_smem ? s_leaf + (nid - 1) : f.t_pred + (nid - 1));
                p[0] = pl[0];
            } else {
                pred_add(loss, f.K, p, f.t_pred + (size_t)(nid - 1) * f.K);
            }
            if (f.compute_grads) {
                grad_row(loss, MSE1 ? 1 : f.K, NCH, MSE1 ? true : f.elided != 0, p, f.y, MSE1 ? 1 : f.ycols, i, f.grad + (size_t)i * f.GS, f.alpha);
                gm = fmaxf(gm, fabsf(f.grad[(size_t)i * f.GS]));
            }
        }
        __syncthreads(); // everybody is done with this buffer: the next iteration refills it
    }
    if (f.gmax && f.compute_grads) block_absmax(gm, f.gmax);
}

// ---------------------------------------------------------------------------------- quantile leaves
// Leaf values of the quantile loss: the alpha-quantile (linear interpolation between the two neighbouring order
// statistics, `Statistics.quantile`) of the residuals of the sampled rows of every leaf (src/predict.jl:264-272).
// The order statistics of all leaves are found together by a radix selection on the order-preserving bit pattern of
// the residual: four passes of 8 bits, each a counting kernel over the rows (one shared-memory-free atomic per row
// and wanted rank into the leaf's 256 counters) and a pick kernel (one warp per leaf walks its counters).
struct QselArgs {
    const uint32_t *nidx;
    const float *grad;        // residual of row i: grad[i * GS + roff]
    const uint8_t *mask;      // rows with mask <= cond are sampled; null: all
    uint32_t *cnt;            // [2][nn + 1][256]
    uint32_t *prefix;         // [2][nn + 1] bits decided so far
    uint32_t *rank;           // [2][nn + 1] rank still to find inside the current prefix
    float *gamma;             // [nn + 1] interpolation weight
    const uint8_t *t_split;
    const double *nsum;
    float *t_pred;
    long long n;
    int GS, roff, nn, C, pass, K, k, clamp; // k: output row being filled; clamp: max(eps, .) on the denominator (quantile)
    uint8_t cond;
    double alpha, eb, lambda, L2; // eb = eta / bagging_size
};
__device__ __forceinline__ uint32_t float_key(float v) { const uint32_t b = __float_as_uint(v); return (b & 0x80000000u) ? ~b : b | 0x80000000u; }
__device__ __forceinline__ float key_float(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? k & 0x7fffffffu : ~k); }
__global__ void __launch_bounds__(256) k_qsel_count(QselArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.n || (a.mask && a.mask[i] > a.cond)) return;
    const uint32_t leaf = a.nidx[i];
    const uint32_t key = float_key(a.grad[(size_t)i * a.GS + a.roff]);
    const int shift = 24 - 8 * a.pass;
    const uint32_t digit = (key >> shift) & 0xffu;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const size_t e = (size_t)r * (a.nn + 1) + leaf;
        // pass 0 counts every row; later passes only the rows that share the bits decided so far
        if (a.pass == 0 || (key >> (shift + 8)) == (a.prefix[e] >> (shift + 8))) atomicAdd(&a.cnt[e * 256 + digit], 1u);
        if (a.pass == 0) break; // the first pass is the same for both ranks: counted once, in the counters of rank 0
    }
}
__global__ void __launch_bounds__(256) k_qsel_pick(QselArgs a) {
    const int leaf = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (leaf < 1 || leaf > a.nn) return;
    const int shift = 24 - 8 * a.pass;
    for (int r = 0; r < 2; ++r) {
        const size_t e = (size_t)r * (a.nn + 1) + leaf;
        uint32_t *cnt = a.cnt + (a.pass == 0 ? (size_t)leaf : e) * 256;
        uint32_t c[8], tot = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) { c[q] = cnt[lane * 8 + q]; tot += c[q]; }
        uint32_t incl = tot;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(FULL, incl, o); if (lane >= o) incl += v; }
        const uint32_t total = __shfl_sync(FULL, incl, 31);
        uint32_t want;
        if (a.pass == 0) {
            // ranks of the two order statistics: h = (n - 1) alpha, lo = floor(h), hi = lo + 1 (clamped)
            const double hpos = total > 0 ? (double)(total - 1) * a.alpha : 0.0;
            const uint32_t lo = (uint32_t)floor(hpos), hi = lo + 1 < total ? lo + 1 : lo;
            if (r == 0 && lane == 0) a.gamma[leaf] = total > 0 ? (float)(hpos - floor(hpos)) : -1.0f; // -1: no sampled row
            want = r == 0 ? lo : hi;
        } else {
            want = a.rank[e];
        }
        // the digit whose cumulative count first exceeds `want`
        const uint32_t excl = incl - tot;
        int found = -1;
        uint32_t before = 0;
        if (total > 0 && want >= excl && want < incl) {
            uint32_t run = excl;
#pragma unroll
            for (int q = 0; q < 8; ++q) { if (found < 0 && want < run + c[q]) { found = lane * 8 + q; before = run; } run += c[q]; }
        }
        const unsigned who = __ballot_sync(FULL, found >= 0);
        if (who) {
            const int src = __ffs(who) - 1;
            found = __shfl_sync(FULL, found, src);
            before = __shfl_sync(FULL, before, src);
            if (lane == 0) {
                a.prefix[e] = (a.pass == 0 ? 0u : a.prefix[e]) | ((uint32_t)found << shift);
                a.rank[e] = want - before;
            }
        } else if (lane == 0) { a.prefix[e] = 0u; a.rank[e] = 0u; }
        __syncwarp();
    }
    // the counters are used again by the next pass
    for (int r = 0; r < 2; ++r) {
        uint32_t *cnt = a.cnt + ((size_t)r * (a.nn + 1) + leaf) * 256;
        for (int q = lane; q < 256; q += 32) cnt[q] = 0u;
    }
}
// leaf value from the two order statistics (their full keys are in `prefix` after the last pass)
__global__ void k_qsel_leaf(QselArgs a) {
    const int leaf = blockIdx.x * blockDim.x + threadIdx.x;
    if (leaf < 1 || leaf > a.nn || a.t_split[leaf - 1]) return;
    const float g = a.gamma[leaf];
    if (g < 0.0f) return; // not a leaf of this tree (or no sampled row reached it): keeps its zero
    const float lo = key_float(a.prefix[leaf]), hi = key_float(a.prefix[(size_t)(a.nn + 1) + leaf]);
    const double q = (double)lo + (double)g * ((double)hi - (double)lo);
    const double w = a.nsum[(size_t)leaf * a.C + a.C - 1];
    const double denom = 1.0 + a.lambda + a.L2 / w;
    a.t_pred[(size_t)(leaf - 1) * a.K + a.k] = (float)(a.eb * q / (a.clamp ? fmax(DBL_EPSILON, denom) : denom));
}

// node of every sampled row from the row lists left by the partition kernels; one CTA per node
__global__ void k_nidx_from_partition(const uint32_t *rows0, const uint32_t *rows1, const int32_t *seg_start,
                                      const int32_t *seg_cnt, const uint8_t *t_split, int nn, uint32_t *out) {
    for (int n = 1 + blockIdx.x; n <= nn; n += gridDim.x) {
        const int cnt = seg_cnt[n];
        if (cnt <= 0 || t_split[n - 1]) continue;
        const int depth = 32 - __clz(n); // root = 1
        const uint32_t *rows = ((depth - 1) & 1) ? rows1 : rows0;
        const int s0 = seg_start[n];
        for (int r = threadIdx.x; r < cnt; r += blockDim.x) out[rows[s0 + r]] = (uint32_t)n;
    }
}

// ---------------------------------------------------------------------------------- inference
struct PredArgs {
    const uint8_t *xT;
    const uint32_t *packed; // [ntrees][nn]
    const float *leaf;      // [ntrees][nn][K]
    float *out;             // [nobs_total x K] column-major, this chunk starts at row0
    uint32_t *leaf_idx;     // [nobs_total x ntrees] column-major or NULL
    long long n, row0, nobs_total;
    int RS, K, loss, ntrees, nn, apply_link;
};
template <int KMAX>
__global__ void __launch_bounds__(256) k_predict(PredArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.n) return;
    const uint8_t *xrow = a.xT + (size_t)i * a.RS;
    float p[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) p[k] = 0.0f;
    const int K = a.K;
    for (int t = 0; t < a.ntrees; ++t) {
        const int nid = traverse(a.packed + (size_t)t * a.nn, xrow);
        if (a.leaf_idx) a.leaf_idx[(size_t)t * a.nobs_total + a.row0 + i] = (uint32_t)nid;
        pred_add(a.loss, K, p, a.leaf + ((size_t)t * a.nn + nid - 1) * K);
    }
    if (a.apply_link) { // apply_prediction_link! (src/predict.jl:105-116)
        if (a.loss == EVB_LOGLOSS) { for (int k = 0; k < K; ++k) p[k] = sigmoidf_(p[k]); }
        else if (a.loss == EVB_GAUSSIAN_MLE || a.loss == EVB_LOGISTIC_MLE) { for (int k = 1; k < K; k += 2) p[k] = softplusf_(p[k]); }
        else if (a.loss == EVB_POISSON || a.loss == EVB_GAMMA || a.loss == EVB_TWEEDIE) { for (int k = 0; k < K; ++k) p[k] = expf(p[k]); }
        else if (a.loss == EVB_MLOGLOSS) {
            float s = 0.0f;
            for (int k = 0; k < K; ++k) { p[k] = expf(p[k]); s += p[k]; }
            for (int k = 0; k < K; ++k) p[k] /= s;
        }
    }
    for (int k = 0; k < K; ++k) a.out[(size_t)k * a.nobs_total + a.row0 + i] = p[k];
}


// The same with everything a thread touches in shared memory: the CTA's rows of bins are staged once, word-major
// ([word of the row][row]: thread t only ever reads column t, so its loads never conflict with its neighbours'
// whatever features the trees test), and the packed trees + their leaf tables stream through two shared-memory buffers
// of TB trees each: while the threads walk the trees of one buffer, `cp.async` fills the other, so a traversal step
// costs two shared-memory loads and the trip to L2 is off the critical path.  One thread = one row; trees are applied
// in order (the clamps of `predict!` do not commute).  `tw` = words per tree in `trees` ([nnp] packed nodes, then
// [nnp * K] leaf values; nnp = nn rounded up to a multiple of four so that every tree starts on a 16-byte boundary).
// Used when 2 * TB trees fit beside the rows.
__device__ __forceinline__ int traverse_wm(const uint32_t *packed, const uint32_t *xcol, int rows) {
    int nid = 1;
    uint32_t pk = packed[0];
    while ((pk >> 24) & 1u) {
        const uint32_t f = pk & 0xffffu, bin = (pk >> 16) & 0xffu;
        const uint32_t x = (xcol[(f >> 2) * rows] >> (8u * (f & 3u))) & 0xffu;
        const bool cond = ((pk >> 25) & 1u) ? (x <= bin) : (x == bin);
        nid = (nid << 1) + (cond ? 0 : 1);
        pk = packed[nid - 1];
    }
    return nid;
}
template <int KMAX>
__global__ void __launch_bounds__(1024) k_predict_staged(PredArgs a, const uint32_t *trees, int nnp, int rows_per_cta, int TB) {
    extern __shared__ __align__(16) uint32_t s_pr[]; // [RS / 4][rows_per_cta] bins, then 2 x TB x tw tree words
    const int rw = a.RS >> 2;
    uint32_t *s_rows = s_pr;
    const int K = a.K, tw = nnp * (1 + K);
    uint32_t *s_trees = s_pr + (size_t)rows_per_cta * rw;
    const long long row0 = (long long)blockIdx.x * rows_per_cta;
    const int nr = (int)min((long long)rows_per_cta, a.n - row0);
    auto load_block = [&](int t0, int buf) { // trees t0 .. t0 + TB - 1 -> buffer `buf`, 16 bytes per copy
        const int nt = min(TB, a.ntrees - t0);
        const uint4 *src = reinterpret_cast<const uint4 *>(trees + (size_t)t0 * tw);
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_trees + (size_t)buf * TB * tw);
        for (int c = threadIdx.x; c < nt * (tw >> 2); c += blockDim.x)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)c * 16u), "l"(src + c) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_block(0, 0);
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.xT + (size_t)row0 * a.RS);
        const int cpr = a.RS >> 4, nchunk = nr * cpr;
        for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
            const uint4 v = src[c];
            const int r = c / cpr, part = c - r * cpr;
            uint32_t *d = s_rows + (size_t)(part * 4) * rows_per_cta + r;
            d[0] = v.x; d[rows_per_cta] = v.y; d[2 * rows_per_cta] = v.z; d[3 * rows_per_cta] = v.w;
        }
    }
    const bool act = (int)threadIdx.x < nr;
    const long long i = row0 + threadIdx.x;
    const uint32_t *xcol = s_rows + threadIdx.x;
    float p[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) p[k] = 0.0f;
    int buf = 0;
    for (int t0 = 0; t0 < a.ntrees; t0 += TB, buf ^= 1) {
        const int nt = min(TB, a.ntrees - t0);
        if (t0 + TB < a.ntrees) load_block(t0 + TB, buf ^ 1); // the other buffer was consumed before the last barrier
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads(); // this block's trees (and, the first time, the rows) are in place for everybody
        if (act) {
            for (int t = 0; t < nt; ++t) {
                const uint32_t *pk = s_trees + ((size_t)buf * TB + t) * tw;
                const int nid = traverse_wm(pk, xcol, rows_per_cta);
                if (a.leaf_idx) a.leaf_idx[(size_t)(t0 + t) * a.nobs_total + a.row0 + i] = (uint32_t)nid;
                pred_add(a.loss, K, p, reinterpret_cast<const float *>(pk + nnp) + (size_t)(nid - 1) * K);
            }
        }
        __syncthreads(); // everybody is done with this buffer: the next iteration refills it
    }
    if (!act) return;
    if (a.apply_link) { // apply_prediction_link! (src/predict.jl:105-116)
        if (a.loss == EVB_LOGLOSS) { for (int k = 0; k < K; ++k) p[k] = sigmoidf_(p[k]); }
        else if (a.loss == EVB_GAUSSIAN_MLE || a.loss == EVB_LOGISTIC_MLE) { for (int k = 1; k < K; k += 2) p[k] = softplusf_(p[k]); }
        else if (a.loss == EVB_POISSON || a.loss == EVB_GAMMA || a.loss == EVB_TWEEDIE) { for (int k = 0; k < K; ++k) p[k] = expf(p[k]); }
        else if (a.loss == EVB_MLOGLOSS) {
            float sm = 0.0f;
            for (int k = 0; k < K; ++k) { p[k] = expf(p[k]); sm += p[k]; }
            for (int k = 0; k < K; ++k) p[k] /= sm;
        }
    }
    for (int k = 0; k < K; ++k) a.out[(size_t)k * a.nobs_total + a.row0 + i] = p[k];
}

// trees in the layout k_predict_staged streams: tree t = [nnp] packed nodes, then [nnp][K] leaf values (zero padded)
__global__ void k_pack_staged(const uint32_t *packed, const float *leaf, int ntrees, int nn, int nnp, int K, uint32_t *out) {
    const int tw = nnp * (1 + K);
    const long long total = (long long)ntrees * tw;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(e / tw), o = (int)(e - (long long)t * tw);
        uint32_t v = 0u;
        if (o < nnp) { if (o < nn) v = packed[(size_t)t * nn + o]; }
        else { const int q = o - nnp; if (q < nn * K) v = __float_as_uint(leaf[(size_t)t * nn * K + q]); }
        out[e] = v;
    }
}

__global__ void k_pack_trees(const long long *feat, const uint8_t *bin, const uint8_t *split, const uint8_t *feattypes,
                             long long total, uint32_t *packed) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    uint32_t pk = 0;
    if (split[i]) {
        const uint32_t f = (uint32_t)(feat[i] - 1);
        pk = f | ((uint32_t)bin[i] << 16) | (1u << 24) | ((feattypes ? (feattypes[f] ? 1u : 0u) : 1u) << 25);
    }
    packed[i] = pk;
}

// ---------------------------------------------------------------------------------- binarize
// searchsortedfirst(edges[j], x): 1 + number of edges strictly below x
template <typename T>
__global__ void __launch_bounds__(256) k_binarize(const T *x, long long ld, long long n, const T *edges, int nedges, uint8_t *out, long long ldo,
                                                   int *nan_err = nullptr) {
    extern __shared__ unsigned char s_raw[];
    T *e = reinterpret_cast<T *>(s_raw);
    const int j = blockIdx.y;
    for (int q = threadIdx.x; q < nedges; q += blockDim.x) e[q] = edges[(size_t)j * nedges + q];
    __syncthreads();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const T v = x[(size_t)j * ld + i];
        if (nan_err && v != v) atomicCAS(nan_err, 0, EVB_DERR_NAN); // missing values are not supported (test/missings.jl)
        int lo = 0, hi = nedges;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (e[mid] < v) lo = mid + 1; else hi = mid; }
        out[(size_t)j * ldo + i] = (uint8_t)(lo + 1);
    }
}

// binarize a block of rows of the raw matrix straight into observation-major bins xT[row][RS] (what the traversal
// reads): 256 rows per CTA, staged through shared memory so that both the reads of x and the writes of xT coalesce
template <typename T>
__global__ void __launch_bounds__(256) k_binarize_rows(const T *x, long long ld, int row_major, long long n, int nfeats, const T *edges,
                                                       int nedges, uint8_t *xT, int RS) {
    extern __shared__ unsigned char s_tile[]; // [256][RS + 4]: one word of padding, so that the same feature of adjacent rows sits in different banks
    const int RSP = RS + 4;
    const long long row0 = (long long)blockIdx.x * 256;
    const int nr = (int)min((long long)256, n - row0);
    for (int e = threadIdx.x; e < 64 * RSP; e += 256) reinterpret_cast<uint32_t *>(s_tile)[e] = 0u;
    __syncthreads();
    const int total = nr * nfeats;
    for (int e = threadIdx.x; e < total; e += 256) {
        int r, j;
        T v;
        if (row_major) { r = e / nfeats; j = e - r * nfeats; v = x[(size_t)(row0 + r) * ld + j]; }
        else { j = e / nr; r = e - j * nr; v = x[(size_t)j * ld + row0 + r]; }
        const T *ed = edges + (size_t)j * nedges;
        int lo = 0, hi = nedges;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (__ldg(ed + mid) < v) lo = mid + 1; else hi = mid; }
        s_tile[r * RSP + j] = (uint8_t)(lo + 1);
    }
    __syncthreads();
    uint4 *dst = reinterpret_cast<uint4 *>(xT + (size_t)row0 * RS);
    const int cpr = RS / 16;
    for (int e = threadIdx.x; e < nr * cpr; e += 256) {
        const int r = e / cpr, part = e - r * cpr;
        const uint32_t *src = reinterpret_cast<const uint32_t *>(s_tile + (size_t)r * RSP) + part * 4;
        dst[e] = make_uint4(src[0], src[1], src[2], src[3]);
    }
}

// ---------------------------------------------------------------------------------- evaluation data
// Per-row metric value in float, as `_metric_value` / `_mle2p_metric_value` / `mlogloss` compute it
// (src/metrics.jl:1-110): the caller multiplies by w and accumulates in double.
__device__ __forceinline__ float metric_row(int metric, int K, const float *p, const void *y, int ycols, long long i, float w, const AlphaSet &al) {
    const float alpha = al.a[0];
    if (metric == EVB_METRIC_MLOGLOSS) {
        const uint32_t yi = ((const uint32_t *)y)[i];
        float isum = 0.0f;
        for (int k = 0; k < K; ++k) isum += expf(p[k]);
        return w * (logf(isum) - p[yi - 1]);
    }
    const float *yf = (const float *)y + (size_t)i * ycols;
    if (metric == EVB_METRIC_MULTIQUANTILE) { // src/metrics.jl:120-141
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) acc += al.a[k] * fmaxf(yf[0] - p[k], 0.0f) + (1.0f - al.a[k]) * fmaxf(p[k] - yf[0], 0.0f);
        return w * acc / (float)K;
    }
    if (metric == EVB_METRIC_GAUSSIAN_MLE || metric == EVB_METRIC_LOGISTIC_MLE) {
        const int Y = K / 2;
        float acc = 0.0f;
        for (int t = 0; t < Y; ++t) {
            const float scale = softplusf_(p[2 * t + 1]), d = yf[t] - p[2 * t];
            if (metric == EVB_METRIC_GAUSSIAN_MLE) acc += -(logf(scale) + d * d / (2.0f * scale * scale));
            else { const float az = fabsf(d / scale); acc += -logf(scale) - az - 2.0f * log1pf(expf(-az)); } // src/metrics.jl:84-89
        }
        return w * acc / (float)Y;
    }
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) {
        const float pk = p[k], yk = yf[k];
        if (metric == EVB_METRIC_MSE) acc += (pk - yk) * (pk - yk);
        else if (metric == EVB_METRIC_MAE) acc += fabsf(pk - yk);
        else if (metric == EVB_METRIC_QUANTILE) acc += alpha * fmaxf(yk - pk, 0.0f) + (1.0f - alpha) * fmaxf(pk - yk, 0.0f); // src/metrics.jl:4-6
        else if (metric == EVB_METRIC_LOGLOSS) { const float s = sigmoidf_(pk); acc += -yk * logf(s) + (yk - 1.0f) * logf(1.0f - s); }
        else if (metric == EVB_METRIC_POISSON) { // src/metrics.jl:13-17; eps(1f-7)
            const float pr = expf(pk);
            acc += 2.0f * (yk * logf(yk / pr + 7.1054274e-15f) + pr - yk);
        } else if (metric == EVB_METRIC_GAMMA) { const float pr = expf(pk); acc += 2.0f * (logf(pr / yk) + yk / pr - 1.0f); }
        else { // tweedie, rho = 1.5 (src/metrics.jl:24-28)
            const float pr = expf(pk), a = sqrtf(pr);
            acc += 2.0f * (sqrtf(yk) / -0.5f / 0.5f - yk * (1.0f / a) / -0.5f + a / 0.5f);
        }
    }
    return w * acc / (float)K;
}

struct EvalArgs {
    const uint8_t *xT;
    const uint32_t *t_packed;
    const float *t_pred;
    const float *fixed_leaf; // non-null: every row receives this leaf (the one-node bias tree), no traversal
    float *pred;
    const void *y;
    const float *w;
    double *part; // [gridDim.x][2]
    long long n;
    int RS, K, loss, metric, nn, ycols, packed_in_smem;
    AlphaSet alpha;
};
// `predict!(cb.p, tree, cb.x_bin, cb.feattypes)` followed by the per-row metric (src/callback.jl:123-128).  Every
// block owns a fixed set of rows and sums them in a fixed order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) k_eval_tree(EvalArgs a) {
    extern __shared__ uint32_t s_packed[];
    __shared__ double s_red[2][8];
    const uint32_t *packed = a.t_packed;
    if (a.packed_in_smem && !a.fixed_leaf) {
        for (int i = threadIdx.x; i < a.nn; i += blockDim.x) s_packed[i] = a.t_packed[i];
        __syncthreads();
        packed = s_packed;
    }
    double sv = 0.0, sw = 0.0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (long long)gridDim.x * blockDim.x) {
        float *p = a.pred + (size_t)i * a.K;
        const float *leaf = a.fixed_leaf ? a.fixed_leaf : a.t_pred + (size_t)(traverse(packed, a.xT + (size_t)i * a.RS) - 1) * a.K;
        pred_add(a.loss, a.K, p, leaf);
        const float w = a.w ? a.w[i] : 1.0f;
        sv += (double)metric_row(a.metric, a.K, p, a.y, a.ycols, i, w, a.alpha);
        sw += (double)w;
    }
    for (int o = 16; o > 0; o >>= 1) { sv += __shfl_down_sync(FULL, sv, o); sw += __shfl_down_sync(FULL, sw, o); }
    if ((threadIdx.x & 31) == 0) { s_red[0][threadIdx.x >> 5] = sv; s_red[1][threadIdx.x >> 5] = sw; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double tv = 0.0, tw = 0.0;
        for (int q = 0; q < 8; ++q) { tv += s_red[0][q]; tw += s_red[1][q]; }
        a.part[2 * blockIdx.x] = tv;
        a.part[2 * blockIdx.x + 1] = tw;
    }
}
__global__ void __launch_bounds__(256) k_eval_sum(const double *part, int nblocks, double *out) {
    __shared__ double s_red[2][256];
    double tv = 0.0, tw = 0.0;
    for (int b = threadIdx.x; b < nblocks; b += 256) { tv += part[2 * b]; tw += part[2 * b + 1]; }
    s_red[0][threadIdx.x] = tv; s_red[1][threadIdx.x] = tw;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) { s_red[0][threadIdx.x] += s_red[0][threadIdx.x + o]; s_red[1][threadIdx.x] += s_red[1][threadIdx.x + o]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) { out[0] = s_red[0][0]; out[1] = s_red[1][0]; }
}

} // namespace

// =====================================================================================================
static AlphaSet evb_alpha_set(const evb_handle *h) {
    AlphaSet s;
    for (int k = 0; k < 8; ++k) s.a[k] = (float)h->p.alphas[k];
    if (h->p.loss != EVB_MULTIQUANTILE) s.a[0] = (float)h->p.alpha;
    return s;
}

int32_t evb_launch_transpose(evb_handle *, const uint8_t *xcol_dev, int64_t ld, int64_t nrows, int j0, int nj, uint8_t *xT,
                             int RS, cudaStream_t st) {
    dim3 grid((unsigned)((nrows + 255) / 256), (unsigned)((nj + 3) / 4));
    k_transpose<<<grid, 256, 0, st>>>(xcol_dev, ld, nrows, j0, nj, xT, RS);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_check_bins(evb_handle *h) {
    k_check_bins<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->xT, h->n, h->RS, h->nfeats, h->B, h->d_err);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_init_state(evb_handle *h, const float *w_dev, const float *pred0_dev, const float *mu_dev) {
    k_init_state<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->grad, h->pred, w_dev, pred0_dev, mu_dev, h->n, h->K, h->GS, h->rec_nch, h->Ce - 1);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_grads(evb_handle *h) {
    if (h->use_q) EVB_CUDA(cudaMemsetAsync(h->d_gmax, 0, sizeof(unsigned), h->st));
    evb_tic(h, EVB_T_GRADS);
    k_grads<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->p.loss, h->K, h->GS, h->rec_nch, h->Ce != h->C, h->ycols, h->n, h->pred, h->y, h->grad,
                                                                h->use_q ? h->d_gmax : nullptr, evb_alpha_set(h));
    evb_toc(h, EVB_T_GRADS);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_quantize(evb_handle *h) {
    evb_tic(h, EVB_T_GRADS);
    k_quantize<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->grad, h->gradq, h->n, h->d_gmax, h->d_qinv, h->wscale, h->winv, h->unit_w ? 1 : 0);
    evb_toc(h, EVB_T_GRADS);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_rows_init(evb_handle *h, bool use_mask, uint8_t mask_cond) {
    evb_tic(h, EVB_T_ROWS_INIT);
    if (!use_mask) {
        k_rows_identity<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->rows[0], h->n, h->nleft);
    } else {
        const int nblocks = (int)((h->n + SEL_CHUNK - 1) / SEL_CHUNK);
        k_sel_count<<<nblocks, SEL_THREADS, 0, h->st>>>(h->mask_d, mask_cond, h->n, h->scan_tmp);
        k_sel_scan<<<1, 1024, 0, h->st>>>(h->scan_tmp, nblocks, h->nleft);
        k_sel_scatter<<<nblocks, SEL_THREADS, 0, h->st>>>(h->mask_d, mask_cond, h->n, h->scan_tmp, h->rows[0]);
    }
    evb_toc(h, EVB_T_ROWS_INIT);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_finalize(evb_handle *h, bool compute_grads, int mode) {
    FinArgs a;
    a.xT = h->xT; a.t_packed = h->t_packed; a.t_pred = h->t_pred; a.pred = h->pred; a.grad = h->grad; a.y = h->y;
    a.nidx = h->nidx; a.n = h->n; a.RS = h->RS; a.K = h->K; a.GS = h->GS; a.NCH = h->rec_nch; a.elided = h->Ce != h->C; a.loss = h->p.loss; a.nn = h->nn;
    a.gmax = h->use_q ? h->d_gmax : nullptr;
    if (h->use_q && compute_grads) EVB_CUDA(cudaMemsetAsync(h->d_gmax, 0, sizeof(unsigned), h->st));
    a.ycols = h->ycols; a.compute_grads = compute_grads ? 1 : 0; a.alpha = evb_alpha_set(h); a.mode = mode;
    const size_t smem = (size_t)h->nn * 4;
    a.packed_in_smem = smem <= 40 * 1024 ? 1 : 0;
    const size_t staged = smem + (size_t)256 * (h->RS + 4);
    static bool attr_set[64] = {}, attr_pipe[64] = {};
    static const bool direct = getenv("EVB_FINALIZE_DIRECT") != nullptr;
    static const bool no_pipe = getenv("EVB_FINALIZE_PIPE") != nullptr && atoi(getenv("EVB_FINALIZE_PIPE")) == 0;
    // pipelined kernel: rows from the chunk layout of the fixed-point histogram kernel when it exists, else from xT
    FinPipeArgs pa;
    pa.f = a;
    const bool from_q2 = h->use_q2; // xH holds feature f at byte f of the row, the tail features follow in xE
    pa.rowsA = from_q2 ? h->xH : h->xT;
    pa.xE = from_q2 && h->q2.ntail > 0 ? h->xE : nullptr;
    pa.strideA = from_q2 ? h->q2.RSH : h->RS;
    pa.wordsA = pa.strideA / 4;
    pa.S = pa.wordsA + 4; // one more chunk: room for the tail word, and an odd chunk count (wordsA / 4 is even or RSH-odd)
    if (((pa.S >> 2) & 1) == 0) pa.S += 4;
    pa.ntiles = (int)((h->n + 255) / 256);
    pa.leaf_in_smem = h->K == 1 ? 1 : 0;
    const size_t pipe_smem = (size_t)((h->nn + 3) & ~3) * 4 * (pa.leaf_in_smem ? 2 : 1) + (size_t)2 * 256 * pa.S * 4;
    evb_tic(h, EVB_T_FINALIZE);
    // measured (B200): 0.33 instead of 0.42 ms per 10M rows x 100 features with one output; with several outputs the
    // prediction and gradient streams outweigh the bins and the one-tile-per-CTA kernel below is faster
    if (mode == 0 && h->K == 1 && pipe_smem <= 100 * 1024 && pa.wordsA <= 64 && !direct && !no_pipe && h->dev < 64) {
        if (!attr_pipe[h->dev]) {
            cudaFuncSetAttribute(k_finalize_pipe<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            cudaFuncSetAttribute(k_finalize_pipe<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            attr_pipe[h->dev] = true;
        }
        int per_sm = (int)((227 * 1024) / (pipe_smem + 1024)); // 1 KB per resident CTA is reserved
        if (per_sm > 6) per_sm = 6;
        if (per_sm < 1) per_sm = 1;
        int grid = h->num_sms * per_sm;
        if (grid > pa.ntiles) grid = pa.ntiles;
        if (h->p.loss == EVB_MSE && a.elided && h->rec_nch == 2 && h->ycols == 1) k_finalize_pipe<true><<<grid, 256, pipe_smem, h->st>>>(pa);
        else k_finalize_pipe<false><<<grid, 256, pipe_smem, h->st>>>(pa);
    } else if (mode == 0 && h->RS <= 256 && staged <= 100 * 1024 && !direct && h->dev < 64) {
        if (!attr_set[h->dev]) { cudaFuncSetAttribute(k_finalize_staged, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); attr_set[h->dev] = true; }
        k_finalize_staged<<<(unsigned)((h->n + 255) / 256), 256, staged, h->st>>>(a);
    } else {
        k_finalize<<<(unsigned)((h->n + 255) / 256), 256, a.packed_in_smem ? smem : 0, h->st>>>(a);
    }
    evb_toc(h, EVB_T_FINALIZE);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// applies the current tree (or, with `fixed_leaf_dev`, one leaf for every row) to the evaluation predictions and
// leaves the metric sums in h->d_evsum
int32_t evb_launch_eval(evb_handle *h, const float *fixed_leaf_dev) {
    EvalArgs a;
    a.xT = h->ev_xT; a.t_packed = h->t_packed; a.t_pred = h->t_pred; a.fixed_leaf = fixed_leaf_dev; a.pred = h->ev_pred;
    a.y = h->ev_y; a.w = h->ev_w; a.part = h->ev_part; a.n = h->ev_n; a.RS = h->RS; a.K = h->K; a.loss = h->p.loss;
    a.metric = h->ev_metric; a.nn = h->nn; a.ycols = h->ycols; a.alpha = evb_alpha_set(h);
    const size_t smem = (size_t)h->nn * 4;
    a.packed_in_smem = smem <= 40 * 1024 ? 1 : 0;
    evb_tic(h, EVB_T_FINALIZE);
    k_eval_tree<<<h->ev_blocks, 256, (a.packed_in_smem && !fixed_leaf_dev) ? smem : 0, h->st>>>(a);
    k_eval_sum<<<1, 256, 0, h->st>>>(h->ev_part, h->ev_blocks, h->d_evsum);
    evb_toc(h, EVB_T_FINALIZE);
    h->tm.launches[EVB_T_FINALIZE] += 1; // two kernels inside one timed bracket
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// quantile loss, K = 1: leaf ids are in h->nidx (finalize mode 1); fills the leaf values of the tree
int32_t evb_launch_quantile_leaves(evb_handle *h, bool use_mask, uint8_t mask_cond) {
    QselArgs a;
    a.nidx = h->nidx; a.grad = h->grad; a.mask = use_mask ? h->mask_d : nullptr; a.cnt = h->qs_cnt; a.prefix = h->qs_prefix;
    a.rank = h->qs_rank; a.gamma = h->qs_gamma; a.t_split = h->t_split; a.nsum = h->nsum; a.t_pred = h->t_pred; a.n = h->n;
    a.GS = h->GS; a.nn = h->nn; a.C = h->C; a.cond = mask_cond;
    a.eb = h->p.eta / (double)h->p.bagging_size; a.lambda = h->p.lambda; a.L2 = h->p.L2; a.K = h->K;
    a.clamp = h->p.loss == EVB_QUANTILE ? 1 : 0; // src/predict.jl:270 has the max(eps, .), :279 has not
    evb_tic(h, EVB_T_FINALIZE);
    for (int k = 0; k < h->K; ++k) { // one selection per output row: the residual of row k sits in the slot of h_k
        const int c = h->K + k;
        a.k = k; a.roff = (c / h->rec_nch) * 4 + (c % h->rec_nch);
        a.alpha = h->p.loss == EVB_QUANTILE ? h->p.alpha : h->p.alphas[k];
        for (int pass = 0; pass < 4; ++pass) {
            a.pass = pass;
            k_qsel_count<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(a);
            if (h->world > 1) {
                // row-sharded: the digit counts of all ranks are added, so every rank walks to the same order
                // statistics of the leaf's rows on all ranks (integer sums: the same leaves as on one GPU)
                int32_t *c32 = reinterpret_cast<int32_t *>(h->qs_cnt);
                EVB_CHECK(evb_nccl_allreduce_i32(h, c32, c32, (size_t)2 * (h->nn + 1) * 256));
            }
            k_qsel_pick<<<(h->nn + 8) / 8, 256, 0, h->st>>>(a);
        }
        k_qsel_leaf<<<(h->nn + 256) / 256, 256, 0, h->st>>>(a);
    }
    evb_toc(h, EVB_T_FINALIZE);
    h->tm.launches[EVB_T_FINALIZE] += 9 * h->K - 1;
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_nidx_from_partition(evb_handle *h, uint32_t *out_dev) {
    EVB_CUDA(cudaMemsetAsync(out_dev, 0, sizeof(uint32_t) * h->n, h->st));
    int blocks = h->nn < 1024 ? h->nn : 1024;
    k_nidx_from_partition<<<blocks, 256, 0, h->st>>>(h->rows[0], h->rows[1], h->seg_start, h->seg_cnt, h->t_split, h->nn, out_dev);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// ---- training matrix from raw features -----------------------------------------------------------------
struct DevBufT {
    void *p = nullptr;
    ~DevBufT() { evb_dev_free(p); }
};
// `binarize(x_train; edges)` of `init_core` (ext/EvoTreesKernelAbstractionsExt/init.jl:3-6, src/fit-utils.jl:66-72) on the
// device: the raw column-major matrix travels in blocks of whole features (each at most 256 MB) and every block is
// binarized straight into the feature-major bin matrix h->xC; the bins never visit the host.  NaN sets the error word.
int32_t evb_upload_binarize(evb_handle *h, const void *x, int32_t dtype, const void *edges, int32_t nedges) {
    const size_t es = dtype == EVB_F64 ? 8 : 4;
    const int64_t n = h->n;
    const int nfeats = h->nfeats;
    int cf = (int)std::max<int64_t>(1, std::min<int64_t>(nfeats, ((int64_t)256 << 20) / (int64_t)(n * es)));
    DevBufT d_x, d_e;
    EVB_CUDA(evb_dev_alloc(&d_x.p, (size_t)cf * n * es));
    EVB_CUDA(evb_dev_alloc(&d_e.p, (size_t)nedges * nfeats * es));
    EVB_CUDA(cudaMemcpyAsync(d_e.p, edges, (size_t)nedges * nfeats * es, cudaMemcpyHostToDevice, h->st));
    unsigned bx = (unsigned)((n + 255) / 256);
    if (bx > 4096) bx = 4096;
    for (int j0 = 0; j0 < nfeats; j0 += cf) {
        const int nj = std::min(cf, nfeats - j0);
        // no wait at the end of a block: its last chunks travel while the host gathers the next block's first ones
        EVB_CHECK(evb_h2d_staged(d_x.p, (const char *)x + (size_t)j0 * n * es, (size_t)nj * n * es, h->st, false));
        dim3 grid(bx, (unsigned)nj);
        if (dtype == EVB_F32)
            k_binarize<float><<<grid, 256, (size_t)nedges * 4, h->st>>>((const float *)d_x.p, n, n, (const float *)d_e.p + (size_t)j0 * nedges, nedges,
                                                                           h->xC + (size_t)j0 * n, n, h->d_err);
        else
            k_binarize<double><<<grid, 256, (size_t)nedges * 8, h->st>>>((const double *)d_x.p, n, n, (const double *)d_e.p + (size_t)j0 * nedges, nedges,
                                                                            h->xC + (size_t)j0 * n, n, h->d_err);
        EVB_CUDA(cudaGetLastError());
    }
    EVB_CUDA(cudaStreamSynchronize(h->st)); // the staging buffers are freed on return
    return EVB_OK;
}

// ---- stateless entry points -----------------------------------------------------------------------
static int32_t check_device(int device) {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) {
        evb_set_error("no CUDA device available (%s): this library has no CPU fallback", cudaGetErrorString(e));
        return EVB_ERR_CUDA;
    }
    if (device < 0 || device >= ndev) { evb_set_error("device %d out of range (0..%d)", device, ndev - 1); return EVB_ERR_ARG; }
    EVB_CUDA(cudaSetDevice(device));
    return EVB_OK;
}

struct DevBuf {
    void *p = nullptr;
    ~DevBuf() { evb_dev_free(p); }
    cudaError_t alloc(size_t bytes) { return evb_dev_alloc(&p, bytes ? bytes : 1); }
    template <typename T> T *as() { return reinterpret_cast<T *>(p); }
};

// Common body of evb_predict (binned input) and evb_predict_x (raw input + edges, binarized on the device).
static int32_t predict_impl(int32_t device, int32_t loss, int32_t K, int32_t ntrees, int32_t nn, const int64_t *feat,
                            const uint8_t *cond_bin, const uint8_t *split, const float *leaf_pred, const uint8_t *x_bin, const void *x,
                            int32_t x_dtype, int32_t x_row_major, const void *edges, int32_t nedges, int64_t nobs, int32_t nfeats,
                            const uint8_t *feattypes, int32_t apply_link, float *out, uint32_t *leaf_idx, double *ms_out) {
    if (!feat || !cond_bin || !split || !leaf_pred || (!x_bin && !x) || !out || nobs < 0 || nfeats < 1 || nfeats > 65535 ||
        ntrees < 0 || nn < 1 || K < 1 || K > 64 || loss < 0 || loss > EVB_LOSS_LAST) {
        evb_set_error("evb_predict: invalid argument");
        return EVB_ERR_ARG;
    }
    if (x && (!edges || nedges < 1 || nedges > 254 || (x_dtype != EVB_F32 && x_dtype != EVB_F64))) {
        evb_set_error("evb_predict_x: edges / dtype invalid");
        return EVB_ERR_ARG;
    }
    EVB_CHECK(check_device(device));
    if (nobs == 0) return EVB_OK;
    cudaStream_t st;
    EVB_CUDA(cudaStreamCreate(&st));
    const int RS = (nfeats + 31) / 32 * 32;
    const size_t es = x_dtype == EVB_F64 ? 8 : 4;
    const long long total = (long long)ntrees * nn;
    const int64_t chunk = nobs < (int64_t)1 << 20 ? nobs : (int64_t)1 << 20;
    // Blocks of `chunk` rows, two of everything: while the kernels of block k run, the host stages block k + 1 through
    // the pinned ring (several threads) and the copy engine brings it over.
    DevBuf d_feat, d_bin, d_split, d_ft, d_packed, d_leaf, d_in[2], d_xT[2], d_out, d_lidx, d_edges;
    cudaEvent_t ev_free[2] = {nullptr, nullptr}, ev_k0[2] = {nullptr, nullptr}, ev_k1[2] = {nullptr, nullptr}, ev_in[2] = {nullptr, nullptr};
    cudaStream_t cs = nullptr;
    float kernel_ms = 0.f;
    // traversal out of shared memory when a tree (packed nodes + leaf table) fits a block of it
    const int nnp = (nn + 3) & ~3;
    const size_t treebytes = (size_t)nnp * (1 + K) * 4;
    int rows_cta = 1024;
    while (rows_cta > 128 && (size_t)rows_cta * RS > (size_t)132 * 1024) rows_cta >>= 1;
    const size_t rows_smem = (size_t)rows_cta * RS;
    int TB = rows_smem < (size_t)200 * 1024 ? (int)(((size_t)200 * 1024 - rows_smem) / (2 * treebytes)) : 0;
    if (TB > 8) TB = 8;
    const bool staged = TB >= 1 && RS % 16 == 0 && !getenv("EVB_PREDICT_DIRECT");
    const size_t pred_smem = rows_smem + (size_t)2 * TB * treebytes;
    DevBuf d_staged;
    auto body = [&]() -> int32_t {
        EVB_CUDA(evb_stream_get(&cs));
        for (int q = 0; q < 2; ++q) {
            EVB_CUDA(cudaEventCreateWithFlags(&ev_free[q], cudaEventDisableTiming));
            EVB_CUDA(cudaEventCreateWithFlags(&ev_in[q], cudaEventDisableTiming));
            EVB_CUDA(cudaEventCreate(&ev_k0[q])); EVB_CUDA(cudaEventCreate(&ev_k1[q]));
            EVB_CUDA(d_in[q].alloc((size_t)chunk * nfeats * (x ? es : 1))); EVB_CUDA(d_xT[q].alloc((size_t)chunk * RS));
            EVB_CUDA(cudaMemsetAsync(d_xT[q].p, 0, (size_t)chunk * RS, st));
        }
        EVB_CUDA(d_feat.alloc(total * 8)); EVB_CUDA(d_bin.alloc(total)); EVB_CUDA(d_split.alloc(total));
        EVB_CUDA(d_packed.alloc(total * 4)); EVB_CUDA(d_leaf.alloc((size_t)total * K * 4));
        EVB_CUDA(d_out.alloc((size_t)nobs * K * 4));
        if (leaf_idx) EVB_CUDA(d_lidx.alloc((size_t)nobs * ntrees * 4));
        if (feattypes) { EVB_CUDA(d_ft.alloc(nfeats)); EVB_CUDA(cudaMemcpyAsync(d_ft.p, feattypes, nfeats, cudaMemcpyHostToDevice, st)); }
        if (x) { EVB_CUDA(d_edges.alloc((size_t)nedges * nfeats * es)); EVB_CUDA(cudaMemcpyAsync(d_edges.p, edges, (size_t)nedges * nfeats * es, cudaMemcpyHostToDevice, st)); }
        EVB_CUDA(cudaMemcpyAsync(d_feat.p, feat, total * 8, cudaMemcpyHostToDevice, st));
        EVB_CUDA(cudaMemcpyAsync(d_bin.p, cond_bin, total, cudaMemcpyHostToDevice, st));
        EVB_CUDA(cudaMemcpyAsync(d_split.p, split, total, cudaMemcpyHostToDevice, st));
        EVB_CUDA(cudaMemcpyAsync(d_leaf.p, leaf_pred, (size_t)total * K * 4, cudaMemcpyHostToDevice, st));
        if (total > 0) {
            k_pack_trees<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_feat.as<long long>(), d_bin.as<uint8_t>(), d_split.as<uint8_t>(),
                                                                           feattypes ? d_ft.as<uint8_t>() : nullptr, total, d_packed.as<uint32_t>());
            EVB_CUDA(cudaGetLastError());
        }
        if (staged && total > 0) {
            EVB_CUDA(d_staged.alloc((size_t)ntrees * treebytes));
            k_pack_staged<<<512, 256, 0, st>>>(d_packed.as<uint32_t>(), d_leaf.as<float>(), ntrees, nn, nnp, K, d_staged.as<uint32_t>());
            EVB_CUDA(cudaGetLastError());
        }
        EVB_CUDA(cudaStreamSynchronize(st)); // trees, edges and the cleared row buffers are in place before the copy stream starts
        int k = 0;
        for (int64_t r0 = 0; r0 < nobs; r0 += chunk, ++k) {
            const int q = k & 1;
            const int64_t nr = nobs - r0 < chunk ? nobs - r0 : chunk;
            if (k >= 2) { // the kernels of block k - 2 are done with these buffers
                EVB_CUDA(cudaEventSynchronize(ev_free[q]));
                float ms = 0.f;
                if (cudaEventElapsedTime(&ms, ev_k0[q], ev_k1[q]) == cudaSuccess) kernel_ms += ms;
            }
            // rows r0 .. r0 + nr of every column (column-major input: one segment per feature), packed as [nfeats][nr]
            // the host does not wait for the copies: the kernels do (event), and the host goes on gathering the next block
            if (x && x_row_major) EVB_CHECK(evb_h2d_staged(d_in[q].p, (const char *)x + (size_t)r0 * nfeats * es, (size_t)nr * nfeats * es, cs, false));
            else if (x) EVB_CHECK(evb_h2d_staged_strided(d_in[q].p, (const char *)x + (size_t)r0 * es, (size_t)nr * es, (size_t)nfeats, (size_t)nobs * es, cs, false));
            else EVB_CHECK(evb_h2d_staged_strided(d_in[q].p, x_bin + r0, (size_t)nr, (size_t)nfeats, (size_t)nobs, cs, false));
            EVB_CUDA(cudaEventRecord(ev_in[q], cs));
            EVB_CUDA(cudaStreamWaitEvent(st, ev_in[q], 0));
            EVB_CUDA(cudaEventRecord(ev_k0[q], st));
            if (x) {
                const unsigned blocks = (unsigned)((nr + 255) / 256);
                const long long ld = x_row_major ? nfeats : nr;
                if (256 * (RS + 4) > 48 * 1024) { // rows of more than 188 bins: the tile needs the opt-in shared memory
                    EVB_CUDA(cudaFuncSetAttribute(k_binarize_rows<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * (RS + 4)));
                    EVB_CUDA(cudaFuncSetAttribute(k_binarize_rows<double>, cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * (RS + 4)));
                }
                if (x_dtype == EVB_F32)
                    k_binarize_rows<float><<<blocks, 256, 256 * (RS + 4), st>>>(d_in[q].as<float>(), ld, x_row_major, nr, nfeats, d_edges.as<float>(), nedges, d_xT[q].as<uint8_t>(), RS);
                else
                    k_binarize_rows<double><<<blocks, 256, 256 * (RS + 4), st>>>(d_in[q].as<double>(), ld, x_row_major, nr, nfeats, d_edges.as<double>(), nedges, d_xT[q].as<uint8_t>(), RS);
                EVB_CUDA(cudaGetLastError());
            } else {
                EVB_CHECK(evb_launch_transpose(nullptr, d_in[q].as<uint8_t>(), nr, nr, 0, nfeats, d_xT[q].as<uint8_t>(), RS, st));
            }
            PredArgs a;
            a.xT = d_xT[q].as<uint8_t>(); a.packed = d_packed.as<uint32_t>(); a.leaf = d_leaf.as<float>(); a.out = d_out.as<float>();
            a.leaf_idx = leaf_idx ? d_lidx.as<uint32_t>() : nullptr; a.n = nr; a.row0 = r0; a.nobs_total = nobs; a.RS = RS; a.K = K;
            a.loss = loss; a.ntrees = ntrees; a.nn = nn; a.apply_link = apply_link;
            if (staged) {
                const unsigned blocks = (unsigned)((nr + rows_cta - 1) / rows_cta);
#define EVB_PRED_STAGED(KM) do { \
                    EVB_CUDA(cudaFuncSetAttribute(k_predict_staged<KM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pred_smem)); \
                    k_predict_staged<KM><<<blocks, rows_cta, pred_smem, st>>>(a, d_staged.as<uint32_t>(), nnp, rows_cta, TB); } while (0)
                if (K <= 1) EVB_PRED_STAGED(1);
                else if (K <= 2) EVB_PRED_STAGED(2);
                else if (K <= 8) EVB_PRED_STAGED(8);
                else EVB_PRED_STAGED(64);
#undef EVB_PRED_STAGED
            } else {
                const unsigned blocks = (unsigned)((nr + 255) / 256);
                if (K <= 1) k_predict<1><<<blocks, 256, 0, st>>>(a);
                else if (K <= 2) k_predict<2><<<blocks, 256, 0, st>>>(a);
                else if (K <= 8) k_predict<8><<<blocks, 256, 0, st>>>(a);
                else k_predict<64><<<blocks, 256, 0, st>>>(a);
            }
            EVB_CUDA(cudaGetLastError());
            EVB_CUDA(cudaEventRecord(ev_k1[q], st));
            EVB_CUDA(cudaEventRecord(ev_free[q], st));
        }
        EVB_CUDA(cudaMemcpyAsync(out, d_out.p, (size_t)nobs * K * 4, cudaMemcpyDeviceToHost, st));
        if (leaf_idx) EVB_CUDA(cudaMemcpyAsync(leaf_idx, d_lidx.p, (size_t)nobs * ntrees * 4, cudaMemcpyDeviceToHost, st));
        EVB_CUDA(cudaStreamSynchronize(st));
        for (int q = 0; q < 2 && q < k; ++q) { // the last (up to) two blocks have not been read yet
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, ev_k0[q], ev_k1[q]) == cudaSuccess) kernel_ms += ms;
        }
        return EVB_OK;
    };
    int32_t rc = body();
    cudaStreamSynchronize(st);
    if (cs) { cudaStreamSynchronize(cs); evb_stream_put(cs); }
    if (ms_out) *ms_out = kernel_ms;
    for (int q = 0; q < 2; ++q) {
        if (ev_free[q]) cudaEventDestroy(ev_free[q]);
        if (ev_in[q]) cudaEventDestroy(ev_in[q]);
        if (ev_k0[q]) cudaEventDestroy(ev_k0[q]);
        if (ev_k1[q]) cudaEventDestroy(ev_k1[q]);
    }
    cudaStreamDestroy(st);
    return rc;
}

extern "C" int32_t evb_predict(int32_t device, int32_t loss, int32_t K, int32_t ntrees, int32_t nn, const int64_t *feat,
                               const uint8_t *cond_bin, const uint8_t *split, const float *leaf_pred, const uint8_t *x_bin,
                               int64_t nobs, int32_t nfeats, const uint8_t *feattypes, int32_t apply_link, float *out,
                               uint32_t *leaf_idx) {
    if (!x_bin) { evb_set_error("evb_predict: x_bin is null"); return EVB_ERR_ARG; }
    return predict_impl(device, loss, K, ntrees, nn, feat, cond_bin, split, leaf_pred, x_bin, nullptr, 0, 0, nullptr, 0, nobs, nfeats,
                        feattypes, apply_link, out, leaf_idx, nullptr);
}

extern "C" int32_t evb_predict_x(int32_t device, int32_t loss, int32_t K, int32_t ntrees, int32_t nn, const int64_t *feat,
                                 const uint8_t *cond_bin, const uint8_t *split, const float *leaf_pred, const void *x, int32_t x_dtype,
                                 int32_t x_row_major, const void *edges, int32_t nedges, int64_t nobs, int32_t nfeats,
                                 const uint8_t *feattypes, int32_t apply_link, float *out, uint32_t *leaf_idx, double *kernel_ms) {
    if (!x) { evb_set_error("evb_predict_x: x is null"); return EVB_ERR_ARG; }
    return predict_impl(device, loss, K, ntrees, nn, feat, cond_bin, split, leaf_pred, nullptr, x, x_dtype, x_row_major, edges, nedges,
                        nobs, nfeats, feattypes, apply_link, out, leaf_idx, kernel_ms);
}

extern "C" int32_t evb_binarize(int32_t device, const void *x, int32_t dtype, int64_t nobs, int32_t nfeats, const void *edges,
                                int32_t nedges, uint8_t *x_bin) {
    if (!x || !edges || !x_bin || nobs < 0 || nfeats < 1 || nedges < 1 || nedges > 254 || (dtype != EVB_F32 && dtype != EVB_F64)) {
        evb_set_error("evb_binarize: invalid argument");
        return EVB_ERR_ARG;
    }
    EVB_CHECK(check_device(device));
    if (nobs == 0) return EVB_OK;
    const size_t es = dtype == EVB_F32 ? 4 : 8;
    cudaStream_t st;
    EVB_CUDA(cudaStreamCreate(&st));
    const int64_t chunk = nobs < (int64_t)4 << 20 ? nobs : (int64_t)4 << 20;
    DevBuf d_x, d_e, d_o;
    auto body = [&]() -> int32_t {
        EVB_CUDA(d_x.alloc((size_t)chunk * nfeats * es)); EVB_CUDA(d_e.alloc((size_t)nedges * nfeats * es)); EVB_CUDA(d_o.alloc((size_t)chunk * nfeats));
        EVB_CUDA(cudaMemcpyAsync(d_e.p, edges, (size_t)nedges * nfeats * es, cudaMemcpyHostToDevice, st));
        for (int64_t r0 = 0; r0 < nobs; r0 += chunk) {
            const int64_t nr = nobs - r0 < chunk ? nobs - r0 : chunk;
            EVB_CUDA(cudaMemcpy2DAsync(d_x.p, (size_t)chunk * es, (const char *)x + (size_t)r0 * es, (size_t)nobs * es, (size_t)nr * es,
                                       (size_t)nfeats, cudaMemcpyHostToDevice, st));
            unsigned bx = (unsigned)((nr + 255) / 256);
            if (bx > 4096) bx = 4096;
            dim3 grid(bx, (unsigned)nfeats);
            if (dtype == EVB_F32)
                k_binarize<float><<<grid, 256, (size_t)nedges * 4, st>>>(d_x.as<float>(), chunk, nr, d_e.as<float>(), nedges, d_o.as<uint8_t>(), chunk);
            else
                k_binarize<double><<<grid, 256, (size_t)nedges * 8, st>>>(d_x.as<double>(), chunk, nr, d_e.as<double>(), nedges, d_o.as<uint8_t>(), chunk);
            EVB_CUDA(cudaGetLastError());
            EVB_CUDA(cudaMemcpy2DAsync(x_bin + r0, (size_t)nobs, d_o.p, (size_t)chunk, (size_t)nr, (size_t)nfeats, cudaMemcpyDeviceToHost, st));
        }
        EVB_CUDA(cudaStreamSynchronize(st));
        return EVB_OK;
    };
    int32_t rc = body();
    cudaStreamSynchronize(st);
    cudaStreamDestroy(st);
    return rc;
}
