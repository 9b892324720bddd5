// Histogram build: `update_hist!` / `_hist!` (src/fit-utils.jl:345-394) and the reference GPU
// `hist_kernel!` (ext/EvoTreesKernelAbstractionsExt/fit-utils.jl:57-95), redesigned for sm_100a.
//
// Design
//   * The rows of every build node are a contiguous segment of a row-index list.  The concatenation of
//     all build segments of a level is cut into gridDim.x equal row ranges, one per CTA, so every CTA
//     streams the same number of rows whatever the node sizes are.  A (CTA, node) intersection is a "piece".
//   * One producer warp stages tiles of 32 rows: each lane issues two TMA bulk copies
//     (cp.async.bulk global->shared, completion on an mbarrier): the row of the observation-major bin
//     matrix (RS bytes) and the row's gradient record (GS floats).  Consumers never touch global memory
//     in the inner loop.
//   * Each consumer warp owns one "unit": 32 feature slots (lane = feature) x up to 4 gradient channels,
//     with a private image img[channel][bin][lane] in shared memory.  Lane l only ever touches bank l, so
//     the accumulation is a plain load/add/store: no atomics, no bank conflicts, and a fixed summation
//     order (ascending rows) inside a piece.
//   * At the end of a piece the image is written to a scratch slot indexed by (CTA, build slot).  A second
//     kernel sums the pieces of every node in ascending CTA order in double precision, so histograms are
//     bit-reproducible from run to run, and transposes them to hcomp[slot][feature][channel][bin].
//   Every wait on an mbarrier is bounded; on expiry the kernel records an error code and returns.
#include "evb_internal.cuh"

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (or as soon as another warp has flagged an error).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, int code) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *(volatile int *)err != 0) return false;
    }
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

struct HistArgs {
    const uint8_t *xT;
    const float *grad;
    const uint32_t *rows;
    const uint32_t *js0;
    const LevelPlan *plan;
    const int32_t *cum;
    const int32_t *slot_node;
    const int32_t *seg_start;
    float *scratch;
    int *err;
    int RS, GS, F, nbins, C, NFG, U, UB, stages, PG;
    uint32_t img_floats;
};

template <int BP, int NCH>
__device__ __forceinline__ void accum_row(float *hl, uint32_t bin, const float4 &g, int nch) {
    const uint32_t bi = min(bin - 1u, (uint32_t)(BP - 1)) * 32u;
    hl[bi] += g.x;
    if (NCH >= 2 && nch >= 2) hl[BP * 32 + bi] += g.y;
    if (NCH >= 3 && nch >= 3) hl[2 * BP * 32 + bi] += g.z;
    if (NCH >= 4 && nch >= 4) hl[3 * BP * 32 + bi] += g.w;
}

template <int BP, int NCH>
__global__ void __launch_bounds__((EVB_MAX_UNITS_PER_BLOCK + 1) * 32) k_hist(HistArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, b = blockIdx.x, ug = blockIdx.y;
    const int nact = min(a.UB, a.U - ug * a.UB);
    const int S = a.stages;
    const int xbytes = EVB_TILE_ROWS * a.RS, gbytes = EVB_TILE_ROWS * a.GS * 4;
    const int stage_bytes = xbytes + gbytes;
    float *imgs = reinterpret_cast<float *>(smem);
    unsigned char *stage0 = smem + (size_t)a.UB * 32 * BP * NCH * 4;
    uint64_t *full = reinterpret_cast<uint64_t *>(stage0 + (size_t)S * stage_bytes);
    uint64_t *empty = full + S;

    const long long R = a.plan->R;
    const long long lo = R * b / G, hi = R * (b + 1) / G;
    if (lo >= hi) return;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], nact); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = tid; i < nact * 32 * BP * NCH; i += blockDim.x) imgs[i] = 0.0f;
    __syncthreads();

    // first build slot that contains row `lo`: largest s with cum[s] <= lo
    const int nbuild = a.plan->nbuild;
    int s;
    {
        int l = 0, r = nbuild - 1;
        while (l < r) { int m = (l + r + 1) >> 1; if ((long long)a.cum[m] <= lo) l = m; else r = m - 1; }
        s = l;
    }

    if (wid == 0) {
        // ---------------- producer: stage tiles of rows with TMA bulk copies -------------------------
        uint32_t it = 0;
        long long pos = lo;
        bool ok = true;
        while (pos < hi && ok) {
            const long long send = min(hi, (long long)a.cum[s + 1]);
            if (send > pos) {
                const int node = a.slot_node[s];
                const long long base = (long long)a.seg_start[node] - a.cum[s];
                for (long long q0 = pos; q0 < send && ok; q0 += EVB_TILE_ROWS, ++it) {
                    const int st = it % S;
                    const int nrows = (int)min((long long)EVB_TILE_ROWS, send - q0);
                    uint32_t row = 0;
                    if (lane < nrows) row = a.rows[base + q0 + lane];
                    ok = mbar_wait(&empty[st], ((it / S) & 1u) ^ 1u, a.err, EVB_DERR_WAIT_EMPTY);
                    if (!ok) break;
                    if (lane == 0) mbar_expect_tx(&full[st], (uint32_t)nrows * (uint32_t)(a.RS + a.GS * 4));
                    __syncwarp();
                    if (lane < nrows) {
                        unsigned char *sb = stage0 + (size_t)st * stage_bytes;
                        bulk_g2s(sb + lane * a.RS, a.xT + (size_t)row * a.RS, (uint32_t)a.RS, &full[st]);
                        bulk_g2s(sb + xbytes + lane * a.GS * 4, a.grad + (size_t)row * a.GS, (uint32_t)a.GS * 4, &full[st]);
                    }
                }
            }
            pos = send;
            ++s;
        }
        if (!ok) {
            // error path: let the copies already issued land before the CTA's shared memory is released
            const uint32_t first = it > (uint32_t)S ? it - S : 0;
            for (uint32_t j = first; j < it; ++j) {
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(&full[j % S], (j / S) & 1u)) break;
            }
        }
        return;
    }
    if (wid - 1 >= nact) return;

    // ---------------- consumers: one unit (32 feature slots x up to NCH channels) per warp ------------
    const int uw = wid - 1;
    const int u = ug * a.UB + uw;
    const int ct = u / a.NFG, fg = u % a.NFG;
    const int slot = fg * 32 + lane;
    const bool act = slot < a.F;
    const uint32_t foff = act ? a.js0[slot] : 0u;
    const int nch = min(NCH, a.C - ct * 4);
    float *img = imgs + (size_t)uw * 32 * BP * NCH;
    float *hl = img + lane;
    const int RS = a.RS, GS = a.GS;

    uint32_t it = 0;
    long long pos = lo;
    while (pos < hi) {
        const long long send = min(hi, (long long)a.cum[s + 1]);
        if (send > pos) {
            for (long long q0 = pos; q0 < send; q0 += EVB_TILE_ROWS, ++it) {
                const int st = it % S;
                const int nrows = (int)min((long long)EVB_TILE_ROWS, send - q0);
                if (!mbar_wait(&full[st], (it / S) & 1u, a.err, EVB_DERR_WAIT_FULL)) return;
                const unsigned char *xs = stage0 + (size_t)st * stage_bytes + foff;
                const float *gs = reinterpret_cast<const float *>(stage0 + (size_t)st * stage_bytes + xbytes) + ct * 4;
                if (act) {
                    int r = 0;
                    for (; r + 4 <= nrows; r += 4) {
                        const uint32_t b0 = xs[(r + 0) * RS], b1 = xs[(r + 1) * RS], b2 = xs[(r + 2) * RS], b3 = xs[(r + 3) * RS];
                        const float4 g0 = *reinterpret_cast<const float4 *>(gs + (r + 0) * GS);
                        const float4 g1 = *reinterpret_cast<const float4 *>(gs + (r + 1) * GS);
                        const float4 g2 = *reinterpret_cast<const float4 *>(gs + (r + 2) * GS);
                        const float4 g3 = *reinterpret_cast<const float4 *>(gs + (r + 3) * GS);
                        accum_row<BP, NCH>(hl, b0, g0, nch);
                        accum_row<BP, NCH>(hl, b1, g1, nch);
                        accum_row<BP, NCH>(hl, b2, g2, nch);
                        accum_row<BP, NCH>(hl, b3, g3, nch);
                    }
                    for (; r < nrows; ++r) {
                        const uint32_t b0 = xs[r * RS];
                        const float4 g0 = *reinterpret_cast<const float4 *>(gs + r * GS);
                        accum_row<BP, NCH>(hl, b0, g0, nch);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }
            // flush the piece (CTA b, slot s) and clear the image
            float *dst = a.scratch + ((size_t)(ug * a.PG + b + s) * a.UB + uw) * a.img_floats + lane;
            for (int c = 0; c < nch; ++c) {
                for (int bin = 0; bin < a.nbins; ++bin) {
                    float *p = hl + (c * BP + bin) * 32;
                    dst[(c * a.nbins + bin) * 32] = *p;
                    *p = 0.0f;
                }
            }
        }
        pos = send;
        ++s;
    }
}

struct ReduceArgs {
    const float *scratch;
    double *hcomp;
    const LevelPlan *plan;
    const int32_t *cum;
    int G, PG, UB, NFG, U, F, C, nbins, NCH;
    uint32_t img_floats;
};

// grid (max build slots of the level, U, ceil(nbins/16)); 512 threads: warp = bin, lane = feature slot
__global__ void __launch_bounds__(512) k_hist_reduce(ReduceArgs a) {
    __shared__ double tile[16][33];
    const int s = blockIdx.x, u = blockIdx.y, bin0 = blockIdx.z * 16;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ug = u / a.UB, uw = u % a.UB, ct = u / a.NFG, fg = u % a.NFG;
    const int nch = min(a.NCH, a.C - ct * 4);
    const int nbuild = a.plan->nbuild;
    const long long R = a.plan->R;
    int bfirst = 0, blast = -1;
    if (s < nbuild && R > 0) {
        const long long c0 = a.cum[s], c1 = a.cum[s + 1];
        if (c1 > c0) {
            bfirst = (int)(((c0 + 1) * a.G - 1) / R);
            blast = (int)((c1 * a.G - 1) / R);
        }
    }
    const int fl = threadIdx.x >> 4, bl = threadIdx.x & 15;
    for (int c = 0; c < nch; ++c) {
        double acc = 0.0;
        const int bin = bin0 + w;
        if (bin < a.nbins) {
            const float *src = a.scratch + ((size_t)(ug * a.PG + s) * a.UB + uw) * a.img_floats + (c * a.nbins + bin) * 32 + lane;
            const size_t bstride = (size_t)a.UB * a.img_floats;
            // CTAs whose row range is empty (R < G) wrote nothing: skip their slots
            for (int b = bfirst; b <= blast; ++b)
                if (R * b / a.G < R * (b + 1) / a.G) acc += (double)src[(size_t)b * bstride];
        }
        tile[w][lane] = acc;
        __syncthreads();
        const int slotf = fg * 32 + fl, binw = bin0 + bl;
        if (slotf < a.F && binw < a.nbins)
            a.hcomp[(((size_t)s * a.F + slotf) * a.C + (ct * 4 + c)) * a.nbins + binw] = tile[bl][fl];
        __syncthreads();
    }
}

template <int BP, int NCH>
cudaError_t launch_hist_t(const HistArgs &a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    static bool attr_set[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_hist<BP, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    k_hist<BP, NCH><<<grid, threads, smem, st>>>(a);
    return cudaGetLastError();
}

template <int BP>
cudaError_t launch_hist_bp(int NCH, const HistArgs &a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    switch (NCH) {
    case 1: return launch_hist_t<BP, 1>(a, grid, threads, smem, st);
    case 2: return launch_hist_t<BP, 2>(a, grid, threads, smem, st);
    case 3: return launch_hist_t<BP, 3>(a, grid, threads, smem, st);
    default: return launch_hist_t<BP, 4>(a, grid, threads, smem, st);
    }
}

template <int BP, int NCH>
int occupancy_t(int threads, size_t smem) {
    cudaFuncSetAttribute(k_hist<BP, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_hist<BP, NCH>, threads, smem) != cudaSuccess) nb = 0;
    return nb;
}
int occupancy(int BP, int NCH, int threads, size_t smem) {
#define OCC_CASE(bp)                                                    \
    case bp:                                                            \
        switch (NCH) {                                                  \
        case 1: return occupancy_t<bp, 1>(threads, smem);               \
        case 2: return occupancy_t<bp, 2>(threads, smem);               \
        case 3: return occupancy_t<bp, 3>(threads, smem);               \
        default: return occupancy_t<bp, 4>(threads, smem);              \
        }
    switch (BP) {
        OCC_CASE(32)
        OCC_CASE(64)
        OCC_CASE(128)
    default:
        switch (NCH) {
        case 1: return occupancy_t<256, 1>(threads, smem);
        case 2: return occupancy_t<256, 2>(threads, smem);
        case 3: return occupancy_t<256, 3>(threads, smem);
        default: return occupancy_t<256, 4>(threads, smem);
        }
    }
#undef OCC_CASE
}

} // namespace

// Geometry for F feature slots.  Called once at create time with F = nfeats (sizes the scratch buffer)
// and again per tree when the column sample is smaller.
int32_t evb_hist_geometry(const evb_handle *h, int F, HistGeom *g) {
    const int B = h->B, C = h->C;
    g->BP = B <= 32 ? 32 : B <= 64 ? 64 : B <= 128 ? 128 : 256;
    g->NCH = C < 4 ? C : 4;
    g->NFG = (F + 31) / 32;
    g->NCT = (C + 3) / 4;
    g->U = g->NFG * g->NCT;
    const size_t img = (size_t)32 * g->BP * g->NCH * 4;
    const size_t stage = (size_t)EVB_TILE_ROWS * (h->RS + h->GS * 4);
    const size_t sm_total = 228 * 1024, blk_max = 227 * 1024, reserve = 1024;
    int UB = g->U < EVB_MAX_UNITS_PER_BLOCK ? g->U : EVB_MAX_UNITS_PER_BLOCK;
    while (UB > 1 && UB * img + 2 * stage + 256 > blk_max) --UB;
    if (UB * img + 2 * stage + 256 > blk_max) {
        evb_set_error("histogram image does not fit shared memory (nbins=%d, nfeats=%d)", B, h->nfeats);
        return EVB_ERR_LIMIT;
    }
    g->UB = UB;
    g->NUG = (g->U + UB - 1) / UB;
    // blocks per SM: as many as fit with >= 3 stages, at most 8
    int t = (int)(sm_total / (UB * img + 3 * stage + 256 + reserve));
    if (t < 1) t = 1;
    if (t > 8) t = 8;
    size_t per_block = sm_total / t - reserve;
    if (per_block > blk_max) per_block = blk_max;
    int S = (int)((per_block - UB * img - 256) / stage);
    if (S > 8) S = 8;
    if (S < 2) S = 2;
    g->stages = S;
    g->smem = UB * img + (size_t)S * stage + 2 * S * 8 + 128;
    const int threads = (UB + 1) * 32;
    int occ = occupancy(g->BP, g->NCH, threads, g->smem);
    if (occ < 1) {
        evb_set_error("histogram kernel cannot be resident (smem=%zu)", g->smem);
        return EVB_ERR_CUDA;
    }
    g->G = occ * h->num_sms;
    g->PG = g->G + h->maxslots;
    g->img_floats = (size_t)g->NCH * B * 32;
    return EVB_OK;
}

int32_t evb_hist_configure(evb_handle *h) {
    EVB_CHECK(evb_hist_geometry(h, h->nfeats, &h->hg));
    h->scratch_floats = (size_t)h->hg.NUG * h->hg.PG * h->hg.UB * h->hg.img_floats;
    return EVB_OK;
}

int32_t evb_launch_hist(evb_handle *h, int level) {
    const HistGeom &g = h->hg;
    HistArgs a;
    a.xT = h->xT; a.grad = h->grad; a.rows = h->rows[(level - 1) & 1]; a.js0 = h->js_d;
    a.plan = h->plan + level; a.cum = h->cum; a.slot_node = h->slot_node; a.seg_start = h->seg_start;
    a.scratch = h->scratch; a.err = h->d_err;
    a.RS = h->RS; a.GS = h->GS; a.F = h->F; a.nbins = h->B; a.C = h->C; a.NFG = g.NFG; a.U = g.U; a.UB = g.UB;
    a.stages = g.stages; a.PG = g.PG; a.img_floats = (uint32_t)g.img_floats;
    dim3 grid(g.G, g.NUG);
    const int threads = (g.UB + 1) * 32;
    evb_tic(h, EVB_T_HIST);
    cudaError_t e;
    switch (g.BP) {
    case 32: e = launch_hist_bp<32>(g.NCH, a, grid, threads, g.smem, h->st); break;
    case 64: e = launch_hist_bp<64>(g.NCH, a, grid, threads, g.smem, h->st); break;
    case 128: e = launch_hist_bp<128>(g.NCH, a, grid, threads, g.smem, h->st); break;
    default: e = launch_hist_bp<256>(g.NCH, a, grid, threads, g.smem, h->st); break;
    }
    evb_toc(h, EVB_T_HIST);
    EVB_CUDA(e);
    return EVB_OK;
}

int32_t evb_launch_hist_reduce(evb_handle *h, int level) {
    const HistGeom &g = h->hg;
    ReduceArgs a;
    a.scratch = h->scratch; a.hcomp = h->hcomp; a.plan = h->plan + level; a.cum = h->cum;
    a.G = g.G; a.PG = g.PG; a.UB = g.UB; a.NFG = g.NFG; a.U = g.U; a.F = h->F; a.C = h->C; a.nbins = h->B; a.NCH = g.NCH;
    a.img_floats = (uint32_t)g.img_floats;
    dim3 grid(evb_level_slots(level), g.U, (h->B + 15) / 16);
    evb_tic(h, EVB_T_HIST_REDUCE);
    k_hist_reduce<<<grid, 512, 0, h->st>>>(a);
    evb_toc(h, EVB_T_HIST_REDUCE);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}
