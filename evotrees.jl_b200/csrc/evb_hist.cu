// Histogram build: `update_hist!` / `_hist!` (src/fit-utils.jl:345-394) and the reference GPU
// `hist_kernel!` (ext/EvoTreesKernelAbstractionsExt/fit-utils.jl:57-95), redesigned for sm_100a.
//
// Design
//   * The rows of every build node are a contiguous segment of a row-index list.  The concatenation of
//     all build segments of a level is cut into gridDim.x equal row ranges, one per CTA, so every CTA
//     streams the same number of rows whatever the node sizes are.  A (CTA, node) intersection is a "piece".
//   * One producer warp stages tiles of 32 rows: the row of the observation-major bin matrix (RS bytes) and the
//     row's gradient record (GS floats), with 16-byte `cp.async` copies that arrive on an mbarrier (the default:
//     measured 7.95 ms per tree at 10M x 100 against 12.16 ms for the other staging path, one TMA bulk copy
//     per row, which EVB_HIST_MODE=0 still selects).  Consumers never touch global memory in the inner loop.
//   * Each consumer warp owns one "unit": 32 feature slots (lane = feature) x up to 4 gradient channels,
//     with a private image img[channel][bin][lane] in shared memory.  Lane l only ever touches bank l, so
//     the accumulation is a plain load/add/store: no atomics, no bank conflicts, and a fixed summation
//     order (ascending rows) inside a piece.
//   * At the end of a piece the image is written to a scratch slot indexed by (CTA, build slot).  A second
//     kernel sums the pieces of every node in ascending CTA order in double precision, so histograms are
//     bit-reproducible from run to run, and transposes them to hcomp[slot][feature][channel][bin].
//   Every wait on an mbarrier is bounded; on expiry the kernel records an error code and returns.
#include "evb_internal.cuh"
#include <mutex>
#include <stdlib.h>

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
// try_wait with a suspend-time hint: the warp sleeps in hardware until the phase completes or the hint (in
// nanoseconds) runs out, instead of burning issue slots in a polling loop.
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(100000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after 2^16 suspended tries of up to 0.1 ms each (or as soon as another warp has flagged an
// error) and records `code` in the error word.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, int code) {
    for (uint32_t i = 0; i < (1u << 16); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && *(volatile int *)err != 0) return false;
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
    int mode;   // bit 0: stage rows with cp.async (LDGSTS) instead of TMA bulk copies (builds with -DEVB_DIAG: bit 4 skips the accumulation)
    int contig; // 1 when feature slot s is feature s (no column sample): a lane's FPL bins are adjacent bytes of the row
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Producer warp of the histogram kernels: stages tiles of 32 rows (bins + gradient record of every row) for the
// consumer warps of the CTA.  Row ids are fetched four tiles (128 rows) at a time and one group ahead, so that the
// latency of reading the row list never sits between two tiles.
__device__ __forceinline__ void produce_tiles(const HistArgs &a, long long lo, long long hi, int s, uint64_t *full, uint64_t *empty,
                                              unsigned char *stage0, int S, int stage_bytes, int xbytes, int lane) {
    uint32_t it = 0;
    long long pos = lo;
    bool ok = true;
    while (pos < hi && ok) {
        const long long send = min(hi, (long long)a.cum[s + 1]);
        if (send > pos) {
            const int node = a.slot_node[s];
            const uint32_t *rows = a.rows + ((long long)a.seg_start[node] - a.cum[s]);
            uint32_t cur[4], nxt[4] = {0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < 4; ++k) { const long long q = pos + k * 32 + lane; cur[k] = q < send ? rows[q] : 0u; }
            for (long long q0 = pos; q0 < send && ok; q0 += 4 * EVB_TILE_ROWS) {
                const long long qn = q0 + 4 * EVB_TILE_ROWS;
                if (qn < send) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const long long q = qn + k * 32 + lane; nxt[k] = q < send ? rows[q] : 0u; }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const long long t0 = q0 + k * EVB_TILE_ROWS;
                    if (t0 < send && ok) {
                        const int st = it % S;
                        const int nrows = (int)min((long long)EVB_TILE_ROWS, send - t0);
                        ok = mbar_wait(&empty[st], ((it / S) & 1u) ^ 1u, a.err, EVB_DERR_WAIT_EMPTY);
                        if (ok && (a.mode & 1)) {
                            unsigned char *sb = stage0 + (size_t)st * stage_bytes;
                            const int cpr = a.RS >> 4, cprg = a.GS >> 2;
                            for (int base = 0; base < EVB_TILE_ROWS * cpr; base += 32) {
                                const int idx = base + lane, rt = idx / cpr, ch = idx - rt * cpr;
                                const uint32_t row = __shfl_sync(0xffffffffu, cur[k], rt & 31);
                                if (rt < nrows) cp_async16(sb + rt * a.RS + ch * 16, a.xT + (size_t)row * a.RS + ch * 16);
                            }
                            for (int base = 0; base < EVB_TILE_ROWS * cprg; base += 32) {
                                const int idx = base + lane, rt = idx / cprg, ch = idx - rt * cprg;
                                const uint32_t row = __shfl_sync(0xffffffffu, cur[k], rt & 31);
                                if (rt < nrows) cp_async16(sb + xbytes + (rt * a.GS + ch * 4) * 4, a.grad + (size_t)row * a.GS + ch * 4);
                            }
                            cp_async_arrive(&full[st]);
                            ++it;
                        } else if (ok) {
                            if (lane == 0) mbar_expect_tx(&full[st], (uint32_t)nrows * (uint32_t)(a.RS + a.GS * 4));
                            __syncwarp();
                            if (lane < nrows) {
                                unsigned char *sb = stage0 + (size_t)st * stage_bytes;
                                bulk_g2s(sb + lane * a.RS, a.xT + (size_t)cur[k] * a.RS, (uint32_t)a.RS, &full[st]);
                                bulk_g2s(sb + xbytes + lane * a.GS * 4, a.grad + (size_t)cur[k] * a.GS, (uint32_t)a.GS * 4, &full[st]);
                            }
                            ++it;
                        }
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) cur[k] = nxt[k];
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
}

// Unit image in shared memory.  A unit is 32 lanes x FPL feature slots per lane x NCH gradient channels.
// For every feature slot j of the lane there is a sub-image; inside it channels are kept in pairs so that one
// 64-bit access moves two of them:
//   region 0: [row 0..BP][lane] float2 (NCH >= 2) or float (NCH == 1)      region 1: the remaining NCH - 2 channels
// Row v holds bin v (bins are 1-based bytes); row 0 is a guard row that absorbs the zero padding bytes of a
// row of bins.  Lane l only touches addresses whose bank is determined by l: no access of a warp conflicts and
// nothing needs an atomic.
template <int BP, int NCH, int FPL>
struct Img {
    static constexpr int W0 = NCH >= 2 ? 2 : 1;
    static constexpr int W1 = NCH - W0;
    static constexpr int RB0 = 32 * W0 * 4;               // bytes per row, region 0
    static constexpr int RB1 = 32 * W1 * 4;
    static constexpr int R1OFF = (BP + 1) * RB0;           // byte offset of region 1 inside a sub-image
    static constexpr int SUB = (BP + 1) * (RB0 + RB1);     // bytes per sub-image
    static constexpr int BYTES = FPL * SUB;                // bytes per unit image
    // o8 = bin << 8 (what one PRMT extracts from the packed bins of a lane); u0 / u1 are 32-bit shared-space
    // addresses of the lane's column in region 0 / region 1 of the unit
    static __device__ __forceinline__ void ld(uint32_t u0, uint32_t u1, int j, uint32_t o8, float (&v)[NCH]) {
        if constexpr (W0 == 2) {
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(u0 + j * SUB + o8));
        } else {
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(u0 + j * SUB + (o8 >> 1)));
        }
        if constexpr (W1 == 2) {
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[2]), "=f"(v[3]) : "r"(u1 + j * SUB + o8));
        } else if constexpr (W1 == 1) {
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[2]) : "r"(u1 + j * SUB + (o8 >> 1)));
        }
    }
    static __device__ __forceinline__ void st(uint32_t u0, uint32_t u1, int j, uint32_t o8, const float (&v)[NCH]) {
        if constexpr (W0 == 2) {
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(u0 + j * SUB + o8), "f"(v[0]), "f"(v[1]) : "memory");
        } else {
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(u0 + j * SUB + (o8 >> 1)), "f"(v[0]) : "memory");
        }
        if constexpr (W1 == 2) {
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(u1 + j * SUB + o8), "f"(v[2]), "f"(v[3]) : "memory");
        } else if constexpr (W1 == 1) {
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(u1 + j * SUB + (o8 >> 1)), "f"(v[2]) : "memory");
        }
    }
};

template <int NCH>
__device__ __forceinline__ void unpack(const float4 &g, float (&v)[NCH]) {
    v[0] = g.x;
    if constexpr (NCH >= 2) v[1] = g.y;
    if constexpr (NCH >= 3) v[2] = g.z;
    if constexpr (NCH >= 4) v[3] = g.w;
}

__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// gradient channels of one row for this unit (the record slice of a unit starts on a 16-byte boundary)
template <int NCH>
__device__ __forceinline__ void lds_grad(uint32_t addr, float (&v)[NCH]) {
    if constexpr (NCH == 1) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(addr));
    else if constexpr (NCH == 2) asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(addr));
    else if constexpr (NCH == 3) {
        float w;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(w) : "r"(addr));
    } else asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
}

// packed bins of one row for this lane: byte j = bin of the lane's j-th feature slot
template <int FPL, bool CONTIG>
__device__ __forceinline__ uint32_t load_bins(uint32_t row, const uint32_t (&foff)[FPL]) {
    if constexpr (CONTIG) {
        if constexpr (FPL == 4) return lds_u32(row + foff[0]);
        else if constexpr (FPL == 2) return lds_u16(row + foff[0]);
        else return lds_u8(row + foff[0]);
    } else {
        uint32_t v = lds_u8(row + foff[0]);
#pragma unroll
        for (int j = 1; j < FPL; ++j) v |= lds_u8(row + foff[j]) << (8 * j);
        return v;
    }
}

// Accumulates the rows of one staged tile into the unit image.  Four rows at a time: all loads first, then the
// adds with forwarding between rows that hit the same bin of the same feature, then the stores in row order.  The
// result is bit-identical to adding the rows one by one, but 4 x FPL read-modify-write chains overlap.
// xs / gs: 32-bit shared-space addresses of the tile's bins and of this unit's slice of the gradient records.
template <int BP, int NCH, int FPL, bool CONTIG>
__device__ __forceinline__ void accumulate_tile(uint32_t xs, uint32_t gs, int nrows, int RS, int GSB,
                                                const uint32_t (&foff)[FPL], uint32_t u0, uint32_t u1) {
    using I = Img<BP, NCH, FPL>;
    int r = 0;
    for (; r + 4 <= nrows; r += 4, xs += 4 * RS, gs += 4 * GSB) {
        uint32_t raw[4];
        float g[4][NCH];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            raw[i] = load_bins<FPL, CONTIG>(xs + i * RS, foff);
            lds_grad<NCH>(gs + i * GSB, g[i]);
        }
        uint32_t o[FPL][4];
        float a[FPL][4][NCH];
#pragma unroll
        for (int j = 0; j < FPL; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                o[j][i] = __byte_perm(raw[i], 0u, 0x4404u | (uint32_t)(j << 4)); // bin << 8
                I::ld(u0, u1, j, o[j][i], a[j][i]);
            }
        }
#pragma unroll
        for (int j = 0; j < FPL; ++j) {
            const bool e10 = o[j][1] == o[j][0], e20 = o[j][2] == o[j][0], e21 = o[j][2] == o[j][1];
            const bool e30 = o[j][3] == o[j][0], e31 = o[j][3] == o[j][1], e32 = o[j][3] == o[j][2];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                a[j][0][c] = a[j][0][c] + g[0][c];
                a[j][1][c] = (e10 ? a[j][0][c] : a[j][1][c]) + g[1][c];
                a[j][2][c] = (e21 ? a[j][1][c] : (e20 ? a[j][0][c] : a[j][2][c])) + g[2][c];
                a[j][3][c] = (e32 ? a[j][2][c] : (e31 ? a[j][1][c] : (e30 ? a[j][0][c] : a[j][3][c]))) + g[3][c];
            }
        }
#pragma unroll
        for (int j = 0; j < FPL; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) I::st(u0, u1, j, o[j][i], a[j][i]);
        }
    }
    for (; r < nrows; ++r, xs += RS, gs += GSB) {
        const uint32_t raw = load_bins<FPL, CONTIG>(xs, foff);
        float g[NCH];
        lds_grad<NCH>(gs, g);
#pragma unroll
        for (int j = 0; j < FPL; ++j) {
            const uint32_t o = __byte_perm(raw, 0u, 0x4404u | (uint32_t)(j << 4));
            float a[NCH];
            I::ld(u0, u1, j, o, a);
#pragma unroll
            for (int c = 0; c < NCH; ++c) a[c] += g[c];
            I::st(u0, u1, j, o, a);
        }
    }
}

template <int BP, int NCH, int FPL>
__global__ void __launch_bounds__((EVB_MAX_UNITS_PER_BLOCK + 1) * 32) k_hist(HistArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    using I = Img<BP, NCH, FPL>;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, b = blockIdx.x, ug = blockIdx.y;
    const int nact = min(a.UB, a.U - ug * a.UB);
    const int S = a.stages;
    const int xbytes = EVB_TILE_ROWS * a.RS, gbytes = EVB_TILE_ROWS * a.GS * 4;
    const int stage_bytes = xbytes + gbytes;
    float *imgs = reinterpret_cast<float *>(smem);
    unsigned char *stage0 = smem + (size_t)a.UB * I::BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(stage0 + (size_t)S * stage_bytes);
    uint64_t *empty = full + S;

    const long long R = a.plan->R;
    const long long lo = R * b / G, hi = R * (b + 1) / G;
    if (lo >= hi) return;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], (a.mode & 1) ? 32 : 1); mbar_init(&empty[s], nact); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = tid; i < nact * (I::BYTES / 4); i += blockDim.x) imgs[i] = 0.0f;
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
        produce_tiles(a, lo, hi, s, full, empty, stage0, S, stage_bytes, xbytes, lane);
        return;
    }
    if (wid - 1 >= nact) return;

    // ---------------- consumers: one unit (32 lanes x FPL feature slots x NCH channels) per warp --------
    const int uw = wid - 1;
    const int u = ug * a.UB + uw;
    const int ct = u / a.NFG, fg = u % a.NFG;
    const int slot0 = (fg * 32 + lane) * FPL;
    const bool act = slot0 < a.F;
    uint32_t foff[FPL];
#pragma unroll
    for (int j = 0; j < FPL; ++j) foff[j] = (slot0 + j < a.F) ? a.js0[slot0 + j] : (act ? a.js0[slot0] : 0u);
    const int nch = min(NCH, a.C - ct * NCH);
    const uint32_t ubase = smem_u32(smem) + (uint32_t)uw * I::BYTES;
    const uint32_t u0 = ubase + lane * I::W0 * 4;
    const uint32_t u1 = ubase + I::R1OFF + lane * I::W1 * 4;
    const int RS = a.RS, GS = a.GS;
    const uint32_t stage0_s = smem_u32(stage0);

    uint32_t it = 0;
    long long pos = lo;
    while (pos < hi) {
        const long long send = min(hi, (long long)a.cum[s + 1]);
        if (send > pos) {
            for (long long q0 = pos; q0 < send; q0 += EVB_TILE_ROWS, ++it) {
                const int st = it % S;
                const int nrows = (int)min((long long)EVB_TILE_ROWS, send - q0);
                if (!mbar_wait(&full[st], (it / S) & 1u, a.err, EVB_DERR_WAIT_FULL)) return;
                const uint32_t xs = stage0_s + (uint32_t)st * stage_bytes;
                const uint32_t gs = xs + xbytes + ct * 16;
#ifdef EVB_DIAG
                if (act && !(a.mode & 16)) { // profiling builds only: mode bit 4 stages the rows and skips the accumulation
#else
                if (act) {
#endif
                    // the common strides are passed as literals so that the row offsets fold into the instructions
                    if (a.contig && RS == 128 && GS == 4) accumulate_tile<BP, NCH, FPL, true>(xs, gs, nrows, 128, 16, foff, u0, u1);
                    else if (a.contig && RS == 64 && GS == 8) accumulate_tile<BP, NCH, FPL, true>(xs, gs, nrows, 64, 32, foff, u0, u1);
                    else if (a.contig && RS == 32 && GS == 12) accumulate_tile<BP, NCH, FPL, true>(xs, gs, nrows, 32, 48, foff, u0, u1);
                    else if (a.contig && RS == 32 && GS == 4) accumulate_tile<BP, NCH, FPL, true>(xs, gs, nrows, 32, 16, foff, u0, u1);
                    else if (a.contig) accumulate_tile<BP, NCH, FPL, true>(xs, gs, nrows, RS, GS * 4, foff, u0, u1);
                    else accumulate_tile<BP, NCH, FPL, false>(xs, gs, nrows, RS, GS * 4, foff, u0, u1);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }
            // flush the piece (CTA b, slot s) and clear the image (guard rows included)
            float *dst = a.scratch + ((size_t)(ug * a.PG + b + s) * a.UB + uw) * a.img_floats + lane;
            const float zero[NCH] = {};
#pragma unroll
            for (int j = 0; j < FPL; ++j) {
                I::st(u0, u1, j, 0u, zero);
                for (int bin = 0; bin < a.nbins; ++bin) {
                    float v[NCH];
                    const uint32_t o8 = (uint32_t)(bin + 1) << 8;
                    I::ld(u0, u1, j, o8, v);
                    I::st(u0, u1, j, o8, zero);
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        if (c < nch) dst[((j * NCH + c) * a.nbins + bin) * 32] = v[c];
                }
            }
        }
        pos = send;
        ++s;
    }
}

// ---------------------------------------------------------------------------------------------------------
// Fixed-point variant for mse with one target.  The quantisation kernel turns the gradient of every row into a
// fixed-point number q = rint(g * 2^s), |q| < 2^29 (and the weight likewise, unless no weights were given: the w
// channel is then a row count).  The kernel splits q into hi = q >> 15 (signed) and lo = q & 0x7fff and adds the
// NW words (hi, lo, 1) or (hi, lo, w_hi, w_lo) into the image [word][bin][lane] of the unit with
// `red.shared.add.u32`: one shared-memory pass per word and row, no read-modify-write chain.  Integer sums do not
// depend on the order of the rows, so
//   * several warps share one image: a CTA (one per SM) keeps a single image per unit of 32 feature slots;
//   * the shared memory that the float variant spends on one image per warp holds row data in flight instead.
//     The warps form QT teams with one warp per unit.  The teams take the 32-row tiles of the CTA's row range in
//     turn; a team stages its tile together with cp.async -- eight adjacent lanes copy the 128 bytes of one row,
//     so a copy instruction touches 4 lines instead of 32 -- into a ring QDR tiles deep (+1 slot so that one
//     named barrier per tile is enough), waits with cp.async.wait_group and the team barrier, and then every warp
//     adds the tile into the image of its unit.  There is no producer warp and no mbarrier.
//     Row r of a tile is stored rotated by 32 * (r & 3) bytes inside its 128 bytes, so that the four rows which
//     the consumers read with one load fall into different banks.
// A piece covers at most 2^17 rows, so neither the sum of the lo words (< 2^32) nor of the hi words (|.| < 2^31)
// can overflow.  The reduce kernel recombines hi * 2^15 + lo in 64-bit integers and scales by 2^-s: every
// histogram entry is the exact sum of the quantised gradients, whatever the order and the number of pieces.
// Needs feature slot s == feature s (no column sample): the unit's bins are then 32 adjacent bytes of a row.
constexpr int QT = 6;                   // teams per CTA
constexpr int QDR = 5;                  // tiles in flight per team
constexpr int QSPLIT = 15;              // scratch words: sum = hi * 2^15 + lo, a piece may hold 2^17 rows (|q| < 2^29)
// Unit weights (NW == 3): the image has two planes only.  q (|q| < 2^26) is split at bit 8 and the row count rides in
// the upper 12 bits of the lo word: plane 0 += q >> 8, plane 1 += (q & 0xff) | 1 << 20.  That holds QSUB * QT tiles
// (at most 4095 rows: lo sum < 2^20, count < 2^12, |hi sum| < 2^30); then the image is flushed into the piece's scratch
// words (hi, lo, count as above), which are private to the CTA (first flush: stores, later ones: red.global.add).
constexpr int QSUB = 4095 / (QT * EVB_TILE_ROWS); // tiles per team between two flushes
__host__ __device__ constexpr int q_planes(int NW) { return NW == 3 ? 2 : 4; }
__host__ __device__ constexpr int q_tile_bytes(int NW) { return EVB_TILE_ROWS * (128 + (NW == 3 ? 4 : 8)); } // bins + q (+ q of w)

template <uint32_t OFF>
__device__ __forceinline__ void red_off(uint32_t addr, uint32_t v) {
    asm volatile("red.shared.add.u32 [%0+%2], %1;" ::"r"(addr), "r"(v), "n"(OFF) : "memory");
}
// the words that one row adds to the image: (q >> 8, (q & 0xff) | 1 << 20) without weights, else hi / lo of g and w
template <int NW>
__device__ __forceinline__ void row_words(uint32_t qg, uint32_t qw, uint32_t (&w)[4]) {
    if constexpr (NW == 3) {
        w[0] = (uint32_t)((int32_t)qg >> 8); w[1] = (qg & 0xffu) | (1u << 20); w[2] = 0u; w[3] = 0u;
    } else {
        w[0] = (uint32_t)((int32_t)qg >> QSPLIT); w[1] = qg & ((1u << QSPLIT) - 1);
        w[2] = qw >> QSPLIT; w[3] = qw & ((1u << QSPLIT) - 1);
    }
}
// adds them into the word planes of the image (plane k starts k * WSZ bytes further)
template <int NW, uint32_t WSZ>
__device__ __forceinline__ void red_row(uint32_t addr, const uint32_t (&w)[4]) {
    red_off<0>(addr, w[0]);
    red_off<WSZ>(addr, w[1]);
    if constexpr (NW == 4) { red_off<2 * WSZ>(addr, w[2]); red_off<3 * WSZ>(addr, w[3]); }
}
// All rows of one staged tile.  4 * REP rows at a time.  With REP = 1 lane (k = lane & 7, rr = lane >> 3) loads the
// 32-bit word with the bins of features 4k .. 4k+3 of row r + rr -- one conflict-free load brings the 128 bins of
// four rows -- and the fixed-point words of that row.  In step j = 0..3 the lane adds its row into feature
// 4k + ((j + rr) & 3): the four lanes that share k work on four different features, so the 32 lanes of every
// reduction hit 32 different banks.  A unit with few features (the last one: 8 / REP groups of four features or
// fewer) keeps REP replicas of its columns instead, k = lane % (8 / REP), rr = lane / (8 / REP), replica rr >> 2,
// and takes 4 * REP rows per step; the replicas are added when the image is flushed.
//   tb: shared-space address of the lane's word of row rr of the tile, tw: of the tile's words + rr * (4 or 8),
//   col[j]: image column of the lane's feature of step j, sel[j]: PRMT selector of that feature's byte.
template <uint32_t OFF>
__device__ __forceinline__ uint32_t lds_u32_at(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
// batch BT of a tile (see q_tile): loads of batch BT + 1 first, then the reductions of batch BT
template <int NW, uint32_t WSZ, int REP, bool FULL, int BT>
__device__ __forceinline__ void q_batch(uint32_t tb, uint32_t tw, int nrows, int rr, const uint32_t (&col)[4], const uint32_t (&sel)[4],
                                        uint32_t bins, uint32_t qg, uint32_t qw) {
    constexpr int RW = NW == 3 ? 1 : 2;
    constexpr int RB = 4 * REP, NB = EVB_TILE_ROWS / RB;
    uint32_t nbins = 0, nqg = 0, nqw = 0;
    if constexpr (BT + 1 < NB) {
        nbins = lds_u32_at<(BT + 1) * RB * 128>(tb);
        nqg = lds_u32_at<(BT + 1) * RB * 4 * RW>(tw);
        if constexpr (RW == 2) nqw = lds_u32_at<(BT + 1) * RB * 8 + 4>(tw);
    }
    if (FULL || BT * RB + rr < nrows) { // FULL: a whole tile of 32 rows, nothing to test
        uint32_t w[4];
        row_words<NW>(qg, qw, w);
        if constexpr (NW == 3) {
            // the four steps of the lane's row as one block: byte select, image address, two reductions each
            asm volatile(
                "{\n .reg .u32 b0, b1, b2, b3, a0, a1, a2, a3;\n"
                " prmt.b32 b0, %0, 0, %1;\n prmt.b32 b1, %0, 0, %2;\n prmt.b32 b2, %0, 0, %3;\n prmt.b32 b3, %0, 0, %4;\n"
                " mad.lo.u32 a0, b0, 128, %5;\n mad.lo.u32 a1, b1, 128, %6;\n mad.lo.u32 a2, b2, 128, %7;\n mad.lo.u32 a3, b3, 128, %8;\n"
                " red.shared.add.u32 [a0], %9;\n red.shared.add.u32 [a0+%11], %10;\n"
                " red.shared.add.u32 [a1], %9;\n red.shared.add.u32 [a1+%11], %10;\n"
                " red.shared.add.u32 [a2], %9;\n red.shared.add.u32 [a2+%11], %10;\n"
                " red.shared.add.u32 [a3], %9;\n red.shared.add.u32 [a3+%11], %10;\n}\n"
                ::"r"(bins), "r"(sel[0]), "r"(sel[1]), "r"(sel[2]), "r"(sel[3]), "r"(col[0]), "r"(col[1]), "r"(col[2]), "r"(col[3]),
                  "r"(w[0]), "r"(w[1]), "n"(WSZ)
                : "memory");
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) red_row<NW, WSZ>(col[j] + __byte_perm(bins, 0u, sel[j]) * 128u, w);
        }
    }
    if constexpr (BT + 1 < NB) q_batch<NW, WSZ, REP, FULL, BT + 1>(tb, tw, nrows, rr, col, sel, nbins, nqg, nqw);
}
template <int NW, uint32_t WSZ, int REP, bool FULL>
__device__ __forceinline__ void q_tile(uint32_t tb, uint32_t tw, int nrows, int rr, const uint32_t (&col)[4], const uint32_t (&sel)[4]) {
    constexpr int RW = NW == 3 ? 1 : 2;
    const uint32_t bins = lds_u32(tb), qg = lds_u32(tw), qw = RW == 2 ? lds_u32(tw + 4) : 0u;
    q_batch<NW, WSZ, REP, FULL, 0>(tb, tw, nrows, rr, col, sel, bins, qg, qw);
}

template <int BP, int NW>
__global__ void __launch_bounds__(EVB_MAX_UNITS_PER_BLOCK * QT * 32) k_histq(HistArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr uint32_t WSZ = (BP + 1) * 128;    // bytes of one word plane [bin 0..BP][lane]
    constexpr uint32_t IMG = q_planes(NW) * WSZ;
    constexpr int QTILE = q_tile_bytes(NW), RW = NW == 3 ? 1 : 2, NSLOT = QDR + 1;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, b = blockIdx.x, ug = blockIdx.y;
    const int nact = min(a.UB, a.U - ug * a.UB);
    const long long R = a.plan->R;
    const long long lo = R * b / G, hi = R * (b + 1) / G;
    if (lo >= hi) return;
    uint32_t *imgs = reinterpret_cast<uint32_t *>(smem);
    for (int i = tid; i < a.UB * (int)(IMG / 4); i += blockDim.x) imgs[i] = 0u;
    __syncthreads();
    const int team = wid / a.UB, uw = wid % a.UB;
    if (uw >= nact) return;

    const int nbuild = a.plan->nbuild;
    int s;
    {
        int l = 0, r = nbuild - 1;
        while (l < r) { int m = (l + r + 1) >> 1; if ((long long)a.cum[m] <= lo) l = m; else r = m - 1; }
        s = l;
    }
    const int fg = ug * a.UB + uw;          // the unit: feature slots fg*32 .. fg*32+31
    const uint32_t u0 = smem_u32(smem) + (uint32_t)uw * IMG + lane * 4; // column of feature slot `lane` (flush)
    // groups of four features in this unit -> replicas of its columns (see q_tile)
    const int nq = min(8, (a.F - fg * 32 + 3) / 4);
    const int rep = nq <= 1 ? 8 : nq <= 2 ? 4 : nq <= 4 ? 2 : 1, nqp = 8 / rep;
    const int k = lane % nqp, rr = lane / nqp;
    uint32_t col[4], sel[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
        const int sh = (jj + rr) & 3;
        col[jj] = smem_u32(smem) + (uint32_t)uw * IMG + (uint32_t)((rr >> 2) * nqp * 4 + 4 * k + sh) * 4;
        sel[jj] = 0x4440u | (uint32_t)sh;
    }
    unsigned char *ring = smem + (size_t)a.UB * IMG + (size_t)team * (NSLOT * QTILE);
    const uint32_t ring_s = smem_u32(ring);
    // the lane's word of row rr inside a tile (rows are rotated by 32 * (row & 3) bytes)
    const uint32_t rd_off = (uint32_t)rr * 128u + ((uint32_t)(uw * 32 + k * 4 + 32 * (rr & 3)) & 127u);
    // staging: the team copies 32 rows x nact * 32 bytes of bins as 16-byte chunks, two per lane
    const int cpr = 2 * nact;               // chunks per row
    int st_row[2], st_src[2], st_dst[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int c = t * nact * 32 + uw * 32 + lane;
        st_row[t] = c / cpr;
        const int pch = c % cpr;
        st_src[t] = pch * 16;
        st_dst[t] = st_row[t] * 128 + ((pch + 2 * (st_row[t] & 3)) & 7) * 16;
    }
    const uint8_t *xsl = a.xT + (size_t)ug * a.UB * 32;  // the CTA's slice of every row of bins
    const int32_t *gq = reinterpret_cast<const int32_t *>(a.grad);
    const size_t RS = a.RS;
    const uint32_t team_bar = 1 + team, unit_bar = 1 + QT + uw;
#ifdef EVB_DIAG
    const bool skip_acc = (a.mode & 16) != 0; // profiling builds only: stage the rows, skip the accumulation
#else
    constexpr bool skip_acc = false;
#endif
    const int team_threads = nact * 32;

    long long pos = lo;
    while (pos < hi) {
        const long long send = min(hi, (long long)a.cum[s + 1]);
        if (send > pos) {
            const uint32_t *rows = a.rows + ((long long)a.seg_start[a.slot_node[s]] - a.cum[s]);
            const long long ntiles = (send - pos + EVB_TILE_ROWS - 1) / EVB_TILE_ROWS;
            const int nmine = ntiles > team ? (int)((ntiles - team + QT - 1) / QT) : 0; // tiles team, team + QT, ...
            // All warps of the unit are done with the rows so far: move the image into the scratch words of the piece
            // (CTA b, slot s) and clear it.  `first`: the piece has no contents yet (store instead of add).
            bool started = false;
            auto flush = [&](bool first) {
                asm volatile("bar.sync %0, %1;" ::"r"(unit_bar), "r"(QT * 32) : "memory");
                uint32_t *dst = reinterpret_cast<uint32_t *>(a.scratch) + ((size_t)(ug * a.PG + b + s) * a.UB + uw) * a.img_floats + lane;
                const int pl = a.nbins * 32; // words per scratch plane
                if constexpr (NW == 3) {
                    if (team == 0) { // guard rows
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(u0), "r"(0u) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(u0 + WSZ), "r"(0u) : "memory");
                    }
                    for (int bin = team; bin < a.nbins; bin += QT) {
                        const uint32_t ai = u0 + (uint32_t)(bin + 1) * 128u;
                        uint32_t vh = lds_u32(ai), vp = lds_u32(ai + WSZ);
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(ai), "r"(0u) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(ai + WSZ), "r"(0u) : "memory");
                        for (int o = 32 / rep; o < 32; o <<= 1) { vh += __shfl_xor_sync(0xffffffffu, vh, o); vp += __shfl_xor_sync(0xffffffffu, vp, o); }
                        const long long sum = (long long)(int32_t)vh * 256 + (long long)(vp & 0xfffffu);
                        uint32_t h = (uint32_t)(int32_t)(sum >> QSPLIT), l = (uint32_t)(sum & ((1 << QSPLIT) - 1)), c = vp >> 20;
                        uint32_t *d = dst + bin * 32;
                        if (first) { d[0] = h; d[pl] = l; d[2 * pl] = c; }
                        else { // nothing waits for the result: reductions into words that only this thread touches
                            asm volatile("red.global.add.u32 [%0], %1;" ::"l"(d), "r"(h) : "memory");
                            asm volatile("red.global.add.u32 [%0], %1;" ::"l"(d + pl), "r"(l) : "memory");
                            asm volatile("red.global.add.u32 [%0], %1;" ::"l"(d + 2 * pl), "r"(c) : "memory");
                        }
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < NW; ++q) {
                        if (team == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(u0 + q * WSZ), "r"(0u) : "memory"); // guard row
                        for (int bin = team; bin < a.nbins; bin += QT) {
                            const uint32_t ai = u0 + q * WSZ + (uint32_t)(bin + 1) * 128u;
                            uint32_t v = lds_u32(ai);
                            asm volatile("st.shared.u32 [%0], %1;" ::"r"(ai), "r"(0u) : "memory");
                            for (int o = 32 / rep; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o); // add the replicas
                            dst[(q * a.nbins + bin) * 32] = v;
                        }
                    }
                }
                asm volatile("bar.sync %0, %1;" ::"r"(unit_bar), "r"(QT * 32) : "memory");
            };
            // Everything below counts in 32-bit offsets from the start of the segment (a row range of a CTA is short).
            const int seglen = (int)(send - pos), ntl = (int)ntiles;
            const uint32_t *rows_seg = rows + pos;
            // row id of row `lane` of the tile at offset o (0 beyond the end of the segment: never copied)
            auto rid_at = [&](int o) -> uint32_t { return o + lane < seglen ? rows_seg[o + lane] : 0u; };
            const int step = QT * EVB_TILE_ROWS;
            int so = team * EVB_TILE_ROWS;       // offset of the tile staged next
            int co = so;                          // offset of the tile consumed next
            uint32_t r0 = rid_at(so), r1 = rid_at(so + step);
            int sslot = 0, cslot = 0, c = 0, until_flush = QSUB;
            for (int i = 0; i < nmine + QDR - 1; ++i) {
                const uint32_t r2 = rid_at(so + 2 * step);
                if (i < nmine) { // stage the team's tile i
                    const int nrows = min(EVB_TILE_ROWS, seglen - so);
                    unsigned char *dst = ring + sslot * QTILE;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const uint32_t rid = __shfl_sync(0xffffffffu, r0, st_row[t]);
                        if (st_row[t] < nrows) cp_async16(dst + st_dst[t], xsl + (size_t)rid * RS + st_src[t]);
                    }
                    if (uw == 0 && lane < nrows) {
                        if constexpr (RW == 1) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst + EVB_TILE_ROWS * 128 + lane * 4)), "l"(gq + r0) : "memory");
                        else asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst + EVB_TILE_ROWS * 128 + lane * 8)), "l"(gq + (size_t)r0 * 2) : "memory");
                    }
                    sslot = sslot + 1 == NSLOT ? 0 : sslot + 1;
                }
                so += step;
                asm volatile("cp.async.commit_group;" ::: "memory");
                r0 = r1; r1 = r2;
                if (i >= QDR - 1) { // consume the team's tile c
                    asm volatile("cp.async.wait_group %0;" ::"n"(QDR - 1) : "memory");
                    // the copies of all warps of the team have landed, and everybody is done with tile c - 1
                    asm volatile("bar.sync %0, %1;" ::"r"(team_bar), "r"(team_threads) : "memory");
                    const int nrows = min(EVB_TILE_ROWS, seglen - co);
                    const uint32_t ts = ring_s + cslot * QTILE;
                    if (!skip_acc) {
                        const uint32_t tb = ts + rd_off, tw = ts + EVB_TILE_ROWS * 128 + rr * 4 * RW;
                        if (rep == 1) { if (nrows == EVB_TILE_ROWS) q_tile<NW, WSZ, 1, true>(tb, tw, nrows, rr, col, sel); else q_tile<NW, WSZ, 1, false>(tb, tw, nrows, rr, col, sel); }
                        else if (rep == 2) q_tile<NW, WSZ, 2, false>(tb, tw, nrows, rr, col, sel);
                        else if (rep == 4) q_tile<NW, WSZ, 4, false>(tb, tw, nrows, rr, col, sel);
                        else q_tile<NW, WSZ, 8, false>(tb, tw, nrows, rr, col, sel);
                    }
                    cslot = cslot + 1 == NSLOT ? 0 : cslot + 1;
                    co += step;
                    ++c;
                    if constexpr (NW == 3) { // the packed counters are full after QSUB tiles of every team
                        if (--until_flush == 0) {
                            until_flush = QSUB;
                            if (ntl > c * QT) { flush(!started); started = true; }
                        }
                    }
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("bar.sync %0, %1;" ::"r"(team_bar), "r"(team_threads) : "memory"); // ring free for the next segment
            flush(!started);
        }
        pos = send;
        ++s;
    }
}

struct ReduceQArgs {
    const uint32_t *scratch;
    double *hcomp;
    const LevelPlan *plan;
    const int32_t *cum;
    const double *qinv; // [2]: 2^-s of the g words, and of the w words (1 when w is a row count)
    int G, PG, UB, NFG, F, nbins, NW;
    uint32_t img_words;
};

// pieces of build slot s: CTAs bfirst..blast (the CTAs whose row range intersects the slot's rows)
__device__ __forceinline__ void slot_pieces(const LevelPlan *plan, const int32_t *cum, int s, int G, int &bfirst, int &blast, long long &R) {
    const int nbuild = plan->nbuild;
    R = plan->R;
    bfirst = 0; blast = -1;
    if (s < nbuild && R > 0) {
        const long long c0 = cum[s], c1 = cum[s + 1];
        if (c1 > c0) {
            bfirst = (int)(((c0 + 1) * G - 1) / R);
            blast = (int)((c1 * G - 1) / R);
        }
    }
}
// hcomp[slot][feature][g, h = 2w, w][bin] from the exact integer sums (K = 1; h: src/loss.jl:52)
__device__ __forceinline__ void store_q(double *hcomp, int s, int F, int nbins, int slotf, int bin, int ch, double v) {
    double *dst = hcomp + ((size_t)s * F + slotf) * 3 * nbins + bin;
    if (ch == 0) dst[0] = v;
    else { dst[(size_t)2 * nbins] = v; dst[nbins] = 2.0 * v; }
}

// Sums the pieces of every build slot of the fixed-point variant: grid (build slots of the level, NFG * 2 channels,
// ceil(nbins / BPB)), 512 threads = NPG piece groups x (BPB bins x 32 feature lanes).
template <int BPB>
__global__ void __launch_bounds__(512) k_histq_reduce(ReduceQArgs a) {
    constexpr int NE = BPB * 32, NPG = 512 / NE;
    __shared__ long long part_hi[NPG][NE], part_lo[NPG][NE];
    __shared__ double tile[BPB][33];
    const int s = blockIdx.x, fg = blockIdx.y >> 1, ch = blockIdx.y & 1, bin0 = blockIdx.z * BPB;
    const int ug = fg / a.UB, uw = fg % a.UB;
    const int e = threadIdx.x % NE, pg = threadIdx.x / NE, binl = e >> 5, lane = e & 31;
    int bfirst, blast;
    long long R;
    slot_pieces(a.plan, a.cum, s, a.G, bfirst, blast, R);
    const bool two = ch == 0 || a.NW == 4;   // hi + lo words, or a single count word
    const int w0 = ch == 0 ? 0 : 2;
    long long hi = 0, lo = 0;
    const int bin = bin0 + binl;
    if (bin < a.nbins) {
        const uint32_t *src = a.scratch + ((size_t)(ug * a.PG + s) * a.UB + uw) * a.img_words + (w0 * a.nbins + bin) * 32 + lane;
        const size_t bstride = (size_t)a.UB * a.img_words, wstride = (size_t)a.nbins * 32;
        const bool all = R >= a.G;
        for (int b = bfirst + pg; b <= blast; b += NPG) {
            if (all || R * b / a.G < R * (b + 1) / a.G) {
                if (two) { hi += (long long)(int32_t)src[(size_t)b * bstride]; lo += (long long)src[(size_t)b * bstride + wstride]; }
                else lo += (long long)src[(size_t)b * bstride];
            }
        }
    }
    part_hi[pg][e] = hi; part_lo[pg][e] = lo;
    __syncthreads();
    if (pg == 0) {
        long long th = 0, tl = 0;
#pragma unroll
        for (int q = 0; q < NPG; ++q) { th += part_hi[q][e]; tl += part_lo[q][e]; }
        tile[binl][lane] = (double)(th * (1ll << QSPLIT) + tl) * a.qinv[ch];
    }
    __syncthreads();
    if (threadIdx.x < NE) {
        const int fl = threadIdx.x / BPB, bl = threadIdx.x % BPB;
        const int slotf = fg * 32 + fl, binw = bin0 + bl;
        if (slotf < a.F && binw < a.nbins) store_q(a.hcomp, s, a.F, a.nbins, slotf, binw, ch, tile[bl][fl]);
    }
}

// deep levels (many build slots, few pieces each): one CTA per (build slot, unit)
__global__ void __launch_bounds__(256) k_histq_reduce_unit(ReduceQArgs a) {
    __shared__ double tile[64][33];
    const int s = blockIdx.x, fg = blockIdx.y;
    const int ug = fg / a.UB, uw = fg % a.UB;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int bfirst, blast;
    long long R;
    slot_pieces(a.plan, a.cum, s, a.G, bfirst, blast, R);
    const bool all = R >= a.G;
    const size_t bstride = (size_t)a.UB * a.img_words, wstride = (size_t)a.nbins * 32;
    const uint32_t *src0 = a.scratch + ((size_t)(ug * a.PG + s) * a.UB + uw) * a.img_words + lane;
    for (int ch = 0; ch < 2; ++ch) {
        const bool two = ch == 0 || a.NW == 4;
        const int w0 = ch == 0 ? 0 : 2;
        for (int bin0 = 0; bin0 < a.nbins; bin0 += 64) {
            for (int bl = w; bl < 64; bl += 8) {
                const int bin = bin0 + bl;
                long long hi = 0, lo = 0;
                if (bin < a.nbins) {
                    const uint32_t *src = src0 + (w0 * a.nbins + bin) * 32;
                    for (int b = bfirst; b <= blast; ++b) {
                        if (all || R * b / a.G < R * (b + 1) / a.G) {
                            if (two) { hi += (long long)(int32_t)src[(size_t)b * bstride]; lo += (long long)src[(size_t)b * bstride + wstride]; }
                            else lo += (long long)src[(size_t)b * bstride];
                        }
                    }
                }
                tile[bl][lane] = (double)(hi * (1ll << QSPLIT) + lo) * a.qinv[ch];
            }
            __syncthreads();
            for (int e = threadIdx.x; e < 64 * 32; e += 256) {
                const int fl = e >> 6, bl = e & 63;
                const int slotf = fg * 32 + fl, binw = bin0 + bl;
                if (slotf < a.F && binw < a.nbins) store_q(a.hcomp, s, a.F, a.nbins, slotf, binw, ch, tile[bl][fl]);
            }
            __syncthreads();
        }
    }
}

template <int BP, int NW>
cudaError_t launch_histq_t(const HistArgs &a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_histq<BP, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    k_histq<BP, NW><<<grid, threads, smem, st>>>(a);
    return cudaGetLastError();
}
template <int BP, int NW>
int occupancy_q_t(int threads, size_t smem) {
    cudaFuncSetAttribute(k_histq<BP, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_histq<BP, NW>, threads, smem) != cudaSuccess) nb = 0;
    return nb;
}
template <int BP>
int dispatch_q_nw(int NW, bool launch, const HistArgs *a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    if (NW == 3) return launch ? (int)launch_histq_t<BP, 3>(*a, grid, threads, smem, st) : occupancy_q_t<BP, 3>(threads, smem);
    return launch ? (int)launch_histq_t<BP, 4>(*a, grid, threads, smem, st) : occupancy_q_t<BP, 4>(threads, smem);
}
int dispatch_q(int BP, int NW, bool launch, const HistArgs *a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    switch (BP) {
    case 32: return dispatch_q_nw<32>(NW, launch, a, grid, threads, smem, st);
    case 64: return dispatch_q_nw<64>(NW, launch, a, grid, threads, smem, st);
    case 128: return dispatch_q_nw<128>(NW, launch, a, grid, threads, smem, st);
    default: return dispatch_q_nw<256>(NW, launch, a, grid, threads, smem, st);
    }
}

struct ReduceArgs {
    const float *scratch;
    double *hcomp;
    const LevelPlan *plan;
    const int32_t *cum;
    int G, PG, UB, NFG, U, F, C, Ce, K, nbins, NCH, FPL; // C: channels of hcomp; Ce: channels accumulated (mse: K + 1)
    uint32_t img_floats;
};

// Sums the pieces of every build slot in a fixed order (double precision) and writes
// hcomp[slot][feature][channel][bin].  grid (max build slots of the level, U * FPL * NCH, ceil(nbins / BPB));
// 512 threads = NPG piece groups x (BPB bins x 32 feature lanes).  Few slots / many pieces per slot (top of
// the tree) use BPB = 4 with four piece groups; many slots use BPB = 16.
template <int BPB>
__global__ void __launch_bounds__(512) k_hist_reduce(ReduceArgs a) {
    constexpr int NE = BPB * 32, NPG = 512 / NE;
    __shared__ double part[NPG][NE];
    __shared__ double tile[BPB][33];
    const int s = blockIdx.x, u = blockIdx.y / (a.NCH * a.FPL), j = (blockIdx.y / a.NCH) % a.FPL, c = blockIdx.y % a.NCH, bin0 = blockIdx.z * BPB;
    const int ug = u / a.UB, uw = u % a.UB, ct = u / a.NFG, fg = u % a.NFG;
    if (c >= min(a.NCH, a.Ce - ct * a.NCH)) return;
    const int e = threadIdx.x % NE, pg = threadIdx.x / NE, binl = e >> 5, lane = e & 31;
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
    double acc = 0.0;
    const int bin = bin0 + binl;
    if (bin < a.nbins) {
        const float *src = a.scratch + ((size_t)(ug * a.PG + s) * a.UB + uw) * a.img_floats + ((j * a.NCH + c) * a.nbins + bin) * 32 + lane;
        const size_t bstride = (size_t)a.UB * a.img_floats;
        if (R >= a.G) { // every CTA owns at least one row: all pieces in [bfirst, blast] exist
#pragma unroll 4
            for (int b = bfirst + pg; b <= blast; b += NPG) acc += (double)src[(size_t)b * bstride];
        } else {        // CTAs with an empty row range wrote nothing: skip their slots
            for (int b = bfirst + pg; b <= blast; b += NPG)
                if (R * b / a.G < R * (b + 1) / a.G) acc += (double)src[(size_t)b * bstride];
        }
    }
    part[pg][e] = acc;
    __syncthreads();
    if (pg == 0) {
        double t = part[0][e];
#pragma unroll
        for (int q = 1; q < NPG; ++q) t += part[q][e];
        tile[binl][lane] = t;
    }
    __syncthreads();
    if (threadIdx.x < NE) {
        const int fl = threadIdx.x / BPB, bl = threadIdx.x % BPB;
        const int slotf = (fg * 32 + fl) * a.FPL + j, binw = bin0 + bl;
        if (slotf < a.F && binw < a.nbins) {
            double *dst = a.hcomp + ((size_t)s * a.F + slotf) * a.C * a.nbins + binw;
            const int ce = ct * a.NCH + c;
            const double v = tile[bl][fl];
            if (a.Ce == a.C) {
                dst[(size_t)ce * a.nbins] = v;
            } else if (ce < a.K) { // mse with elided hessians: accumulated channels are g_1..g_K, w
                dst[(size_t)ce * a.nbins] = v;
            } else {
                dst[(size_t)(2 * a.K) * a.nbins] = v;                                           // w
                for (int k = 0; k < a.K; ++k) dst[(size_t)(a.K + k) * a.nbins] = 2.0 * v;       // h_k = 2w (src/loss.jl:52)
            }
        }
    }
}

// Variant for levels with many build slots (each with few pieces): one CTA per (build slot, unit, feature slot
// of the lane) sums all channels and bins of that sub-image, so that deep levels launch a thousand CTAs with real
// work each instead of many thousands of tiny ones.  Same fixed summation order as k_hist_reduce.
__global__ void __launch_bounds__(256) k_hist_reduce_unit(ReduceArgs a) {
    __shared__ double tile[64][33];
    const int s = blockIdx.x, u = blockIdx.y / a.FPL, j = blockIdx.y % a.FPL;
    const int ug = u / a.UB, uw = u % a.UB, ct = u / a.NFG, fg = u % a.NFG;
    const int nch = min(a.NCH, a.Ce - ct * a.NCH);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
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
    const bool all_exist = R >= a.G;
    const size_t bstride = (size_t)a.UB * a.img_floats;
    const float *src0 = a.scratch + ((size_t)(ug * a.PG + s) * a.UB + uw) * a.img_floats + lane;
    for (int c = 0; c < nch; ++c) {
        for (int bin0 = 0; bin0 < a.nbins; bin0 += 64) {
            for (int bl = w; bl < 64; bl += 8) {
                const int bin = bin0 + bl;
                double acc = 0.0;
                if (bin < a.nbins) {
                    const float *src = src0 + ((j * a.NCH + c) * a.nbins + bin) * 32;
                    for (int b = bfirst; b <= blast; ++b)
                        if (all_exist || R * b / a.G < R * (b + 1) / a.G) acc += (double)src[(size_t)b * bstride];
                }
                tile[bl][lane] = acc;
            }
            __syncthreads();
            for (int e = threadIdx.x; e < 64 * 32; e += 256) {
                const int fl = e >> 6, bl = e & 63;
                const int slotf = (fg * 32 + fl) * a.FPL + j, binw = bin0 + bl;
                if (slotf < a.F && binw < a.nbins) {
                    double *dst = a.hcomp + ((size_t)s * a.F + slotf) * a.C * a.nbins + binw;
                    const int ce = ct * a.NCH + c;
                    const double v = tile[bl][fl];
                    if (a.Ce == a.C || ce < a.K) {
                        dst[(size_t)ce * a.nbins] = v;
                    } else { // mse with elided hessians: w, and h_k = 2w
                        dst[(size_t)(2 * a.K) * a.nbins] = v;
                        for (int k = 0; k < a.K; ++k) dst[(size_t)(a.K + k) * a.nbins] = 2.0 * v;
                    }
                }
            }
            __syncthreads();
        }
    }
}

template <int BP, int NCH, int FPL>
cudaError_t launch_hist_t(const HistArgs &a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_hist<BP, NCH, FPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    k_hist<BP, NCH, FPL><<<grid, threads, smem, st>>>(a);
    return cudaGetLastError();
}
template <int BP, int NCH, int FPL>
int occupancy_t(int threads, size_t smem) {
    cudaFuncSetAttribute(k_hist<BP, NCH, FPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_hist<BP, NCH, FPL>, threads, smem) != cudaSuccess) nb = 0;
    return nb;
}

// Runtime (BP, NCH, FPL) -> template instance.  `launch` selects between launching and an occupancy query.
template <int BP, int NCH>
int dispatch_fpl(int FPL, bool launch, const HistArgs *a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    switch (FPL) {
    case 1: return launch ? (int)launch_hist_t<BP, NCH, 1>(*a, grid, threads, smem, st) : occupancy_t<BP, NCH, 1>(threads, smem);
    case 2: return launch ? (int)launch_hist_t<BP, NCH, 2>(*a, grid, threads, smem, st) : occupancy_t<BP, NCH, 2>(threads, smem);
    default: return launch ? (int)launch_hist_t<BP, NCH, 4>(*a, grid, threads, smem, st) : occupancy_t<BP, NCH, 4>(threads, smem);
    }
}
template <int BP>
int dispatch_nch(int NCH, int FPL, bool launch, const HistArgs *a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    switch (NCH) {
    case 1: return dispatch_fpl<BP, 1>(FPL, launch, a, grid, threads, smem, st);
    case 2: return dispatch_fpl<BP, 2>(FPL, launch, a, grid, threads, smem, st);
    case 3: return dispatch_fpl<BP, 3>(FPL, launch, a, grid, threads, smem, st);
    default: return dispatch_fpl<BP, 4>(FPL, launch, a, grid, threads, smem, st);
    }
}
int dispatch(int BP, int NCH, int FPL, bool launch, const HistArgs *a, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    switch (BP) {
    case 32: return dispatch_nch<32>(NCH, FPL, launch, a, grid, threads, smem, st);
    case 64: return dispatch_nch<64>(NCH, FPL, launch, a, grid, threads, smem, st);
    case 128: return dispatch_nch<128>(NCH, FPL, launch, a, grid, threads, smem, st);
    default: return dispatch_nch<256>(NCH, FPL, launch, a, grid, threads, smem, st);
    }
}
cudaError_t launch_hist(const HistGeom &g, const HistArgs &a, dim3 grid, int threads, cudaStream_t st) {
    return (cudaError_t)dispatch(g.BP, g.NCH, g.FPL, true, &a, grid, threads, g.smem, st);
}
int occupancy(const HistGeom &g, int threads) { return dispatch(g.BP, g.NCH, g.FPL, false, nullptr, dim3(), threads, g.smem, 0); }

size_t unit_image_bytes(int BP, int NCH, int FPL) {
    const int W0 = NCH >= 2 ? 2 : 1, W1 = NCH - W0;
    return (size_t)FPL * (BP + 1) * (32 * W0 * 4 + 32 * W1 * 4);
}

} // namespace

// Geometry for F feature slots.  Called once at create time with F = nfeats (sizes the scratch buffer)
// and again per tree when the column sample is smaller.
// fixed-point variant: one unit per 32 feature slots, NCH = words per row, one CTA per SM
static int32_t histq_geometry(const evb_handle *h, int F, HistGeom *g) {
    const int B = h->B;
    g->BP = B <= 32 ? 32 : B <= 64 ? 64 : B <= 128 ? 128 : 256;
    g->q = true;
    g->NCT = 1; g->NCH = h->unit_w ? 3 : 4; g->FPL = 1;
    g->NFG = (F + 31) / 32;
    g->U = g->NFG;
    const size_t img = (size_t)q_planes(g->NCH) * (g->BP + 1) * 128, rings = (size_t)QT * (QDR + 1) * q_tile_bytes(g->NCH); // rings: per CTA
    int UB = g->U < EVB_MAX_UNITS_PER_BLOCK ? g->U : EVB_MAX_UNITS_PER_BLOCK;
    while (UB > 1 && UB * img + rings > 227 * 1024) --UB;
    if (UB * img + rings > 227 * 1024) return EVB_ERR_LIMIT; // 256 bins with weights: the caller falls back to the float kernel
    g->UB = UB; g->NUG = (g->U + UB - 1) / UB; g->stages = QDR;
    g->smem = UB * img + rings;
    const int occ = dispatch_q(g->BP, g->NCH, false, nullptr, dim3(), UB * QT * 32, g->smem, 0);
    if (occ < 1) { evb_set_error("histogram kernel cannot be resident (smem=%zu)", g->smem); return EVB_ERR_CUDA; }
    g->G = occ * h->num_sms;
    // the 32-bit partial sums of a piece hold at most 2^17 rows: more (equal) row ranges than resident CTAs if needed
    if ((long long)g->G * 130000 < h->n) g->G = (int)((h->n + 129999) / 130000 + g->G - 1) / g->G * g->G;
    g->PG = g->G + h->maxslots;
    g->img_floats = (size_t)g->NCH * B * 32;
    return EVB_OK;
}

int32_t evb_hist_geometry(const evb_handle *h, int F, HistGeom *g) {
    if (h->use_q && F == h->nfeats) {
        const int32_t rc = histq_geometry(h, F, g);
        if (rc != EVB_ERR_LIMIT) return rc;
    }
    const int B = h->B, C = h->Ce;
    g->q = false;
    g->BP = B <= 32 ? 32 : B <= 64 ? 64 : B <= 128 ? 128 : 256;
    g->NCT = (C + 3) / 4;              // channel groups; channels are spread evenly over them
    g->NCH = (C + g->NCT - 1) / g->NCT;
    // feature slots per lane: as many as the feature count asks for, as long as a unit image stays <= 64 KB
    int FPL = 1; // measured on B200: 2 or 4 slots per lane (fewer, fatter warps) are slower than more resident warps
    if (const char *e = getenv("EVB_HIST_FPL")) { const int want = atoi(e); if (want == 1 || want == 2 || want == 4) FPL = want; }
    while (FPL > 1 && unit_image_bytes(g->BP, g->NCH, FPL) > 65 * 1024) FPL >>= 1;
    g->FPL = FPL;
    g->NFG = (F + 32 * FPL - 1) / (32 * FPL);
    g->U = g->NFG * g->NCT;
    const size_t img = unit_image_bytes(g->BP, g->NCH, FPL);
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
    // CTAs per SM: resident warps matter more than stage depth, so take as many CTAs as fit with two stages
    int t = (int)(sm_total / (UB * img + 2 * stage + 256 + reserve));
    if (const char *e = getenv("EVB_HIST_BLOCKS_PER_SM")) {           // tuning override
        const int want = atoi(e);
        if (want >= 1 && UB * img + 2 * stage + 256 + reserve <= sm_total / want) t = want;
    }
    if (t < 1) t = 1;
    if (t > 8) t = 8;
    size_t per_block = sm_total / t - reserve;
    if (per_block > blk_max) per_block = blk_max;
    int S = (int)((per_block - UB * img - 256) / stage);
    if (S > 8) S = 8;
    if (const char *e = getenv("EVB_HIST_STAGES")) { const int want = atoi(e); if (want >= 2 && want < S) S = want; }
    if (S < 2) S = 2;
    g->stages = S;
    g->smem = UB * img + (size_t)S * stage + 2 * S * 8 + 128;
    const int threads = (UB + 1) * 32;
    int occ = occupancy(*g, threads);
    if (occ < 1) {
        evb_set_error("histogram kernel cannot be resident (smem=%zu)", g->smem);
        return EVB_ERR_CUDA;
    }
    g->G = occ * h->num_sms;
    // Few rows: fewer, longer row ranges (every CTA costs one partial image that the reduce kernel has to read),
    // but never fewer CTAs than SMs.
    if (h->n > 0) {
        long long cap = h->n / 1024;
        if (cap < h->num_sms) cap = h->num_sms;
        if ((long long)g->G > cap) g->G = (int)cap;
    }
    g->PG = g->G + h->maxslots;
    g->img_floats = (size_t)FPL * g->NCH * B * 32;
    return EVB_OK;
}

int32_t evb_hist_configure(evb_handle *h) {
    EVB_CHECK(evb_hist_geometry(h, h->nfeats, &h->hg));
    h->q_active = h->hg.q;
    h->scratch_floats = (size_t)h->hg.NUG * h->hg.PG * h->hg.UB * h->hg.img_floats;
    return EVB_OK;
}

int32_t evb_launch_hist(evb_handle *h, int level) {
    const HistGeom &g = h->hg;
    HistArgs a;
    a.xT = h->xT; a.grad = h->q_active ? reinterpret_cast<const float *>(h->gradq) : h->grad; a.rows = h->rows[(level - 1) & 1]; a.js0 = h->js_d;
    a.plan = h->plan + level; a.cum = h->cum; a.slot_node = h->slot_node; a.seg_start = h->seg_start;
    a.scratch = h->scratch; a.err = h->d_err;
    a.RS = h->RS; a.GS = h->GS; a.F = h->F; a.nbins = h->B; a.C = h->Ce; a.NFG = g.NFG; a.U = g.U; a.UB = g.UB;
    a.stages = g.stages; a.PG = g.PG; a.img_floats = (uint32_t)g.img_floats;
    a.mode = h->hist_mode;
    a.contig = h->F == h->nfeats ? 1 : 0;
    dim3 grid(g.G, g.NUG);
    const int threads = h->q_active ? g.UB * QT * 32 : (g.UB + 1) * 32;
    evb_tic(h, EVB_T_HIST);
    cudaError_t e = h->q_active ? (cudaError_t)dispatch_q(g.BP, g.NCH, true, &a, grid, threads, g.smem, h->st) : launch_hist(g, a, grid, threads, h->st);
    evb_toc(h, EVB_T_HIST);
    EVB_CUDA(e);
    return EVB_OK;
}

int32_t evb_launch_hist_reduce(evb_handle *h, int level) {
    const HistGeom &g = h->hg;
    if (h->q_active) {
        ReduceQArgs a;
        a.scratch = reinterpret_cast<const uint32_t *>(h->scratch); a.hcomp = h->hcomp; a.plan = h->plan + level; a.cum = h->cum;
        a.qinv = h->d_qinv; a.G = g.G; a.PG = g.PG; a.UB = g.UB; a.NFG = g.NFG; a.F = h->F; a.nbins = h->B; a.NW = g.NCH;
        a.img_words = (uint32_t)g.img_floats;
        const int slots = evb_level_slots(level);
        evb_tic(h, EVB_T_HIST_REDUCE);
        if (slots <= 2) k_histq_reduce<1><<<dim3(slots, g.NFG * 2, h->B), 512, 0, h->st>>>(a);
        else if (slots <= 8) k_histq_reduce<4><<<dim3(slots, g.NFG * 2, (h->B + 3) / 4), 512, 0, h->st>>>(a);
        else if (slots <= 32) k_histq_reduce<16><<<dim3(slots, g.NFG * 2, (h->B + 15) / 16), 512, 0, h->st>>>(a);
        else k_histq_reduce_unit<<<dim3(slots, g.NFG), 256, 0, h->st>>>(a);
        evb_toc(h, EVB_T_HIST_REDUCE);
        EVB_CUDA(cudaGetLastError());
        return EVB_OK;
    }
    ReduceArgs a;
    a.scratch = h->scratch; a.hcomp = h->hcomp; a.plan = h->plan + level; a.cum = h->cum;
    a.G = g.G; a.PG = g.PG; a.UB = g.UB; a.NFG = g.NFG; a.U = g.U; a.F = h->F; a.C = h->C; a.Ce = h->Ce; a.K = h->K; a.nbins = h->B; a.NCH = g.NCH; a.FPL = g.FPL;
    a.img_floats = (uint32_t)g.img_floats;
    const int slots = evb_level_slots(level);
    evb_tic(h, EVB_T_HIST_REDUCE);
    if (slots <= 2) {           // top of the tree: hundreds of pieces per slot -> 16 piece groups per CTA
        dim3 grid(slots, g.U * g.FPL * g.NCH, h->B);
        k_hist_reduce<1><<<grid, 512, 0, h->st>>>(a);
    } else if (slots <= 8) {
        dim3 grid(slots, g.U * g.FPL * g.NCH, (h->B + 3) / 4);
        k_hist_reduce<4><<<grid, 512, 0, h->st>>>(a);
    } else if (slots <= 32) {
        dim3 grid(slots, g.U * g.FPL * g.NCH, (h->B + 15) / 16);
        k_hist_reduce<16><<<grid, 512, 0, h->st>>>(a);
    } else {                    // deep levels: few pieces per slot -> one CTA per sub-image
        dim3 grid(slots, g.U * g.FPL);
        k_hist_reduce_unit<<<grid, 256, 0, h->st>>>(a);
    }
    evb_toc(h, EVB_T_HIST_REDUCE);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// =====================================================================================================
// Stand-alone histogram of one list of rows, for callers that hold their own device buffers.
// evb_hist_rows allocates its work buffers per call; evb_hist_rows_noalloc allocates nothing.
// =====================================================================================================
namespace {

constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)2 << 20; // 8 MiB of partial images
constexpr int NOALLOC_MAX_FEATS = 1024;

struct RowsPlan {
    LevelPlan plan;
    int32_t cum[2];
    int32_t slot_node[2];
    int32_t seg_start[2];
    int err;
    int pad;
};

// Work memory of evb_hist_rows_noalloc.  It is part of the loaded library image on every GPU that uses the
// library and is shared by all calls on that GPU.
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) RowsPlan g_noalloc_plan;
static __device__ __align__(256) uint32_t g_noalloc_js[NOALLOC_MAX_FEATS];

__global__ void k_rows_plan_fill(RowsPlan *p, uint32_t *js, int nfeats, long long nrows) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < nfeats) js[t] = (uint32_t)t;
    if (t == 0) {
        p->plan.nbuild = 1; p->plan.nitems = 0; p->plan.R = nrows; p->plan.n_sel = (int32_t)nrows; p->plan.pad = 0;
        p->cum[0] = 0; p->cum[1] = (int32_t)nrows;
        p->slot_node[0] = 1; p->slot_node[1] = 0;
        p->seg_start[0] = 0; p->seg_start[1] = 0;
        p->err = 0;
    }
}

struct NoAllocDev {
    float *scratch = nullptr;
    RowsPlan *plan = nullptr;
    uint32_t *js = nullptr;
    bool ready = false;
};
NoAllocDev g_noalloc_dev[64];
std::mutex g_noalloc_mu;

int32_t rows_hist_check_args(int32_t device, const void *x_rows, int64_t nobs, int32_t nfeats, int32_t row_stride, int32_t nbins,
                             const void *grad, int32_t nch, const void *rows, int64_t nrows, const void *out) {
    if (!x_rows || !grad || !rows || !out) { evb_set_error("evb_hist_rows: null pointer"); return EVB_ERR_ARG; }
    if (nobs < 1 || nobs > 2000000000ll || nrows < 0 || nrows > 2000000000ll) { evb_set_error("evb_hist_rows: nobs / nrows out of range"); return EVB_ERR_ARG; }
    if (nfeats < 1 || row_stride < nfeats || (row_stride & 15)) { evb_set_error("evb_hist_rows: row_stride must be >= nfeats and a multiple of 16"); return EVB_ERR_ARG; }
    if (nbins < 2 || nbins > 255 || nch < 1 || nch > 4) { evb_set_error("evb_hist_rows: nbins must be 2..255 and nch 1..4"); return EVB_ERR_ARG; }
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) { evb_set_error("no CUDA device available (%s): this library has no CPU fallback", cudaGetErrorString(e)); return EVB_ERR_CUDA; }
    if (device < 0 || device >= ndev || device >= 64) { evb_set_error("evb_hist_rows: device %d out of range", device); return EVB_ERR_ARG; }
    return EVB_OK;
}

// Launches hist + reduce for one list of rows with the given work buffers; `max_pieces` bounds the grid.
int32_t rows_hist_run(int device, cudaStream_t st, const uint8_t *x_rows, int32_t nfeats, int32_t row_stride, int32_t nbins,
                      const float *grad, int32_t nch, const uint32_t *rows, int64_t nrows, double *out, float *scratch,
                      size_t scratch_floats, RowsPlan *plan, uint32_t *js, int hist_mode) {
    evb_handle hh{};
    hh.B = nbins; hh.C = nch; hh.Ce = nch; hh.K = 1; hh.RS = row_stride; hh.GS = 4; hh.nfeats = nfeats; hh.maxslots = 1; hh.n = nrows;
    int sms = 0;
    EVB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    hh.num_sms = sms;
    HistGeom g;
    EVB_CHECK(evb_hist_geometry(&hh, nfeats, &g));
    const size_t per_piece = (size_t)g.NUG * g.UB * g.img_floats;
    if (2 * per_piece > scratch_floats) {
        evb_set_error("evb_hist_rows: nfeats x nbins x nch too large for the work buffer (%zu floats per partial image, %zu available)",
                      per_piece, scratch_floats);
        return EVB_ERR_LIMIT;
    }
    const int gmax = (int)(scratch_floats / per_piece) - 1;
    if (g.G > gmax) g.G = gmax;
    g.PG = g.G + 1;
    k_rows_plan_fill<<<(nfeats + 255) / 256, 256, 0, st>>>(plan, js, nfeats, nrows);
    EVB_CUDA(cudaGetLastError());
    HistArgs a;
    a.xT = x_rows; a.grad = grad; a.rows = rows; a.js0 = js; a.plan = &plan->plan; a.cum = plan->cum; a.slot_node = plan->slot_node;
    a.seg_start = plan->seg_start; a.scratch = scratch; a.err = &plan->err;
    a.RS = row_stride; a.GS = 4; a.F = nfeats; a.nbins = nbins; a.C = nch; a.NFG = g.NFG; a.U = g.U; a.UB = g.UB;
    a.stages = g.stages; a.PG = g.PG; a.img_floats = (uint32_t)g.img_floats; a.mode = hist_mode; a.contig = 1;
    dim3 grid(g.G, g.NUG);
    const int threads = (g.UB + 1) * 32;
    EVB_CUDA(launch_hist(g, a, grid, threads, st));
    ReduceArgs r;
    r.scratch = scratch; r.hcomp = out; r.plan = &plan->plan; r.cum = plan->cum;
    r.G = g.G; r.PG = g.PG; r.UB = g.UB; r.NFG = g.NFG; r.U = g.U; r.F = nfeats; r.C = nch; r.Ce = nch; r.K = 1; r.nbins = nbins; r.NCH = g.NCH; r.FPL = g.FPL;
    r.img_floats = (uint32_t)g.img_floats;
    dim3 rgrid(1, g.U * g.FPL * g.NCH, (nbins + 3) / 4);
    k_hist_reduce<4><<<rgrid, 512, 0, st>>>(r);
    EVB_CUDA(cudaGetLastError());
    int derr = 0;
    EVB_CUDA(cudaMemcpyAsync(&derr, &plan->err, sizeof(int), cudaMemcpyDeviceToHost, st));
    EVB_CUDA(cudaStreamSynchronize(st));
    if (derr != 0) { evb_set_error("evb_hist_rows: device self-check failed (code %d)", derr); return EVB_ERR_DEVICE; }
    return EVB_OK;
}

} // namespace

extern "C" int32_t evb_hist_rows(int32_t device, void *stream, const uint8_t *x_rows, int64_t nobs, int32_t nfeats, int32_t row_stride,
                                 int32_t nbins, const float *grad, int32_t nch, const uint32_t *rows, int64_t nrows, double *out) {
    EVB_CHECK(rows_hist_check_args(device, x_rows, nobs, nfeats, row_stride, nbins, grad, nch, rows, nrows, out));
    EVB_CUDA(cudaSetDevice(device));
    cudaStream_t st = (cudaStream_t)stream;
    evb_handle hh{};
    hh.B = nbins; hh.C = nch; hh.Ce = nch; hh.RS = row_stride; hh.GS = 4; hh.nfeats = nfeats; hh.maxslots = 1; hh.n = nrows;
    int sms = 0;
    EVB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    hh.num_sms = sms;
    HistGeom g;
    EVB_CHECK(evb_hist_geometry(&hh, nfeats, &g));
    const size_t floats = (size_t)g.NUG * g.PG * g.UB * g.img_floats;
    float *scratch = nullptr;
    RowsPlan *plan = nullptr;
    uint32_t *js = nullptr;
    int32_t rc = EVB_OK;
    if (cudaMalloc((void **)&scratch, floats * sizeof(float)) != cudaSuccess || cudaMalloc((void **)&plan, sizeof(RowsPlan)) != cudaSuccess ||
        cudaMalloc((void **)&js, sizeof(uint32_t) * nfeats) != cudaSuccess) {
        evb_set_error("evb_hist_rows: out of device memory");
        rc = EVB_ERR_CUDA;
    } else {
        rc = rows_hist_run(device, st, x_rows, nfeats, row_stride, nbins, grad, nch, rows, nrows, out, scratch, floats, plan, js, evb_hist_mode_env());
    }
    cudaStreamSynchronize(st);
    if (scratch) cudaFree(scratch);
    if (plan) cudaFree(plan);
    if (js) cudaFree(js);
    return rc;
}

extern "C" int32_t evb_hist_rows_noalloc(int32_t device, void *stream, const uint8_t *x_rows, int64_t nobs, int32_t nfeats,
                                         int32_t row_stride, int32_t nbins, const float *grad, int32_t nch, const uint32_t *rows,
                                         int64_t nrows, double *out) {
    EVB_CHECK(rows_hist_check_args(device, x_rows, nobs, nfeats, row_stride, nbins, grad, nch, rows, nrows, out));
    if (nfeats > NOALLOC_MAX_FEATS) {
        evb_set_error("evb_hist_rows_noalloc: nfeats=%d exceeds the built-in limit of %d features", nfeats, NOALLOC_MAX_FEATS);
        return EVB_ERR_LIMIT;
    }
    EVB_CUDA(cudaSetDevice(device));
    NoAllocDev &d = g_noalloc_dev[device];
    {
        // once per device, with that device current: the symbols' names are host-side stand-ins, the kernels need
        // the device addresses.  The lock makes two host threads that call for the first time at once safe.
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (!d.ready) {
            EVB_CUDA(cudaGetSymbolAddress((void **)&d.scratch, g_noalloc_scratch));
            EVB_CUDA(cudaGetSymbolAddress((void **)&d.plan, g_noalloc_plan));
            EVB_CUDA(cudaGetSymbolAddress((void **)&d.js, g_noalloc_js));
            d.ready = true;
        }
    }
    return rows_hist_run(device, (cudaStream_t)stream, x_rows, nfeats, row_stride, nbins, grad, nch, rows, nrows, out, d.scratch,
                         NOALLOC_SCRATCH_FLOATS, d.plan, d.js, evb_hist_mode_env());
}
