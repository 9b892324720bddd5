// Fixed-point histogram build for mse with one target and unit weights: `update_hist!` / `_hist!`
// (src/fit-utils.jl:345-394; GPU counterpart `hist_kernel!`, ext/EvoTreesKernelAbstractionsExt/fit-utils.jl:57-95).
//
// Data layout.  The bins of a row live in two arrays: xH[row][RSH] holds the features in 16-byte chunks (16 features
// each) and xE[row] = {q, tail} holds the row's fixed-point gradient q = rint(g * 2^s) (written once per boosting
// round) and, when nfeats % 16 is 1..4, the bins of those last features, so that a row of 100 features is 96 + 8
// bytes: three whole sectors plus one, wherever the row is gathered from.
//
// Kernel.  Warps work on their own: there is no producer, no staging buffer and no barrier between tiles.  A warp
// takes tiles of 32 rows.  Lane l loads chunk (32 s + l) % NC of row (32 s + l) / NC in step s with one 128-bit
// load straight into registers (a row's chunks sit in adjacent lanes, so a request covers whole lines); the
// registers of a step are refilled for a later step (of this tile or of the warp's next one) as soon as they have
// been accumulated, so a few loads per lane are always in flight and no shared memory is spent on rows.
// A CTA keeps one packed image [bin][plane][column] of 32-bit words in shared memory; a row adds two
// words per feature with `red.shared.add.u32`: q >> 6 into plane 0 and (q & 0x3f) | 1 << 19 into plane 1 (the row
// count rides in the top 13 bits; |q| < 2^24).  Integer sums do not depend on the order, so all warps share the image.  The 32
// lanes of a reduction always hit 32 different banks: lanes differ in the chunk's parity, in the word of the chunk
// they work on (the four registers of a chunk are rotated by (l >> 1) & 3) and in the byte of that word
// ((l >> 3) & 3).
// The packed counters hold 8191 rows: after at most 255 tiles, and at the end of a node's rows, the CTA adds the packed
// image to the node's accumulators in global memory (`red.global.add.u64 / .u32`, cell by cell: consecutive lanes,
// consecutive addresses) and clears it.  Two CTAs share an SM, so one accumulates while the other flushes.  (Optional:
// one CTA per SM that keeps a wide image -- 64-bit sums, 32-bit counts -- in shared memory between the flushes to global
// memory.)  Every histogram entry is therefore the exact integer sum of the quantised gradients, whatever the order of
// the rows and however the rows are cut into pieces.
#include "evb_internal.cuh"
#include <stdlib.h>

namespace {

constexpr unsigned FULL = 0xffffffffu;
// Measured on B200 (10M x 100, depth 11, ms of this kernel per tree).  One CTA per SM with a wide image (64-bit sums in shared
// memory between the flushes to global memory): 768 threads 1.91, 1024: 2.29, 512: 2.33 (the last two before later
// changes).  Two CTAs of 384 threads per SM without the wide image, every flush going to global memory: 1.83; three
// CTAs of 256: 2.28.
constexpr int Q2_THREADS = 384;
// Word format.  q has QB bits (|q| < 2^QB); plane 0 takes q >> LB, plane 1 takes (q & (2^LB - 1)) | 1 << CS, and an image
// cell must hold 2^CB - 1 rows: QB - LB + CB <= 31 (signed plane 0), LB + CB <= CS and CS + CB <= 32 (plane 1).
// QB = 26: LB 8, CS 20, CB 12 (4095 rows, 127 tiles between flushes); QB = 24: LB 6, CS 19, CB 13 (8191 rows, 255 tiles).
constexpr int Q2_MAX_EPOCH_26 = 127, Q2_MAX_EPOCH_24 = 255;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

struct Q2Args {
    const uint8_t *xH;
    const uint2 *xE;
    const uint32_t *rows;
    const LevelPlan *plan;
    const int32_t *cum, *slot_node, *seg_start;
    unsigned long long *hsum; // [slot][bin][SC] sums of q
    uint32_t *hcnt;           // [slot][bin][SC] row counts
    int RSH, B, SC;
    int nmain;                // features held in xH
    int ntail;                // features held in xE (0..4)
    int TE;                   // tiles between two flushes
    int LB, CS;               // word format: low bits in plane 1, position of the row count
    int wide;                 // 1: epochs end in the CTA's wide image in shared memory; 0: no wide image, every flush goes to global memory
    int min_rows;             // rows per CTA below which fewer CTAs take part
    uint32_t zrow;            // index of an all-zero row of xH / xE (bins 0, q 0)
};

// image geometry for NC chunks of 16 features (+ 8 replicas of the 4 tail features): NCOL columns per plane row
template <int NC, bool TAIL>
struct Q2Cfg {
    static constexpr int NEED = 16 * NC + (TAIL ? 32 : 0);
    static_assert(NEED <= 128, "at most 128 image columns per CTA");
    static constexpr int NCOL = NEED <= 32 ? 32 : NEED <= 64 ? 64 : 128;
    static constexpr int TAILCOL = NCOL - 32;
    static constexpr uint32_t ROWB = NCOL * 4; // bytes of one plane row; a bin owns two of them (plane 0, plane 1)
    static constexpr uint32_t X = NCOL / 32;   // (bin << 8 | column byte) * X = bin * 2 * ROWB + 4 * column
};

__device__ __forceinline__ uint4 ldg_chunk(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// row id: issued where it stands (a plain load may be moved next to its first use, a whole tile later)
__device__ __forceinline__ uint32_t ldg_rid(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_ext(const uint2 *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Four features (one word of bins) of one row.  u: the word; Cb: bytes {column byte of register byte k}; sel[k]: PRMT
// selector that builds (bin << 8 | column byte) of the lane's k-th feature; As: image address of the lane's column
// group in bin row 0.  (bin << 8 | column byte) * X = bin * 2 * ROWB + 4 * column.
template <uint32_t ROWB, uint32_t X>
__device__ __forceinline__ void q2_word(uint32_t u, uint32_t As, uint32_t Cb, const uint32_t (&sel)[4], uint32_t w0, uint32_t w1) {
    asm volatile(
        "{\n .reg .u32 b0, b1, b2, b3, a0, a1, a2, a3;\n"
        " prmt.b32 b0, %0, %1, %2;\n prmt.b32 b1, %0, %1, %3;\n prmt.b32 b2, %0, %1, %4;\n prmt.b32 b3, %0, %1, %5;\n"
        " mad.lo.u32 a0, b0, %10, %6;\n mad.lo.u32 a1, b1, %10, %6;\n mad.lo.u32 a2, b2, %10, %6;\n mad.lo.u32 a3, b3, %10, %6;\n"
        " red.shared.add.u32 [a0], %7;\n red.shared.add.u32 [a0+%9], %8;\n"
        " red.shared.add.u32 [a1], %7;\n red.shared.add.u32 [a1+%9], %8;\n"
        " red.shared.add.u32 [a2], %7;\n red.shared.add.u32 [a2+%9], %8;\n"
        " red.shared.add.u32 [a3], %7;\n red.shared.add.u32 [a3+%9], %8;\n}\n"
        ::"r"(u), "r"(Cb), "r"(sel[0]), "r"(sel[1]), "r"(sel[2]), "r"(sel[3]), "r"(As), "r"(w0), "r"(w1), "n"(ROWB), "n"(X)
        : "memory");
}

// iterator over the non-empty pieces (CTA row range x build slot) of a CTA, addressed by the CTA's tile index
struct PieceIt {
    int s, g0, nt, pstart, pend;
    const uint32_t *rows;
    bool end;
};
__device__ __forceinline__ void piece_load(const Q2Args &a, PieceIt &it, int lo, int hi, int nbuild) {
    for (;;) {
        if (it.s >= nbuild) { it.end = true; return; }
        const int c0 = a.cum[it.s], c1 = a.cum[it.s + 1];
        if (c0 >= hi) { it.end = true; return; }
        const int ps = max(lo, c0), pe = min(hi, c1);
        if (pe > ps) {
            it.pstart = ps; it.pend = pe; it.nt = (pe - ps + 31) >> 5;
            it.rows = a.rows + ((long long)a.seg_start[a.slot_node[it.s]] - c0);
            return;
        }
        ++it.s;
    }
}
__device__ __forceinline__ void piece_next(const Q2Args &a, PieceIt &it, int lo, int hi, int nbuild) {
    it.g0 += it.nt;
    ++it.s;
    piece_load(a, it, lo, hi, nbuild);
}

// register sets of chunk loads in flight per lane: step s of a tile uses set s % NSET and refills it for step s + NSET
__host__ __device__ constexpr int q2_nset(int NC) { return NC == 6 ? 3 : NC == 8 ? 4 : NC; }

template <int NC, bool TAIL, int NT>
__global__ void __launch_bounds__(NT, NT <= 384 ? 2 : 1) k_histq2(Q2Args a) {
    using Cf = Q2Cfg<NC, TAIL>;
    constexpr int NCOL = Cf::NCOL, NSET = q2_nset(NC);
    constexpr uint32_t ROWB = Cf::ROWB, X = Cf::X;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, wid = tid >> 5, l = tid & 31;
    constexpr int NW = NT / 32;
    const int b = blockIdx.x, chunk0 = blockIdx.y * NC;
    const long long R = a.plan->R;
    // few rows: fewer CTAs take part (every CTA costs one pass over its image)
    int G = gridDim.x;
    {
        const long long want = (R + a.min_rows - 1) / a.min_rows;
        if (want < G) G = want < 1 ? 1 : (int)want;
    }
    if (b >= G) return;
    const int lo = (int)(R * b / G), hi = (int)(R * (b + 1) / G);
    if (lo >= hi) return;
    uint32_t *img_w = reinterpret_cast<uint32_t *>(smem);
    for (int i = tid; i < ((a.B + 1) * 2 * NCOL * 4 + (a.wide ? a.B * (16 * NC + (TAIL ? 4 : 0)) * 12 : 0)) / 4; i += NT) img_w[i] = 0u; // packed (+ wide) image
    __syncthreads();

    const int nbuild = a.plan->nbuild;
    int s0;
    {
        int lft = 0, rgt = nbuild - 1; // largest s with cum[s] <= lo
        while (lft < rgt) { const int m = (lft + rgt + 1) >> 1; if (a.cum[m] <= lo) lft = m; else rgt = m - 1; }
        s0 = lft;
    }
    // per-lane constants
    const int rot_w = (l >> 1) & 3, rot_b = (l >> 3) & 3;
    uint32_t sel[4], Cb0 = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t cb = (uint32_t)((k + rot_b) & 3);
        Cb0 |= (cb * (4u / X)) << (8 * k);
        sel[k] = ((0xCu + k) << 12) | ((0xCu + k) << 8) | (cb << 4) | (4u + k);
    }
    const uint32_t img = smem_u32(smem);
    uint32_t A0[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) A0[p] = img + 16u * (uint32_t)((p + rot_w) & 3);
    const uint32_t At = img + 4u * (uint32_t)(Cf::TAILCOL + 4 * (l & 7));
    const bool r1 = (rot_w & 1) != 0, r2 = (rot_w & 2) != 0;
    // step s of a tile: the lane works on chunk (32 s + l) % NC of row (32 s + l) / NC.  rowsel packs the rows (5 bits
    // per step); the chunk of step 0 is ch0 and every step adds 32 % NC (mod NC).
    uint32_t rowsel = 0;
#pragma unroll
    for (int s = 0; s < NC && s < 6; ++s) rowsel |= (uint32_t)((32 * s + l) / NC) << (5 * s);
    auto row_of = [&](int s) -> int { return NC <= 6 ? (int)(rowsel >> (5 * s)) : (32 * s + l) / NC; }; // shuffles use the low 5 bits
    const int ch0 = l % NC;
    const uint8_t *xH = a.xH + (size_t)chunk0 * 16;
    const uint32_t RSH = (uint32_t)a.RSH;
    const uint32_t zrow = a.zrow; // an all-zero row: its bins land in the image's guard row

    // The packed image is emptied at every boundary.  Inside a node's rows it goes into the CTA's wide image in shared
    // memory (64-bit sums, 32-bit counts; every cell belongs to one thread, so plain adds); at the end of the node's
    // rows (`final`) packed + wide go to the accumulators of build slot `slot` in global memory.  All threads of the CTA.
    constexpr int WC = 16 * NC + (TAIL ? 4 : 0); // columns of the wide image
    long long *wsum = reinterpret_cast<long long *>(smem + (size_t)(a.B + 1) * 2 * NCOL * 4);
    uint32_t *wcnt = reinterpret_cast<uint32_t *>(wsum + (size_t)a.B * WC);
    const int LB = a.LB, CS = a.CS;
    const uint32_t cmask = (1u << CS) - 1u, lmask = (1u << LB) - 1u, one = 1u << CS;
    auto flush = [&](int slot, bool final) {
        __syncthreads();
        if (!a.wide) {
            // no wide image: the packed image goes to the slot's accumulators cell by cell (consecutive lanes, consecutive
            // addresses), whether the node's rows end here or only the count field is full
            const size_t base = (size_t)slot * a.B;
            constexpr int MC = 16 * NC;
            for (int c = tid; c < a.B * MC; c += NT) {
                const int bin = c / MC, col = c - bin * MC;
                uint32_t *p = img_w + (size_t)(bin + 1) * 2 * NCOL + col;
                const uint32_t vh = p[0], vp = p[NCOL];
                if ((vh | vp) == 0u) continue;
                p[0] = 0u; p[NCOL] = 0u;
                const int f = chunk0 * 16 + col;
                if (f < a.nmain) {
                    const long long sum = ((long long)(int32_t)vh << LB) + (long long)(vp & cmask);
                    const size_t o = (base + bin) * a.SC + f;
                    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(a.hsum + o), "l"(sum) : "memory");
                    asm volatile("red.global.add.u32 [%0], %1;" ::"l"(a.hcnt + o), "r"(vp >> CS) : "memory");
                }
            }
            if (TAIL) {
                for (int bin = wid; bin < a.B; bin += NW) {
                    uint32_t *p = img_w + (size_t)(bin + 1) * 2 * NCOL + Cf::TAILCOL + l;
                    const uint32_t vh = p[0], vp = p[NCOL];
                    if (__ballot_sync(FULL, (vh | vp) != 0u) == 0u) continue;
                    p[0] = 0u; p[NCOL] = 0u;
                    long long sum = ((long long)(int32_t)vh << LB) + (long long)(vp & cmask);
                    uint32_t cnt = vp >> CS;
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) { sum += __shfl_xor_sync(FULL, sum, o); cnt += __shfl_xor_sync(FULL, cnt, o); }
                    if (l < a.ntail && cnt != 0u) {
                        const size_t o = (base + bin) * a.SC + a.nmain + l;
                        asm volatile("red.global.add.u64 [%0], %1;" ::"l"(a.hsum + o), "l"(sum) : "memory");
                        asm volatile("red.global.add.u32 [%0], %1;" ::"l"(a.hcnt + o), "r"(cnt) : "memory");
                    }
                }
            }
            __syncthreads();
            return;
        }
        constexpr int QPR = 4 * NC; // quads of main columns per bin row
        for (int e = tid; e < a.B * QPR; e += NT) {
            const int bin = e / QPR, col = (e % QPR) * 4;
            uint32_t *p = img_w + (size_t)(bin + 1) * 2 * NCOL + col;
            const uint4 vh = *reinterpret_cast<const uint4 *>(p), vp = *reinterpret_cast<const uint4 *>(p + NCOL);
            if ((vh.x | vh.y | vh.z | vh.w | vp.x | vp.y | vp.z | vp.w) == 0u) continue;
            *reinterpret_cast<uint4 *>(p) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4 *>(p + NCOL) = make_uint4(0u, 0u, 0u, 0u);
            const uint32_t h4[4] = {vh.x, vh.y, vh.z, vh.w}, p4[4] = {vp.x, vp.y, vp.z, vp.w};
            long long sm4[4];
            uint32_t c4[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) { sm4[k] = ((long long)(int32_t)h4[k] << LB) + (long long)(p4[k] & cmask); c4[k] = p4[k] >> CS; }
            longlong2 *ws = reinterpret_cast<longlong2 *>(wsum + (size_t)bin * WC + col);
            uint4 *wc = reinterpret_cast<uint4 *>(wcnt + (size_t)bin * WC + col);
            longlong2 s0 = ws[0], s1 = ws[1];
            uint4 cw = *wc;
            s0.x += sm4[0]; s0.y += sm4[1]; s1.x += sm4[2]; s1.y += sm4[3];
            cw.x += c4[0]; cw.y += c4[1]; cw.z += c4[2]; cw.w += c4[3];
            ws[0] = s0; ws[1] = s1; *wc = cw;
        }
        if (TAIL) { // 8 replicas of the 4 tail features: one warp per bin row, lane = column of the packed image
            for (int bin = wid; bin < a.B; bin += NW) {
                uint32_t *p = img_w + (size_t)(bin + 1) * 2 * NCOL + Cf::TAILCOL + l;
                const uint32_t vh = p[0], vp = p[NCOL];
                if (__ballot_sync(FULL, (vh | vp) != 0u) == 0u) continue;
                p[0] = 0u; p[NCOL] = 0u;
                long long sum = ((long long)(int32_t)vh << LB) + (long long)(vp & cmask);
                uint32_t cnt = vp >> CS;
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) { sum += __shfl_xor_sync(FULL, sum, o); cnt += __shfl_xor_sync(FULL, cnt, o); }
                if (l < 4) {
                    wsum[(size_t)bin * WC + 16 * NC + l] += sum;
                    wcnt[(size_t)bin * WC + 16 * NC + l] += cnt;
                }
            }
        }
        if (final) {
            // the wide image goes to the slot's accumulators cell by cell: consecutive lanes, consecutive addresses
            __syncthreads();
            const size_t base = (size_t)slot * a.B;
            for (int c = tid; c < a.B * WC; c += NT) {
                const uint32_t cnt = wcnt[c];
                if (cnt == 0u) continue;
                const long long sum = wsum[c];
                wsum[c] = 0; wcnt[c] = 0u;
                const int bin = c / WC, col = c - bin * WC;
                const bool main_col = col < 16 * NC;
                const int f = main_col ? chunk0 * 16 + col : a.nmain + col - 16 * NC;
                if (main_col ? f < a.nmain : col - 16 * NC < a.ntail) {
                    const size_t o = (base + bin) * a.SC + f;
                    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(a.hsum + o), "l"(sum) : "memory");
                    asm volatile("red.global.add.u32 [%0], %1;" ::"l"(a.hcnt + o), "r"(cnt) : "memory");
                }
            }
        }
        __syncthreads();
    };

    // the two piece iterators of a warp (accumulate stage, row-id fetch stage) are warp-uniform and touched once per
    // tile: they live in shared memory so that the registers stay with the loads in flight
    __shared__ PieceIt s_it[NT / 32][2];
    PieceIt &pc = s_it[wid][0], &pa = s_it[wid][1];
    pc.s = s0; pc.g0 = 0; pc.end = false;
    piece_load(a, pc, lo, hi, nbuild);
    pa = pc;
    __syncwarp();
    int ep_end = pc.end ? 0 : min(pc.nt, a.TE);

    // row ids of tile g of this CTA (lane = row of the tile); rows past the end of the tile read the zero row
    auto fetch = [&](int g) -> uint32_t {
        while (!pa.end && g >= pa.g0 + pa.nt) piece_next(a, pa, lo, hi, nbuild);
        if (pa.end) return zrow;
        const int off = pa.pstart + ((g - pa.g0) << 5);
        return off + l < pa.pend ? ldg_rid(pa.rows + off + l) : zrow;
    };
    // chunk of step s for the tile whose row ids are `rid`; ch = the lane's chunk in that step
    auto load_chunk = [&](uint32_t rid, int s, int ch) -> uint4 {
        const uint32_t r = __shfl_sync(FULL, rid, row_of(s));
        return ldg_chunk(xH + (size_t)(r * RSH + (uint32_t)ch * 16u));
    };
    auto ch_of = [&](int s) -> int { return (ch0 + (32 * s) % NC) % NC; };

    uint32_t ridC, ridB;
    uint4 v[NSET];
    uint2 extC;
    ridC = fetch(wid);
    ridB = fetch(wid + NW);
    extC = ldg_ext(a.xE + ridC);
#pragma unroll
    for (int s = 0; s < NSET; ++s) v[s] = load_chunk(ridC, s, ch_of(s));
    for (int g = wid;; g += NW) {
        bool done = false;
        for (;;) {
            if (pc.end) { done = true; break; }
            if (g < pc.g0 + ep_end) break;
            flush(pc.s, ep_end == pc.nt);
            if (ep_end == pc.nt) { piece_next(a, pc, lo, hi, nbuild); if (!pc.end) ep_end = min(pc.nt, a.TE); }
            else ep_end = min(pc.nt, ep_end + a.TE);
        }
        if (done) break;
        const uint2 extN = ldg_ext(a.xE + ridB);
        const uint32_t ridA = fetch(g + 2 * NW);
#pragma unroll
        for (int s = 0; s < NC; ++s) {
            const int ch = ch_of(s);
            const uint32_t q = __shfl_sync(FULL, extC.x, row_of(s));
            const uint32_t w0 = (uint32_t)((int32_t)q >> LB), w1 = (q & lmask) | one;
            const uint4 c = v[s % NSET];
            const uint32_t t0 = r1 ? c.y : c.x, t1 = r1 ? c.z : c.y, t2 = r1 ? c.w : c.z, t3 = r1 ? c.x : c.w;
            const uint32_t u0 = r2 ? t2 : t0, u1 = r2 ? t3 : t1, u2 = r2 ? t0 : t2, u3 = r2 ? t1 : t3;
            const uint32_t Cb = Cb0 + (uint32_t)ch * ((64u / X) * 0x01010101u); // column byte += 16 columns per chunk
            q2_word<ROWB, X>(u0, A0[0], Cb, sel, w0, w1);
            q2_word<ROWB, X>(u1, A0[1], Cb, sel, w0, w1);
            q2_word<ROWB, X>(u2, A0[2], Cb, sel, w0, w1);
            q2_word<ROWB, X>(u3, A0[3], Cb, sel, w0, w1);
            // the same registers, for step s + NSET: of this tile, or of the warp's next tile
            if (s + NSET < NC) v[s % NSET] = load_chunk(ridC, s + NSET, ch_of(s + NSET));
            else v[s % NSET] = load_chunk(ridB, s + NSET - NC, ch_of(s + NSET - NC));
        }
        if (TAIL) { // lane = row of the tile
            const uint32_t q = extC.x;
            const uint32_t w0 = (uint32_t)((int32_t)q >> LB), w1 = (q & lmask) | one;
            q2_word<ROWB, X>(extC.y, At, Cb0, sel, w0, w1);
        }
        extC = extN;
        ridC = ridB; ridB = ridA;
    }
}

// hcomp[slot][f][g, h = 2w, w][bin] (doubles) from the integer accumulators, which are cleared for the next level.
// One CTA per (build slot, 32 feature slots).
struct Q2ConvArgs {
    unsigned long long *hsum;
    uint32_t *hcnt;
    double *hcomp;
    const LevelPlan *plan;
    const uint32_t *js0;
    const double *qinv;
    int B, SC, F;
};
__global__ void __launch_bounds__(256) k_q2_to_hcomp(Q2ConvArgs a) {
    __shared__ double tg[64][33], tw[64][33];
    const int s = blockIdx.x, f0 = blockIdx.y * 32;
    if (s >= a.plan->nbuild) return;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const double qi = a.qinv[0];
    const int f = f0 + lane;
    const int col = f < a.F ? (int)a.js0[f] : -1;
    for (int bin0 = 0; bin0 < a.B; bin0 += 64) {
        for (int bl = w; bl < 64; bl += 8) {
            const int bin = bin0 + bl;
            double g = 0.0, c = 0.0;
            if (bin < a.B && col >= 0) {
                const size_t o = ((size_t)s * a.B + bin) * a.SC + col;
                g = (double)(long long)a.hsum[o] * qi;
                c = (double)a.hcnt[o];
            }
            tg[bl][lane] = g; tw[bl][lane] = c;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 64 * 32; e += 256) {
            const int fl = e >> 6, bl = e & 63;
            const int ff = f0 + fl, bin = bin0 + bl;
            if (ff < a.F && bin < a.B) {
                double *dst = a.hcomp + ((size_t)s * a.F + ff) * 3 * a.B + bin;
                const double wv = tw[bl][fl];
                dst[0] = tg[bl][fl]; dst[a.B] = 2.0 * wv; dst[(size_t)2 * a.B] = wv; // h = 2w (src/loss.jl:52)
            }
        }
        __syncthreads();
    }
}
// clears the accumulators of the level's build slots (all feature columns, sampled or not)
__global__ void __launch_bounds__(256) k_q2_clear(unsigned long long *hsum, uint32_t *hcnt, const LevelPlan *plan, size_t per_slot) {
    const size_t n = (size_t)plan->nbuild * per_slot;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) { hsum[i] = 0ull; hcnt[i] = 0u; }
}

// tail features of every row: xE[i].y = bins of features nmain .. nmain + ntail - 1 (one byte each, zero padded)
__global__ void __launch_bounds__(256) k_q2_tail(const uint8_t *xC, long long n, int nmain, int ntail, uint2 *xE) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t t = 0;
    for (int k = 0; k < ntail; ++k) t |= (uint32_t)xC[(size_t)(nmain + k) * n + i] << (8 * k);
    xE[i] = make_uint2(0u, t);
}

// q = rint(g * 2^s), 2^s the largest power of two with max |g| * 2^s < 2^QB, into xE[i].x; 2^-s into qinv[0]
__global__ void __launch_bounds__(256) k_q2_quantize(const float *grad, int GS, uint2 *xE, long long n, const unsigned *gmax, double *qinv, int QB) {
    const float m = __uint_as_float(*gmax);
    float sc = 1.0f;
    double inv = 1.0;
    if (m > 0.0f && m < INFINITY) {
        int e;
        frexpf(m, &e);
        sc = ldexpf(1.0f, QB - e);
        inv = ldexp(1.0, e - QB);
    }
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) { qinv[0] = inv; qinv[1] = 1.0; }
    if (i >= n) return;
    reinterpret_cast<int32_t *>(xE)[2 * i] = __float2int_rn(grad[(size_t)i * GS] * sc);
}

template <int NC, bool TAIL, int NT>
int q2_instance_t(bool launch, const Q2Args *a, dim3 grid, size_t smem, cudaStream_t st) {
    static size_t attr_set[64] = {}; // dynamic shared memory the kernel has been allowed on each device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && attr_set[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(k_histq2<NC, TAIL, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return launch ? (int)e : 0;
        attr_set[dev] = smem;
    }
    if (!launch) {
        int nb = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k_histq2<NC, TAIL, NT>, NT, smem) != cudaSuccess) nb = 0;
        return nb;
    }
    k_histq2<NC, TAIL, NT><<<grid, NT, smem, st>>>(*a);
    return (int)cudaGetLastError();
}
int g_q2_threads = Q2_THREADS;
template <int NC, bool TAIL>
int q2_instance(bool launch, const Q2Args *a, dim3 grid, size_t smem, cudaStream_t st) {
    if (g_q2_threads == 384) return q2_instance_t<NC, TAIL, 384>(launch, a, grid, smem, st);
    if (g_q2_threads == 512) return q2_instance_t<NC, TAIL, 512>(launch, a, grid, smem, st);
    if (g_q2_threads == 768) return q2_instance_t<NC, TAIL, 768>(launch, a, grid, smem, st);
    return q2_instance_t<NC, TAIL, 1024>(launch, a, grid, smem, st);
}
template <bool TAIL>
int q2_dispatch_nc(int NC, bool launch, const Q2Args *a, dim3 grid, size_t smem, cudaStream_t st) {
    switch (NC) {
    case 1: return q2_instance<1, TAIL>(launch, a, grid, smem, st);
    case 2: return q2_instance<2, TAIL>(launch, a, grid, smem, st);
    case 3: return q2_instance<3, TAIL>(launch, a, grid, smem, st);
    case 4: return q2_instance<4, TAIL>(launch, a, grid, smem, st);
    case 5: return q2_instance<5, TAIL>(launch, a, grid, smem, st);
    default: return q2_instance<6, TAIL>(launch, a, grid, smem, st);
    }
}
int q2_dispatch(int NC, bool tail, bool launch, const Q2Args *a, dim3 grid, size_t smem, cudaStream_t st) {
    if (tail) return q2_dispatch_nc<true>(NC, launch, a, grid, smem, st);
    switch (NC) {
    case 7: return q2_instance<7, false>(launch, a, grid, smem, st);
    case 8: return q2_instance<8, false>(launch, a, grid, smem, st);
    default: return q2_dispatch_nc<false>(NC, launch, a, grid, smem, st);
    }
}
int q2_ncol(int NC, bool tail) { const int need = 16 * NC + (tail ? 32 : 0); return need <= 32 ? 32 : need <= 64 ? 64 : 128; }
// shared memory of a CTA: packed image [B + 1][2][NCOL] words + wide image [B][16 NC (+ 4)] x (64-bit sum, 32-bit count)
bool g_q2_wide = false;
size_t q2_smem(int B, int NC, bool tail) { return (size_t)(B + 1) * 2 * q2_ncol(NC, tail) * 4 + (g_q2_wide ? (size_t)B * (16 * NC + (tail ? 4 : 0)) * 12 : 0); }

} // namespace

// Chooses the layout: chunks per CTA group, number of groups, tail features.  Returns EVB_ERR_LIMIT when the shape
// does not fit (the caller then uses the other histogram kernels).
int32_t evb_q2_configure(evb_handle *h) {
    const int nf = h->nfeats, B = h->B;
    Q2Geom &g = h->q2;
    const size_t smem_max = 224 * 1024; // the kernel also holds a few KB of static shared memory
    // Default: no wide image -- the packed image alone lets two CTAs of 384 threads share an SM, and while one of them
    // flushes the other one accumulates.  EVB_Q2_WIDE=1: one CTA of 768 threads with the wide image.
    if (const char *e = getenv("EVB_Q2_WIDE")) g_q2_wide = atoi(e) != 0;
    g_q2_threads = g_q2_wide ? 768 : 384;
    const int t = nf % 16;
    const int nc_all = (nf + 15) / 16;
    // one group with the tail in xE if it fits
    g.ntail = 0;
    g.NC = 0;
    if (t >= 1 && t <= 4 && nf / 16 >= 1 && nf / 16 <= 6) {
        const int NC = nf / 16;
        if (q2_smem(B, NC, true) <= smem_max) { g.NC = NC; g.ngroups = 1; g.ntail = t; }
    }
    if (g.NC == 0) {
        // groups of equal chunk counts; the widest image that fits shared memory
        int ncmax = 8;
        while (ncmax > 1 && q2_smem(B, ncmax, false) > smem_max) ncmax >>= 1;
        if (q2_smem(B, ncmax, false) > smem_max) return EVB_ERR_LIMIT;
        g.ngroups = (nc_all + ncmax - 1) / ncmax;
        g.NC = (nc_all + g.ngroups - 1) / g.ngroups;
    }
    if (g.ngroups > 64) return EVB_ERR_LIMIT;
    if (const char *e = getenv("EVB_Q2_THREADS")) { const int want = atoi(e); if (want == 384 || want == 512 || want == 768 || want == 1024) g_q2_threads = want; }
    g.nmain = nf - g.ntail;
    g.RSH = g.ngroups * g.NC * 16;
    if ((unsigned long long)(h->n + 1) * g.RSH >= (1ull << 32)) return EVB_ERR_LIMIT; // 32-bit byte offsets into xH
    g.SC = (nf + 3) / 4 * 4;
    g.smem = q2_smem(B, g.NC, g.ntail > 0);
    const int occ = q2_dispatch(g.NC, g.ntail > 0, false, nullptr, dim3(), g.smem, 0);
    if (occ < 1) { evb_set_error("fixed-point histogram kernel cannot be resident (smem=%zu)", g.smem); return EVB_ERR_CUDA; }
    g.G = occ * h->num_sms;
    const int NW = g_q2_threads / 32;
    g.QB = 24;
    if (const char *e = getenv("EVB_Q2_QBITS")) { const int want = atoi(e); if (want == 24 || want == 26) g.QB = want; }
    const int max_epoch = g.QB == 26 ? Q2_MAX_EPOCH_26 : Q2_MAX_EPOCH_24;
    g.TE = max_epoch / NW * NW;
    if (const char *e = getenv("EVB_Q2_EPOCH")) { const int want = atoi(e); if (want >= 1 && want <= max_epoch) g.TE = want; }
    g.min_rows = 512; // measured: 100k x 10 rows 0.054 ms per tree at 512, 0.059 at 1024, 0.088 at 4096; no difference at 10M rows
    if (const char *e = getenv("EVB_Q2_MIN_ROWS")) { const int want = atoi(e); if (want >= 32) g.min_rows = want; }
    return EVB_OK;
}

// xH / xE from the feature-major matrix on the device (h->xC), once at create time
int32_t evb_q2_build_layout(evb_handle *h) {
    const Q2Geom &g = h->q2;
    EVB_CUDA(cudaMemsetAsync(h->xH, 0, (size_t)(h->n + 1) * g.RSH, h->st)); // row n: the all-zero row
    EVB_CUDA(cudaMemsetAsync(h->xE + h->n, 0, sizeof(uint2), h->st));
    EVB_CHECK(evb_launch_transpose(h, h->xC, h->n, h->n, 0, g.nmain, h->xH, g.RSH, h->st));
    k_q2_tail<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->xC, h->n, g.nmain, g.ntail, h->xE);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_q2_quantize(evb_handle *h) {
    evb_tic(h, EVB_T_GRADS);
    k_q2_quantize<<<(unsigned)((h->n + 255) / 256), 256, 0, h->st>>>(h->grad, h->GS, h->xE, h->n, h->d_gmax, h->d_qinv, h->q2.QB);
    evb_toc(h, EVB_T_GRADS);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

int32_t evb_launch_histq2(evb_handle *h, int level) {
    const Q2Geom &g = h->q2;
    Q2Args a;
    a.xH = h->xH; a.xE = h->xE; a.rows = h->rows[(level - 1) & 1];
    a.plan = h->plan + level; a.cum = h->cum; a.slot_node = h->slot_node; a.seg_start = h->seg_start;
    a.hsum = h->hsum_q; a.hcnt = h->hcnt_q;
    a.RSH = g.RSH; a.B = h->B; a.SC = g.SC; a.nmain = g.nmain; a.ntail = g.ntail; a.TE = g.TE; a.min_rows = g.min_rows; a.zrow = (uint32_t)h->n;
    a.LB = g.QB == 26 ? 8 : 6; a.CS = g.QB == 26 ? 20 : 19;
    a.wide = g_q2_wide ? 1 : 0;
    evb_tic(h, EVB_T_HIST);
    const cudaError_t e = (cudaError_t)q2_dispatch(g.NC, g.ntail > 0, true, &a, dim3(g.G, g.ngroups), g.smem, h->st);
    evb_toc(h, EVB_T_HIST);
    EVB_CUDA(e);
    return EVB_OK;
}

// The split scan reads the integer accumulators itself when nothing else needs the doubles: one GPU (no exchange of
// hcomp between ranks).  EVB_Q2_DIRECT=0 keeps the conversion kernel.
bool evb_q2_direct(const evb_handle *h) {
    static const bool off = getenv("EVB_Q2_DIRECT") != nullptr && atoi(getenv("EVB_Q2_DIRECT")) == 0;
    return h->use_q2 && h->world == 1 && !off;
}

// clears the accumulators of the level's build slots (after the scan has read them)
int32_t evb_launch_q2_clear(evb_handle *h, int level) {
    const Q2Geom &g = h->q2;
    const int slots = evb_level_slots(level);
    const size_t per_slot = (size_t)h->B * g.SC;
    size_t blocks = ((size_t)slots * per_slot + 255) / 256;
    if (blocks > (size_t)h->num_sms * 8) blocks = (size_t)h->num_sms * 8;
    evb_tic(h, EVB_T_HIST_REDUCE);
    k_q2_clear<<<(unsigned)blocks, 256, 0, h->st>>>(h->hsum_q, h->hcnt_q, h->plan + level, per_slot);
    evb_toc(h, EVB_T_HIST_REDUCE);
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}

// integer accumulators -> hcomp (doubles, the layout of the other histogram kernels), accumulators cleared
int32_t evb_launch_q2_reduce(evb_handle *h, int level) {
    const Q2Geom &g = h->q2;
    Q2ConvArgs a;
    a.hsum = h->hsum_q; a.hcnt = h->hcnt_q; a.hcomp = h->hcomp; a.plan = h->plan + level; a.js0 = h->js_d; a.qinv = h->d_qinv;
    a.B = h->B; a.SC = g.SC; a.F = h->F;
    const int slots = evb_level_slots(level);
    evb_tic(h, EVB_T_HIST_REDUCE);
    k_q2_to_hcomp<<<dim3(slots, (h->F + 31) / 32), 256, 0, h->st>>>(a);
    const size_t per_slot = (size_t)h->B * g.SC;
    size_t blocks = ((size_t)slots * per_slot + 255) / 256;
    if (blocks > (size_t)h->num_sms * 8) blocks = (size_t)h->num_sms * 8;
    k_q2_clear<<<(unsigned)blocks, 256, 0, h->st>>>(h->hsum_q, h->hcnt_q, h->plan + level, per_slot);
    evb_toc(h, EVB_T_HIST_REDUCE);
    h->tm.launches[EVB_T_HIST_REDUCE] += 1;
    EVB_CUDA(cudaGetLastError());
    return EVB_OK;
}
