// Q4_K dequant-fused GEMV / skinny GEMM for the verify rows of a speculative-decode pass.
//
// Replaces the reference's decode GEMVs: k_gemv_q8 / k_gemv_multi (engine/kernels/gemv.hip:291-367,1042-1067),
// the T-invariant production kernel k_gemv_wmma<Q4_K> (gemv.hip:602-672) and the f32-activation baseline
// k_gemv_q4_K_f32 (gemv.hip:1177-1216).
//
// Design (sm_100a). Weights stay in the 144-byte ggml Q4_K block format, [N][K/256] blocks, rows contiguous, and
// every weight byte is read from HBM once per launch. The launch is one persistent CTA per SM (148 CTAs x 12 warps).
// K is cut into P equal parts (P = 1, 2 or 4, a function of the tensor shape only, chosen so that the 16-row tiles
// divide evenly over the SMs); the 148/P CTAs of part p share the tiles evenly, and inside a CTA the stream of units
// (16 rows x 2 blocks, tile-major then along K) is divided evenly and contiguously over the 12 warps. Each warp runs
// its own ring of 1-D bulk async copies (cp.async.bulk + mbarrier; 16 row pieces of 288 B per stage in the ggml layout,
// one 4608-byte copy per stage in the engine's tile-major layout), unpacks the nibbles in registers and feeds the int8
// tensor-core tile mma.m16n8k32 (weights on M, verify rows on N = 8), which yields the exact int32 dot of every
// 32-element sub-block. The 6-bit scales of a lane's two rows are decoded in registers. The quantised activations of
// the CTA's K part are staged once per CTA in shared memory by bulk copies. One fp32 update per sub-block follows, in
// block order:
//     acc = fmaf((d*sc) * xd, (float)idot, acc);  acc = fmaf(-(dmin*mn), xs, acc);
// A tile whose blocks are spread over several warps of the CTA is finished through shared memory: the partial sums
// are added in warp order. Each K part writes its own output plane; the planes are added in part order by the
// consumer (or by the small reduction kernel of the public entry point). No atomics, no cross-CTA traffic.
// The partition is a function of (N, K) only, never of the number of verify rows, so a row of an n+1-row verify pass
// is bit-identical to the same row of a 1-row pass (the reference's "T-invariance", gemv.hip:600-601), and a CPU can
// reproduce the result bit for bit.
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

constexpr int SK_STAGES = GEMV_STAGES;
constexpr int SK_THREADS = GEMV_WARPS * 32;
constexpr int SK_XG = 4;   // copy pairs per column tile of the activations; NT * SK_XG <= 32
// Two weight layouts. Row-major ggml (TILED = false): a stage holds 16 row pieces of CB blocks, one bulk copy per row.
// Tile-major (TILED = true, the engine repacks to it at load; same bytes, permuted): for every 16-row tile and block a
// contiguous 2304-byte chunk = 16 headers (16 B each) + nibbles stored [j][lane][row g 8 B | row g+8 8 B], so a stage
// is ONE bulk copy and every lane fetches its two rows of a 64-element group with one 128-bit shared-memory load.
template <int CB, bool TILED> struct SkGeom {
    static constexpr int ROW_STRIDE = CB == 2 ? 288 : 160;   // 288 = 2*128+32, 160 = 128+32: rows land on distinct 32-byte bank groups
    static constexpr int STAGE_BYTES = TILED ? CB * 2304 : 16 * ROW_STRIDE;
    static constexpr int FIXED = GEMV_WARPS * SK_STAGES * STAGE_BYTES + 1024;
};

// XG: the activations are read from global memory (L2) inside the loop instead of being staged in shared memory: the
// form for several column tiles whose activations do not fit beside the rings (small matrices with a long K).
template <int NT, int CB, bool TILED, bool XG = false>
__global__ void __launch_bounds__(SK_THREADS, 1) k_gemv_q4k_sk(const uint8_t* __restrict__ W, const uint4* __restrict__ xq, const float4* __restrict__ xsc,
                                                                float* __restrict__ y, int N, int nb, int P, int R, int ldy, size_t part_stride,
                                                                int* __restrict__ err) {
    using Geo = SkGeom<CB, TILED>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring_all = smem;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + GEMV_WARPS * SK_STAGES * Geo::STAGE_BYTES);
    const int nbp = nb / P;                                // blocks of this CTA's K part
    const int xstride = XG ? nb : nbp;                     // blocks between two column tiles of the activations
    const uint4* xq_s = XG ? xq : reinterpret_cast<const uint4*>(smem + Geo::FIXED);
    const float4* xsc_s = XG ? xsc : reinterpret_cast<const float4*>(smem + Geo::FIXED + NT * nbp * 2048);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const GemvCta ct = gemv_cta(N, nb, P, blockIdx.x);
    const int C = nbp / CB, kb0 = ct.part * nbp;
    const int cu = (ct.t1 - ct.t0) * C;                    // units of this CTA
    const int weff = cu < GEMV_WARPS ? cu : GEMV_WARPS;
    const int u0 = warp < weff ? gemv_warp_start(cu, weff, warp) : 0, u1 = warp < weff ? gemv_warp_start(cu, weff, warp + 1) : 0;
    const int nunits = u1 - u0;
    uint8_t* ring = ring_all + warp * SK_STAGES * Geo::STAGE_BYTES;
    const uint32_t bar0 = smem_u32(&bars[warp * SK_STAGES]);
    const uint32_t xbar = smem_u32(&bars[GEMV_WARPS * SK_STAGES]);
    const uint32_t row_bytes = (uint32_t)nb * 144u;
    constexpr uint32_t unit_bytes = CB * 144u;
    y += (size_t)ct.part * part_stride;
    pdl_launch_dependents();   // the next kernel may be scheduled; it waits for this one to finish before using its output
    if (lane == 0) {
        for (int s = 0; s < SK_STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        if (warp == 0) mbar_init(xbar, 1);
        fence_barrier_init();
    }
    __syncthreads();

    // issue cursor (tile, chunk) of the next unit to fetch; advanced incrementally, no divisions in the loop
    const int first_tile = ct.t0 + (nunits ? u0 / C : 0);
    int it_tile = first_tile, it_chunk = nunits ? u0 % C : 0, it_i = 0;
    const uint8_t* it_src = TILED ? W + ((size_t)it_tile * nb + kb0 + it_chunk * CB) * 2304
                                  : W + ((size_t)it_tile * 16 + (lane & 15)) * row_bytes + (size_t)(kb0 + it_chunk * CB) * 144;
    const uint32_t ring_lane = smem_u32(ring) + (TILED ? 0 : (lane & 15) * Geo::ROW_STRIDE);
    auto issue = [&]() {
        const int s = it_i % SK_STAGES;
        const uint32_t bar = bar0 + 8 * s;
        if constexpr (TILED) {
            if (lane == 0) { mbar_expect_tx(bar, CB * 2304u); bulk_g2s(ring_lane + s * Geo::STAGE_BYTES, it_src, CB * 2304u, bar); }
            ++it_i; ++it_chunk; it_src += CB * 2304;
            if (it_chunk == C) { it_chunk = 0; ++it_tile; it_src += (size_t)(nb - C * CB) * 2304; }
        } else {
            const int nrows = min(16, N - it_tile * 16);
            if (lane == 0) mbar_expect_tx(bar, unit_bytes * (uint32_t)nrows);
            __syncwarp();
            if (lane < nrows) bulk_g2s(ring_lane + s * Geo::STAGE_BYTES, it_src, unit_bytes, bar);
            ++it_i; ++it_chunk; it_src += unit_bytes;
            if (it_chunk == C) { it_chunk = 0; ++it_tile; it_src += (size_t)16 * row_bytes - (size_t)C * unit_bytes; }
        }
    };
    // the weight stream does not depend on the previous kernel: prime the ring before waiting for it
    for (int i = 0; i < SK_STAGES && i < nunits; ++i) issue();

    pdl_wait();

    if (!XG && warp == 0) {   // quantised activations of blocks [kb0, kb0 + nbp), all NT column tiles, by bulk copies. Per column
        // tile the int8 fragments (2048 B per block) and the scales (512 B per block) of consecutive blocks are
        // contiguous. Issuing a bulk copy costs ~45 ns (one copy pair per block took 1.8 us), so each column tile is
        // fetched as SK_XG copy pairs over ranges of blocks, each CTA starting at a different range so that the 148 CTAs
        // do not walk the same L2 lines in lockstep.
        if (lane == 0) mbar_expect_tx(xbar, (uint32_t)NT * nbp * 2560u);
        __syncwarp();
        if (lane < NT * SK_XG) {
            const int n = lane / SK_XG, gx = (lane % SK_XG + blockIdx.x) % SK_XG;
            const int b0 = (gx * nbp) / SK_XG, b1 = ((gx + 1) * nbp) / SK_XG;
            if (b1 > b0) {
                bulk_g2s(smem_u32(smem + Geo::FIXED + (n * nbp + b0) * 2048), xq + ((size_t)n * nb + kb0 + b0) * 128, (uint32_t)(b1 - b0) * 2048u, xbar);
                bulk_g2s(smem_u32(smem + Geo::FIXED + NT * nbp * 2048 + (n * nbp + b0) * 512), xsc + ((size_t)n * nb + kb0 + b0) * 32, (uint32_t)(b1 - b0) * 512u, xbar);
            }
        }
    }

    float2 acc[NT][2];   // [n][0] = row g, cols 2t,2t+1 ; [n][1] = row g+8
    auto zero_acc = [&]() {
#pragma unroll
        for (int n = 0; n < NT; ++n) { acc[n][0] = make_float2(0.f, 0.f); acc[n][1] = make_float2(0.f, 0.f); }
    };
    zero_acc();
    auto store_tile = [&](int tile, const float (&v)[NT][4]) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int row = tile * 16 + g + ((k & 2) ? 8 : 0), col = n * 8 + 2 * t + (k & 1);
                if (row < N && col < R) y[(size_t)col * ldy + row] = v[n][k];
            }
    };
    // a tile covered by this warp alone is stored at once; otherwise the partial sum goes to shared memory
    // (slot 0 = the warp's first tile, slot 1 = its last tile) and is combined after the CTA barrier
    float* red = reinterpret_cast<float*>(ring_all);   // reused after every warp has drained its ring
    float part_v[2][NT][4]; bool part_on[2] = {false, false}; int part_tile[2] = {0, 0};
    auto flush = [&](int tile, bool whole) {
        float v[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) { v[n][0] = acc[n][0].x; v[n][1] = acc[n][0].y; v[n][2] = acc[n][1].x; v[n][3] = acc[n][1].y; }
        if (whole) { store_tile(tile, v); return; }
        const int slot = tile == first_tile ? 0 : 1;
        part_on[slot] = true; part_tile[slot] = tile;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) part_v[slot][n][k] = v[n][k];
    };

    // per-lane constant offsets
    const uint32_t w_lane = TILED ? 256 + lane * 16 : g * Geo::ROW_STRIDE + 16 + 8 * t;   // weights: row g (+8 rows: + 8*ROW_STRIDE)
    const uint32_t hdr_lane = TILED ? g * 16 : g * Geo::ROW_STRIDE;      // header of row g (+8 rows: + HDR8)
    constexpr int HDR8 = TILED ? 128 : 8 * Geo::ROW_STRIDE;
    constexpr int BLK_STRIDE = TILED ? 2304 : 144;

    int cur_tile = first_tile, chunk = nunits ? u0 % C : 0;
    bool cur_from_start = chunk == 0;
    bool ok = XG ? true : mbar_wait(xbar, 0, err);
    for (int i = 0; i < nunits && ok; ++i) {
        const int s = i % SK_STAGES;
        ok = mbar_wait(bar0 + 8 * s, (i / SK_STAGES) & 1, err);
        if (!ok) break;
        const uint8_t* st = ring + s * Geo::STAGE_BYTES;
        const uint4* xqp = xq_s + ((XG ? kb0 : 0) + chunk * CB) * 128 + lane;
        const float4* xsp = xsc_s + ((XG ? kb0 : 0) + chunk * CB) * 32 + t;
#pragma unroll
        for (int blk = 0; blk < CB; ++blk) {
            // Scales of this lane's two rows (g, g+8), decoded in registers from the 16-byte headers. A 6-bit value v
            // becomes the float 8388608 + v by a byte permute into the mantissa of 0x4B000000, and
            // fmaf(d, 8388608 + v, -(d * 8388608)) is exactly d * v (one rounding of an exactly representable
            // product). Odd sub-blocks take the high nibbles unshifted (16 * q): their d carries the exact 1/16.
            const RowScales ra = decode_scales(*reinterpret_cast<const uint4*>(st + hdr_lane + blk * BLK_STRIDE));
            const RowScales rb = decode_scales(*reinterpret_cast<const uint4*>(st + hdr_lane + HDR8 + blk * BLK_STRIDE));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint2 w0, w1;
                if constexpr (TILED) {
                    const uint4 ww = *reinterpret_cast<const uint4*>(st + w_lane + blk * 2304 + 512 * j);
                    w0 = make_uint2(ww.x, ww.y); w1 = make_uint2(ww.z, ww.w);
                } else {
                    w0 = *reinterpret_cast<const uint2*>(st + w_lane + blk * 144 + 32 * j);
                    w1 = *reinterpret_cast<const uint2*>(st + w_lane + 8 * Geo::ROW_STRIDE + blk * 144 + 32 * j);
                }
                const uint32_t alo[4] = {w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu};
                const uint32_t ahi[4] = {w0.x & 0xF0F0F0F0u, w1.x & 0xF0F0F0F0u, w0.y & 0xF0F0F0F0u, w1.y & 0xF0F0F0F0u};
                const float4 sa0 = ra.get(2 * j), sb0 = rb.get(2 * j);           // low-nibble sub-block: rows g, g+8
                const float4 sa1 = ra.get(2 * j + 1), sb1 = rb.get(2 * j + 1);   // high-nibble sub-block
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4* xfp = xqp + n * xstride * 128 + (blk * 4 + j) * 32;
                    const float4* x0p = xsp + n * xstride * 32 + (blk * 8 + 2 * j) * 4;
                    const uint4 xf = XG ? __ldcg(xfp) : *xfp;
                    const float4 x0 = XG ? __ldcg(x0p) : *x0p;
                    const float4 x1 = XG ? __ldcg(x0p + 4) : x0p[4];
                    // The accumulator input carries 0x4B400000: the int32 result, read as fp32, is 12582912 + idot
                    // exactly (|idot| < 2^22), so the int -> float conversion is one exact packed subtraction.
                    int c0[4], c1[4];
                    mma_u8s8_magic(c0, alo, xf.x, xf.y);
                    mma_u8s8_magic(c1, ahi, xf.z, xf.w);
                    const float2 xd0 = make_float2(x0.x, x0.y), xs0 = make_float2(x0.z, x0.w);
                    const float2 xd1 = make_float2(x1.x, x1.y), xs1 = make_float2(x1.z, x1.w);
                    const float2 mg = make_float2(-12582912.f, -12582912.f);
                    // low-nibble sub-block 2j, then high-nibble sub-block 2j+1 (block order)
                    fma2(acc[n][0], mul2(make_float2(sa0.x, sa0.y), xd0), add2(make_float2(__int_as_float(c0[0]), __int_as_float(c0[1])), mg));
                    fma2(acc[n][0], make_float2(sa0.z, sa0.w), xs0);
                    fma2(acc[n][1], mul2(make_float2(sb0.x, sb0.y), xd0), add2(make_float2(__int_as_float(c0[2]), __int_as_float(c0[3])), mg));
                    fma2(acc[n][1], make_float2(sb0.z, sb0.w), xs0);
                    fma2(acc[n][0], mul2(make_float2(sa1.x, sa1.y), xd1), add2(make_float2(__int_as_float(c1[0]), __int_as_float(c1[1])), mg));
                    fma2(acc[n][0], make_float2(sa1.z, sa1.w), xs1);
                    fma2(acc[n][1], mul2(make_float2(sb1.x, sb1.y), xd1), add2(make_float2(__int_as_float(c1[2]), __int_as_float(c1[3])), mg));
                    fma2(acc[n][1], make_float2(sb1.z, sb1.w), xs1);
                }
            }
        }
        __syncwarp();   // every lane has read the stage before it is refilled
        if (it_i < nunits) issue();
        if (++chunk == C) {
            flush(cur_tile, cur_from_start);
            zero_acc();
            chunk = 0; ++cur_tile; cur_from_start = true;
        } else if (i + 1 == nunits) {
            flush(cur_tile, false);
        }
    }
    // ---------------- tiles shared by several warps of this CTA: combine through shared memory in warp order
    __syncthreads();   // every ring is drained: its memory becomes the exchange buffer [warp][slot][NT*4][32]
#pragma unroll
    for (int sl = 0; sl < 2; ++sl)
        if (part_on[sl])
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int k = 0; k < 4; ++k) red[((warp * 2 + sl) * NT * 4 + n * 4 + k) * 32 + lane] = part_v[sl][n][k];
    __syncthreads();
    if (!ok) return;
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
        if (!part_on[sl]) continue;
        const int tile = part_tile[sl], tl = tile - ct.t0;
        if ((tl + 1) * C > u1) continue;                     // the tile ends in a later warp: that warp finishes it
        const int w_first = gemv_warp_owner(cu, weff, tl * C);
        // exchange-buffer rows of the contributors (slot 0 when the tile is the contributor's first tile)
        int src[GEMV_WARPS];
#pragma unroll
        for (int ww = 0; ww < GEMV_WARPS; ++ww)
            src[ww] = (ww >= w_first && ww <= warp) ? (ww * 2 + ((gemv_warp_start(cu, weff, ww) / C == tl) ? 0 : 1)) * NT * 4 : -1;
        float v[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a = 0.f;
#pragma unroll
                for (int ww = 0; ww < GEMV_WARPS; ++ww)
                    if (src[ww] >= 0) {
                        const float pv = red[(src[ww] + n * 4 + k) * 32 + lane];
                        a = ww == w_first ? pv : a + pv;
                    }
                v[n][k] = a;
            }
        store_tile(tile, v);
    }
}

// ---- f32-activation GEMV (the arithmetic of the reference's k_gemv_q4_K_f32, gemv.hip:1177-1216, kept as a numerics
// contract: four partial sums per output row, partial l over blocks l, l+4, ... in order; per 64-element group
// t = d0*s0 - m0*sx0 + d1*s1 - m1*sx1 with s = fmaf chain over the 32 elements and sx = their serial sum; the four
// partials combined by the xor tree 2, 1). Structure for sm_100a: one CTA per 32 output rows, thread = (row, partial);
// the 32 row pieces of a 4-block K chunk and the matching activations arrive by bulk async copies into a 2-stage
// shared-memory ring (HBM sees 576-byte coalesced row pieces instead of per-thread 16-byte loads strided by the row
// size), activation blocks padded to 260 floats so that the four partials of a row read distinct banks, and the
// weight-independent sums sx computed once per chunk for all rows. ----
constexpr int F32_ROWS = 32, F32_THREADS = 128, F32_XPAD = 260, F32_CHUNK = 4;
template <int NCOL>
__global__ void __launch_bounds__(F32_THREADS) k_gemv_q4k_f32(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int N, int K, int* __restrict__ err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* wst = smem;                                                          // [2][32 rows][4 blocks * 144]
    float* xst = reinterpret_cast<float*>(smem + 2 * F32_ROWS * F32_CHUNK * 144);  // [2][NCOL][4][260]
    float* sxs = xst + 2 * NCOL * F32_CHUNK * F32_XPAD;                           // [NCOL][4 blocks * 8 sub-blocks]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sxs + NCOL * 32);
    const int tid = threadIdx.x, r = tid >> 2, l = tid & 3;
    const int nb = K / 256, nch = (nb + F32_CHUNK - 1) / F32_CHUNK, row0 = blockIdx.x * F32_ROWS, nrows = min(F32_ROWS, N - row0);
    const uint32_t bar0 = smem_u32(bars);
    if (tid == 0) { mbar_init(bar0, 1); mbar_init(bar0 + 8, 1); fence_barrier_init(); }
    __syncthreads();
    auto issue = [&](int ci) {   // warp 0: one copy per row piece, one per (column, block) of activations
        if (tid >= 32) return;
        const int s = ci & 1, b0 = ci * F32_CHUNK, cb = min(F32_CHUNK, nb - b0);
        const uint32_t bar = bar0 + 8 * s;
        if (tid == 0) mbar_expect_tx(bar, (uint32_t)(nrows * cb * 144 + NCOL * cb * 1024));
        __syncwarp();
        if (tid < nrows) bulk_g2s(smem_u32(wst + (s * F32_ROWS + tid) * F32_CHUNK * 144), W + ((size_t)(row0 + tid) * nb + b0) * 144, (uint32_t)cb * 144u, bar);
        for (int i = tid; i < NCOL * cb; i += 32) {
            const int c = i / cb, bl = i - c * cb;
            bulk_g2s(smem_u32(xst + ((s * NCOL + c) * F32_CHUNK + bl) * F32_XPAD), x + (size_t)c * K + (size_t)(b0 + bl) * 256, 1024u, bar);
        }
    };
    float acc[NCOL];
#pragma unroll
    for (int c = 0; c < NCOL; ++c) acc[c] = 0.f;
    issue(0);
    if (nch > 1) issue(1);
    bool ok = true;
    for (int ci = 0; ci < nch; ++ci) {
        const int s = ci & 1, cb = min(F32_CHUNK, nb - ci * F32_CHUNK);
        ok = __syncthreads_and(mbar_wait(bar0 + 8 * s, (ci >> 1) & 1, err) ? 1 : 0) != 0;
        if (!ok) break;
        for (int i = tid; i < NCOL * cb * 8; i += F32_THREADS) {   // sx of (column, block, sub-block): serial sum in element order
            const int c = i / (cb * 8), rem = i - c * (cb * 8), bl = rem >> 3, k = rem & 7;
            const float* xp = xst + ((s * NCOL + c) * F32_CHUNK + bl) * F32_XPAD + 32 * k;
            float a = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) a = a + xp[e];
            sxs[c * 32 + bl * 8 + k] = a;
        }
        __syncthreads();
        if (r < nrows && l < cb) {
            const uint8_t* blk = wst + (s * F32_ROWS + r) * F32_CHUNK * 144 + l * 144;
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
            const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t sc0, mn0, sc1, mn1; q4k_scale_min(hdr, 2 * j, sc0, mn0); q4k_scale_min(hdr, 2 * j + 1, sc1, mn1);
                const float d0 = d * (float)sc0, m0 = dmin * (float)mn0, d1 = d * (float)sc1, m1 = dmin * (float)mn1;
                const uint4 qa = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j), qb = *reinterpret_cast<const uint4*>(blk + 32 + 32 * j);
                const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    const float* xc = xst + ((s * NCOL + c) * F32_CHUNK + l) * F32_XPAD + 64 * j;
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int e4 = 0; e4 < 8; ++e4) {
                        const float4 x0 = *reinterpret_cast<const float4*>(xc + 4 * e4), x1 = *reinterpret_cast<const float4*>(xc + 32 + 4 * e4);
                        const uint32_t q = qw[e4];
                        s0 = fmaf(x0.x, (float)(q & 0xFu), s0); s1 = fmaf(x1.x, (float)((q >> 4) & 0xFu), s1);
                        s0 = fmaf(x0.y, (float)((q >> 8) & 0xFu), s0); s1 = fmaf(x1.y, (float)((q >> 12) & 0xFu), s1);
                        s0 = fmaf(x0.z, (float)((q >> 16) & 0xFu), s0); s1 = fmaf(x1.z, (float)((q >> 20) & 0xFu), s1);
                        s0 = fmaf(x0.w, (float)((q >> 24) & 0xFu), s0); s1 = fmaf(x1.w, (float)(q >> 28), s1);
                    }
                    const float sx0 = sxs[c * 32 + l * 8 + 2 * j], sx1 = sxs[c * 32 + l * 8 + 2 * j + 1];
                    float tt = d0 * s0; tt = tt - m0 * sx0; tt = tt + d1 * s1; tt = tt - m1 * sx1;
                    acc[c] = acc[c] + tt;
                }
            }
        }
        __syncthreads();   // the stage and sxs are free again
        if (ci + 2 < nch) issue(ci + 2);
    }
    if (!ok) return;
#pragma unroll
    for (int c = 0; c < NCOL; ++c) {
        acc[c] = acc[c] + __shfl_xor_sync(0xffffffffu, acc[c], 2);
        acc[c] = acc[c] + __shfl_xor_sync(0xffffffffu, acc[c], 1);
        if (l == 0 && r < nrows) y[(size_t)c * N + row0 + r] = acc[c];
    }
}

template <int NT, int CB, bool TILED, bool XG = false>
int launch_sk2(const uint8_t* W, const void* xq, const void* xsc, float* y, int N, int nb, int P, int R, int ldy, size_t part_stride,
               int* err, cudaStream_t s, bool pdl) {
    const size_t smem = SkGeom<CB, TILED>::FIXED + (XG ? 0 : (size_t)NT * (nb / P) * 2560);
    static size_t attr_smem[MAX_DEVICES] = {};   // per device: the opt-in belongs to the device's copy of the kernel
    const int dev = current_device(); if (dev < 0) return HP_ECUDA;
    if (smem > attr_smem[dev]) { HP_CUDA(cudaFuncSetAttribute(k_gemv_q4k_sk<NT, CB, TILED, XG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_smem[dev] = smem; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(GEMV_NCTA); cfg.blockDim = dim3(SK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl && !(pdl_off_mask(s) & 64) ? 1 : 0;
    HP_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_q4k_sk<NT, CB, TILED, XG>, W, (const uint4*)xq, (const float4*)xsc, y, N, nb, P, R, ldy, part_stride, err));
    return HP_OK;
}
template <int NT, bool XG = false>
int launch_sk(const uint8_t* W, bool tiled, const void* xq, const void* xsc, float* y, int N, int nb, int P, int R, int ldy, size_t part_stride,
              int* err, cudaStream_t s, bool pdl) {
    const bool cb2 = (nb / P) % 2 == 0;
    if (tiled) return cb2 ? launch_sk2<NT, 2, true, XG>(W, xq, xsc, y, N, nb, P, R, ldy, part_stride, err, s, pdl)
                          : launch_sk2<NT, 1, true, XG>(W, xq, xsc, y, N, nb, P, R, ldy, part_stride, err, s, pdl);
    return cb2 ? launch_sk2<NT, 2, false, XG>(W, xq, xsc, y, N, nb, P, R, ldy, part_stride, err, s, pdl)
               : launch_sk2<NT, 1, false, XG>(W, xq, xsc, y, N, nb, P, R, ldy, part_stride, err, s, pdl);
}

// row-major ggml blocks -> tile-major chunks (see SkGeom); rows beyond N are zero (they contribute nothing).
// half > 0: the tensor is a stack of matrices of 2 * half rows (gate rows then up rows of an expert); tile q of a matrix
// then holds gate rows 8q..8q+7 followed by up rows 8q..8q+7, so that one lane of the tensor-core tile owns gate and up
// of the same feature.
__global__ void __launch_bounds__(256) k_repack_tiled(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int nb, int half) {
    const size_t chunk = blockIdx.x;                       // (tile, block)
    const int tile = (int)(chunk / nb), b = (int)(chunk % nb);
    uint8_t* out = dst + chunk * 2304;
    for (int i = threadIdx.x; i < 2304 / 4; i += 256) {    // one 32-bit word per step
        const int o = i * 4; uint32_t v = 0;
        int row, off;                                      // source row in the tile and byte offset in its 144-byte block
        if (o < 256) { row = o / 16; off = o % 16; }
        else { const int q = o - 256, j = q / 512, lane = (q % 512) / 16, w = q % 16, g = lane >> 2, t = lane & 3; row = g + (w >= 8 ? 8 : 0); off = 16 + 32 * j + 8 * t + (w & 7); }
        int r = tile * 16 + row;
        if (half > 0) { const int tpe = half / 8, eb = tile / tpe, q = tile % tpe; r = eb * 2 * half + (row < 8 ? 8 * q + row : half + 8 * q + row - 8); }
        if (r < N) v = *reinterpret_cast<const uint32_t*>(src + ((size_t)r * nb + b) * 144 + off);
        *reinterpret_cast<uint32_t*>(out + o) = v;
    }
}

// sum the K-part planes in part order: y[r][n] = ((p0 + p1) + p2) + p3
__global__ void k_reduce_parts(const float* __restrict__ parts, size_t part_stride, int P, float* __restrict__ y, int N, int R, int ldp, int ldy) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (n >= N || r >= R) return;
    float v = parts[(size_t)r * ldp + n];
    for (int p = 1; p < P; ++p) v = v + parts[(size_t)p * part_stride + (size_t)r * ldp + n];
    y[(size_t)r * ldy + n] = v;
}

}  // namespace

int gemv_parts(int N, int K) { return gemv_num_parts(N, K / 256); }

size_t gemv_tiled_bytes(size_t N, int K) { return ((N + 15) / 16) * (size_t)(K / 256) * 2304; }
int gemv_repack_tiled(const void* src, void* dst, size_t N, int K, cudaStream_t s, int interleave_half) {
    HP_REQUIRE(N > 0 && N < ((size_t)1 << 31) && K > 0 && K % 256 == 0, "gemv_repack_tiled: bad shape");
    HP_REQUIRE(interleave_half == 0 || (interleave_half % 8 == 0 && N % (2 * (size_t)interleave_half) == 0), "gemv_repack_tiled: the gate|up interleave needs stacks of 2 * half rows, half a multiple of 8");
    k_repack_tiled<<<(unsigned)(((N + 15) / 16) * (K / 256)), 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, (int)N, K / 256, interleave_half);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

int gemv_q4k_q8_parts(const void* W, const XQ8F& x, float* yparts, int N, int K, int R, int ldy, size_t part_stride, int* err, cudaStream_t s, bool pdl, bool tiled) {
    HP_REQUIRE(K > 0 && K % 256 == 0, "gemv_q4k_q8: K=%d must be a positive multiple of 256", K);
    HP_REQUIRE(N > 0 && R >= 1 && R <= 32 && ldy >= N, "gemv_q4k_q8: bad shape N=%d R=%d ldy=%d", N, R, ldy);
    const int nb = K / 256, P = gemv_num_parts(N, nb);
    HP_REQUIRE(P > 0, "gemv_q4k_q8: K=%d is too large for the activation staging buffer", K);
    const int ntile = (R + 7) / 8, nbp = nb / P;
    // all column tiles in one launch: their activations staged in shared memory beside the rings when they fit, read
    // from L2 inside the loop otherwise (small matrices with a long K: one launch instead of one per tile of 8 columns;
    // same per-column arithmetic either way)
    const bool staged = ntile == 1 || (size_t)SkGeom<2, false>::FIXED + (size_t)ntile * nbp * 2560 <= (size_t)GEMV_SMEM_LIMIT;
    const uint8_t* w = (const uint8_t*)W;
    int rc;
    if (staged) {
        switch (ntile) {
            case 1: rc = launch_sk<1>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
            case 2: rc = launch_sk<2>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
            case 3: rc = launch_sk<3>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
            default: rc = launch_sk<4>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
        }
    } else {
        switch (ntile) {
            case 2: rc = launch_sk<2, true>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
            case 3: rc = launch_sk<3, true>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
            default: rc = launch_sk<4, true>(w, tiled, x.q, x.sc, yparts, N, nb, P, R, ldy, part_stride, err, s, pdl); break;
        }
    }
    if (rc != HP_OK) return rc;
    return HP_OK;
}

int gemv_q4k_q8(const void* W, const XQ8F& x, float* y, int N, int K, int R, int ldy, const GemvWorkspace& ws, cudaStream_t s, bool pdl) {
    HP_REQUIRE(K > 0 && K % 256 == 0 && N > 0, "gemv_q4k_q8: bad shape N=%d K=%d", N, K);
    const int P = gemv_num_parts(N, K / 256);
    if (P == 1) return gemv_q4k_q8_parts(W, x, y, N, K, R, ldy, 0, ws.err, s, pdl, false);
    HP_REQUIRE(ws.part && (size_t)P * R * N * sizeof(float) <= ws.part_bytes, "gemv_q4k_q8: workspace too small for %d K-part planes of %d x %d", P, R, N);
    const size_t stride = (size_t)R * N;
    const int rc = gemv_q4k_q8_parts(W, x, ws.part, N, K, R, N, stride, ws.err, s, pdl, false);
    if (rc != HP_OK) return rc;
    k_reduce_parts<<<dim3((N + 255) / 256, R), 256, 0, s>>>(ws.part, stride, P, y, N, R, N, ldy);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}

template <int NCOL>
static int launch_f32(const uint8_t* W, const float* x, float* y, int N, int K, int* err, cudaStream_t s) {
    const size_t smem = (size_t)2 * F32_ROWS * F32_CHUNK * 144 + (size_t)2 * NCOL * F32_CHUNK * F32_XPAD * 4 + (size_t)NCOL * 32 * 4 + 16;
    static bool attr[MAX_DEVICES] = {};
    const int dev = current_device(); if (dev < 0) return HP_ECUDA;
    if (!attr[dev]) { HP_CUDA(cudaFuncSetAttribute(k_gemv_q4k_f32<NCOL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[dev] = true; }
    k_gemv_q4k_f32<NCOL><<<(N + F32_ROWS - 1) / F32_ROWS, F32_THREADS, smem, s>>>(W, x, y, N, K, err);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int gemv_q4k_f32(const void* W, const float* x, float* y, int N, int K, int R, int* err, cudaStream_t s) {
    HP_REQUIRE(K > 0 && K % 256 == 0, "gemv_q4k_f32: K=%d must be a positive multiple of 256", K);
    HP_REQUIRE(N > 0 && R >= 1 && R <= 8, "gemv_q4k_f32: bad shape N=%d R=%d (R <= 8)", N, R);
    HP_REQUIRE(((uintptr_t)x & 15) == 0, "gemv_q4k_f32: activations must be 16-byte aligned");
    const uint8_t* w = (const uint8_t*)W;
    switch (R) {
        case 1: return launch_f32<1>(w, x, y, N, K, err, s); case 2: return launch_f32<2>(w, x, y, N, K, err, s);
        case 3: return launch_f32<3>(w, x, y, N, K, err, s); case 4: return launch_f32<4>(w, x, y, N, K, err, s);
        case 5: return launch_f32<5>(w, x, y, N, K, err, s); case 6: return launch_f32<6>(w, x, y, N, K, err, s);
        case 7: return launch_f32<7>(w, x, y, N, K, err, s); default: return launch_f32<8>(w, x, y, N, K, err, s);
    }
}

}  // namespace hp
