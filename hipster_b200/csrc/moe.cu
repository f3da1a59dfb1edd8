// Mixture-of-experts FFN of the Flash-Next-shaped model: exact f32 router GEMV, softmax top-k routing with a shared
// expert slot, grouped routed-expert GEMV (gate|up), SiLU-gated product + quantisation per (row, slot), and the
// down-projection with the in-order weighted combine (no atomics: deterministic and independent of the row count).
//
// Reference: k_f32_gemv (engine/kernels/fn.hip:252-266), k_moe_route (fn.hip:167-205), k_moe_silu_quant (fn.hip:206-211),
// k_gemv_moe / k_gemv_moe_down (engine/kernels/gemv.hip:1075-1129), Qwen4Exp::moe_layer (engine/src/qwen4exp.cpp:345-354).
//
// Expert GEMV numerics: exact int32 dot per 32-element sub-block (int8 tensor-core tile), one fp32 update per sub-block,
// blocks in order along K, no split: acc = fmaf((d*sc)*xd, idot, acc); acc = fmaf(-(dmin*mn), xs, acc).
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

// ---- router + routing + grouping in ONE launch ------------------------------------------------------------------------
// Phase 1, router (exact f32; reference k_f32_gemv, fn.hip:252-266): per (weight row n, pass row t) lane l takes
// k = 4l + 128 i as float4, four fmaf per step in element order, then the xor-shuffle tree 16..1; a warp computes two
// weight rows against four pass rows at once. Phase 2, in the CTA that finishes last (ticket counter), routing (k_moe_route,
// fn.hip:167-205), two warps per row: softmax over the first E logits (sum: xor tree inside each group of 32 experts, the
// group sums added in group order), top-k by (value desc, index asc), weights renormalised by the sum of the selected
// probabilities taken in rank order; slot k = shared expert, id -1, weight sigmoid(logit[E]). Phase 3, same CTA: the
// (row, slot) pairs are grouped by expert into segments of up to 8 pairs (see below).
// synth_key != 0: the E expert logits fed to the softmax are seeded N(0, 1) draws keyed by (layer key, slot, token,
// position, expert) instead of the GEMV's (benchmark input control: with random-init weights every row's hidden state is
// nearly the same vector, so a linear router would send all rows to the same experts); the shared expert's gate keeps its logit.
struct MoeSeg { int expert, ncols, cols[8]; int pad[6]; };   // 64 bytes; cols = pair indices t * nslot + e
__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) { if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
__device__ __forceinline__ void row_barrier(int row) { asm volatile("bar.sync %0, 64;" ::"r"(row + 1) : "memory"); }   // the two warps of a row
struct RouteArgs {
    const float* W; const float* x; float* y; int N, K, T;       // router [N = E + 1][K], rows x [T][K], logits y [T][N]
    int* ids; float* w; int E, k;                                 // outputs [T][k + 1]
    int* ticket;                                                  // five zero-initialised ints (left zero)
    const int* row_tok; const int* row_pos; const int* row_slot; unsigned long long synth_key;
    int e_lo, e_hi, own_shared; MoeSeg* segs; int* ctl; unsigned long long* touched;   // grouping (segs == nullptr: skipped)
    int stage_w, stage_x; int* err;                               // router rows / pass rows staged in shared memory; status word for the bounded waits
};
constexpr int RG_THREADS = 512;
constexpr int RG_ROUTE_SMEM = 8 * 1024 * 4;   // routing scratch: the probabilities of 8 rows x up to 1024 experts
__global__ void __launch_bounds__(RG_THREADS) k_route_group(RouteArgs a) {
    pdl_launch_dependents();
    __shared__ int scnt[1026]; __shared__ int soff[1026]; __shared__ int swt[RG_THREADS / 32]; __shared__ int s_last;
    __shared__ __align__(8) unsigned long long wbar, xbar;
    __shared__ float s_max[8][2], s_gsum[8][32], s_sel[8][16]; __shared__ uint32_t s_ck[8][32]; __shared__ int s_ci[8][32];
    // dynamic shared memory: the CTA's 16 router rows [16][K] f32 (a.stage_w), then its 8 pass rows [8][K] f32 (a.stage_x);
    // the routing phase reuses the front of it
    extern __shared__ __align__(128) uint8_t rg_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Router GEMV: CTA (bx, by) covers weight rows 16 bx .. 16 bx + 15 for pass rows 8 by .. 8 by + 7; warp w takes the
    // weight rows 2 (w & 7), +1 against the pass rows 4 (w >> 3) .. +3. Spreading the 2 N T K fmaf over ~100 CTAs keeps
    // the load pipes of any one SM out of the critical path. The 16 weight rows do not depend on the previous kernel:
    // they are fetched by bulk async copies before the dependency wait; the pass rows by bulk copies right after it,
    // all at once, instead of one dependent L2 round trip per 128 columns.
    const float* wsm = reinterpret_cast<const float*>(rg_smem);
    const float* xsm = reinterpret_cast<const float*>(rg_smem + (size_t)16 * a.K * 4);
    const uint32_t wb = smem_u32(&wbar), xb = smem_u32(&xbar);
    if (a.stage_w) {
        if (tid == 0) { mbar_init(wb, 1); mbar_init(xb, 1); fence_barrier_init(); }
        __syncthreads();
        if (warp == 0) {
            const int nrow = min(16, a.N - (int)blockIdx.x * 16);
            if (lane == 0) mbar_expect_tx(wb, (uint32_t)nrow * (uint32_t)a.K * 4u);
            __syncwarp();
            if (lane < nrow) bulk_g2s(smem_u32(rg_smem + (size_t)lane * a.K * 4), a.W + (size_t)(blockIdx.x * 16 + lane) * a.K, (uint32_t)a.K * 4u, wb);
        }
    }
    pdl_wait();
    if (a.stage_x && warp == 0) {
        const int nrow = min(8, a.T - (int)blockIdx.y * 8);
        if (lane == 0) mbar_expect_tx(xb, (uint32_t)nrow * (uint32_t)a.K * 4u);
        __syncwarp();
        if (lane < nrow) bulk_g2s(smem_u32(xsm + (size_t)lane * a.K), a.x + (size_t)(blockIdx.y * 8 + lane) * a.K, (uint32_t)a.K * 4u, xb);
    }
    // the routing phase's row key does not depend on the logits: fetched here, under the copies of the pass rows
    const int row = warp >> 1, sub = warp & 1, t = blockIdx.y * 8 + row;   // routing: two warps per row, half of the expert groups each
    unsigned long long base = 0ull;   // synthetic logits: rnd64(key + slot, (token, position), expert) = splitmix64(base + expert)
    if (a.synth_key && t < a.T) base = splitmix64((a.synth_key + (unsigned long long)a.row_slot[t]) ^ ((((unsigned long long)(unsigned)a.row_tok[t] << 32) | (unsigned)a.row_pos[t]) * 0x9E3779B97F4A7C15ull));
    {
        const int n0 = blockIdx.x * 16 + 2 * (warp & 7), q0 = 4 * (warp >> 3), t0 = blockIdx.y * 8 + q0;
        const bool live0 = n0 < a.N, live1 = n0 + 1 < a.N;
        bool ok = true;
        const float* wr0; const float* wr1;
        if (a.stage_w) { ok = mbar_wait(wb, 0, a.err); wr0 = wsm + (size_t)(2 * (warp & 7)) * a.K; wr1 = wsm + (size_t)(live1 ? 2 * (warp & 7) + 1 : 2 * (warp & 7)) * a.K; }
        else { wr0 = a.W + (size_t)(live0 ? n0 : 0) * a.K; wr1 = a.W + (size_t)(live1 ? n0 + 1 : 0) * a.K; }
        if (a.stage_x) ok = mbar_wait(xb, 0, a.err) && ok;
        const float* xr = a.stage_x ? xsm + (size_t)q0 * a.K : a.x + (size_t)t0 * a.K;
        float acc0[4], acc1[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc0[q] = 0.f; acc1[q] = 0.f; }
        if (ok && live0 && t0 < a.T) {
#pragma unroll 2
            for (int i = lane * 4; i < a.K; i += 128) {
                const float4 w0 = *reinterpret_cast<const float4*>(wr0 + i), w1 = *reinterpret_cast<const float4*>(wr1 + i);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (t0 + q < a.T) {
                        const float4 xv = *reinterpret_cast<const float4*>(xr + (size_t)q * a.K + i);
                        acc0[q] = fmaf(w0.x, xv.x, acc0[q]); acc0[q] = fmaf(w0.y, xv.y, acc0[q]); acc0[q] = fmaf(w0.z, xv.z, acc0[q]); acc0[q] = fmaf(w0.w, xv.w, acc0[q]);
                        acc1[q] = fmaf(w1.x, xv.x, acc1[q]); acc1[q] = fmaf(w1.y, xv.y, acc1[q]); acc1[q] = fmaf(w1.z, xv.z, acc1[q]); acc1[q] = fmaf(w1.w, xv.w, acc1[q]);
                    }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) { acc0[q] = acc0[q] + __shfl_xor_sync(0xffffffffu, acc0[q], off); acc1[q] = acc1[q] + __shfl_xor_sync(0xffffffffu, acc1[q], off); }
            if (lane == 0 && t0 + q < a.T) {
                if (live0) a.y[(size_t)(t0 + q) * a.N + n0] = acc0[q];
                if (live1) a.y[(size_t)(t0 + q) * a.N + n0 + 1] = acc1[q];
            }
        }
    }
    // ---- routing of the 8 rows of group `by`, by the CTA that completes their logits last (ticket per group), so that
    // the groups are routed on different SMs at the same time: warps 2 r and 2 r + 1 route row 8 by + r. This code runs once per
    // launch on an SM that has not executed it before, so it is written for a small instruction footprint (rolled loops
    // over values kept in shared memory): unrolled over 32 register values it was bound by instruction fetch.
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.ticket + blockIdx.y, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int ns = a.k + 1;
    if (t < a.T) {
        const float* lg = a.y + (size_t)t * a.N;
        const float shared_logit = __ldcg(lg + a.E);
        float* sv = reinterpret_cast<float*>(rg_smem) + row * 1024;   // lane l owns the entries l + 32 q of its warp's groups
        uint32_t* sk = reinterpret_cast<uint32_t*>(sv);
        const int nq = (a.E + 31) >> 5, hq = (nq + 1) >> 1, qa = sub * hq, qb = min(nq, qa + hq);
        float mx = -INFINITY;
#pragma unroll 4
        for (int q = qa; q < qb; ++q) {
            const int i = 32 * q + lane;
            const float val = i < a.E ? (a.synth_key ? irwin(splitmix64(base + (uint64_t)i)) : __ldcg(lg + i)) : -INFINITY;
            sv[i] = val; mx = fmaxf(mx, val);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) s_max[row][sub] = mx;
        row_barrier(row);
        mx = fmaxf(s_max[row][0], s_max[row][1]);
        // softmax denominator: xor tree inside each group of 32 experts, the group sums added in group order
#pragma unroll 4
        for (int q = qa; q < qb; ++q) {
            const int i = 32 * q + lane;
            const float pr = i < a.E ? expf_det(sv[i] - mx) : 0.f;
            sv[i] = pr;
            float sg = pr;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sg = sg + __shfl_xor_sync(0xffffffffu, sg, off);
            if (lane == 0) s_gsum[row][q] = sg;
        }
        row_barrier(row);
        float sum = s_gsum[row][0];
        for (int q = 1; q < nq; ++q) sum = sum + s_gsum[row][q];
        // Selection keys: a probability is a non-negative float, so its bit pattern orders like an unsigned integer;
        // key = bits + 1, 0 = no entry (padding, or already taken). The warp's own k best by (key desc, index asc): one
        // integer max and one integer min across the warp per winner; every global winner is among the 2 k candidates.
        uint32_t lk = 0u; int li = 0x7fffffff;
#pragma unroll 4
        for (int q = qa; q < qb; ++q) {
            const int i = 32 * q + lane;
            const uint32_t key = i < a.E ? __float_as_uint(sv[i] / sum) + 1u : 0u;
            sk[i] = key;
            if (key > lk) { lk = key; li = i; }
        }
        uint32_t myk = 0u; int myi = 0x7fffffff;
        for (int r = 0; r < a.k; ++r) {
            const uint32_t m = __reduce_max_sync(0xffffffffu, lk);
            const int wi = (int)__reduce_min_sync(0xffffffffu, lk == m ? (uint32_t)li : 0x7fffffffu);
            if (lane == r) { myk = m; myi = wi; }
            if (m != 0u && (wi & 31) == lane) {   // the owner retires the entry and looks for its next best
                sk[wi] = 0u; lk = 0u; li = 0x7fffffff;
#pragma unroll 4
                for (int q = qa; q < qb; ++q) { const uint32_t key = sk[32 * q + lane]; if (key > lk) { lk = key; li = 32 * q + lane; } }
            }
        }
        if (lane < a.k) { s_ck[row][16 * sub + lane] = myk; s_ci[row][16 * sub + lane] = myi; }
        row_barrier(row);
        if (sub == 0) {
            // merge by rank: candidate c is the winner number (count of candidates that beat it)
            const bool valid = lane < 2 * a.k;
            const int slot = lane < a.k ? lane : 16 + lane - a.k;
            const uint32_t ck = valid ? s_ck[row][slot] : 0u; const int ci = valid ? s_ci[row][slot] : 0x7fffffff;
            int rank = 0;
            for (int j = 0; j < 2 * a.k; ++j) {
                const int sj = j < a.k ? j : 16 + j - a.k;
                const uint32_t kj = s_ck[row][sj]; const int ij = s_ci[row][sj];
                rank += (kj > ck || (kj == ck && ij < ci)) ? 1 : 0;
            }
            if (ck != 0u && rank < a.k) { a.ids[t * ns + rank] = ci; s_sel[row][rank] = __uint_as_float(ck - 1u); }
            __syncwarp();
            float wsum = s_sel[row][0];   // the selected probabilities added in rank order
            for (int r = 1; r < a.k; ++r) wsum = wsum + s_sel[row][r];
            if (lane < a.k) a.w[t * ns + lane] = s_sel[row][lane] / wsum;
            if (lane == 0) { a.ids[t * ns + a.k] = -1; a.w[t * ns + a.k] = sigmoid_det(shared_logit); }
        }
    }
    if (tid == 0) a.ticket[blockIdx.y] = 0;   // ready for the next launch
    if (!a.segs) return;
    // ---- grouping, by the CTA that routes last (second-level ticket): bucket b = expert e_lo + b (b < nown), then the
    // shared expert; segments in bucket order, the pairs of a bucket in increasing pair index
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.ticket + 4, 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int nown = a.e_hi - a.e_lo, nb = nown + (a.own_shared ? 1 : 0), np = a.T * ns;
    // scnt[b] = bit mask of the rows that picked bucket b (a row picks an expert at most once, T <= 32): a pair's place in
    // its bucket is the number of lower rows in the mask
    for (int b = tid; b < 1026; b += RG_THREADS) scnt[b] = 0;
    __syncthreads();
    int my_b = -1, my_rank = 0, my_id = 0;
    if (tid < np) {
        my_id = __ldcg(a.ids + tid);
        my_b = my_id >= 0 ? ((my_id >= a.e_lo && my_id < a.e_hi) ? my_id - a.e_lo : -1) : (a.own_shared ? nown : -1);
        if (my_b >= 0) atomicOr(reinterpret_cast<unsigned*>(&scnt[my_b]), 1u << (tid / ns));
    }
    __syncthreads();
    if (my_b >= 0) my_rank = __popc((unsigned)scnt[my_b] & ((1u << (tid / ns)) - 1u));
    {   // exclusive scan of the segments per bucket: thread = buckets 2 tid and 2 tid + 1 (0..1023), bucket 1024 appended
        const int b0 = 2 * tid, c0 = b0 < nb ? (__popc((unsigned)scnt[b0]) + 7) >> 3 : 0, c1 = b0 + 1 < nb ? (__popc((unsigned)scnt[b0 + 1]) + 7) >> 3 : 0;
        int inc = c0 + c1;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const int o = __shfl_up_sync(0xffffffffu, inc, off); if (lane >= off) inc += o; }
        if (lane == 31) swt[warp] = inc;
        const int ntouch = __syncthreads_count(b0 < nb && scnt[b0] != 0) + __syncthreads_count(b0 + 1 < nb && scnt[b0 + 1] != 0);
        if (warp == 0) {
            int wv = lane < RG_THREADS / 32 ? swt[lane] : 0, winc = wv;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) { const int o = __shfl_up_sync(0xffffffffu, winc, off); if (lane >= off) winc += o; }
            if (lane < RG_THREADS / 32) swt[lane] = winc - wv;   // exclusive offset of each warp
        }
        __syncthreads();
        const int ex = swt[warp] + inc - (c0 + c1);
        soff[b0] = ex; soff[b0 + 1] = ex + c0;
        if (tid == RG_THREADS - 1) {
            const int tot1024 = ex + c0 + c1;
            soff[1024] = tot1024;
            const int c2 = nb > 1024 ? (__popc((unsigned)scnt[1024]) + 7) >> 3 : 0;
            a.ctl[0] = tot1024 + c2; a.ctl[1] = 0; a.ctl[2] = 0;   // segments, ticket counters of the two GEMVs
            if (a.touched) atomicAdd(a.touched, (unsigned long long)(ntouch + (nb > 1024 && scnt[1024] != 0 ? 1 : 0)));
            a.ticket[4] = 0;
        }
    }
    __syncthreads();
    if (my_b >= 0) {
        MoeSeg* sg = a.segs + soff[my_b] + (my_rank >> 3); const int c = my_rank & 7;
        sg->cols[c] = tid;
        if (c == 0) sg->expert = my_id;
        if (c == 7 || my_rank == __popc((unsigned)scnt[my_b]) - 1) sg->ncols = c + 1;
    }
}

// ---- routed-expert GEMVs, grouped by expert -------------------------------------------------------------------------
// After routing, the (row, slot) pairs of a pass are grouped by expert: one SEGMENT per touched expert this GPU owns
// (and one for the shared expert), holding up to 8 pairs as the columns of the tensor-core tile; an expert with more
// than 8 pairs gets several segments. Every touched expert matrix is therefore streamed from HBM once per pass for all
// the rows that routed to it (once per 8 of them). Work unit = (segment, 4 consecutive 16-row tiles); warps take units
// from a global ticket counter (which warp computes a unit has no influence on the result: a unit is computed by one
// warp alone, blocks in order along K, no split), and stream their tiles through a private ring of bulk async copies.
// Expert tensors are kept tile-major (the layout of gemv_q4k.cu: per (16-row tile, block) 2304 contiguous bytes); the
// gate|up tensor is repacked with gate rows 8q..8q+7 and up rows 8q..8q+7 sharing tile q, so that a lane holds gate
// and up of the same feature and the SiLU-gated product and its int8 quantisation (fn.hip:206-211) finish in registers:
// a unit's 4 tiles are exactly one 32-feature quantisation group.
constexpr int MOE_UNIT_TILES = 4;
// Ring geometry (warps per CTA x stages per warp), chosen by the number of rows of the pass: the shared memory of an SM
// buys either many warps with a short ring (many units: throughput) or few warps with a long one (few units, e.g. the
// 3 rows of a single-slot verify pass: each busy warp must keep enough bytes in flight by itself to hide the DRAM latency).

struct MoeGArgs {
    const uint8_t* w_exp; const uint8_t* w_sh;     // tile-major expert tensors: this GPU's experts [e_hi - e_lo][tiles][nb] chunks, and the shared expert's
    int e_lo, tiles, nb;                            // tiles of 16 rows per expert, blocks per row
    const MoeSeg* segs; int* ctl; int ticket;      // ticket counter index in ctl (1 = gate|up, 2 = down)
    const uint8_t* xq; const float* xsc; int xK, xdiv;   // activations: fragment-major rows of xK elements; row of pair p = p / xdiv
    float* y; int N;                                // MODE 1: y[pair][N]
    int8_t* oq; float* osc; int F;                  // MODE 0: quantised silu(gate) * up per pair, F features
    int* err;
    int ep_world, ep_rank; float* ep_x[8]; unsigned* ep_ctl[8]; size_t ep_half;   // MODE 1 of the quad form: peers to deliver y to (ep_world <= 1: none)
};
// MODE 0: gate|up with the fused SiLU-gated product + quantisation; MODE 1: down projection (per-pair f32 outputs)
template <int MODE, int SB, int MOE_WARPS, int MOE_DEPTH>
__global__ void __launch_bounds__(MOE_WARPS * 32, 1) k_moe_gemv_grouped(MoeGArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int STAGE = SB * 2304;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint8_t* ring = smem + warp * MOE_DEPTH * STAGE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + MOE_WARPS * MOE_DEPTH * STAGE);
    const uint32_t bar0 = smem_u32(&bars[warp * MOE_DEPTH]);
    pdl_launch_dependents();
    if (lane == 0) { for (int s = 0; s < MOE_DEPTH; ++s) mbar_init(bar0 + 8 * s, 1); fence_barrier_init(); }
    __syncwarp();
    pdl_wait();
    const int spt = a.nb / SB;                                 // stages per tile
    const int ups = a.tiles / MOE_UNIT_TILES, total = a.ctl[0] * ups, spu = MOE_UNIT_TILES * spt;   // units per segment, units, stages per unit
    auto grab = [&]() { int u = 0; if (lane == 0) u = atomicAdd(a.ctl + a.ticket, 1); return __shfl_sync(0xffffffffu, u, 0); };
    auto unit_base = [&](int u) -> const uint8_t* {           // first chunk of the unit's first tile
        const MoeSeg& sg = a.segs[u / ups];
        const uint8_t* w = sg.expert >= 0 ? a.w_exp + (size_t)(sg.expert - a.e_lo) * a.tiles * a.nb * 2304 : a.w_sh;
        return w + (size_t)(u % ups) * MOE_UNIT_TILES * a.nb * 2304;
    };
    // issue cursor: unit iu, stage is (0..spu) of it; the copies of a unit are consecutive in memory (4 tiles x nb chunks).
    // It runs MOE_DEPTH stages ahead of the compute cursor, i.e. up to MOE_DEPTH / spu + 1 units ahead: the units it has
    // moved on to wait in a short queue (q0 = next to compute) until the compute cursor reaches them.
    int iu = grab(), is = 0, icount = 0; const uint8_t* isrc = iu < total ? unit_base(iu) : nullptr;
    int q0 = -1, q1 = -1, q2 = -1, q3 = -1, qn = 0;
    auto issue = [&]() {
        if (iu >= total) return;
        const uint32_t bar = bar0 + 8 * (icount % MOE_DEPTH);
        if (lane == 0) { mbar_expect_tx(bar, STAGE); bulk_g2s(smem_u32(ring + (icount % MOE_DEPTH) * STAGE), isrc, STAGE, bar); }
        ++icount; isrc += STAGE;
        if (++is == spu) {
            is = 0; iu = grab(); isrc = iu < total ? unit_base(iu) : nullptr;
            if (qn == 0) q0 = iu; else if (qn == 1) q1 = iu; else if (qn == 2) q2 = iu; else q3 = iu;
            ++qn;
        }
    };
    int cu = iu;
    for (int i = 0; i < MOE_DEPTH; ++i) issue();
    int ccount = 0; bool ok = true;
    while (cu < total && ok) {
        const MoeSeg sg = a.segs[cu / ups];
        // this lane's columns: B fragments of column g, scales of columns 2t and 2t + 1
        const int rg = g < sg.ncols ? sg.cols[g] / a.xdiv : -1;
        const int c0 = 2 * t < sg.ncols ? sg.cols[2 * t] : -1, c1 = 2 * t + 1 < sg.ncols ? sg.cols[2 * t + 1] : -1;
        const int r0 = c0 >= 0 ? c0 / a.xdiv : -1, r1 = c1 >= 0 ? c1 / a.xdiv : -1;
        const uint4* xq_g = rg >= 0 ? reinterpret_cast<const uint4*>(a.xq) + ((size_t)(rg >> 3) * (a.xK >> 6)) * 32 + ((rg & 7) * 4 + t) : nullptr;
        const float* xs0 = r0 >= 0 ? a.xsc + xq_d_index(r0, 0, a.xK) : nullptr;
        const float* xs1 = r1 >= 0 ? a.xsc + xq_d_index(r1, 0, a.xK) : nullptr;
        float act[MOE_UNIT_TILES][2];
        for (int ti = 0; ti < MOE_UNIT_TILES && ok; ++ti) {
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
            for (int st = 0; st < spt && ok; ++st) {
                const int s = ccount % MOE_DEPTH;
                ok = mbar_wait(bar0 + 8 * s, (ccount / MOE_DEPTH) & 1, a.err);
                if (!ok) break;
                const uint8_t* sp = ring + s * STAGE;
#pragma unroll
                for (int blk = 0; blk < SB; ++blk) {
                    const int b = st * SB + blk;
                    const RowScales ra = decode_scales(*reinterpret_cast<const uint4*>(sp + g * 16 + blk * 2304));
                    const RowScales rb = decode_scales(*reinterpret_cast<const uint4*>(sp + g * 16 + 128 + blk * 2304));
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 ww = *reinterpret_cast<const uint4*>(sp + 256 + lane * 16 + blk * 2304 + 512 * j);
                        const uint32_t alo[4] = {ww.x & 0x0F0F0F0Fu, ww.z & 0x0F0F0F0Fu, ww.y & 0x0F0F0F0Fu, ww.w & 0x0F0F0F0Fu};
                        const uint32_t ahi[4] = {ww.x & 0xF0F0F0F0u, ww.z & 0xF0F0F0F0u, ww.y & 0xF0F0F0F0u, ww.w & 0xF0F0F0F0u};
                        const float4 sa0 = ra.get(2 * j), sb0 = rb.get(2 * j), sa1 = ra.get(2 * j + 1), sb1 = rb.get(2 * j + 1);
                        const uint4 xf = xq_g ? __ldg(xq_g + (size_t)(b * 4 + j) * 32) : make_uint4(0, 0, 0, 0);
                        // scales {d, s} of sub-blocks 2j (low nibbles) and 2j + 1 (high nibbles) for this lane's two columns
                        const int sb = b * 8 + 2 * j;
                        float2 xd0 = make_float2(0.f, 0.f), xs0v = xd0, xd1 = xd0, xs1v = xd0;
                        if (xs0) { xd0.x = __ldg(xs0 + sb * 16); xs0v.x = __ldg(xs0 + sb * 16 + 2); xd1.x = __ldg(xs0 + (sb + 1) * 16); xs1v.x = __ldg(xs0 + (sb + 1) * 16 + 2); }
                        if (xs1) { xd0.y = __ldg(xs1 + sb * 16); xs0v.y = __ldg(xs1 + sb * 16 + 2); xd1.y = __ldg(xs1 + (sb + 1) * 16); xs1v.y = __ldg(xs1 + (sb + 1) * 16 + 2); }
                        int m0[4], m1[4];
                        mma_u8s8_magic(m0, alo, xf.x, xf.y);
                        mma_u8s8_magic(m1, ahi, xf.z, xf.w);
                        const float2 mg = make_float2(-12582912.f, -12582912.f);
                        fma2(acc0, mul2(make_float2(sa0.x, sa0.y), xd0), add2(make_float2(__int_as_float(m0[0]), __int_as_float(m0[1])), mg));
                        fma2(acc0, make_float2(sa0.z, sa0.w), xs0v);
                        fma2(acc1, mul2(make_float2(sb0.x, sb0.y), xd0), add2(make_float2(__int_as_float(m0[2]), __int_as_float(m0[3])), mg));
                        fma2(acc1, make_float2(sb0.z, sb0.w), xs0v);
                        fma2(acc0, mul2(make_float2(sa1.x, sa1.y), xd1), add2(make_float2(__int_as_float(m1[0]), __int_as_float(m1[1])), mg));
                        fma2(acc0, make_float2(sa1.z, sa1.w), xs1v);
                        fma2(acc1, mul2(make_float2(sb1.x, sb1.y), xd1), add2(make_float2(__int_as_float(m1[2]), __int_as_float(m1[3])), mg));
                        fma2(acc1, make_float2(sb1.z, sb1.w), xs1v);
                    }
                }
                __syncwarp();   // every lane has read the stage before it is refilled
                ++ccount;
                issue();
            }
            if (!ok) break;
            const int tile = (cu % ups) * MOE_UNIT_TILES + ti;
            if constexpr (MODE == 1) {
                if (c0 >= 0) { a.y[(size_t)c0 * a.N + tile * 16 + g] = acc0.x; a.y[(size_t)c0 * a.N + tile * 16 + g + 8] = acc1.x; }
                if (c1 >= 0) { a.y[(size_t)c1 * a.N + tile * 16 + g] = acc0.y; a.y[(size_t)c1 * a.N + tile * 16 + g + 8] = acc1.y; }
            } else {   // rows g = gate of feature 8 * tile + g, rows g + 8 = up of the same feature
                act[ti][0] = silu_det(acc0.x) * acc1.x; act[ti][1] = silu_det(acc0.y) * acc1.y;
            }
        }
        if (!ok) break;
        if constexpr (MODE == 0) {
            // quantise the unit's 32 features (8 * ti + g over the 4 tiles and the 8 lanes that share t) per column:
            // amax / 127, q = rint(v * (127 / amax)), s = d * sum(q) (gemv.hip:36-51)
            const int sbk = cu % ups;                           // 32-feature sub-block of the F features
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float amax = 0.f;
#pragma unroll
                for (int ti = 0; ti < MOE_UNIT_TILES; ++ti) amax = fmaxf(amax, fabsf(act[ti][c]));
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                const float dd = amax / 127.f, id = amax > 0.f ? 127.f / amax : 0.f;
                int q[MOE_UNIT_TILES], sum = 0;
#pragma unroll
                for (int ti = 0; ti < MOE_UNIT_TILES; ++ti) { q[ti] = __float2int_rn(act[ti][c] * id); sum += q[ti]; }
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                const int pair = c ? c1 : c0;
                if (pair >= 0) {
#pragma unroll
                    for (int ti = 0; ti < MOE_UNIT_TILES; ++ti) a.oq[xq_q_index(pair, sbk * 32 + 8 * ti + g, a.F)] = (int8_t)q[ti];
                    if (g == 0) { const size_t di = xq_d_index(pair, sbk, a.F); a.osc[di] = dd; a.osc[di + 2] = dd * (float)sum; }
                }
            }
        }
        cu = q0; q0 = q1; q1 = q2; q2 = q3; q3 = -1; --qn;   // the next unit is the oldest one the issue cursor moved on to
    }
}

// ---- the same GEMVs with the work cut by quads of warps ------------------------------------------------------------
// A CTA is three quads of four warps. A quad owns a contiguous range of work units (segment, 4 tiles), i.e. mostly one
// or two segments: it gathers the segment's <= 8 activation columns ONCE into shared memory in the layout of the dense
// kernel (so a lane fetches its int8 fragment and its columns' scales with three 128-bit shared loads per 64 weights
// instead of nine global loads), and its warps take one tile of every unit each (warp w: tile w), streamed through a
// private ring. A warp's pipeline thus runs over ~7 tiles per launch instead of ~1.75 four-tile units, which removes
// the quantisation of the launch time to whole units. MODE 0: the 32-feature quantisation group spans the quad's four
// tiles: amax (a maximum) and the integer sum of the quantised values go through shared memory between two quad
// barriers. Per output element the arithmetic is unchanged: one warp, blocks in order along K, no split.
constexpr int MQ_WARPS = 12, MQ_QUADS = 3, MQ_AUX = 2048;   // bytes after the rings: barriers + the quads' exchange words
__device__ __forceinline__ void quad_barrier(int quad) { asm volatile("bar.sync %0, 128;" ::"r"(quad + 1) : "memory"); }
template <int MODE, int SB, int DEPTH>
__global__ void __launch_bounds__(MQ_WARPS * 32, 1) k_moe_gemv_quad(MoeGArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int STAGE = SB * 2304;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, quad = warp >> 2, w4 = warp & 3, qtid = threadIdx.x & 127;
    uint8_t* ring = smem + warp * DEPTH * STAGE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + MQ_WARPS * DEPTH * STAGE);
    float* ex_amax = reinterpret_cast<float*>(smem + MQ_WARPS * DEPTH * STAGE + 1024) + quad * 32;   // [warp of the quad][t * 2 + c]
    int* ex_sum = reinterpret_cast<int*>(smem + MQ_WARPS * DEPTH * STAGE + 1536) + quad * 32;
    uint8_t* xbuf = smem + MQ_WARPS * DEPTH * STAGE + MQ_AUX + (size_t)quad * a.nb * 2560;          // int8 fragments [nb][2048], then scales [nb][512]
    uint4* xq_s = reinterpret_cast<uint4*>(xbuf);
    float* xsc_s = reinterpret_cast<float*>(xbuf + (size_t)a.nb * 2048);
    const uint32_t bar0 = smem_u32(&bars[warp * DEPTH]);
    pdl_launch_dependents();
    if (lane == 0) { for (int s = 0; s < DEPTH; ++s) mbar_init(bar0 + 8 * s, 1); fence_barrier_init(); }
    __syncwarp();
    pdl_wait();
    const int spt = a.nb / SB, ups = a.tiles / MOE_UNIT_TILES;   // stages per tile, units per segment
    // expert parallelism: number of the exchange this launch feeds, and the half of the peers' buffers it goes to
    unsigned ep_e = 0u; size_t ep_off = 0;
    if constexpr (MODE == 1) { if (a.ep_world > 1) { ep_e = __ldcg(a.ep_ctl[a.ep_rank] + 8) + 1u; ep_off = (size_t)(ep_e & 1u) * a.ep_half; } }
    const int total = a.ctl[0] * ups, nquads = (int)gridDim.x * MQ_QUADS, gq = (int)blockIdx.x * MQ_QUADS + quad;
    const int u_lo = (int)((long long)gq * total / nquads), u_hi = (int)((long long)(gq + 1) * total / nquads);
    const size_t tile_bytes = (size_t)a.nb * 2304;
    auto seg_weights = [&](int seg) -> const uint8_t* {
        const int e = __ldcg(&a.segs[seg].expert);
        return e >= 0 ? a.w_exp + (size_t)(e - a.e_lo) * a.tiles * tile_bytes : a.w_sh;
    };
    // issue cursor: unit iu (segment iseg, unit i_us of it), stage ist of this warp's tile of the unit
    int iu = u_lo, iseg = u_lo < u_hi ? u_lo / ups : 0, i_us = u_lo < u_hi ? u_lo % ups : 0, ist = 0, icount = 0;
    const uint8_t* ibase = u_lo < u_hi ? seg_weights(iseg) : nullptr;
    const uint8_t* isrc = ibase ? ibase + (size_t)(i_us * MOE_UNIT_TILES + w4) * tile_bytes : nullptr;
    bool ok = true;
    auto issue = [&]() {
        if (iu >= u_hi || !ok) return;
        const uint32_t bar = bar0 + 8 * (icount % DEPTH);
        if (lane == 0) { mbar_expect_tx(bar, STAGE); bulk_g2s(smem_u32(ring + (icount % DEPTH) * STAGE), isrc, STAGE, bar); }
        ++icount; isrc += STAGE;
        if (++ist == spt) {
            ist = 0; ++iu;
            if (iu < u_hi) {
                if (++i_us == ups) { i_us = 0; ++iseg; ibase = seg_weights(iseg); }
                isrc = ibase + (size_t)(i_us * MOE_UNIT_TILES + w4) * tile_bytes;
            }
        }
    };
    for (int i = 0; i < DEPTH; ++i) issue();
    int cseg = u_lo < u_hi ? u_lo / ups : 0, c_us = u_lo < u_hi ? u_lo % ups : 0, staged = -1, ccount = 0;
    int c0 = -1, c1 = -1;   // pair indices of this lane's columns 2t, 2t + 1
    const uint4* xq4 = reinterpret_cast<const uint4*>(a.xq);
    const int nsb = a.xK >> 5, nk64 = a.xK >> 6;
    for (int cu = u_lo; cu < u_hi; ++cu) {
        if (cseg != staged) {
            // gather the segment's columns: fragment (k block of 64, column gg, quarter tt) and scales (sub-block, column)
            quad_barrier(quad);   // everybody has finished with the previous segment's activations
            const MoeSeg* sg = a.segs + cseg;
            const int ncols = __ldcg(&sg->ncols);
            {   // a thread's column and quarter are the same for all its items (the items are 128 apart): the column's row
                // is looked up once, and the item loads are independent of each other (one L2 round trip, not one per item)
                const int gg = (qtid & 31) >> 2, tt = qtid & 3;
                const int r = gg < ncols ? __ldcg(&sg->cols[gg]) / a.xdiv : -1;
                const uint4* src = r >= 0 ? xq4 + (size_t)(r >> 3) * nk64 * 32 + (r & 7) * 4 + tt : nullptr;
#pragma unroll 8
                for (int kb = qtid >> 5; kb < nk64; kb += 4) xq_s[kb * 32 + (qtid & 31)] = src ? __ldcg(src + (size_t)kb * 32) : make_uint4(0u, 0u, 0u, 0u);
                const int w = qtid & 15, gs = (w >> 2) * 2 + (w & 1), is_s = (w >> 1) & 1;
                const int rs = gs < ncols ? __ldcg(&sg->cols[gs]) / a.xdiv : -1;
                const float* ssrc = rs >= 0 ? a.xsc + (size_t)(rs >> 3) * nsb * 16 + ((rs & 7) >> 1) * 4 + (rs & 1) + 2 * is_s : nullptr;
#pragma unroll 8
                for (int sb = qtid >> 4; sb < nsb; sb += 8) xsc_s[sb * 16 + w] = ssrc ? __ldcg(ssrc + (size_t)sb * 16) : 0.f;
            }
            c0 = 2 * t < ncols ? __ldcg(&sg->cols[2 * t]) : -1; c1 = 2 * t + 1 < ncols ? __ldcg(&sg->cols[2 * t + 1]) : -1;
            staged = cseg;
            quad_barrier(quad);
        }
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
        for (int st = 0; st < spt; ++st) {
            const int s = ccount % DEPTH;
            if (ok) ok = mbar_wait(bar0 + 8 * s, (ccount / DEPTH) & 1, a.err);
            if (ok) {
                const uint8_t* sp = ring + s * STAGE;
#pragma unroll
                for (int blk = 0; blk < SB; ++blk) {
                    const int b = st * SB + blk;
                    const RowScales ra = decode_scales(*reinterpret_cast<const uint4*>(sp + g * 16 + blk * 2304));
                    const RowScales rb = decode_scales(*reinterpret_cast<const uint4*>(sp + g * 16 + 128 + blk * 2304));
                    const uint4* xqp = xq_s + (size_t)b * 128 + lane;
                    const float4* xsp = reinterpret_cast<const float4*>(xsc_s) + (size_t)b * 32 + t;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 ww = *reinterpret_cast<const uint4*>(sp + 256 + lane * 16 + blk * 2304 + 512 * j);
                        const uint32_t alo[4] = {ww.x & 0x0F0F0F0Fu, ww.z & 0x0F0F0F0Fu, ww.y & 0x0F0F0F0Fu, ww.w & 0x0F0F0F0Fu};
                        const uint32_t ahi[4] = {ww.x & 0xF0F0F0F0u, ww.z & 0xF0F0F0F0u, ww.y & 0xF0F0F0F0u, ww.w & 0xF0F0F0F0u};
                        const float4 sa0 = ra.get(2 * j), sb0 = rb.get(2 * j), sa1 = ra.get(2 * j + 1), sb1 = rb.get(2 * j + 1);
                        const uint4 xf = xqp[j * 32];
                        const float4 x0 = xsp[(2 * j) * 4], x1 = xsp[(2 * j + 1) * 4];
                        const float2 xd0 = make_float2(x0.x, x0.y), xs0v = make_float2(x0.z, x0.w), xd1 = make_float2(x1.x, x1.y), xs1v = make_float2(x1.z, x1.w);
                        int m0[4], m1[4];
                        mma_u8s8_magic(m0, alo, xf.x, xf.y);
                        mma_u8s8_magic(m1, ahi, xf.z, xf.w);
                        const float2 mg = make_float2(-12582912.f, -12582912.f);
                        fma2(acc0, mul2(make_float2(sa0.x, sa0.y), xd0), add2(make_float2(__int_as_float(m0[0]), __int_as_float(m0[1])), mg));
                        fma2(acc0, make_float2(sa0.z, sa0.w), xs0v);
                        fma2(acc1, mul2(make_float2(sb0.x, sb0.y), xd0), add2(make_float2(__int_as_float(m0[2]), __int_as_float(m0[3])), mg));
                        fma2(acc1, make_float2(sb0.z, sb0.w), xs0v);
                        fma2(acc0, mul2(make_float2(sa1.x, sa1.y), xd1), add2(make_float2(__int_as_float(m1[0]), __int_as_float(m1[1])), mg));
                        fma2(acc0, make_float2(sa1.z, sa1.w), xs1v);
                        fma2(acc1, mul2(make_float2(sb1.x, sb1.y), xd1), add2(make_float2(__int_as_float(m1[2]), __int_as_float(m1[3])), mg));
                        fma2(acc1, make_float2(sb1.z, sb1.w), xs1v);
                    }
                }
            }
            __syncwarp();   // every lane has read the stage before it is refilled
            ++ccount;
            issue();
        }
        const int tile = c_us * MOE_UNIT_TILES + w4;
        if constexpr (MODE == 1) {
            if (ok) {
                if (c0 >= 0) { a.y[(size_t)c0 * a.N + tile * 16 + g] = acc0.x; a.y[(size_t)c0 * a.N + tile * 16 + g + 8] = acc1.x; }
                if (c1 >= 0) { a.y[(size_t)c1 * a.N + tile * 16 + g] = acc0.y; a.y[(size_t)c1 * a.N + tile * 16 + g + 8] = acc1.y; }
                // the same values into every other rank's exchange buffer: the transfer rides on the stores, tile by tile
                // (the 8 lanes that share t write 32 consecutive bytes of a pair's row)
                for (int q = 0; q < a.ep_world; ++q) {
                    if (a.ep_world <= 1 || q == a.ep_rank) continue;
                    float* py = a.ep_x[q] + ep_off;
                    if (c0 >= 0) { py[(size_t)c0 * a.N + tile * 16 + g] = acc0.x; py[(size_t)c0 * a.N + tile * 16 + g + 8] = acc1.x; }
                    if (c1 >= 0) { py[(size_t)c1 * a.N + tile * 16 + g] = acc0.y; py[(size_t)c1 * a.N + tile * 16 + g + 8] = acc1.y; }
                }
            }
        } else {
            // rows g = gate of feature 8 * tile + g, rows g + 8 = up of the same feature; the unit's 4 tiles (this quad's 4
            // warps) are one 32-feature quantisation group per column: amax / 127, q = rint(v * (127 / amax)),
            // s = d * sum(q) (gemv.hip:36-51)
            const float act[2] = {silu_det(acc0.x) * acc1.x, silu_det(acc0.y) * acc1.y};
            float am[2] = {fabsf(act[0]), fabsf(act[1])};
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) { am[0] = fmaxf(am[0], __shfl_xor_sync(0xffffffffu, am[0], off)); am[1] = fmaxf(am[1], __shfl_xor_sync(0xffffffffu, am[1], off)); }
            if (g == 0) { ex_amax[w4 * 8 + t * 2] = am[0]; ex_amax[w4 * 8 + t * 2 + 1] = am[1]; }
            quad_barrier(quad);
            int qs[2]; float dd[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float amax = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) amax = fmaxf(amax, ex_amax[w * 8 + t * 2 + c]);
                dd[c] = amax / 127.f;
                const float id = amax > 0.f ? 127.f / amax : 0.f;
                const int q = __float2int_rn(act[c] * id);
                int sum = q;
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                qs[c] = sum;
                const int pair = c ? c1 : c0;
                if (pair >= 0 && ok) a.oq[xq_q_index(pair, c_us * 32 + 8 * w4 + g, a.F)] = (int8_t)q;
            }
            if (g == 0) { ex_sum[w4 * 8 + t * 2] = qs[0]; ex_sum[w4 * 8 + t * 2 + 1] = qs[1]; }
            quad_barrier(quad);
            if (w4 == 0 && g == 0 && ok) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int pair = c ? c1 : c0;
                    if (pair >= 0) {
                        const int sum = ex_sum[t * 2 + c] + ex_sum[8 + t * 2 + c] + ex_sum[16 + t * 2 + c] + ex_sum[24 + t * 2 + c];
                        const size_t di = xq_d_index(pair, c_us, a.F); a.osc[di] = dd[c]; a.osc[di + 2] = dd[c] * (float)sum;
                    }
                }
            }
        }
        if (++c_us == ups) { c_us = 0; ++cseg; }
    }
    if constexpr (MODE == 1) {
        if (a.ep_world > 1) {   // every CTA's deliveries are visible system-wide before the last one raises this rank's flag on the peers
            unsigned* ctl = a.ep_ctl[a.ep_rank];
            __threadfence_system();
            __syncthreads();
            if (threadIdx.x == 0 && atomicAdd(ctl + 9, 1u) == gridDim.x - 1) {
                __threadfence_system();
                for (int q = 0; q < a.ep_world; ++q)
                    if (q != a.ep_rank) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.ep_ctl[q] + a.ep_rank), "r"(ep_e) : "memory");
                ctl[9] = 0u; __threadfence();
                atomicExch(ctl + 8, ep_e);
            }
        }
    }
}

// in-order weighted combine of the per-(row, slot) expert outputs (gemv.hip:1104-1112); used by the kernel-level entry
// point (inside the engine the combine runs in the norm kernel that follows)
__global__ void __launch_bounds__(256) k_moe_combine(const float* __restrict__ v, const float* __restrict__ slotw, float* __restrict__ y, int nslot, int E) {
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x; if (i >= E) return;
    float acc = 0.f;
    for (int e = 0; e < nslot; ++e) acc = fmaf(slotw[t * nslot + e], v[(size_t)(t * nslot + e) * E + i], acc);
    y[(size_t)t * E + i] = acc;
}

}  // namespace

int moe_route_group(const MoeRouteParams& p, cudaStream_t s) {
    HP_REQUIRE(p.E >= 1 && p.E <= 1024 && p.k >= 1 && p.k <= 15 && p.k <= p.E && p.K > 0 && p.K % 128 == 0 && p.T >= 1 && p.T <= 32 && p.ticket, "moe_route_group: bad shape E=%d K=%d k=%d T=%d", p.E, p.K, p.k, p.T);
    HP_REQUIRE(p.synth_key == 0 || (p.row_tok && p.row_pos && p.row_slot), "moe_route_group: synthetic logits need the rows' tokens, positions and slots");
    HP_REQUIRE(!p.segs || (p.ctl && p.T * (p.k + 1) <= MOE_MAX_PAIRS && p.e_lo >= 0 && p.e_hi <= p.E && p.e_lo <= p.e_hi), "moe_route_group: bad grouping arguments");
    RouteArgs a; a.W = p.W; a.x = p.x; a.y = p.logits; a.N = p.E + 1; a.K = p.K; a.T = p.T; a.ids = p.ids; a.w = p.w; a.E = p.E; a.k = p.k; a.ticket = p.ticket;
    a.row_tok = p.row_tok; a.row_pos = p.row_pos; a.row_slot = p.row_slot; a.synth_key = p.synth_key;
    a.e_lo = p.e_lo; a.e_hi = p.e_hi; a.own_shared = p.own_shared; a.segs = (MoeSeg*)p.segs; a.ctl = p.ctl; a.touched = p.touched;
    // the CTA's 16 router rows are staged in shared memory when they fit (K <= 3072 floats per row), its 8 pass rows too
    // when both fit (K <= 2176); the routing phase needs RG_ROUTE_SMEM bytes of the same buffer
    const size_t wbytes = (size_t)16 * a.K * 4, xbytes = (size_t)8 * a.K * 4;
    a.stage_w = wbytes <= 192 * 1024 && ((uintptr_t)a.W & 15) == 0 ? 1 : 0;
    a.stage_x = a.stage_w && wbytes + xbytes <= 204 * 1024 && ((uintptr_t)a.x & 15) == 0 ? 1 : 0; a.err = p.err;
    size_t smem = a.stage_w ? wbytes + (a.stage_x ? xbytes : 0) : 0;
    if (smem < (size_t)RG_ROUTE_SMEM) smem = RG_ROUTE_SMEM;
    if (smem > 32 * 1024) {   // the kernel also has ~12 KB of static shared memory: opt in above 48 KB in total
        static size_t attr[MAX_DEVICES] = {};
        const int dev = current_device(); if (dev < 0) return HP_ECUDA;
        if (smem > attr[dev]) { HP_CUDA(cudaFuncSetAttribute(k_route_group, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[dev] = smem; }
    }
    HP_CUDA(launch_pdl<8>(k_route_group, dim3((a.N + 15) / 16, (a.T + 7) / 8), dim3(RG_THREADS), smem, s, a));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
size_t moe_seg_bytes() { return (size_t)MOE_MAX_PAIRS * sizeof(MoeSeg); }
template <int MODE, int SB, int WARPS, int DEPTH>
static int launch_grouped(const MoeGArgs& a, cudaStream_t s) {
    const size_t smem = (size_t)WARPS * DEPTH * SB * 2304 + WARPS * DEPTH * 8;
    static bool attr[MAX_DEVICES] = {};
    const int dev = current_device(); if (dev < 0) return HP_ECUDA;
    if (!attr[dev]) { HP_CUDA(cudaFuncSetAttribute(k_moe_gemv_grouped<MODE, SB, WARPS, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[dev] = true; }
    HP_CUDA(launch_pdl<8>(k_moe_gemv_grouped<MODE, SB, WARPS, DEPTH>, dim3(GEMV_NCTA), dim3(WARPS * 32), smem, s, a));
    return HP_OK;
}
// few rows (units <= T * nslot * tiles / 4 stay below ~4 per SM): 4 warps x 6 stages; otherwise 12 warps x 2 stages
template <int MODE, int SB>
static int launch_grouped_geo(const MoeGArgs& a, bool few, cudaStream_t s) {
    return few ? launch_grouped<MODE, SB, 4, 6>(a, s) : launch_grouped<MODE, SB, 12, 2>(a, s);
}
template <int MODE>
static int launch_grouped_sb(const MoeGArgs& a, bool few, cudaStream_t s) {
    return a.nb % 4 == 0 ? launch_grouped_geo<MODE, 4>(a, few, s) : a.nb % 2 == 0 ? launch_grouped_geo<MODE, 2>(a, few, s) : launch_grouped_geo<MODE, 1>(a, few, s);
}
template <int MODE, int SB, int DEPTH>
static int launch_quad(const MoeGArgs& a, size_t smem, cudaStream_t s) {
    static size_t attr[MAX_DEVICES] = {};
    const int dev = current_device(); if (dev < 0) return HP_ECUDA;
    if (smem > attr[dev]) { HP_CUDA(cudaFuncSetAttribute(k_moe_gemv_quad<MODE, SB, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr[dev] = smem; }
    HP_CUDA(launch_pdl<8>(k_moe_gemv_quad<MODE, SB, DEPTH>, dim3(GEMV_NCTA), dim3(MQ_WARPS * 32), smem, s, a));
    return HP_OK;
}
// the quad form when the three quads' activation buffers fit beside the rings (K <= 2048 for the gate|up projection),
// the one-warp-per-unit form otherwise
static size_t quad_smem(const MoeGArgs& a) { const int sb = a.nb % 2 == 0 ? 2 : 1, depth = sb == 2 ? 3 : 6; return (size_t)MQ_WARPS * depth * sb * 2304 + MQ_AUX + (size_t)MQ_QUADS * a.nb * 2560; }
static bool quad_form(const MoeGArgs& a) {
    static const bool v1 = getenv("HIPSTER_B200_MOE_UNITS") != nullptr;
    return !v1 && quad_smem(a) <= 227 * 1024 && a.tiles % MOE_UNIT_TILES == 0;
}
template <int MODE>
static int launch_experts(const MoeGArgs& a, bool few, cudaStream_t s) {
    const int sb = a.nb % 2 == 0 ? 2 : 1;
    const size_t smem = quad_smem(a);
    if (!quad_form(a)) return launch_grouped_sb<MODE>(a, few, s);
    return sb == 2 ? launch_quad<MODE, 2, 3>(a, smem, s) : launch_quad<MODE, 1, 6>(a, smem, s);
}
int moe_experts_grouped(const MoeGroupParams& p, cudaStream_t s, int* pushed) {
    HP_REQUIRE(p.E % 256 == 0 && p.F % 256 == 0 && p.T >= 1 && p.nslot >= 1 && p.T * p.nslot <= MOE_MAX_PAIRS, "moe_experts_grouped: bad shape");
    HP_REQUIRE(p.segs && p.ctl && p.v, "moe_experts_grouped: null pointer");
    MoeGArgs a; a.e_lo = p.e_lo; a.segs = (const MoeSeg*)p.segs; a.ctl = p.ctl; a.err = p.err;
    // gate|up: [2F rows][E]; tile q = gate rows 8q.. | up rows 8q..; 4 tiles = one 32-feature quantisation group
    a.w_exp = (const uint8_t*)p.w_gate_up; a.w_sh = (const uint8_t*)p.sh_gate_up; a.tiles = 2 * p.F / 16; a.nb = p.E / 256; a.ticket = 1;
    a.xq = (const uint8_t*)p.xq.q; a.xsc = (const float*)p.xq.sc; a.xK = p.E; a.xdiv = p.nslot;
    a.y = nullptr; a.N = 0; a.oq = (int8_t*)p.xq2.q; a.osc = (float*)p.xq2.sc; a.F = p.F;
    a.ep_world = 1; a.ep_rank = 0; a.ep_half = 0; for (int q = 0; q < 8; ++q) { a.ep_x[q] = nullptr; a.ep_ctl[q] = nullptr; }
    if (pushed) *pushed = 0;
    const bool few = p.T <= 4;
    { const int rc = launch_experts<0>(a, few, s); if (rc != HP_OK) return rc; }
    // down: [E rows][F]; per-pair outputs
    a.w_exp = (const uint8_t*)p.w_down; a.w_sh = (const uint8_t*)p.sh_down; a.tiles = p.E / 16; a.nb = p.F / 256; a.ticket = 2;
    a.xq = (const uint8_t*)p.xq2.q; a.xsc = (const float*)p.xq2.sc; a.xK = p.F; a.xdiv = 1;
    a.y = p.v; a.N = p.E; a.oq = nullptr; a.osc = nullptr;
    if (p.ep_world > 1 && p.ep_x[p.ep_rank] && quad_form(a)) {
        HP_REQUIRE(p.ep_world <= 8 && p.ep_rank >= 0 && p.ep_rank < p.ep_world && p.ep_half >= (size_t)p.T * p.nslot * p.E, "moe_experts_grouped: bad peer arguments");
        a.ep_world = p.ep_world; a.ep_rank = p.ep_rank; a.ep_half = p.ep_half;
        for (int q = 0; q < p.ep_world; ++q) { a.ep_x[q] = p.ep_x[q]; a.ep_ctl[q] = p.ep_ctl[q]; }
        if (pushed) *pushed = 1;
    }
    { const int rc = launch_experts<1>(a, few, s); if (rc != HP_OK) return rc; }
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int moe_combine(const float* v, const float* slotw, float* y, int T, int nslot, int E, cudaStream_t s) {
    HP_REQUIRE(T >= 1 && nslot >= 1 && E >= 1, "moe_combine: bad shape");
    k_moe_combine<<<dim3((E + 255) / 256, T), 256, 0, s>>>(v, slotw, y, nslot, E);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
}  // namespace hp
