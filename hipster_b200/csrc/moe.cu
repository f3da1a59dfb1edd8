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

// ---- router (exact f32: one warp per weight row; lane l takes k = 4l + 128 i as float4, four fmaf per step in element
// order, then the xor-shuffle tree 16..1) and routing (softmax over the first E logits, top-k by (value desc, index asc),
// weights renormalised by the sum of the selected probabilities taken in rank order; slot k = shared expert, id -1, with
// weight sigmoid(logit[E])). Reference: k_f32_gemv (fn.hip:252-266), k_moe_route (fn.hip:167-205). ----
__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) { if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
// Both in one launch: the CTA that finishes a row's logits last (ticket counter per row) routes that row. The softmax
// sums follow a fixed order: xor tree inside each 32-element group, the 32 group results combined in group order (warp w
// of the 256-thread CTA does groups w, w+8, w+16, w+24).
__global__ void __launch_bounds__(256) k_router_route(const float* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int N, int K,
                                                     int* __restrict__ ids, float* __restrict__ w, int E, int k, int* __restrict__ cnt) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh[32]; __shared__ float selp[16]; __shared__ int seli[16]; __shared__ float sp[1024]; __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, t = blockIdx.y;
    const int n = (blockIdx.x * 256 + tid) >> 5;
    if (n < N) {
        const float* wr = W + (size_t)n * K; const float* xr = x + (size_t)t * K;
        float acc = 0.f;
#pragma unroll 8
        for (int i = lane * 4; i < K; i += 128) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(wr + i)), b = *reinterpret_cast<const float4*>(xr + i);
            acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc = acc + __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) { y[(size_t)t * N + n] = acc; __threadfence(); }
    }
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&cnt[t], 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* lg = y + (size_t)t * N;   // N = E + 1 logits of this row, written by all the CTAs of the row
    float v[4], e[4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = 32 * (warp + 8 * j) + lane;
        v[j] = i < E ? __ldcg(lg + i) : -INFINITY;
        float m = v[j];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        if (lane == 0) sh[warp + 8 * j] = m;
    }
    __syncthreads();
    mx = sh[0]; for (int q = 1; q < 32; ++q) mx = fmaxf(mx, sh[q]);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = 32 * (warp + 8 * j) + lane;
        e[j] = i < E ? expf_det(v[j] - mx) : 0.f;
        float sacc = e[j];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sacc = sacc + __shfl_xor_sync(0xffffffffu, sacc, off);
        if (lane == 0) sh[warp + 8 * j] = sacc;
    }
    __syncthreads();
    float sum = sh[0]; for (int q = 1; q < 32; ++q) sum = sum + sh[q];
#pragma unroll
    for (int j = 0; j < 4; ++j) { const int i = 32 * (warp + 8 * j) + lane; sp[i] = i < E ? e[j] / sum : -2.f; }
    __syncthreads();
    if (warp == 0) {   // top-k by (value desc, index asc); lane l owns indices l, l+32, ...
        float pv[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) pv[q] = sp[lane + 32 * q];
        for (int r = 0; r < k; ++r) {
            float bv = pv[0]; int bi = lane;
#pragma unroll
            for (int q = 1; q < 32; ++q) better(bv, bi, pv[q], lane + 32 * q);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) { const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off); better(bv, bi, ov, oi); }
            if (lane == 0) { selp[r] = bv; seli[r] = bi; }
#pragma unroll
            for (int q = 0; q < 32; ++q) if (bi == lane + 32 * q) pv[q] = -1.f;
        }
    }
    __syncthreads();
    if (tid == 0) {
        float wsum = 0.f; for (int r = 0; r < k; ++r) wsum = wsum + selp[r];
        for (int r = 0; r < k; ++r) { ids[t * (k + 1) + r] = seli[r]; w[t * (k + 1) + r] = selp[r] / wsum; }
        ids[t * (k + 1) + k] = -1; w[t * (k + 1) + k] = sigmoid_det(__ldcg(lg + E));
        cnt[t] = 0;   // ready for the next launch
    }
}

// ---- one 16-row tile of an expert matrix against one activation row: blocks in order, weights read straight from
// global memory (each expert tile is touched once), CH blocks per batch so that their loads share one round trip.
// Returns the column of interest in r0 / r1 (rows g, g+8). Scales are decoded in registers per lane (rows g, g+8):
// a 6-bit value v becomes the float 2^23 + v by a byte permute, and fmaf(d, 2^23 + v, -(d * 2^23)) is exactly d * v;
// odd sub-blocks take the high nibbles unshifted (16 * q), their d carries the exact 1/16. ----
struct MoeRowScales {
    float d, cd, dq, cdq, nd, cnd; uint32_t sc[2], mn[2];
    __device__ __forceinline__ void get(int k, float& s0, float& nm) const {
        const float fs = __uint_as_float(__byte_perm(sc[k >> 2], 0x4B000000u, 0x7540u | (k & 3)));
        const float fm = __uint_as_float(__byte_perm(mn[k >> 2], 0x4B000000u, 0x7540u | (k & 3)));
        s0 = (k & 1) ? fmaf(dq, fs, cdq) : fmaf(d, fs, cd);
        nm = fmaf(nd, fm, cnd);
    }
};
__device__ __forceinline__ MoeRowScales moe_decode_scales(const uint4 hdr) {
    MoeRowScales r;
    r.d = h2f((uint16_t)(hdr.x & 0xFFFF)); r.nd = -h2f((uint16_t)(hdr.x >> 16));
    r.dq = r.d * 0.0625f;
    r.cd = -(r.d * 8388608.f); r.cdq = -(r.dq * 8388608.f); r.cnd = -(r.nd * 8388608.f);
    r.sc[0] = hdr.y & 0x3F3F3F3Fu; r.mn[0] = hdr.z & 0x3F3F3F3Fu;
    r.sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    r.mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    return r;
}
template <int CH>
__device__ __forceinline__ void expert_tile(const uint8_t* __restrict__ W, int row_bytes, int nb, const uint4* __restrict__ xq, const float4* __restrict__ xsc,
                                            int xtile, int xcol, int lane, float& r0, float& r1) {
    const int g = lane >> 2, t = lane & 3;
    float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
    const uint8_t* rowa = W + (size_t)g * row_bytes;
    const uint8_t* rowb = W + (size_t)(g + 8) * row_bytes;
    for (int b0 = 0; b0 < nb; b0 += CH) {
        uint4 ha[CH], hb[CH]; uint2 wa[CH][4], wb[CH][4];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int b = b0 + c < nb ? b0 + c : nb - 1;
            ha[c] = __ldg(reinterpret_cast<const uint4*>(rowa + (size_t)b * 144)); hb[c] = __ldg(reinterpret_cast<const uint4*>(rowb + (size_t)b * 144));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                wa[c][j] = __ldg(reinterpret_cast<const uint2*>(rowa + (size_t)b * 144 + 16 + 8 * t + 32 * j));
                wb[c][j] = __ldg(reinterpret_cast<const uint2*>(rowb + (size_t)b * 144 + 16 + 8 * t + 32 * j));
            }
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int b = b0 + c;
            if (b < nb) {
                const MoeRowScales ra = moe_decode_scales(ha[c]), rb = moe_decode_scales(hb[c]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint2 w0 = wa[c][j], w1 = wb[c][j];
                    const uint32_t alo[4] = {w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu};
                    const uint32_t ahi[4] = {w0.x & 0xF0F0F0F0u, w1.x & 0xF0F0F0F0u, w0.y & 0xF0F0F0F0u, w1.y & 0xF0F0F0F0u};
                    float sa0, na0, sb0, nb0, sa1, na1, sb1, nb1;
                    ra.get(2 * j, sa0, na0); rb.get(2 * j, sb0, nb0); ra.get(2 * j + 1, sa1, na1); rb.get(2 * j + 1, sb1, nb1);
                    const uint4 xf = __ldg(xq + ((size_t)xtile * nb * 4 + b * 4 + j) * 32 + lane);
                    const float4 x0 = __ldg(xsc + ((size_t)xtile * nb * 8 + b * 8 + 2 * j) * 4 + t), x1 = __ldg(xsc + ((size_t)xtile * nb * 8 + b * 8 + 2 * j + 1) * 4 + t);
                    int c0[4], c1[4];
                    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                 : "=r"(c0[0]), "=r"(c0[1]), "=r"(c0[2]), "=r"(c0[3]) : "r"(alo[0]), "r"(alo[1]), "r"(alo[2]), "r"(alo[3]), "r"(xf.x), "r"(xf.y), "r"(0));
                    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                 : "=r"(c1[0]), "=r"(c1[1]), "=r"(c1[2]), "=r"(c1[3]) : "r"(ahi[0]), "r"(ahi[1]), "r"(ahi[2]), "r"(ahi[3]), "r"(xf.z), "r"(xf.w), "r"(0));
                    // columns 2t, 2t+1 of the activation tile; only column xcol is kept at the end
                    acc0.x = fmaf(sa0 * x0.x, (float)c0[0], acc0.x); acc0.x = fmaf(na0, x0.z, acc0.x);
                    acc0.y = fmaf(sa0 * x0.y, (float)c0[1], acc0.y); acc0.y = fmaf(na0, x0.w, acc0.y);
                    acc1.x = fmaf(sb0 * x0.x, (float)c0[2], acc1.x); acc1.x = fmaf(nb0, x0.z, acc1.x);
                    acc1.y = fmaf(sb0 * x0.y, (float)c0[3], acc1.y); acc1.y = fmaf(nb0, x0.w, acc1.y);
                    acc0.x = fmaf(sa1 * x1.x, (float)c1[0], acc0.x); acc0.x = fmaf(na1, x1.z, acc0.x);
                    acc0.y = fmaf(sa1 * x1.y, (float)c1[1], acc0.y); acc0.y = fmaf(na1, x1.w, acc0.y);
                    acc1.x = fmaf(sb1 * x1.x, (float)c1[2], acc1.x); acc1.x = fmaf(nb1, x1.z, acc1.x);
                    acc1.y = fmaf(sb1 * x1.y, (float)c1[3], acc1.y); acc1.y = fmaf(nb1, x1.w, acc1.y);
                }
            }
        }
    }
    // hand column xcol to every lane of its row group: it lives in lane (g, xcol/2), component xcol & 1
    const float m0 = (xcol & 1) ? acc0.y : acc0.x, m1 = (xcol & 1) ? acc1.y : acc1.x;
    r0 = __shfl_sync(0xffffffffu, m0, (lane & ~3) | (xcol >> 1));
    r1 = __shfl_sync(0xffffffffu, m1, (lane & ~3) | (xcol >> 1));
}

struct MoeArgs {
    const uint8_t* w_exp; const uint8_t* w_sh; size_t ebytes; int N, K;     // expert matrices [E][N][K/256 blocks], shared [N][K/256]
    const int* ids; const float* slotw; int nslot;                           // [T][nslot]
    const uint4* xq; const float4* xsc;                                      // quantised activations (rows = T, or T*nslot for the down projection)
    float* y; int T;
    int e_lo, e_hi, own_shared;                                              // routed experts owned by this GPU [e_lo, e_hi) and whether it computes the shared slot
};
__device__ __forceinline__ bool moe_owned(const MoeArgs& a, int id) { return id >= 0 ? (id >= a.e_lo && id < a.e_hi) : a.own_shared != 0; }
// gate|up: y[(t,e)][N] = W[ids[t,e]] . x[t]; one warp per (pair, 16-row tile)
__global__ void __launch_bounds__(256) k_moe_gemv(MoeArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = a.N / 16, unit = blockIdx.x * 8 + warp;
    if (unit >= a.T * a.nslot * tiles) return;
    const int pair = unit / tiles, tile = unit % tiles, t = pair / a.nslot;
    const int id = a.ids[pair];
    if (!moe_owned(a, id)) return;                                           // expert lives on another GPU
    const int nb = a.K / 256, row_bytes = nb * 144;
    const uint8_t* W = (id >= 0 ? a.w_exp + (size_t)id * a.ebytes : a.w_sh) + (size_t)tile * 16 * row_bytes;
    float r0, r1;
    expert_tile<4>(W, row_bytes, nb, a.xq, a.xsc, t >> 3, t & 7, lane, r0, r1);
    const int g = lane >> 2;
    if ((lane & 3) == 0) { a.y[(size_t)pair * a.N + tile * 16 + g] = r0; a.y[(size_t)pair * a.N + tile * 16 + g + 8] = r1; }
}
// per-pair expert output of the down projection: v[(t,e)][N] = W_down[ids[t,e]] . act[(t,e)] (expert-parallel form)
__global__ void __launch_bounds__(256) k_moe_down_pairs(MoeArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = a.N / 16, unit = blockIdx.x * 8 + warp;
    if (unit >= a.T * a.nslot * tiles) return;
    const int pair = unit / tiles, tile = unit % tiles;
    const int id = a.ids[pair];
    const int g = lane >> 2;
    if (!moe_owned(a, id)) {   // not ours: contribute exact zeros to the exchange buffer
        if ((lane & 3) == 0) { a.y[(size_t)pair * a.N + tile * 16 + g] = 0.f; a.y[(size_t)pair * a.N + tile * 16 + g + 8] = 0.f; }
        return;
    }
    const int nb = a.K / 256, row_bytes = nb * 144;
    const uint8_t* W = (id >= 0 ? a.w_exp + (size_t)id * a.ebytes : a.w_sh) + (size_t)tile * 16 * row_bytes;
    float r0, r1;
    expert_tile<2>(W, row_bytes, nb, a.xq, a.xsc, pair >> 3, pair & 7, lane, r0, r1);
    if ((lane & 3) == 0) { a.y[(size_t)pair * a.N + tile * 16 + g] = r0; a.y[(size_t)pair * a.N + tile * 16 + g + 8] = r1; }
}
// q8(silu(g) * u) per (t,e) row: gu [pairs][2F] (fn.hip:206-211); pairs of experts that live elsewhere are skipped
__global__ void __launch_bounds__(256) k_moe_silu_quant(const float* __restrict__ gu, int F, const int* __restrict__ ids, int e_lo, int e_hi, int own_shared, int8_t* __restrict__ q, float* __restrict__ sc) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.y, sb = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (sb * 32 >= F) return;
    const int id = ids[pair]; if (id >= 0 ? (id < e_lo || id >= e_hi) : !own_shared) return;
    const int i = sb * 32 + lane;
    warp_quant32_store(silu_det(gu[(size_t)pair * 2 * F + i]) * gu[(size_t)pair * 2 * F + F + i], pair, sb, F, q, sc, lane);
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

int router_route(const float* W, const float* x, float* logits, int* ids, float* w, int* counters, int E, int K, int k, int T, cudaStream_t s) {
    HP_REQUIRE(E >= 1 && E <= 1024 && k >= 1 && k <= 15 && k <= E && K > 0 && K % 128 == 0 && T >= 1 && T <= 32 && counters, "router_route: bad shape E=%d K=%d k=%d T=%d", E, K, k, T);
    const int N = E + 1;
    HP_CUDA(launch_pdl<8>(k_router_route, dim3((N * 32 + 255) / 256, T), dim3(256), 0, s, W, x, logits, N, K, ids, w, E, k, counters));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
static MoeArgs moe_args(const MoeParams& p) {
    MoeArgs a; a.w_exp = (const uint8_t*)p.w_exp; a.w_sh = (const uint8_t*)p.w_sh; a.ebytes = p.ebytes; a.N = p.N; a.K = p.K; a.ids = p.ids; a.slotw = p.slotw; a.nslot = p.nslot;
    a.xq = (const uint4*)p.xq.q; a.xsc = (const float4*)p.xq.sc; a.y = p.y; a.T = p.T; a.e_lo = p.e_lo; a.e_hi = p.e_hi; a.own_shared = p.own_shared; return a;
}
int moe_gemv_up(const MoeParams& p, cudaStream_t s) {
    HP_REQUIRE(p.N % 16 == 0 && p.K % 256 == 0 && p.T >= 1 && p.nslot >= 1, "moe_gemv_up: bad shape");
    const int units = p.T * p.nslot * (p.N / 16);
    HP_CUDA(launch_pdl<8>(k_moe_gemv, dim3((units + 7) / 8), dim3(256), 0, s, moe_args(p)));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int moe_silu_quant(const float* gu, int F, const int* ids, int e_lo, int e_hi, int own_shared, XQ8F xq, int pairs, cudaStream_t s) {
    HP_REQUIRE(F % 64 == 0 && pairs >= 1, "moe_silu_quant: bad shape");
    HP_CUDA(launch_pdl<8>(k_moe_silu_quant, dim3((F / 32 + 7) / 8, pairs), dim3(256), 0, s, gu, F, ids, e_lo, e_hi, own_shared, (int8_t*)xq.q, (float*)xq.sc));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int moe_combine(const float* v, const float* slotw, float* y, int T, int nslot, int E, cudaStream_t s) {
    HP_REQUIRE(T >= 1 && nslot >= 1 && E >= 1, "moe_combine: bad shape");
    k_moe_combine<<<dim3((E + 255) / 256, T), 256, 0, s>>>(v, slotw, y, nslot, E);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int moe_down_pairs(const MoeParams& p, cudaStream_t s) {
    HP_REQUIRE(p.N % 16 == 0 && p.K % 256 == 0 && p.T >= 1 && p.nslot >= 1, "moe_down_pairs: bad shape");
    const int units = p.T * p.nslot * (p.N / 16);
    HP_CUDA(launch_pdl<8>(k_moe_down_pairs, dim3((units + 7) / 8), dim3(256), 0, s, moe_args(p)));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

}  // namespace hp
