// Q4_K dequant-fused GEMV / skinny GEMM for the verify rows of a speculative-decode pass.
//
// Replaces the reference's decode GEMVs: k_gemv_q8 / k_gemv_multi (engine/kernels/gemv.hip:291-367,1042-1067),
// the T-invariant production kernel k_gemv_wmma<Q4_K> (gemv.hip:602-672) and the f32-activation baseline
// k_gemv_q4_K_f32 (gemv.hip:1177-1216).
//
// Design (sm_100a): weights stay in the 144-byte ggml Q4_K block format, [N][K/256] blocks, rows contiguous.
// A CTA owns 16 consecutive weight rows. A producer warp streams them with 1-D bulk async copies
// (cp.async.bulk + mbarrier) through a ring of shared-memory stages, 4 blocks (576 B) of every row per stage;
// four consumer warps take one block of the stage each (block b belongs to warp b % 4), unpack the nibbles in
// registers and feed them to the int8 tensor-core tile mma.m16n8k32 (weights on M, verify rows on N = 8), which
// yields the exact int32 dot of every 32-element sub-block. One fp32 update per sub-block follows, in block order:
//     acc = fmaf((d*sc) * xd, (float)idot, acc);  acc = fmaf(-(dmin*mn), xs, acc);
// and the four per-warp partial sums are added in warp order. The order depends on the tensor shape only, never on
// the number of verify rows, so a row of an n+1-row verify pass is bit-identical to the same row of a 1-row pass
// (the reference's "T-invariance", gemv.hip:600-601). Each weight byte is read from HBM once per pass.
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

constexpr int GEMV_ROWS = 16;            // weight rows per CTA (one mma M tile)
constexpr int GEMV_KS = 4;               // consumer warps = K slices
constexpr int GEMV_STAGES = 6;
constexpr int GEMV_ROW_BYTES = 4 * 144;  // bytes of one row in one stage
constexpr int GEMV_ROW_STRIDE = GEMV_ROW_BYTES + 96;   // 672 = 5*128 + 32: rows land on distinct 32-byte bank groups
constexpr int GEMV_STAGE_BYTES = GEMV_ROWS * GEMV_ROW_STRIDE;
constexpr int GEMV_THREADS = (GEMV_KS + 1) * 32;

struct GemvSmem {
    alignas(128) uint8_t ring[GEMV_STAGES][GEMV_STAGE_BYTES];
    alignas(16) float4 scr[GEMV_KS][4][GEMV_ROWS];   // per warp: {s0(2j), -m(2j), s0(2j+1), -m(2j+1)} [j][row]
    alignas(8) unsigned long long full[GEMV_STAGES];
    alignas(8) unsigned long long empty[GEMV_STAGES];
};

template <int NT>
__global__ void __launch_bounds__(GEMV_THREADS) k_gemv_q4k_q8(const uint8_t* __restrict__ W, const uint4* __restrict__ xq, const float4* __restrict__ xsc,
                                                               float* __restrict__ y, int N, int nb, int R, int ldy, int* __restrict__ err) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    GemvSmem& sm = *reinterpret_cast<GemvSmem*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * GEMV_ROWS;
    const int nrows = min(GEMV_ROWS, N - row0);
    const int nst = (nb + 3) >> 2;
    const size_t row_bytes = (size_t)nb * 144;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMV_STAGES; ++s) { mbar_init(smem_u32(&sm.full[s]), 1); mbar_init(smem_u32(&sm.empty[s]), GEMV_KS); }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == GEMV_KS) {
        // ---------------- producer: weights do not depend on the previous kernel, so streaming starts at once
        const uint8_t* src = W + (size_t)(row0 + lane) * row_bytes;
        for (int i = 0; i < nst; ++i) {
            const int s = i % GEMV_STAGES;
            if (i >= GEMV_STAGES) { if (!mbar_wait(smem_u32(&sm.empty[s]), ((i / GEMV_STAGES) - 1) & 1, err)) break; }
            const uint32_t bytes = (uint32_t)min(4, nb - 4 * i) * 144u;
            if (lane == 0) mbar_expect_tx(smem_u32(&sm.full[s]), bytes * (uint32_t)nrows);
            __syncwarp();
            if (lane < nrows) bulk_g2s(smem_u32(&sm.ring[s][lane * GEMV_ROW_STRIDE]), src + (size_t)i * GEMV_ROW_BYTES, bytes, smem_u32(&sm.full[s]));
        }
    } else {
        // ---------------- consumers
        const int g = lane >> 2, t = lane & 3;
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
        const int njj = nb * 4, nsb = nb * 8;
        pdl_wait();   // activations come from the previous kernel
        bool ok = true;
        for (int i = 0; i < nst && ok; ++i) {
            const int s = i % GEMV_STAGES;
            ok = mbar_wait(smem_u32(&sm.full[s]), (i / GEMV_STAGES) & 1, err);
            const int b = 4 * i + warp;
            if (ok && b < nb) {
                const uint8_t* st = sm.ring[s] + warp * 144;
                {   // scale pre-pass: lane -> (row = lane/2, half = lane&1) decodes 4 sub-blocks
                    const int r = lane >> 1, hf = lane & 1;
                    const uint4 hdr = *reinterpret_cast<const uint4*>(st + r * GEMV_ROW_STRIDE);
                    const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t sc, mn; q4k_scale_min(hdr, 4 * hf + k, sc, mn);
                        v[2 * k] = d * (float)sc; v[2 * k + 1] = -(dmin * (float)mn);
                    }
                    sm.scr[warp][2 * hf][r] = make_float4(v[0], v[1], v[2], v[3]);
                    sm.scr[warp][2 * hf + 1][r] = make_float4(v[4], v[5], v[6], v[7]);
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint2 w0 = *reinterpret_cast<const uint2*>(st + g * GEMV_ROW_STRIDE + 16 + 32 * j + 8 * t);
                    const uint2 w1 = *reinterpret_cast<const uint2*>(st + (g + 8) * GEMV_ROW_STRIDE + 16 + 32 * j + 8 * t);
                    const uint32_t alo[4] = {w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu};
                    const uint32_t ahi[4] = {(w0.x >> 4) & 0x0F0F0F0Fu, (w1.x >> 4) & 0x0F0F0F0Fu, (w0.y >> 4) & 0x0F0F0F0Fu, (w1.y >> 4) & 0x0F0F0F0Fu};
                    const float4 sa = sm.scr[warp][j][g], sb8 = sm.scr[warp][j][g + 8];
                    const int jj = b * 4 + j, sb = b * 8 + 2 * j;
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const uint4 xf = __ldg(xq + ((size_t)n * njj + jj) * 32 + lane);
                        const float4 x0 = __ldg(xsc + ((size_t)n * nsb + sb) * 4 + t);
                        const float4 x1 = __ldg(xsc + ((size_t)n * nsb + sb + 1) * 4 + t);
                        int c0[4], c1[4];
                        mma_u8s8(c0, alo, xf.x, xf.y);
                        mma_u8s8(c1, ahi, xf.z, xf.w);
                        // low-nibble sub-block 2j
                        acc[n][0] = fmaf(sa.x * x0.x, (float)c0[0], acc[n][0]);  acc[n][0] = fmaf(sa.y, x0.z, acc[n][0]);
                        acc[n][1] = fmaf(sa.x * x0.y, (float)c0[1], acc[n][1]);  acc[n][1] = fmaf(sa.y, x0.w, acc[n][1]);
                        acc[n][2] = fmaf(sb8.x * x0.x, (float)c0[2], acc[n][2]); acc[n][2] = fmaf(sb8.y, x0.z, acc[n][2]);
                        acc[n][3] = fmaf(sb8.x * x0.y, (float)c0[3], acc[n][3]); acc[n][3] = fmaf(sb8.y, x0.w, acc[n][3]);
                        // high-nibble sub-block 2j+1
                        acc[n][0] = fmaf(sa.z * x1.x, (float)c1[0], acc[n][0]);  acc[n][0] = fmaf(sa.w, x1.z, acc[n][0]);
                        acc[n][1] = fmaf(sa.z * x1.y, (float)c1[1], acc[n][1]);  acc[n][1] = fmaf(sa.w, x1.w, acc[n][1]);
                        acc[n][2] = fmaf(sb8.z * x1.x, (float)c1[2], acc[n][2]); acc[n][2] = fmaf(sb8.w, x1.z, acc[n][2]);
                        acc[n][3] = fmaf(sb8.z * x1.y, (float)c1[3], acc[n][3]); acc[n][3] = fmaf(sb8.w, x1.w, acc[n][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.empty[s]));
        }
        // ---------------- split-K reduction in warp order (the ring is free: every stage has been consumed)
        asm volatile("bar.sync 1, %0;" ::"n"(GEMV_KS * 32));
        float* red = reinterpret_cast<float*>(sm.ring);   // [KS][NT*4][32]
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) red[(warp * NT * 4 + n * 4 + k) * 32 + lane] = acc[n][k];
        asm volatile("bar.sync 1, %0;" ::"n"(GEMV_KS * 32));
        if (warp == 0) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float v = red[(n * 4 + k) * 32 + lane];
#pragma unroll
                    for (int w = 1; w < GEMV_KS; ++w) v = v + red[(w * NT * 4 + n * 4 + k) * 32 + lane];
                    const int row = row0 + g + ((k & 2) ? 8 : 0), col = n * 8 + 2 * t + (k & 1);
                    if (row < N && col < R) y[(size_t)col * ldy + row] = v;
                }
        }
    }
}

// ---- f32-activation baseline: lane l of TPR takes blocks l, l+TPR, ...; xor-shuffle tree (gemv.hip:1177-1216) ----
template <int TPR, int NCOL>
__global__ void __launch_bounds__(256) k_gemv_q4k_f32(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int N, int K) {
    constexpr int ROWS = 256 / TPR;
    const int lane = threadIdx.x % TPR, row = blockIdx.x * ROWS + threadIdx.x / TPR;
    const int nb = K / 256;
    const bool live = row < N;
    const uint8_t* wrow = W + (size_t)(live ? row : 0) * nb * 144;
    float acc[NCOL];
#pragma unroll
    for (int c = 0; c < NCOL; ++c) acc[c] = 0.f;
    for (int b = lane; b < nb && live; b += TPR) {
        const uint4* blk = reinterpret_cast<const uint4*>(wrow + (size_t)b * 144);
        const uint4 hdr = __ldg(blk);
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t sc0, mn0, sc1, mn1; q4k_scale_min(hdr, 2 * j, sc0, mn0); q4k_scale_min(hdr, 2 * j + 1, sc1, mn1);
            const float d0 = d * (float)sc0, m0 = dmin * (float)mn0, d1 = d * (float)sc1, m1 = dmin * (float)mn1;
            const uint4 qa = __ldg(blk + 1 + 2 * j), qb = __ldg(blk + 2 + 2 * j);
            const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                const float* xc = x + (size_t)c * K + (size_t)b * 256 + 64 * j;
                float s0 = 0.f, s1 = 0.f, sx0 = 0.f, sx1 = 0.f;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const uint32_t q = (qw[e >> 2] >> (8 * (e & 3))) & 0xFFu;
                    const float x0 = __ldg(xc + e), x1 = __ldg(xc + 32 + e);
                    s0 = fmaf(x0, (float)(q & 0xFu), s0); s1 = fmaf(x1, (float)(q >> 4), s1);
                    sx0 = sx0 + x0; sx1 = sx1 + x1;
                }
                float tt = d0 * s0; tt = tt - m0 * sx0; tt = tt + d1 * s1; tt = tt - m1 * sx1;
                acc[c] = acc[c] + tt;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < NCOL; ++c)
#pragma unroll
        for (int off = TPR / 2; off > 0; off >>= 1) acc[c] = acc[c] + __shfl_xor_sync(0xffffffffu, acc[c], off, TPR);
    if (lane == 0 && live)
#pragma unroll
        for (int c = 0; c < NCOL; ++c) y[(size_t)c * N + row] = acc[c];
}

template <int NT>
int launch_q8(const uint8_t* W, const void* xq, const void* xsc, float* y, int N, int nb, int R, int ldy, int* err, cudaStream_t s, bool pdl) {
    static bool attr_set = false;
    if (!attr_set) { HP_CUDA(cudaFuncSetAttribute(k_gemv_q4k_q8<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(GemvSmem))); attr_set = true; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + GEMV_ROWS - 1) / GEMV_ROWS); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = sizeof(GemvSmem); cfg.stream = s;
    cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    HP_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_q4k_q8<NT>, W, (const uint4*)xq, (const float4*)xsc, y, N, nb, R, ldy, err));
    return HP_OK;
}

}  // namespace

int gemv_q4k_q8(const void* W, const XQ8F& x, float* y, int N, int K, int R, int ldy, int* err, cudaStream_t s, bool pdl) {
    HP_REQUIRE(K > 0 && K % 256 == 0, "gemv_q4k_q8: K=%d must be a positive multiple of 256", K);
    HP_REQUIRE(N > 0 && R >= 1 && R <= 32 && ldy >= N, "gemv_q4k_q8: bad shape N=%d R=%d ldy=%d", N, R, ldy);
    const int nb = K / 256;
    switch ((R + 7) / 8) {
        case 1: return launch_q8<1>((const uint8_t*)W, x.q, x.sc, y, N, nb, R, ldy, err, s, pdl);
        case 2: return launch_q8<2>((const uint8_t*)W, x.q, x.sc, y, N, nb, R, ldy, err, s, pdl);
        case 3: return launch_q8<3>((const uint8_t*)W, x.q, x.sc, y, N, nb, R, ldy, err, s, pdl);
        default: return launch_q8<4>((const uint8_t*)W, x.q, x.sc, y, N, nb, R, ldy, err, s, pdl);
    }
}

int gemv_q4k_f32(const void* W, const float* x, float* y, int N, int K, int R, cudaStream_t s) {
    HP_REQUIRE(K > 0 && K % 256 == 0, "gemv_q4k_f32: K=%d must be a positive multiple of 256", K);
    HP_REQUIRE(N > 0 && R >= 1 && R <= 8, "gemv_q4k_f32: bad shape N=%d R=%d (R <= 8)", N, R);
    constexpr int TPR = 4; const int grid = (N + 256 / TPR - 1) / (256 / TPR);
#define HP_F32(NC) k_gemv_q4k_f32<TPR, NC><<<grid, 256, 0, s>>>((const uint8_t*)W, x, y, N, K)
    switch (R) { case 1: HP_F32(1); break; case 2: HP_F32(2); break; case 3: HP_F32(3); break; case 4: HP_F32(4); break;
                 case 5: HP_F32(5); break; case 6: HP_F32(6); break; case 7: HP_F32(7); break; default: HP_F32(8); break; }
#undef HP_F32
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}

}  // namespace hp
