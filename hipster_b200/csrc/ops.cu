// Layer kernels of the decode / verify pass other than the GEMV: embedding gather, fused residual-add + RMSNorm +
// int8 quantisation, MTP input (two norms concatenated), SiLU-gated product + quantisation, and the Gated-DeltaNet
// short convolution + delta-rule recurrence with deferred commit ("rollback") and optional per-row state snapshots.
//
// Reference: engine/kernels/ops.hip -- k_add_rmsnorm_quant (:79-98), k_norm2_concat_quant (:99-116),
// k_silu_mul_quant (:146-151), k_embed_q4_K (:154-171), k_gdn_conv (:188-202), k_gdn_step (:205-256); replay buffers and
// Qwen35::accept (engine/src/qwen35.cpp:383-403).
//
// Every reduction has a fixed order (stated at each kernel) so that the CPU oracle reproduces the results bit for bit.
#include <type_traits>
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

// Sum of one value per thread over the block, in a fixed order: xor-shuffle tree inside each warp (offsets 16..1),
// then the warp sums added sequentially in warp order. All threads return the same value. NW = warps per block.
template <int NW>
__device__ __forceinline__ float block_sum_det(float v, float* sh) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, off);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float tot = sh[0];
#pragma unroll
    for (int i = 1; i < NW; ++i) tot = tot + sh[i];
    return tot;
}

// ---- embedding gather: bf16 table [V][E] -> f32 rows (reference: k_embed_q4_K, ops.hip:154-171; this build's
// configurations keep embeddings in bf16) ----
__global__ void __launch_bounds__(256) k_embed_bf16(const int* __restrict__ tok, const uint16_t* __restrict__ table, float* __restrict__ out, int E, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x; int id = tok[r]; if (id < 0 || id >= V) id = 0;
    const uint16_t* src = table + (size_t)id * E;
    for (int i = threadIdx.x; i < E; i += 256) out[(size_t)r * E + i] = bf2f(src[i]);
}

// ---- row norms. A cluster of 4 CTAs x 320 threads per row: thread t (0..1279 over the cluster) owns the 4-element
// groups t, t+1280, ... (128-bit accesses, kept in registers), so that the row's traffic is spread over four SMs.
// Sum of squares: per-thread fmaf chain over its elements in index order, xor tree inside each warp, then the 40 warp
// sums (warp index over the cluster) added in order by every thread after the cluster barrier. Quantisation: a
// 32-element sub-block is held by 8 consecutive lanes.
constexpr int NORM_CL = 4, NORM_TPB = 1280 / NORM_CL, NORM_ROWT = NORM_CL * NORM_TPB, NORM_NW = NORM_ROWT / 32, NORM_MAXG = 2;   // rows of up to 10240 elements
// warp part of the cluster-wide sum: leaves this warp's sum in slot (10 * rank + warp) of every CTA's table
__device__ __forceinline__ void norm_publish(float v, float* tab, int rank) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, off);
    const int lane = threadIdx.x & 31;
    if (lane < NORM_CL) st_cluster_f32(&tab[rank * (NORM_TPB / 32) + (threadIdx.x >> 5)], (uint32_t)lane, v);
}
__device__ __forceinline__ float norm_total(const float* tab) {
    float tot = tab[0];
#pragma unroll
    for (int i = 1; i < NORM_NW; ++i) tot = tot + tab[i];
    return tot;
}
// 4 consecutive activations of row r starting at element i0 (a multiple of 4), owned by one lane; the 8 lanes of a
// sub-block are consecutive. Same arithmetic as warp_quant32_store.
__device__ __forceinline__ void quant4_store(const float (&o)[4], int r, int i0, int K, int8_t* __restrict__ q, float* __restrict__ sc, int lane, bool live = true) {
    float amax = fmaxf(fmaxf(fabsf(o[0]), fabsf(o[1])), fmaxf(fabsf(o[2]), fabsf(o[3])));
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float dd = amax / 127.f, id = amax > 0.f ? 127.f / amax : 0.f;
    const int q0 = __float2int_rn(o[0] * id), q1 = __float2int_rn(o[1] * id), q2 = __float2int_rn(o[2] * id), q3 = __float2int_rn(o[3] * id);
    int sum = (q0 + q1) + (q2 + q3);
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (!live) return;   // every lane of the warp took part in the shuffles above
    *reinterpret_cast<uint32_t*>(q + xq_q_index(r, i0, K)) = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    if ((lane & 7) == 0) { const size_t di = xq_d_index(r, i0 >> 5, K); sc[di] = dd; sc[di + 2] = dd * (float)sum; }
}
__device__ __forceinline__ void bf4(const uint16_t* w, float (&o)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(w);
    o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xFFFF0000u); o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xFFFF0000u);
}

// ---- x += y (y = sum of P K-part planes in part order); xn = x * (1/sqrt(mean x^2 + eps)) * w; xq = q8(xn) ----
template <int PT, int NG>   // PT > 0: the number of planes, known at compile time so that every load is in flight at once; 0: run-time P. NG: groups per thread
__global__ void __cluster_dims__(NORM_CL, 1, 1) __launch_bounds__(NORM_TPB) k_add_rmsnorm_quant(float* __restrict__ x, const float* __restrict__ y, int P, size_t part_stride, int ldy,
                                                                     const uint16_t* __restrict__ w, float* __restrict__ xn, int8_t* __restrict__ q, float* __restrict__ sc,
                                                                     int n, float eps, int assign, const float* __restrict__ slotw, int nslot) {
    __shared__ float tab[NORM_NW];
    pdl_launch_dependents();
    cluster_arrive_relaxed();   // matched by cluster_wait() before the first store into another CTA
    const int rank = blockIdx.x % NORM_CL, r = blockIdx.x / NORM_CL, lane = threadIdx.x & 31, t = rank * NORM_TPB + threadIdx.x;
    float* xr = x + (size_t)r * n;
    float wv[NG][4];
#pragma unroll
    for (int k = 0; k < NG; ++k) { const int i = 4 * (t + k * NORM_ROWT); if (i < n) bf4(w + i, wv[k]); }   // weights do not depend on the previous kernel
    pdl_wait();
    float4 v[NG];
#pragma unroll
    for (int k = 0; k < NG; ++k) { const int i = 4 * (t + k * NORM_ROWT); v[k] = (i < n && !assign) ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f); }
    if (y) {
        float4 s[NG];
#pragma unroll
        for (int k = 0; k < NG; ++k) { const int i = 4 * (t + k * NORM_ROWT); s[k] = (i < n && !slotw) ? *reinterpret_cast<const float4*>(y + (size_t)r * ldy + i) : make_float4(0.f, 0.f, 0.f, 0.f); }
        if constexpr (PT > 0) {
            float4 u[PT > 1 ? PT - 1 : 1][NG];
#pragma unroll
            for (int p = 1; p < PT; ++p)
#pragma unroll
                for (int k = 0; k < NG; ++k) { const int i = 4 * (t + k * NORM_ROWT); u[p - 1][k] = i < n ? *reinterpret_cast<const float4*>(y + (size_t)p * part_stride + (size_t)r * ldy + i) : make_float4(0.f, 0.f, 0.f, 0.f); }
#pragma unroll
            for (int p = 1; p < PT; ++p)
#pragma unroll
                for (int k = 0; k < NG; ++k) { s[k].x = s[k].x + u[p - 1][k].x; s[k].y = s[k].y + u[p - 1][k].y; s[k].z = s[k].z + u[p - 1][k].z; s[k].w = s[k].w + u[p - 1][k].w; }
        } else if (slotw) {
            // MoE combine (gemv.hip:1104-1112): y holds one row per (row, slot) pair; acc = fmaf(weight, value, acc) in slot order
#pragma unroll
            for (int k = 0; k < NG; ++k) s[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int e = 0; e < nslot; ++e) {
                const float we = slotw[r * nslot + e];
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    const int i = 4 * (t + k * NORM_ROWT);
                    if (i < n) { const float4 uu = *reinterpret_cast<const float4*>(y + (size_t)(r * nslot + e) * ldy + i); s[k].x = fmaf(we, uu.x, s[k].x); s[k].y = fmaf(we, uu.y, s[k].y); s[k].z = fmaf(we, uu.z, s[k].z); s[k].w = fmaf(we, uu.w, s[k].w); }
                }
            }
        } else {
            for (int p = 1; p < P; ++p)
#pragma unroll
                for (int k = 0; k < NG; ++k) {
                    const int i = 4 * (t + k * NORM_ROWT);
                    if (i < n) { const float4 uu = *reinterpret_cast<const float4*>(y + (size_t)p * part_stride + (size_t)r * ldy + i); s[k].x = s[k].x + uu.x; s[k].y = s[k].y + uu.y; s[k].z = s[k].z + uu.z; s[k].w = s[k].w + uu.w; }
                }
        }
#pragma unroll
        for (int k = 0; k < NG; ++k) {
            const int i = 4 * (t + k * NORM_ROWT);
            if (i < n) {
                if (assign) v[k] = s[k];   // x = y exactly (no 0 + y: it would turn -0 into +0)
                else { v[k].x = v[k].x + s[k].x; v[k].y = v[k].y + s[k].y; v[k].z = v[k].z + s[k].z; v[k].w = v[k].w + s[k].w; }
                *reinterpret_cast<float4*>(xr + i) = v[k];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NG; ++k) { ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss); }   // absent groups hold zeros
    cluster_wait();
    norm_publish(ss, tab, rank);
    cluster_sync_all();
    ss = norm_total(tab);
    const float scl = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int k = 0; k < NG; ++k) {
        const int i = 4 * (t + k * NORM_ROWT);
        const bool live = i < n;   // n is a multiple of 32: the 8 lanes of a sub-block are live together; dead lanes still shuffle
        const float o[4] = {live ? (v[k].x * scl) * wv[k][0] : 0.f, live ? (v[k].y * scl) * wv[k][1] : 0.f, live ? (v[k].z * scl) * wv[k][2] : 0.f, live ? (v[k].w * scl) * wv[k][3] : 0.f};
        if (live && xn) *reinterpret_cast<float4*>(xn + (size_t)r * n + i) = make_float4(o[0], o[1], o[2], o[3]);
        quant4_store(o, r, i, n, q, sc, lane, live);
    }
}

// ---- MTP input: out[r] = [rmsnorm(a[r]) * wa | rmsnorm(b[r]) * wb], quantised (ops.hip:99-116) ----
template <int NG>
__global__ void __cluster_dims__(NORM_CL, 1, 1) __launch_bounds__(NORM_TPB) k_norm2_concat_quant(const float* __restrict__ a, const uint16_t* __restrict__ wa, const float* __restrict__ b, int ldb,
                                                                      const uint16_t* __restrict__ wb, float* __restrict__ out, int8_t* __restrict__ q, float* __restrict__ sc,
                                                                      int n, float eps) {
    __shared__ float taba[NORM_NW], tabb[NORM_NW];
    pdl_launch_dependents();
    cluster_arrive_relaxed();
    const int rank = blockIdx.x % NORM_CL, r = blockIdx.x / NORM_CL, lane = threadIdx.x & 31, t = rank * NORM_TPB + threadIdx.x;
    float wav[NG][4], wbv[NG][4];
#pragma unroll
    for (int k = 0; k < NG; ++k) { const int i = 4 * (t + k * NORM_ROWT); if (i < n) { bf4(wa + i, wav[k]); bf4(wb + i, wbv[k]); } }
    pdl_wait();
    const float* ar = a + (size_t)r * n; const float* br = b + (size_t)r * ldb;
    float4 va[NG], vb[NG];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int k = 0; k < NG; ++k) {
        const int i = 4 * (t + k * NORM_ROWT);
        va[k] = i < n ? *reinterpret_cast<const float4*>(ar + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        vb[k] = i < n ? *reinterpret_cast<const float4*>(br + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < NG; ++k) {
        sa = fmaf(va[k].x, va[k].x, sa); sa = fmaf(va[k].y, va[k].y, sa); sa = fmaf(va[k].z, va[k].z, sa); sa = fmaf(va[k].w, va[k].w, sa);
        sb = fmaf(vb[k].x, vb[k].x, sb); sb = fmaf(vb[k].y, vb[k].y, sb); sb = fmaf(vb[k].z, vb[k].z, sb); sb = fmaf(vb[k].w, vb[k].w, sb);
    }
    cluster_wait();
    norm_publish(sa, taba, rank); norm_publish(sb, tabb, rank);
    cluster_sync_all();
    const float ca = 1.0f / sqrtf(norm_total(taba) / (float)n + eps), cb = 1.0f / sqrtf(norm_total(tabb) / (float)n + eps);
#pragma unroll
    for (int k = 0; k < NG; ++k) {
        const int i = 4 * (t + k * NORM_ROWT);
        const bool live = i < n;
        const float oa[4] = {live ? (va[k].x * ca) * wav[k][0] : 0.f, live ? (va[k].y * ca) * wav[k][1] : 0.f, live ? (va[k].z * ca) * wav[k][2] : 0.f, live ? (va[k].w * ca) * wav[k][3] : 0.f};
        const float ob[4] = {live ? (vb[k].x * cb) * wbv[k][0] : 0.f, live ? (vb[k].y * cb) * wbv[k][1] : 0.f, live ? (vb[k].z * cb) * wbv[k][2] : 0.f, live ? (vb[k].w * cb) * wbv[k][3] : 0.f};
        if (live && out) {
            *reinterpret_cast<float4*>(out + (size_t)r * 2 * n + i) = make_float4(oa[0], oa[1], oa[2], oa[3]);
            *reinterpret_cast<float4*>(out + (size_t)r * 2 * n + n + i) = make_float4(ob[0], ob[1], ob[2], ob[3]);
        }
        quant4_store(oa, r, i, 2 * n, q, sc, lane, live);
        quant4_store(ob, r, n + i, 2 * n, q, sc, lane, live);
    }
}

// ---- xq = q8(silu(gate) * up); gate = columns [0, F), up = [F, 2F) of gu [R][ldg] (ops.hip:146-151) ----
// one thread per 4 consecutive features (128-bit loads), 8 consecutive lanes per 32-element sub-block
__global__ void __launch_bounds__(256) k_silu_mul_quant(const float* __restrict__ gu, int ldg, int F, int8_t* __restrict__ q, float* __restrict__ sc) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, i = (blockIdx.x * 256 + threadIdx.x) * 4, lane = threadIdx.x & 31;
    const bool live = i < F;   // F is a multiple of 32: the 8 lanes of a sub-block are live together
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 g = live ? *reinterpret_cast<const float4*>(gu + (size_t)r * ldg + i) : z4, u = live ? *reinterpret_cast<const float4*>(gu + (size_t)r * ldg + F + i) : z4;
    const float o[4] = {silu_det(g.x) * u.x, silu_det(g.y) * u.y, silu_det(g.z) * u.z, silu_det(g.w) * u.w};
    quant4_store(o, r, i, F, q, sc, lane, live);
}

// ---- Gated DeltaNet: causal 4-tap depthwise conv + SiLU, then the gated delta rule, for one (v-head, sequence) ----
// A cluster of 4 CTAs per (v-head, sequence); CTA `rank` owns value rows 32*rank .. 32*rank+31 of the head's state
// M[j][i] (j = value row, i = key index). 256 threads: thread tid holds columns 16*(tid&7) .. +15 of row 32*rank + tid/8
// in registers, read and written straight from / to HBM (a warp covers 2 KB of consecutive state). Every CTA convolves
// and normalises the head's 128 q and 128 k channels itself (thread tid: q channel tid, or k channel tid-128) and its
// own 32 v channels (threads 0..31).
// Rows are processed in order: first `n_replay` rows of the previous pass (their raw inputs were saved per head by
// that pass; no output) -- this is the deferred commit of the accepted prefix: the state and conv history reached
// after them are written back --, then the T new rows (outputs only; state stays in registers, optional snapshots),
// whose raw inputs are saved in turn. The saved rows and the history are shared by the cluster: a cluster barrier
// separates everybody's reads from the writes (q|k parts written by rank 0, v parts by their owner).
// Row math (ops.hip:221-250): q,k <- x / max(||x||, eps); beta = sigmoid(b); decay = exp(a_neg * softplus(alpha + dt));
// M *= decay; dot_j = sum_i M[j][i] k[i]; delta_j = (v_j - dot_j) beta; M[j][i] += delta_j k[i];
// o_j = sum_i M[j][i] q[i] / sqrt(128); out = rmsnorm_128(o) * w * gate(z). Sums over i: fmaf chain over the thread's
// 16 columns in index order, the 8 partial sums combined by an xor tree (1, 2, 4); sums over 128 channels: xor tree
// inside each warp of 32 channels, the four warp sums added in channel order.
struct GdnArgs {
    const float* rows; int ld;                                    // merged GEMV output [rows][ld]: qkv | z | beta | alpha
    float* saved; size_t saved_stride;                            // per slot: [n_v][8 rows][388]: raw q|k|v channels, beta, alpha of the last pass
    int off_z, off_b, off_a;                                      // column offsets inside a row
    int n_qk, n_v;                                                // heads (dim 128)
    const float* conv_w; const uint16_t* dt_bias; const uint16_t* a_neg; const uint16_t* norm_w;   // conv_w f32 [C][4]
    float* state; float* conv_state; size_t state_stride, conv_stride;   // per slot: [n_v][128][128], [n_v][3][384] (each v-head keeps its own q|k|v history)
    const int* seq;                                               // device descriptors: per sequence {r0, T, slot, -}
    const int* replay_n;                                          // device: rows of the previous pass to commit, per slot
    int imm_T, imm_replay;                                        // used instead when seq == nullptr (a single sequence described by value)
    float* out; int8_t* oq; float* osc;                           // out f32 [rows][n_v*128] (nullable), quantised out
    float* snap; size_t snap_row_stride;                          // optional state snapshots after each new row
    float eps; int sigmoid_gate;
};
constexpr int GDN_MAXROWS = 16, GDN_CL = 4;   // replayed rows (<= 8) + new rows (<= 8) of one sequence; CTAs per head
__device__ __forceinline__ float2 gdn_mul2(float2 a, float2 b) {
    float2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(r)) : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return r;
}
__device__ __forceinline__ float2 gdn_fma2(float2 a, float2 b, float2 c) {   // a * b + c per lane, one rounding each
    float2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(r))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)), "l"(reinterpret_cast<unsigned long long&>(c)));
    return r;
}
// MINB = resident CTAs per SM the register budget is cut for: 3 (80 registers) for one or two sequences (one wave either
// way), 4 (64 registers, a few bytes of spills) for passes over several sequences, where the grid runs in several waves
// of this latency-bound kernel and a fourth CTA per SM shortens them. Same instructions, same results.
template <int MINB>
__global__ void __cluster_dims__(GDN_CL, 1, 1) __launch_bounds__(256, MINB) k_gdn(GdnArgs a) {
    constexpr int D = 128, NLD = 8, NCV = 6;   // items per thread: (16 + 3) * 96 <= 8 * 256 raw values, 16 * 96 = 6 * 256 conv outputs
    // conv'ed, then normalised q | k of every row (filled by all four CTAs); 16-float chunks padded to 20 so that the
    // eight chunk owners of a state row read 128 bits each from distinct banks
    __shared__ __align__(16) float sqk[GDN_MAXROWS][2 * 160];
    __shared__ float raw[GDN_MAXROWS + 3][96], sv[GDN_MAXROWS][32], sout[8][32];
    __shared__ float csum[GDN_MAXROWS][2][GDN_CL], snrm[GDN_MAXROWS][2], sbeta[GDN_MAXROWS], sdecay[GDN_MAXROWS];
    __shared__ float cred[8][GDN_CL];
    pdl_launch_dependents();
    cluster_arrive_relaxed();   // matched by cluster_wait() before the first store into another CTA: every CTA has started by then
    const int rank = blockIdx.x % GDN_CL, h = blockIdx.x / GDN_CL, hk = h % a.n_qk, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Item e = tid + 256 k of this thread is (row index e / 96, local channel c = e % 96) both for the raw loads and for
    // the conv outputs. Local channel c: group c/32 = q, k, v; channel 32*rank + c%32 of the head. Its slot in a
    // history / saved row, its column in a row of the merged projection, its conv taps (independent of the predecessor):
    int e_rr[NLD], e_c[NLD], e_slot[NLD], e_col[NLD];
    float4 cw[NCV];
#pragma unroll
    for (int k = 0; k < NLD; ++k) {
        const int e = tid + 256 * k, rr = e / 96, c = e - rr * 96, g3 = c >> 5, cl = 32 * rank + (c & 31);
        e_rr[k] = rr; e_c[k] = c; e_slot[k] = g3 * D + cl;
        e_col[k] = g3 == 0 ? hk * D + cl : g3 == 1 ? a.n_qk * D + hk * D + cl : 2 * a.n_qk * D + h * D + cl;
        if (k < NCV) cw[k] = *reinterpret_cast<const float4*>(a.conv_w + (size_t)e_col[k] * 4);
    }
    const float nw = bf2f(a.norm_w[32 * rank + lane]);
    pdl_wait();
    const int r0 = a.seq ? a.seq[blockIdx.y * 4 + 0] : 0, T = min(a.seq ? a.seq[blockIdx.y * 4 + 1] : a.imm_T, 8), slot = a.seq ? a.seq[blockIdx.y * 4 + 2] : 0;
    float* sav = a.saved + (size_t)slot * a.saved_stride + (size_t)h * 8 * 388;   // [8][q 128 | k 128 | v 128 | beta | alpha | pad]
    const int jl = tid >> 3, ck = tid & 7, j = 32 * rank + jl;
    float* Mrow = a.state + (size_t)slot * a.state_stride + ((size_t)h * D + j) * D + 16 * ck;
    float2 m[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2) { const float4 v = *reinterpret_cast<const float4*>(Mrow + 2 * i); m[i] = make_float2(v.x, v.y); m[i + 1] = make_float2(v.z, v.w); }
    auto commit_state = [&]() {
#pragma unroll
        for (int i = 0; i < 8; i += 2) *reinterpret_cast<float4*>(Mrow + 2 * i) = make_float4(m[i].x, m[i].y, m[i + 1].x, m[i + 1].y);
    };
    // conv history of this head: [3 taps][q 128 | k 128 | v 128]; private per v-head
    float* cst = a.conv_state + (size_t)slot * a.conv_stride + (size_t)h * 3 * 384;
    const int Z = a.n_v * D;
    // gate input z of this lane's channel for the row that warp `warp` finishes in phase 3
    const float zz = warp < T ? a.rows[(size_t)(r0 + warp) * a.ld + a.off_z + h * D + 32 * rank + lane] : 0.f;

    // ---- phase 1: history (3 taps) + raw inputs of all rows -> raw[tap or 3 + row][c]. The history and the new rows do
    // not depend on the replay count: their loads go out first, together with the load of the count itself; the saved
    // rows of the accepted prefix follow once the count is known.
    constexpr int NLA = 5, NLB = 3;   // (8 + 3) * 96 <= 5 * 256 history + new values, 8 * 96 = 3 * 256 replayed values
    float tmpa[NLA], tmpb[NLB];
#pragma unroll
    for (int k = 0; k < NLA; ++k) {
        const int rr = e_rr[k];
        if (rr < T + 3) tmpa[k] = rr < 3 ? cst[rr * 384 + e_slot[k]] : a.rows[(size_t)(r0 + rr - 3) * a.ld + e_col[k]];
    }
    const int nrep = min(a.seq ? (a.replay_n ? a.replay_n[slot] : 0) : a.imm_replay, 8);
    const int nrows = nrep + T;
#pragma unroll
    for (int k = 0; k < NLB; ++k) { const int it = e_rr[k]; if (it < nrep) tmpb[k] = sav[it * 388 + e_slot[k]]; }
#pragma unroll
    for (int k = 0; k < NLA; ++k) { const int rr = e_rr[k]; if (rr < T + 3) raw[rr < 3 ? rr : rr + nrep][e_c[k]] = tmpa[k]; }
#pragma unroll
    for (int k = 0; k < NLB; ++k) { const int it = e_rr[k]; if (it < nrep) raw[3 + it][e_c[k]] = tmpb[k]; }
    // gates of every row (all four CTAs compute them: no exchange), by the last warp, which has the fewest conv items
    float raw_b = 0.f, raw_a = 0.f;
    if (warp == 7 && lane < nrows) {
        const bool replay = lane < nrep;
        const float* row = a.rows + (size_t)(replay ? 0 : r0 + (lane - nrep)) * a.ld;
        raw_b = replay ? sav[lane * 388 + 384] : row[a.off_b + h];
        raw_a = replay ? sav[lane * 388 + 385] : row[a.off_a + h];
        sbeta[lane] = sigmoid_det(raw_b);
        sdecay[lane] = expf_det(bf2f(a.a_neg[h]) * softplus_det(raw_a + bf2f(a.dt_bias[h])));
    }
    __syncthreads();
    // Every CTA reads and writes only its own channels of the saved rows and of the history, so they can be rewritten at
    // once: raw inputs of the new rows for a later commit, history after the accepted prefix. (beta / alpha are read by
    // all four CTAs and rewritten by rank 0 after the first cluster barrier.)
#pragma unroll
    for (int k = 0; k < 3; ++k) { const int t = e_rr[k]; if (t < T) sav[t * 388 + e_slot[k]] = raw[3 + nrep + t][e_c[k]]; }
    if (nrep > 0) {
#pragma unroll
        for (int k = 0; k < 2; ++k) { const int tap = e_rr[k]; if (tap < 3) cst[tap * 384 + e_slot[k]] = raw[nrep + tap][e_c[k]]; }
    }
    cluster_wait();
    // conv + SiLU of every (row, channel) independently. q and k go to all four CTAs; their squared l2 norms: xor tree
    // over the warp's 32 channels, the warp sum goes to all four CTAs (slot = this CTA's rank)
#pragma unroll
    for (int k = 0; k < NCV; ++k) {
        const int it = e_rr[k], c = e_c[k];
        if (it < nrows) {   // warp-uniform: a warp covers one group of one row
            const float4 w = cw[k];
            float t = w.x * raw[it][c]; t = fmaf(w.y, raw[it + 1][c], t); t = fmaf(w.z, raw[it + 2][c], t); t = fmaf(w.w, raw[it + 3][c], t);
            const float v = silu_det(t);
            if (c >= 64) sv[it][c - 64] = v;
            else {
                const int g2 = c >> 5, ch = 32 * rank + (c & 31);
                float* dst = &sqk[it][g2 * 160 + (ch >> 4) * 20 + (ch & 15)];
#pragma unroll
                for (int r = 0; r < GDN_CL; ++r) st_cluster_f32(dst, r, v);
                float p = v * v;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) p = p + __shfl_xor_sync(0xffffffffu, p, off);
                if (lane < GDN_CL) st_cluster_f32(&csum[it][g2][rank], (uint32_t)lane, p);
            }
        }
    }
    cluster_sync_all();
    if (rank == 0 && warp == 7 && lane >= nrep && lane < nrows) { sav[(lane - nrep) * 388 + 384] = raw_b; sav[(lane - nrep) * 388 + 385] = raw_a; }
    if (tid < 2 * nrows) {
        const float* cs = &csum[tid >> 1][tid & 1][0];
        float tot = cs[0]; tot = tot + cs[1]; tot = tot + cs[2]; tot = tot + cs[3];
        snrm[tid >> 1][tid & 1] = fmaxf(sqrtf(tot), a.eps);
    }
    __syncthreads();
    {   // normalise q | k of every row in place: thread tid owns channel tid (q for tid < 128, k otherwise)
        const int off = (tid >> 7) * 160 + ((tid & 127) >> 4) * 20 + (tid & 15);
#pragma unroll 4
        for (int it = 0; it < nrows; ++it) sqk[it][off] = sqk[it][off] / snrm[it][tid >> 7];
    }
    __syncthreads();

    // ---- phase 2: the recurrence, row after row, state in registers; no block-wide synchronisation inside
    for (int it = 0; it < nrows; ++it) {
        if (it == nrep && nrep > 0) commit_state();
        const float beta = sbeta[it], decay = sdecay[it];
        const float* kk = &sqk[it][160 + 20 * ck]; const float* qq = &sqk[it][20 * ck];
        float2 kr[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2) { const float4 v = *reinterpret_cast<const float4*>(kk + 2 * i); kr[i] = make_float2(v.x, v.y); kr[i + 1] = make_float2(v.z, v.w); }
        const float2 dc2 = make_float2(decay, decay);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { m[i] = gdn_mul2(m[i], dc2); dot = fmaf(m[i].x, kr[i].x, dot); dot = fmaf(m[i].y, kr[i].y, dot); }
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) dot = dot + __shfl_xor_sync(0xffffffffu, dot, off);
        const float delta = (sv[it][jl] - dot) * beta;
        const float2 dl2 = make_float2(delta, delta);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const float4 qv = *reinterpret_cast<const float4*>(qq + 2 * i);
            m[i] = gdn_fma2(dl2, kr[i], m[i]); o = fmaf(m[i].x, qv.x, o); o = fmaf(m[i].y, qv.y, o);
            m[i + 1] = gdn_fma2(dl2, kr[i + 1], m[i + 1]); o = fmaf(m[i + 1].x, qv.z, o); o = fmaf(m[i + 1].y, qv.w, o);
        }
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) o = o + __shfl_xor_sync(0xffffffffu, o, off);
        if (it >= nrep) {
            if (ck == 0) sout[it - nrep][jl] = o * 0.08838834764831845f;
            if (a.snap) {
                float* sp = a.snap + (size_t)(it - nrep) * a.snap_row_stride + ((size_t)h * D + j) * D + 16 * ck;
#pragma unroll
                for (int i = 0; i < 8; i += 2) *reinterpret_cast<float4*>(sp + 2 * i) = make_float4(m[i].x, m[i].y, m[i + 1].x, m[i + 1].y);
            }
        }
    }
    if (T == 0 && nrep > 0) commit_state();
    __syncthreads();

    // ---- phase 3: per-head RMSNorm * w * gate(z) + quantisation of the new rows; warp t takes row t, lane = channel.
    // The sum of squares over the head's 128 channels: every CTA sends its warp sum to all four CTAs of the cluster.
    if (warp < T) {
        float ps = sout[warp][lane] * sout[warp][lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ps = ps + __shfl_xor_sync(0xffffffffu, ps, off);
        if (lane < GDN_CL) st_cluster_f32(&cred[warp][rank], (uint32_t)lane, ps);
    }
    const float gate = warp < T ? (a.sigmoid_gate ? sigmoid_det(zz) : silu_det(zz)) : 0.f;
    cluster_sync_all();
    if (warp < T) {
        float ss = cred[warp][0]; ss = ss + cred[warp][1]; ss = ss + cred[warp][2]; ss = ss + cred[warp][3];
        const int row = r0 + warp, c = 32 * rank + lane;
        const size_t oi = (size_t)row * Z + h * D + c;
        const float v = ((sout[warp][lane] * (1.0f / sqrtf(ss / (float)D + a.eps))) * nw) * gate;
        if (a.out) a.out[oi] = v;
        if (a.oq) warp_quant32_store(v, row, (h * D + c) >> 5, Z, a.oq, a.osc, lane);
    }
}

}  // namespace

int embed_bf16(const int* tok, const void* table, float* out, int R, int E, int V, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && E > 0 && V > 0, "embed_bf16: bad shape");
    HP_CUDA(launch_pdl<16>(k_embed_bf16, dim3(R), dim3(256), 0, s, tok, (const uint16_t*)table, out, E, V));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int add_rmsnorm_quant(float* x, const float* y, int P, size_t part_stride, int ldy, const void* w_bf16, float* xn, XQ8F xq, int R, int n, float eps, cudaStream_t s, bool assign,
                      const float* slotw, int nslot) {
    HP_REQUIRE(!assign || y, "add_rmsnorm_quant: assign needs planes");
    HP_REQUIRE(!slotw || (y && nslot >= 1), "add_rmsnorm_quant: the slot-weighted form needs the per-pair rows");
    HP_REQUIRE(R >= 1 && n > 0 && n % 64 == 0, "add_rmsnorm_quant: n=%d must be a positive multiple of 64", n);
    HP_REQUIRE(n <= NORM_ROWT * 4 * NORM_MAXG, "add_rmsnorm_quant: n=%d exceeds %d", n, NORM_ROWT * 4 * NORM_MAXG);
    HP_REQUIRE(!y || (ldy % 4 == 0 && part_stride % 4 == 0), "add_rmsnorm_quant: plane strides must be multiples of 4 floats");
    const int pt = slotw ? 0 : !y || P == 1 ? 1 : P == 2 ? 2 : P == 4 ? 4 : 0;
    auto pick = [&](auto ng_tag) {
        constexpr int NG = decltype(ng_tag)::value;
        return pt == 1 ? k_add_rmsnorm_quant<1, NG> : pt == 2 ? k_add_rmsnorm_quant<2, NG> : pt == 4 ? k_add_rmsnorm_quant<4, NG> : k_add_rmsnorm_quant<0, NG>;
    };
    auto kern = n <= NORM_ROWT * 4 ? pick(std::integral_constant<int, 1>()) : pick(std::integral_constant<int, NORM_MAXG>());
    HP_CUDA(launch_pdl(kern, dim3(R * NORM_CL), dim3(NORM_TPB), 0, s, x, y, P, part_stride, ldy, (const uint16_t*)w_bf16, xn, (int8_t*)xq.q, (float*)xq.sc, n, eps, assign ? 1 : 0, slotw, nslot));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int norm2_concat_quant(const float* a, const void* wa, const float* b, int ldb, const void* wb, float* out, XQ8F xq, int R, int n, float eps, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n > 0 && n % 64 == 0 && ldb % 4 == 0, "norm2_concat_quant: n=%d must be a positive multiple of 64 (ldb a multiple of 4)", n);
    HP_REQUIRE(n <= NORM_ROWT * 4 * NORM_MAXG, "norm2_concat_quant: n=%d exceeds %d", n, NORM_ROWT * 4 * NORM_MAXG);
    auto kern = n <= NORM_ROWT * 4 ? k_norm2_concat_quant<1> : k_norm2_concat_quant<NORM_MAXG>;
    HP_CUDA(launch_pdl(kern, dim3(R * NORM_CL), dim3(NORM_TPB), 0, s, a, (const uint16_t*)wa, b, ldb, (const uint16_t*)wb, out, (int8_t*)xq.q, (float*)xq.sc, n, eps));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int silu_mul_quant(const float* gu, int ldg, int F, XQ8F xq, int R, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && F > 0 && F % 64 == 0 && ldg >= 2 * F, "silu_mul_quant: bad shape F=%d ldg=%d", F, ldg);
    HP_REQUIRE(ldg % 4 == 0, "silu_mul_quant: ldg must be a multiple of 4");
    launch_pdl<256>(k_silu_mul_quant, dim3((F / 4 + 255) / 256, R), dim3(256), 0, s, gu, ldg, F, (int8_t*)xq.q, (float*)xq.sc);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int gdn_forward(const GdnParams& p, int nseq, cudaStream_t s) {
    HP_REQUIRE(nseq >= 1 && nseq <= 8 && p.n_qk >= 1 && p.n_v >= p.n_qk, "gdn_forward: bad shape");
    GdnArgs a;
    a.rows = p.rows; a.saved = p.saved; a.saved_stride = p.saved_stride; a.ld = p.ld; a.off_z = p.off_z; a.off_b = p.off_b; a.off_a = p.off_a;
    a.n_qk = p.n_qk; a.n_v = p.n_v; a.conv_w = p.conv_w; a.dt_bias = (const uint16_t*)p.dt_bias; a.a_neg = (const uint16_t*)p.a_neg; a.norm_w = (const uint16_t*)p.norm_w;
    a.state = p.state; a.conv_state = p.conv_state; a.state_stride = p.state_stride; a.conv_stride = p.conv_stride;
    a.seq = p.seq; a.replay_n = p.replay_n; a.imm_T = p.imm_T; a.imm_replay = p.imm_replay; a.out = p.out; a.oq = (int8_t*)p.xq.q; a.osc = (float*)p.xq.sc;
    a.snap = p.snap; a.snap_row_stride = p.snap_row_stride; a.eps = p.eps; a.sigmoid_gate = p.sigmoid_gate;
    if (nseq >= 3) HP_CUDA(launch_pdl<128>(k_gdn<4>, dim3(p.n_v * GDN_CL, nseq), dim3(256), 0, s, a));
    else HP_CUDA(launch_pdl<128>(k_gdn<3>, dim3(p.n_v * GDN_CL, nseq), dim3(256), 0, s, a));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

}  // namespace hp
