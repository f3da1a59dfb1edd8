// Layer kernels of the decode / verify pass other than the GEMV: embedding gather, fused residual-add + RMSNorm +
// int8 quantisation, MTP input (two norms concatenated), SiLU-gated product + quantisation, and the Gated-DeltaNet
// short convolution + delta-rule recurrence with deferred commit ("rollback") and optional per-row state snapshots.
//
// Reference: engine/kernels/ops.hip -- k_add_rmsnorm_quant (:79-98), k_norm2_concat_quant (:99-116),
// k_silu_mul_quant (:146-151), k_embed_q4_K (:154-171), k_gdn_conv (:188-202), k_gdn_step (:205-256); replay buffers and
// Qwen35::accept (engine/src/qwen35.cpp:383-403).
//
// Every reduction has a fixed order (stated at each kernel) so that the CPU oracle reproduces the results bit for bit.
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
    const int r = blockIdx.x; int id = tok[r]; if (id < 0 || id >= V) id = 0;
    const uint16_t* src = table + (size_t)id * E;
    for (int i = threadIdx.x; i < E; i += 256) out[(size_t)r * E + i] = bf2f(src[i]);
}

// ---- x += y (y = sum of P K-part planes in part order); xn = x * (1/sqrt(mean x^2 + eps)) * w; xq = q8(xn) ----
// One 1024-thread block per row. Thread i owns elements i, i+1024, ... (kept in registers); sum of squares: per-thread
// fmaf chain in that order, then block_sum_det over the 32 warps. Quantisation per 32 consecutive elements (one warp).
constexpr int NORM_THREADS = 1024, NORM_MAXE = 10;   // rows of up to 10240 elements
__global__ void __launch_bounds__(NORM_THREADS) k_add_rmsnorm_quant(float* __restrict__ x, const float* __restrict__ y, int P, size_t part_stride, int ldy,
                                                                     const uint16_t* __restrict__ w, float* __restrict__ xn, int8_t* __restrict__ q, float* __restrict__ sc,
                                                                     int n, float eps) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    const int r = blockIdx.x, lane = threadIdx.x & 31;
    float* xr = x + (size_t)r * n;
    float wv[NORM_MAXE];
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; wv[k] = i < n ? bf2f(w[i]) : 0.f; }   // weights do not depend on the previous kernel
    pdl_wait();
    float v[NORM_MAXE];
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; v[k] = i < n ? xr[i] : 0.f; }
    if (y) {
        float s[NORM_MAXE];
#pragma unroll
        for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; s[k] = i < n ? y[(size_t)r * ldy + i] : 0.f; }
        for (int p = 1; p < P; ++p)
#pragma unroll
            for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; if (i < n) s[k] = s[k] + y[(size_t)p * part_stride + (size_t)r * ldy + i]; }
#pragma unroll
        for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; if (i < n) { v[k] = v[k] + s[k]; xr[i] = v[k]; } }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; if (i < n) ss = fmaf(v[k], v[k], ss); }
    ss = block_sum_det<32>(ss, sh);
    const float scl = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < n) {   // n is a multiple of 32: a warp is wholly inside or wholly outside
            const float o = (v[k] * scl) * wv[k];
            if (xn) xn[(size_t)r * n + i] = o;
            warp_quant32_store(o, r, i >> 5, n, q, sc, lane);
        }
    }
}

// ---- MTP input: out[r] = [rmsnorm(a[r]) * wa | rmsnorm(b[r]) * wb], quantised (ops.hip:99-116) ----
__global__ void __launch_bounds__(NORM_THREADS) k_norm2_concat_quant(const float* __restrict__ a, const uint16_t* __restrict__ wa, const float* __restrict__ b, int ldb,
                                                                      const uint16_t* __restrict__ wb, float* __restrict__ out, int8_t* __restrict__ q, float* __restrict__ sc,
                                                                      int n, float eps) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, lane = threadIdx.x & 31;
    const float* ar = a + (size_t)r * n; const float* br = b + (size_t)r * ldb;
    float va[NORM_MAXE], vb[NORM_MAXE];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; va[k] = i < n ? ar[i] : 0.f; vb[k] = i < n ? br[i] : 0.f; }
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) { const int i = threadIdx.x + k * NORM_THREADS; if (i < n) { sa = fmaf(va[k], va[k], sa); sb = fmaf(vb[k], vb[k], sb); } }
    sa = block_sum_det<32>(sa, sh); sb = block_sum_det<32>(sb, sh);
    const float ca = 1.0f / sqrtf(sa / (float)n + eps), cb = 1.0f / sqrtf(sb / (float)n + eps);
#pragma unroll
    for (int k = 0; k < NORM_MAXE; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < n) {
            const float oa = (va[k] * ca) * bf2f(wa[i]), ob = (vb[k] * cb) * bf2f(wb[i]);
            if (out) { out[(size_t)r * 2 * n + i] = oa; out[(size_t)r * 2 * n + n + i] = ob; }
            warp_quant32_store(oa, r, i >> 5, 2 * n, q, sc, lane);
            warp_quant32_store(ob, r, (n + i) >> 5, 2 * n, q, sc, lane);
        }
    }
}

// ---- xq = q8(silu(gate) * up); gate = columns [0, F), up = [F, 2F) of gu [R][ldg] (ops.hip:146-151) ----
__global__ void __launch_bounds__(256) k_silu_mul_quant(const float* __restrict__ gu, int ldg, int F, int8_t* __restrict__ q, float* __restrict__ sc) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, sb = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (sb * 32 >= F) return;
    const int i = sb * 32 + lane;
    const float g = gu[(size_t)r * ldg + i], u = gu[(size_t)r * ldg + F + i];
    warp_quant32_store(silu_det(g) * u, r, sb, F, q, sc, lane);
}

// ---- Gated DeltaNet: causal 4-tap depthwise conv + SiLU, then the gated delta rule, for one (v-head, sequence) ----
// 256 threads. Threads 0..127 own q channel c and k channel c of q/k head hk = h % n_qk, threads 128..255 own v channel
// c of head h. State M[j][i] (j = value row, i = key index): thread tid holds row j = tid/2, columns 64*(tid&1)..+63.
// Rows are processed in order: first `n_replay` rows of the previous pass (their raw inputs were saved per head by
// that pass; no output) -- this is the deferred commit of the accepted prefix: the state and conv history reached
// after them are written back --, then the T new rows (outputs only; state stays in registers, optional snapshots),
// whose raw inputs are saved in turn.
// Row math (ops.hip:221-250): q,k <- x / max(||x||, eps); beta = sigmoid(b); decay = exp(a_neg * softplus(alpha + dt));
// M *= decay; dot_j = sum_i M[j][i] k[i]; delta_j = (v_j - dot_j) beta; M[j][i] += delta_j k[i];
// o_j = sum_i M[j][i] q[i] / sqrt(128); out = rmsnorm_128(o) * w * gate(z). Sums over i: fmaf chain over the thread's
// 64 columns in index order, the two halves added; sums over 128 channels: block_sum_det.
struct GdnArgs {
    const float* rows; int ld;                                    // merged GEMV output [rows][ld]: qkv | z | beta | alpha
    float* saved; size_t saved_stride;                            // per slot: [n_v][8 rows][388]: raw q|k|v channels, beta, alpha of the last pass
    int off_z, off_b, off_a;                                      // column offsets inside a row
    int n_qk, n_v;                                                // heads (dim 128)
    const float* conv_w; const uint16_t* dt_bias; const uint16_t* a_neg; const uint16_t* norm_w;   // conv_w f32 [C][4]
    float* state; float* conv_state; size_t state_stride, conv_stride;   // per slot: [n_v][128][128], [n_v][3][384] (each v-head keeps its own q|k|v history)
    const int* seq;                                               // device descriptors: per sequence {r0, T, slot, -}
    const int* replay_n;                                          // device: rows of the previous pass to commit, per slot
    float* out; int8_t* oq; float* osc;                           // out f32 [rows][n_v*128] (nullable), quantised out
    float* snap; size_t snap_row_stride;                          // optional state snapshots after each new row
    float eps; int sigmoid_gate;
};
constexpr int GDN_MAXROWS = 16, GDN_STG_LD = 132;   // replayed rows (<= 8) + new rows (<= 8) of one sequence
__global__ void __launch_bounds__(256) k_gdn(GdnArgs a) {
    constexpr int D = 128;
    __shared__ __align__(16) float sall[GDN_MAXROWS][3 * D], sout[8][D];
    __shared__ float red[GDN_MAXROWS * 2][8], tot[GDN_MAXROWS * 2], sbeta[GDN_MAXROWS], sdecay[GDN_MAXROWS], sraw_b[GDN_MAXROWS], sraw_a[GDN_MAXROWS];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, hk = h % a.n_qk, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = a.seq[blockIdx.y * 4 + 0], T = min(a.seq[blockIdx.y * 4 + 1], 8), slot = a.seq[blockIdx.y * 4 + 2];
    float* sav = a.saved + (size_t)slot * a.saved_stride + (size_t)h * 8 * 388;   // [8][q 128 | k 128 | v 128 | beta | alpha | pad]
    const int nrep = a.replay_n ? min(a.replay_n[slot], 8) : 0;
    const int nrows = nrep + T;
    const int Z = a.n_v * D;
    const int j = tid >> 1, ih = tid & 1;
    // conv history of this head: [3 taps][q 128 | k 128 | v 128]; private per v-head so that no CTA reads what another writes
    float* cst = a.conv_state + (size_t)slot * a.conv_stride + (size_t)h * 3 * 384;
    const int sa_ = tid < D ? tid : D + tid, sb_ = D + (tid & (D - 1));   // history / saved-row slots of channels ca / cb
    // the 64 KB state of this head moves between HBM and registers through shared memory, so that global accesses are
    // fully coalesced 128-bit rows (each thread owns 64 consecutive floats of one state row)
    extern __shared__ __align__(16) float stg[];                 // [128][GDN_STG_LD]
    float* Mhead = a.state + (size_t)slot * a.state_stride + (size_t)h * D * D;
    for (int idx = tid; idx < D * D / 4; idx += 256) {
        const float4 v = reinterpret_cast<const float4*>(Mhead)[idx];
        *reinterpret_cast<float4*>(stg + (idx >> 5) * GDN_STG_LD + (idx & 31) * 4) = v;
    }
    __syncthreads();
    float m[64];
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(stg + j * GDN_STG_LD + 64 * ih + i);
        m[i] = v.x; m[i + 1] = v.y; m[i + 2] = v.z; m[i + 3] = v.w;
    }
    auto commit_state = [&]() {   // block-uniform call sites only
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(stg + j * GDN_STG_LD + 64 * ih + i) = make_float4(m[i], m[i + 1], m[i + 2], m[i + 3]);
        __syncthreads();
        for (int idx = tid; idx < D * D / 4; idx += 256)
            reinterpret_cast<float4*>(Mhead)[idx] = *reinterpret_cast<const float4*>(stg + (idx >> 5) * GDN_STG_LD + (idx & 31) * 4);
    };
    // conv channels of this thread: ca (q for tid < 128, v otherwise), cb (k, tid < 128 only)
    const int ca = tid < D ? hk * D + tid : 2 * a.n_qk * D + h * D + (tid - D);
    const int cb = a.n_qk * D + hk * D + (tid & (D - 1));
    float ha0 = cst[sa_], ha1 = cst[384 + sa_], ha2 = cst[768 + sa_];
    float hb0 = 0.f, hb1 = 0.f, hb2 = 0.f;
    if (tid < D) { hb0 = cst[sb_]; hb1 = cst[384 + sb_]; hb2 = cst[768 + sb_]; }
    const float wa0 = a.conv_w[ca * 4 + 0], wa1 = a.conv_w[ca * 4 + 1], wa2 = a.conv_w[ca * 4 + 2], wa3 = a.conv_w[ca * 4 + 3];
    const float wb0 = a.conv_w[cb * 4 + 0], wb1 = a.conv_w[cb * 4 + 1], wb2 = a.conv_w[cb * 4 + 2], wb3 = a.conv_w[cb * 4 + 3];

    // ---- phase 1: raw inputs of all rows fetched with asynchronous 4-byte copies (all in flight at once, compact
    // code), then conv + SiLU in place, squared norms, gates. sall[it] = [q 128 | k 128 | v 128] of row it.
    for (int it = 0; it < nrows; ++it) {
        const bool replay = it < nrep;
        const float* row = a.rows + (size_t)(replay ? 0 : r0 + (it - nrep)) * a.ld;
        const float* srow = sav + (replay ? it : 0) * 388;
        cp_async4(&sall[it][sa_], replay ? srow + sa_ : row + ca);
        if (tid < D) cp_async4(&sall[it][sb_], replay ? srow + sb_ : row + cb);
        if (tid == 0) { cp_async4(&sraw_b[it], replay ? srow + 384 : row + a.off_b + h); cp_async4(&sraw_a[it], replay ? srow + 385 : row + a.off_a + h); }
    }
    cp_async_wait_all();
    __syncthreads();
    if (tid < nrows) {
        sbeta[tid] = sigmoid_det(sraw_b[tid]);
        sdecay[tid] = expf_det(bf2f(a.a_neg[h]) * softplus_det(sraw_a[tid] + bf2f(a.dt_bias[h])));
    }
    // keep the raw inputs of the new rows for a later commit (every replayed row has been read: they are in shared memory)
    for (int it = nrep; it < nrows; ++it) {
        float* srow = sav + (it - nrep) * 388;
        srow[sa_] = sall[it][sa_]; if (tid < D) srow[sb_] = sall[it][sb_];
        if (tid == 0) { srow[384] = sraw_b[it]; srow[385] = sraw_a[it]; }
    }
    for (int it = 0; it < nrows; ++it) {
        if (it == nrep && nrep > 0) {   // history after the accepted prefix: committed
            cst[sa_] = ha0; cst[384 + sa_] = ha1; cst[768 + sa_] = ha2;
            if (tid < D) { cst[sb_] = hb0; cst[384 + sb_] = hb1; cst[768 + sb_] = hb2; }
        }
        const float xa = sall[it][sa_];
        float t = wa0 * ha0; t = fmaf(wa1, ha1, t); t = fmaf(wa2, ha2, t); t = fmaf(wa3, xa, t);
        const float va = silu_det(t); ha0 = ha1; ha1 = ha2; ha2 = xa;
        sall[it][sa_] = va;
        float vb = 0.f;
        if (tid < D) {
            const float xb = sall[it][sb_];
            float u = wb0 * hb0; u = fmaf(wb1, hb1, u); u = fmaf(wb2, hb2, u); u = fmaf(wb3, xb, u);
            vb = silu_det(u); hb0 = hb1; hb1 = hb2; hb2 = xb;
            sall[it][sb_] = vb;
        }
        // squared l2 norms: xor tree inside the warp, warp sums added in warp order afterwards
        float pq = tid < D ? va * va : 0.f, pk = tid < D ? vb * vb : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) { pq = pq + __shfl_xor_sync(0xffffffffu, pq, off); pk = pk + __shfl_xor_sync(0xffffffffu, pk, off); }
        if (lane == 0) { red[2 * it][warp] = pq; red[2 * it + 1][warp] = pk; }
    }
    if (T == 0 && nrep > 0) {   // pure commit: the loop above never reached it == nrep
        cst[sa_] = ha0; cst[384 + sa_] = ha1; cst[768 + sa_] = ha2;
        if (tid < D) { cst[sb_] = hb0; cst[384 + sb_] = hb1; cst[768 + sb_] = hb2; }
    }
    __syncthreads();
    if (tid < 2 * nrows) { float t = red[tid][0]; for (int w = 1; w < 8; ++w) t = t + red[tid][w]; tot[tid] = t; }
    __syncthreads();
    if (tid < D)
        for (int it = 0; it < nrows; ++it) {
            sall[it][tid] = sall[it][tid] / fmaxf(sqrtf(tot[2 * it]), a.eps);
            sall[it][D + tid] = sall[it][D + tid] / fmaxf(sqrtf(tot[2 * it + 1]), a.eps);
        }
    __syncthreads();

    // ---- phase 2: the recurrence, row after row, state in registers; no block-wide synchronisation inside
    for (int it = 0; it < nrows; ++it) {
        if (it == nrep && nrep > 0) commit_state();
        const float beta = sbeta[it], decay = sdecay[it];
        const float* kk = &sall[it][D + 64 * ih]; const float* qq = &sall[it][64 * ih];
        float kr[64];
#pragma unroll
        for (int i = 0; i < 64; i += 4) { const float4 v = *reinterpret_cast<const float4*>(kk + i); kr[i] = v.x; kr[i + 1] = v.y; kr[i + 2] = v.z; kr[i + 3] = v.w; }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) { m[i] = m[i] * decay; dot = fmaf(m[i], kr[i], dot); }
        dot = dot + __shfl_xor_sync(0xffffffffu, dot, 1);
        const float delta = (sall[it][2 * D + j] - dot) * beta;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
            const float4 qv = *reinterpret_cast<const float4*>(qq + i);
            m[i] = fmaf(delta, kr[i], m[i]); o = fmaf(m[i], qv.x, o);
            m[i + 1] = fmaf(delta, kr[i + 1], m[i + 1]); o = fmaf(m[i + 1], qv.y, o);
            m[i + 2] = fmaf(delta, kr[i + 2], m[i + 2]); o = fmaf(m[i + 2], qv.z, o);
            m[i + 3] = fmaf(delta, kr[i + 3], m[i + 3]); o = fmaf(m[i + 3], qv.w, o);
        }
        o = o + __shfl_xor_sync(0xffffffffu, o, 1);
        if (it >= nrep) {
            if (ih == 0) sout[it - nrep][j] = o * 0.08838834764831845f;
            if (a.snap) {
                float* sp = a.snap + (size_t)(it - nrep) * a.snap_row_stride + ((size_t)h * D + j) * D + 64 * ih;
#pragma unroll
                for (int i = 0; i < 64; ++i) sp[i] = m[i];
            }
        }
    }
    if (T == 0 && nrep > 0) commit_state();
    __syncthreads();

    // ---- phase 3: per-head RMSNorm * w * gate(z) + quantisation of the new rows
    for (int t = 0; t < T; ++t) {
        float ps = tid < D ? sout[t][tid] * sout[t][tid] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ps = ps + __shfl_xor_sync(0xffffffffu, ps, off);
        if (lane == 0) red[t][warp] = ps;
    }
    __syncthreads();
    if (tid < T) { float t = red[tid][0]; for (int w = 1; w < 8; ++w) t = t + red[tid][w]; tot[tid] = t; }
    __syncthreads();
    if (tid < D)
        for (int t = 0; t < T; ++t) {
            const int row = r0 + t;
            const size_t oi = (size_t)row * Z + h * D + tid;
            const float zz = a.rows[(size_t)row * a.ld + a.off_z + h * D + tid];
            const float v = ((sout[t][tid] * (1.0f / sqrtf(tot[t] / (float)D + a.eps))) * bf2f(a.norm_w[tid])) * (a.sigmoid_gate ? sigmoid_det(zz) : silu_det(zz));
            if (a.out) a.out[oi] = v;
            if (a.oq) warp_quant32_store(v, row, (h * D + tid) >> 5, Z, a.oq, a.osc, lane);
        }
}

}  // namespace

int embed_bf16(const int* tok, const void* table, float* out, int R, int E, int V, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && E > 0 && V > 0, "embed_bf16: bad shape");
    k_embed_bf16<<<R, 256, 0, s>>>(tok, (const uint16_t*)table, out, E, V);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int add_rmsnorm_quant(float* x, const float* y, int P, size_t part_stride, int ldy, const void* w_bf16, float* xn, XQ8F xq, int R, int n, float eps, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n > 0 && n % 64 == 0, "add_rmsnorm_quant: n=%d must be a positive multiple of 64", n);
    HP_REQUIRE(n <= NORM_THREADS * NORM_MAXE, "add_rmsnorm_quant: n=%d exceeds %d", n, NORM_THREADS * NORM_MAXE);
    launch_pdl(k_add_rmsnorm_quant, dim3(R), dim3(NORM_THREADS), 0, s, x, y, P, part_stride, ldy, (const uint16_t*)w_bf16, xn, (int8_t*)xq.q, (float*)xq.sc, n, eps);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int norm2_concat_quant(const float* a, const void* wa, const float* b, int ldb, const void* wb, float* out, XQ8F xq, int R, int n, float eps, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n > 0 && n % 64 == 0, "norm2_concat_quant: n=%d must be a positive multiple of 64", n);
    HP_REQUIRE(n <= NORM_THREADS * NORM_MAXE, "norm2_concat_quant: n=%d exceeds %d", n, NORM_THREADS * NORM_MAXE);
    launch_pdl(k_norm2_concat_quant, dim3(R), dim3(NORM_THREADS), 0, s, a, (const uint16_t*)wa, b, ldb, (const uint16_t*)wb, out, (int8_t*)xq.q, (float*)xq.sc, n, eps);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int silu_mul_quant(const float* gu, int ldg, int F, XQ8F xq, int R, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && F > 0 && F % 64 == 0 && ldg >= 2 * F, "silu_mul_quant: bad shape F=%d ldg=%d", F, ldg);
    launch_pdl(k_silu_mul_quant, dim3((F / 32 + 7) / 8, R), dim3(256), 0, s, gu, ldg, F, (int8_t*)xq.q, (float*)xq.sc);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int gdn_forward(const GdnParams& p, int nseq, cudaStream_t s) {
    HP_REQUIRE(nseq >= 1 && nseq <= 8 && p.n_qk >= 1 && p.n_v >= p.n_qk, "gdn_forward: bad shape");
    GdnArgs a;
    a.rows = p.rows; a.saved = p.saved; a.saved_stride = p.saved_stride; a.ld = p.ld; a.off_z = p.off_z; a.off_b = p.off_b; a.off_a = p.off_a;
    a.n_qk = p.n_qk; a.n_v = p.n_v; a.conv_w = p.conv_w; a.dt_bias = (const uint16_t*)p.dt_bias; a.a_neg = (const uint16_t*)p.a_neg; a.norm_w = (const uint16_t*)p.norm_w;
    a.state = p.state; a.conv_state = p.conv_state; a.state_stride = p.state_stride; a.conv_stride = p.conv_stride;
    a.seq = p.seq; a.replay_n = p.replay_n; a.out = p.out; a.oq = (int8_t*)p.xq.q; a.osc = (float*)p.xq.sc;
    a.snap = p.snap; a.snap_row_stride = p.snap_row_stride; a.eps = p.eps; a.sigmoid_gate = p.sigmoid_gate;
    static bool attr = false;
    if (!attr) { HP_CUDA(cudaFuncSetAttribute(k_gdn, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * GDN_STG_LD * 4)); attr = true; }
    HP_CUDA(launch_pdl(k_gdn, dim3(p.n_v, nseq), dim3(256), 128 * GDN_STG_LD * 4, s, a));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

}  // namespace hp
