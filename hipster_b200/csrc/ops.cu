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
// One 256-thread block per row. Thread i owns elements i, i+256, ...; sum of squares: per-thread fmaf chain in that
// order, then block_sum_det. Quantisation per 32 consecutive elements (one warp).
__global__ void __launch_bounds__(256) k_add_rmsnorm_quant(float* __restrict__ x, const float* __restrict__ y, int P, size_t part_stride, int ldy,
                                                            const uint16_t* __restrict__ w, float* __restrict__ xn, int8_t* __restrict__ q, float* __restrict__ sc,
                                                            int n, float eps) {
    __shared__ float sh[8];
    const int r = blockIdx.x, lane = threadIdx.x & 31;
    float* xr = x + (size_t)r * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        float t = xr[i];
        if (y) {
            float s = y[(size_t)r * ldy + i];
            for (int p = 1; p < P; ++p) s = s + y[(size_t)p * part_stride + (size_t)r * ldy + i];
            t = t + s; xr[i] = t;
        }
        ss = fmaf(t, t, ss);
    }
    ss = block_sum_det<8>(ss, sh);
    const float scl = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = (xr[i] * scl) * bf2f(w[i]);
        if (xn) xn[(size_t)r * n + i] = v;
        warp_quant32_store(v, r, i >> 5, n, q, sc, lane);
    }
}

// ---- MTP input: out[r] = [rmsnorm(a[r]) * wa | rmsnorm(b[r]) * wb], quantised (ops.hip:99-116) ----
__global__ void __launch_bounds__(256) k_norm2_concat_quant(const float* __restrict__ a, const uint16_t* __restrict__ wa, const float* __restrict__ b, int ldb,
                                                             const uint16_t* __restrict__ wb, float* __restrict__ out, int8_t* __restrict__ q, float* __restrict__ sc,
                                                             int n, float eps) {
    __shared__ float sh[8];
    const int r = blockIdx.x, lane = threadIdx.x & 31;
    const float* ar = a + (size_t)r * n; const float* br = b + (size_t)r * ldb;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { sa = fmaf(ar[i], ar[i], sa); sb = fmaf(br[i], br[i], sb); }
    sa = block_sum_det<8>(sa, sh); sb = block_sum_det<8>(sb, sh);
    const float ca = 1.0f / sqrtf(sa / (float)n + eps), cb = 1.0f / sqrtf(sb / (float)n + eps);
    for (int i = threadIdx.x; i < 2 * n; i += 256) {
        const float v = i < n ? (ar[i] * ca) * bf2f(wa[i]) : (br[i - n] * cb) * bf2f(wb[i - n]);
        if (out) out[(size_t)r * 2 * n + i] = v;
        warp_quant32_store(v, r, i >> 5, 2 * n, q, sc, lane);
    }
}

// ---- xq = q8(silu(gate) * up); gate = columns [0, F), up = [F, 2F) of gu [R][ldg] (ops.hip:146-151) ----
__global__ void __launch_bounds__(256) k_silu_mul_quant(const float* __restrict__ gu, int ldg, int F, int8_t* __restrict__ q, float* __restrict__ sc) {
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
__global__ void __launch_bounds__(256) k_gdn(GdnArgs a) {
    constexpr int D = 128;
    __shared__ float sq[D], sk[D], sv[D], sout[D], sh[8];
    const int h = blockIdx.x, hk = h % a.n_qk, tid = threadIdx.x;
    const int r0 = a.seq[blockIdx.y * 4 + 0], T = a.seq[blockIdx.y * 4 + 1], slot = a.seq[blockIdx.y * 4 + 2];
    float* sav = a.saved + (size_t)slot * a.saved_stride + (size_t)h * 8 * 388;   // [8][q 128 | k 128 | v 128 | beta | alpha | pad]
    const int nrep = a.replay_n ? a.replay_n[slot] : 0;
    const int Z = a.n_v * D;
    const int j = tid >> 1, ih = tid & 1;
    float* Mst = a.state + (size_t)slot * a.state_stride + ((size_t)h * D + j) * D + 64 * ih;
    // conv history of this head: [3 taps][q 128 | k 128 | v 128]; private per v-head so that no CTA reads what another writes
    float* cst = a.conv_state + (size_t)slot * a.conv_stride + (size_t)h * 3 * 384;
    const int sa_ = tid < D ? tid : D + tid, sb_ = D + (tid & (D - 1));   // history slots of channels ca / cb
    float m[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) m[i] = Mst[i];
    // conv channels of this thread: ca (q for tid < 128, v otherwise), cb (k, tid < 128 only)
    const int ca = tid < D ? hk * D + tid : 2 * a.n_qk * D + h * D + (tid - D);
    const int cb = a.n_qk * D + hk * D + (tid & (D - 1));
    float ha0 = cst[sa_], ha1 = cst[384 + sa_], ha2 = cst[768 + sa_];
    float hb0 = 0.f, hb1 = 0.f, hb2 = 0.f;
    if (tid < D) { hb0 = cst[sb_]; hb1 = cst[384 + sb_]; hb2 = cst[768 + sb_]; }
    const float wa0 = a.conv_w[ca * 4 + 0], wa1 = a.conv_w[ca * 4 + 1], wa2 = a.conv_w[ca * 4 + 2], wa3 = a.conv_w[ca * 4 + 3];
    const float wb0 = a.conv_w[cb * 4 + 0], wb1 = a.conv_w[cb * 4 + 1], wb2 = a.conv_w[cb * 4 + 2], wb3 = a.conv_w[cb * 4 + 3];
    const float dtb = bf2f(a.dt_bias[h]), aneg = bf2f(a.a_neg[h]);

    for (int it = 0; it < nrep + T; ++it) {
        const bool replay = it < nrep;
        const int t = r0 + (it - nrep);                      // row of this pass (new rows only)
        const float* row = a.rows + (size_t)(replay ? 0 : t) * a.ld;
        float* srow = sav + (replay ? it : it - nrep) * 388;
        if (it == nrep) {   // the accepted prefix has been applied: commit state and conv history (also when nrep == 0: no-op values)
            if (nrep > 0) {
#pragma unroll
                for (int i = 0; i < 64; ++i) Mst[i] = m[i];
                cst[sa_] = ha0; cst[384 + sa_] = ha1; cst[768 + sa_] = ha2;
                if (tid < D) { cst[sb_] = hb0; cst[384 + sb_] = hb1; cst[768 + sb_] = hb2; }
            }
        }
        // conv + silu
        const float xa = replay ? srow[sa_] : row[ca];
        float va = wa0 * ha0; va = fmaf(wa1, ha1, va); va = fmaf(wa2, ha2, va); va = fmaf(wa3, xa, va);
        va = silu_det(va); ha0 = ha1; ha1 = ha2; ha2 = xa;
        float vb = 0.f, vb_raw = 0.f;
        if (tid < D) {
            const float xb = replay ? srow[sb_] : row[cb];
            vb = wb0 * hb0; vb = fmaf(wb1, hb1, vb); vb = fmaf(wb2, hb2, vb); vb = fmaf(wb3, xb, vb);
            vb = silu_det(vb); hb0 = hb1; hb1 = hb2; hb2 = xb; vb_raw = xb;
        }
        const float qn = block_sum_det<8>(tid < D ? va * va : 0.f, sh);
        const float kn = block_sum_det<8>(tid < D ? vb * vb : 0.f, sh);
        if (tid < D) { sq[tid] = va / fmaxf(sqrtf(qn), a.eps); sk[tid] = vb / fmaxf(sqrtf(kn), a.eps); }
        else sv[tid - D] = va;
        __syncthreads();
        const float braw = replay ? srow[384] : row[a.off_b + h], araw = replay ? srow[385] : row[a.off_a + h];
        if (!replay) {   // keep the raw inputs of this row for a later commit (rows beyond 8 per sequence are never replayed)
            srow[sa_] = xa; if (tid < D) srow[sb_] = vb_raw; if (tid == 0) { srow[384] = braw; srow[385] = araw; }
        }
        const float beta = sigmoid_det(braw);
        const float decay = expf_det(aneg * softplus_det(araw + dtb));
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) { m[i] = m[i] * decay; dot = fmaf(m[i], sk[64 * ih + i], dot); }
        dot = dot + __shfl_xor_sync(0xffffffffu, dot, 1);
        const float delta = (sv[j] - dot) * beta;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) { m[i] = fmaf(delta, sk[64 * ih + i], m[i]); o = fmaf(m[i], sq[64 * ih + i], o); }
        o = o + __shfl_xor_sync(0xffffffffu, o, 1);
        if (!replay) {
            if (ih == 0) sout[j] = o * 0.08838834764831845f;
            __syncthreads();
            const float ss = block_sum_det<8>(tid < D ? sout[tid] * sout[tid] : 0.f, sh);
            if (tid < D) {
                const size_t oi = (size_t)t * Z + h * D + tid;
                const float zz = row[a.off_z + h * D + tid];
                const float v = ((sout[tid] * (1.0f / sqrtf(ss / (float)D + a.eps))) * bf2f(a.norm_w[tid])) * (a.sigmoid_gate ? sigmoid_det(zz) : silu_det(zz));
                if (a.out) a.out[oi] = v;
                if (a.oq) warp_quant32_store(v, t, (h * D + tid) >> 5, Z, a.oq, a.osc, tid & 31);
            }
            if (a.snap) {
                float* sp = a.snap + (size_t)(it - nrep) * a.snap_row_stride + ((size_t)h * D + j) * D + 64 * ih;
#pragma unroll
                for (int i = 0; i < 64; ++i) sp[i] = m[i];
            }
        }
        __syncthreads();
    }
    if (T == 0 && nrep > 0) {   // pure commit (no new rows): the loop above never reached it == nrep
#pragma unroll
        for (int i = 0; i < 64; ++i) Mst[i] = m[i];
        cst[sa_] = ha0; cst[384 + sa_] = ha1; cst[768 + sa_] = ha2;
        if (tid < D) { cst[sb_] = hb0; cst[384 + sb_] = hb1; cst[768 + sb_] = hb2; }
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
    k_add_rmsnorm_quant<<<R, 256, 0, s>>>(x, y, P, part_stride, ldy, (const uint16_t*)w_bf16, xn, (int8_t*)xq.q, (float*)xq.sc, n, eps);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int norm2_concat_quant(const float* a, const void* wa, const float* b, int ldb, const void* wb, float* out, XQ8F xq, int R, int n, float eps, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n > 0 && n % 64 == 0, "norm2_concat_quant: n=%d must be a positive multiple of 64", n);
    k_norm2_concat_quant<<<R, 256, 0, s>>>(a, (const uint16_t*)wa, b, ldb, (const uint16_t*)wb, out, (int8_t*)xq.q, (float*)xq.sc, n, eps);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int silu_mul_quant(const float* gu, int ldg, int F, XQ8F xq, int R, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && F > 0 && F % 64 == 0 && ldg >= 2 * F, "silu_mul_quant: bad shape F=%d ldg=%d", F, ldg);
    k_silu_mul_quant<<<dim3((F / 32 + 7) / 8, R), 256, 0, s>>>(gu, ldg, F, (int8_t*)xq.q, (float*)xq.sc);
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
    k_gdn<<<dim3(p.n_v, nseq), 256, 0, s>>>(a);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

}  // namespace hp
