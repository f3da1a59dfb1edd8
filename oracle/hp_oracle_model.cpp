// CPU oracle, part 2: layer kernels, seeded weight generation and the engine (forward / accept / mtp_forward).
// TEST INFRASTRUCTURE ONLY -- see hp_oracle.h. Scalar restatement of the reference's device kernels, which have no host
// twin in the reference (engine/kernels/ops.hip, fn.hip) and of its engine control flow (engine/src/qwen35.cpp).
// Reduction orders are the ones this build's CUDA kernels document, so results agree bit for bit.
#include "hp_oracle.h"
#include <cmath>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <stdexcept>

namespace {

inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint32_t fbits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

// fixed-order block sum: 256 partials = 8 groups of 32; inside a group the xor tree (offsets 16..1), then groups in order
float det_block_sum(const float* part, int nthreads) {
    float tot = 0.f;
    for (int w = 0; w < nthreads / 32; ++w) {
        float a[32], b[32];
        for (int l = 0; l < 32; ++l) a[l] = part[w * 32 + l];
        for (int off = 16; off > 0; off >>= 1) { for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ off]; memcpy(a, b, sizeof a); }
        tot = w == 0 ? a[0] : tot + a[0];
    }
    return tot;
}
// IEEE round-to-nearest-even f32 -> f16 (what __float2half_rn does; the KV cache is written with it, ops.hip:391-396)
uint16_t f32_to_f16_rne(float f) {
    const uint32_t x = fbits(f); const uint32_t sign = (x >> 16) & 0x8000; const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00 | ((ax > 0x7f800000u) ? 0x200 : 0));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00);                       // rounds to infinity
    if (ax < 0x33000001u) return (uint16_t)sign;                                   // rounds to zero
    int e = (int)(ax >> 23) - 127; uint32_t m = (ax & 0x7fffff) | 0x800000;
    int shift; uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; } else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffff; }
    const uint32_t half = 1u << (shift - 1), rem = m & ((1u << shift) - 1); uint32_t r = m >> shift;
    if (rem > half || (rem == half && (r & 1))) r++;
    return (uint16_t)(sign | (base + r));
}

// ---- seeded generation (restated from the engine's description: splitmix64 counter hash, Irwin-Hall(4) normals) ----
inline uint64_t splitmix64(uint64_t x) { x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull; return x ^ (x >> 31); }
inline uint64_t rnd64(uint64_t seed, uint64_t tid, uint64_t idx) { return splitmix64(splitmix64(seed ^ (tid * 0x9E3779B97F4A7C15ull)) + idx); }
inline float irwin(uint64_t u) {
    const int sum = (int)(u & 0xFFFF) + (int)((u >> 16) & 0xFFFF) + (int)((u >> 32) & 0xFFFF) + (int)(u >> 48) - 131070;
    return (float)sum * 2.6429e-5f;
}
inline uint16_t f32_to_bf16(float f) { uint32_t u = fbits(f); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }
void gen_q4k(std::vector<uint8_t>& w, int N, int K, uint64_t seed, uint64_t tid) {
    const size_t nwords = (size_t)N * (K / 256) * 18; w.resize(nwords * 8);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < nwords; ++i) {
        uint64_t v = rnd64(seed, tid, i);
        if (i % 18 == 0) {
            const size_t b = i / 18;
            const uint16_t d = orc_f32_to_f16(fabsf(irwin(rnd64(seed, tid ^ 0xD00Dull, b))) * 0.01f);
            const uint16_t dm = orc_f32_to_f16(fabsf(irwin(rnd64(seed, tid ^ 0xE00Eull, b))) * 0.01f);
            v = (v & 0xFFFFFFFF00000000ull) | (uint64_t)d | ((uint64_t)dm << 16);
        }
        memcpy(&w[i * 8], &v, 8);
    }
}
void gen_bf16(std::vector<uint16_t>& p, size_t n, uint64_t seed, uint64_t tid, float mean, float sd, bool neg_abs = false) {
    p.resize(n);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) { float v = mean + sd * irwin(rnd64(seed, tid, i)); if (neg_abs) v = -fabsf(v); p[i] = f32_to_bf16(v); }
}
void gen_f32(std::vector<float>& p, size_t n, uint64_t seed, uint64_t tid, float mean, float sd, bool neg_abs) {
    p.resize(n); for (size_t i = 0; i < n; ++i) { float v = mean + sd * irwin(rnd64(seed, tid, i)); if (neg_abs) v = -fabsf(v); p[i] = v; }
}

struct XQ { std::vector<int8_t> q; std::vector<float> d, s; int K = 0; void set(int R, int k) { K = k; q.assign((size_t)R * k, 0); d.assign((size_t)R * k / 32, 0.f); s.assign((size_t)R * k / 32, 0.f); } };

}  // namespace

// ---------------------------------------------------------------- layer kernels (row layout)
// ops.hip:79-98: x += y; xn = x * rsqrt(mean x^2 + eps) * w; q8. Here y = sum of P planes in plane order; the sum of
// squares: 1280 workers, worker t takes the 4-element groups t, t+1280, ... (fmaf chain in index order), then det_block_sum.
extern "C" void orc_add_rmsnorm_quant(float* x, const float* y, int P, size_t part_stride, int ldy, const uint16_t* w, float* xn,
                                      int8_t* q, float* d, float* s, int R, int n, float eps) {
    std::vector<float> v(n);
    for (int r = 0; r < R; ++r) {
        float* xr = x + (size_t)r * n; float part[1280];
        for (int t = 0; t < 1280; ++t) {
            float ss = 0.f;
            for (int g = t; g < n / 4; g += 1280)
                for (int i = 4 * g; i < 4 * g + 4; ++i) {
                    float a = xr[i];
                    if (y) { float sum = y[(size_t)r * ldy + i]; for (int p = 1; p < P; ++p) sum = sum + y[(size_t)p * part_stride + (size_t)r * ldy + i]; a = a + sum; xr[i] = a; }
                    ss = fmaf(a, a, ss);
                }
            part[t] = ss;
        }
        const float tot = det_block_sum(part, 1280);
        const float scl = 1.0f / sqrtf(tot / (float)n + eps);
        for (int i = 0; i < n; ++i) { v[i] = (xr[i] * scl) * bf2f(w[i]); if (xn) xn[(size_t)r * n + i] = v[i]; }
        orc_quantize_x_q8(v.data(), 1, n, q + (size_t)r * n, d + (size_t)r * (n / 32), s + (size_t)r * (n / 32));
    }
}
// ops.hip:99-116
extern "C" void orc_norm2_concat_quant(const float* a, const uint16_t* wa, const float* b, int ldb, const uint16_t* wb, float* out,
                                       int8_t* q, float* d, float* s, int R, int n, float eps) {
    std::vector<float> v(2 * n);
    for (int r = 0; r < R; ++r) {
        const float* ar = a + (size_t)r * n; const float* br = b + (size_t)r * ldb; float pa[1280], pb[1280];
        for (int t = 0; t < 1280; ++t) {
            float sa = 0.f, sb = 0.f;
            for (int g = t; g < n / 4; g += 1280) for (int i = 4 * g; i < 4 * g + 4; ++i) { sa = fmaf(ar[i], ar[i], sa); sb = fmaf(br[i], br[i], sb); }
            pa[t] = sa; pb[t] = sb;
        }
        const float ca = 1.0f / sqrtf(det_block_sum(pa, 1280) / (float)n + eps), cb = 1.0f / sqrtf(det_block_sum(pb, 1280) / (float)n + eps);
        for (int i = 0; i < n; ++i) { v[i] = (ar[i] * ca) * bf2f(wa[i]); v[n + i] = (br[i] * cb) * bf2f(wb[i]); }
        if (out) memcpy(out + (size_t)r * 2 * n, v.data(), (size_t)2 * n * 4);
        orc_quantize_x_q8(v.data(), 1, 2 * n, q + (size_t)r * 2 * n, d + (size_t)r * (2 * n / 32), s + (size_t)r * (2 * n / 32));
    }
}
// ops.hip:146-151
extern "C" void orc_silu_mul_quant(const float* gu, int ldg, int F, int8_t* q, float* d, float* s, int R) {
    std::vector<float> v(F);
    for (int r = 0; r < R; ++r) {
        for (int i = 0; i < F; ++i) v[i] = orc_silu(gu[(size_t)r * ldg + i]) * gu[(size_t)r * ldg + F + i];
        orc_quantize_x_q8(v.data(), 1, F, q + (size_t)r * F, d + (size_t)r * (F / 32), s + (size_t)r * (F / 32));
    }
}

// Gated DeltaNet: conv (ops.hip:188-202) + recurrent step (ops.hip:205-256) over T rows of one sequence, all heads.
// rows [T][ld]: qkv (q: n_qk*128 | k: n_qk*128 | v: n_v*128) | z (n_v*128) | beta (n_v) | alpha (n_v).
// state [n_v][128][128] (M[j][i]), conv history [3][C] oldest first (reference layout). out [T][n_v*128] (nullable).
// snap (nullable): state after each row, [T][n_v][128][128].
extern "C" void orc_gdn_rows(const float* rows, int ld, int T, int n_qk, int n_v, const float* conv_w, const uint16_t* dt_bias, const uint16_t* a_neg,
                             const uint16_t* norm_w, float* state, float* conv_hist, float* out, float* snap, float eps, int sigmoid_gate) {
    const int D = 128, C = (2 * n_qk + n_v) * D, Z = n_v * D, off_z = C, off_b = C + Z, off_a = off_b + n_v;
    std::vector<float> cv(C);
    for (int t = 0; t < T; ++t) {
        const float* row = rows + (size_t)t * ld;
        for (int c = 0; c < C; ++c) {
            float* h0 = conv_hist + c; float* h1 = conv_hist + C + c; float* h2 = conv_hist + 2 * C + c;
            const float* w = conv_w + (size_t)c * 4; const float x = row[c];
            float a = w[0] * *h0; a = fmaf(w[1], *h1, a); a = fmaf(w[2], *h2, a); a = fmaf(w[3], x, a);
            cv[c] = orc_silu(a); *h0 = *h1; *h1 = *h2; *h2 = x;
        }
#pragma omp parallel for schedule(static)
        for (int h = 0; h < n_v; ++h) {
            const int hk = h % n_qk;
            const float* q = cv.data() + hk * D; const float* k = cv.data() + n_qk * D + hk * D; const float* v = cv.data() + 2 * n_qk * D + h * D;
            float part[256], sq[128], sk[128], so[128];
            for (int i = 0; i < 256; ++i) part[i] = i < D ? q[i] * q[i] : 0.f;
            const float qn = det_block_sum(part, 256);
            for (int i = 0; i < 256; ++i) part[i] = i < D ? k[i] * k[i] : 0.f;
            const float kn = det_block_sum(part, 256);
            for (int i = 0; i < D; ++i) { sq[i] = q[i] / fmaxf(sqrtf(qn), eps); sk[i] = k[i] / fmaxf(sqrtf(kn), eps); }
            const float beta = orc_sigmoid(row[off_b + h]);
            const float decay = orc_expf(bf2f(a_neg[h]) * orc_softplus(row[off_a + h] + bf2f(dt_bias[h])));
            float* M = state + (size_t)h * D * D;
            for (int j = 0; j < D; ++j) {
                // 8 partial sums over 16 consecutive key indices each, combined by an xor tree (offsets 1, 2, 4)
                float dd[8], oo[8];
                for (int c = 0; c < 8; ++c) { float dot = 0.f; float* m = M + (size_t)j * D + 16 * c; for (int i = 0; i < 16; ++i) { m[i] = m[i] * decay; dot = fmaf(m[i], sk[16 * c + i], dot); } dd[c] = dot; }
                const float delta = (v[j] - (((dd[0] + dd[1]) + (dd[2] + dd[3])) + ((dd[4] + dd[5]) + (dd[6] + dd[7])))) * beta;
                for (int c = 0; c < 8; ++c) { float o = 0.f; float* m = M + (size_t)j * D + 16 * c; for (int i = 0; i < 16; ++i) { m[i] = fmaf(delta, sk[16 * c + i], m[i]); o = fmaf(m[i], sq[16 * c + i], o); } oo[c] = o; }
                so[j] = (((oo[0] + oo[1]) + (oo[2] + oo[3])) + ((oo[4] + oo[5]) + (oo[6] + oo[7]))) * 0.08838834764831845f;
            }
            if (out) {
                for (int i = 0; i < 256; ++i) part[i] = i < D ? so[i] * so[i] : 0.f;
                const float ss = det_block_sum(part, 256);
                for (int i = 0; i < D; ++i) {
                    const float zz = row[off_z + h * D + i];
                    out[(size_t)t * Z + h * D + i] = ((so[i] * (1.0f / sqrtf(ss / (float)D + eps))) * bf2f(norm_w[i])) * (sigmoid_gate ? orc_sigmoid(zz) : orc_silu(zz));
                }
            }
            if (snap) memcpy(snap + ((size_t)t * n_v + h) * D * D, M, (size_t)D * D * 4);
        }
    }
}

// Attention for one row (ops.hip:363-465 semantics; split structure of ops.hip:831-948 with 128-key splits).
// qkv row: [q_full n_head x (256 q | 256 gate) | k n_kv x 256 | v n_kv x 256] (q and k are normalised + rotated in place).
// kc / vc: f16 [n_kv][max_ctx][256] of the row's slot. rope: (cos, sin) [max_ctx][n_rot/2]. out [n_head*256].
extern "C" void orc_attn_row(float* qkv, int n_head, int n_kv, int n_rot, const uint16_t* qw, const uint16_t* kw, const float* rope, int pos,
                             uint16_t* kc, uint16_t* vc, int max_ctx, float* out, float eps) {
    const int HD = 256, half = n_rot / 2, G = n_head / n_kv, SPL = 128;
    for (int hb = 0; hb < n_head + n_kv; ++hb) {
        const bool isq = hb < n_head;
        float* x = isq ? qkv + hb * 512 : qkv + n_head * 512 + (hb - n_head) * HD;
        float part[256]; for (int t = 0; t < HD; ++t) part[t] = x[t] * x[t];
        const float ss = det_block_sum(part, 256);
        float buf[256];
        for (int t = 0; t < HD; ++t) buf[t] = (x[t] * (1.0f / sqrtf(ss / (float)HD + eps))) * bf2f((isq ? qw : kw)[t]);
        for (int t = 0; t < HD; ++t) {
            float n = buf[t];
            if (t < n_rot) {
                const int i = t % half; const float c = rope[((size_t)pos * half + i) * 2], sn = rope[((size_t)pos * half + i) * 2 + 1];
                const float x0 = buf[i], x1 = buf[i + half];
                n = t < half ? fmaf(-x1, sn, x0 * c) : fmaf(x1, c, x0 * sn);
            }
            x[t] = n;
        }
        if (!isq) {
            const int kh = hb - n_head; const float* v = qkv + n_head * 512 + n_kv * HD + kh * HD;
            for (int t = 0; t < HD; ++t) { kc[((size_t)kh * max_ctx + pos) * HD + t] = f32_to_f16_rne(x[t]); vc[((size_t)kh * max_ctx + pos) * HD + t] = f32_to_f16_rne(v[t]); }
        }
    }
    const int nsplit = (pos + 1 + SPL - 1) / SPL;
    std::vector<float> pO((size_t)nsplit * HD), e(SPL);
    std::vector<float> pm(nsplit), pl(nsplit);
    for (int head = 0; head < n_head; ++head) {
        const int kh = head / G; const float* q = qkv + head * 512;
        for (int sp = 0; sp < nsplit; ++sp) {
            const int k_lo = sp * SPL, nk = std::min(SPL, pos + 1 - k_lo);
            float mx = -INFINITY;
            for (int k = 0; k < nk; ++k) {
                const uint16_t* kr = kc + ((size_t)kh * max_ctx + k_lo + k) * HD;
                float sc = 0.f; for (int d = 0; d < HD; ++d) sc = fmaf(q[d], orc_f16_to_f32(kr[d]), sc);
                e[k] = sc * 0.0625f; mx = fmaxf(mx, e[k]);
            }
            // sum of the weights: 32 partial sums over keys l, l+32, l+64, l+96 (ascending), then an xor tree (offsets 16..1)
            float part[32];
            for (int k = 0; k < nk; ++k) e[k] = orc_expf(e[k] - mx);
            for (int ln = 0; ln < 32; ++ln) { float a = ln < nk ? e[ln] : 0.f; for (int i = 1; i < 4; ++i) a = a + (ln + 32 * i < nk ? e[ln + 32 * i] : 0.f); part[ln] = a; }
            const float l = det_block_sum(part, 32);
            for (int d = 0; d < HD; ++d) {
                float o = 0.f;
                for (int k = 0; k < nk; ++k) o = fmaf(e[k], orc_f16_to_f32(vc[((size_t)kh * max_ctx + k_lo + k) * HD + d]), o);
                pO[(size_t)sp * HD + d] = o;
            }
            pm[sp] = mx; pl[sp] = l;
        }
        float mx = -INFINITY; for (int sp = 0; sp < nsplit; ++sp) mx = fmaxf(mx, pm[sp]);
        for (int d = 0; d < HD; ++d) {
            float o = 0.f, l = 0.f;
            for (int sp = 0; sp < nsplit; ++sp) { const float w = orc_expf(pm[sp] - mx); o = fmaf(w, pO[(size_t)sp * HD + d], o); l = fmaf(w, pl[sp], l); }
            out[head * HD + d] = (o / l) * orc_sigmoid(q[HD + d]);
        }
    }
}

// ---------------------------------------------------------------- mixture of experts
// fn.hip:252-266: one 32-lane worker group per weight row; lane l takes k = 4l + 128i, four fmaf per step, xor tree.
extern "C" void orc_router_gemv(const float* W, const float* x, float* y, int N, int K, int T) {
    for (int t = 0; t < T; ++t)
        for (int n = 0; n < N; ++n) {
            float a[32], b[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.f;
                for (int i = l * 4; i < K; i += 128) for (int e = 0; e < 4; ++e) acc = fmaf(W[(size_t)n * K + i + e], x[(size_t)t * K + i + e], acc);
                a[l] = acc;
            }
            for (int off = 16; off > 0; off >>= 1) { for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ off]; memcpy(a, b, sizeof a); }
            y[(size_t)t * N + n] = a[0];
        }
}
// fn.hip:167-205: softmax over E logits, top-k (value desc, index asc), renormalise by the sum of the selected
// probabilities in rank order; slot k = shared expert, id -1, weight sigmoid(logit[E]). Arrays [T][k+1].
extern "C" void orc_moe_route(const float* logits, int* ids, float* w, int T, int E, int k) {
    std::vector<float> p(E); float part[1024];
    for (int t = 0; t < T; ++t) {
        const float* lg = logits + (size_t)t * (E + 1);
        float mx = -INFINITY; for (int i = 0; i < E; ++i) mx = fmaxf(mx, lg[i]);
        for (int i = 0; i < 1024; ++i) part[i] = i < E ? orc_expf(lg[i] - mx) : 0.f;
        const float sum = det_block_sum(part, 1024);
        for (int i = 0; i < E; ++i) p[i] = part[i] / sum;
        float wsum = 0.f; float sel[16];
        for (int r = 0; r < k; ++r) {
            int bi = 0; float bv = p[0];
            for (int i = 1; i < E; ++i) if (p[i] > bv) { bv = p[i]; bi = i; }
            ids[t * (k + 1) + r] = bi; sel[r] = bv; p[bi] = -1.f; wsum = wsum + bv;
        }
        for (int r = 0; r < k; ++r) w[t * (k + 1) + r] = sel[r] / wsum;
        ids[t * (k + 1) + k] = -1; w[t * (k + 1) + k] = orc_sigmoid(lg[E]);
    }
}
// gemv.hip:1075-1114 numerics for one activation row against one expert matrix: blocks in order, no split.
extern "C" void orc_gemv_q4k_q8_seq(const uint8_t* W, const int8_t* q, const float* xd, const float* xs, float* y, int N, int K) {
    const int nb = K / 256;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < N; ++row) {
        const uint8_t* wrow = W + (size_t)row * nb * 144; float acc = 0.f;
        for (int b = 0; b < nb; ++b) {
            const uint8_t* bp = wrow + (size_t)b * 144;
            uint16_t dh, mh; memcpy(&dh, bp, 2); memcpy(&mh, bp + 2, 2);
            const float d = orc_f16_to_f32(dh), dmin = orc_f16_to_f32(mh);
            uint8_t sc[8], mn[8]; orc_q4k_scale_min(bp + 4, sc, mn);
            for (int sb = 0; sb < 8; ++sb) {
                const int grp = sb >> 1, hi = sb & 1; const uint8_t* qs = bp + 16 + 32 * grp; const int8_t* xe = q + (size_t)b * 256 + 32 * sb;
                int idot = 0; for (int e = 0; e < 32; ++e) idot += (int)(hi ? (qs[e] >> 4) : (qs[e] & 0xF)) * (int)xe[e];
                acc = fmaf((d * (float)sc[sb]) * xd[b * 8 + sb], (float)idot, acc);
                acc = fmaf(-(dmin * (float)mn[sb]), xs[b * 8 + sb], acc);
            }
        }
        y[row] = acc;
    }
}

// helpers for the Python restatement of one MoE layer: act = silu(g) * u (fn.hip:206-211), acc = fmaf(w, v, acc) (gemv.hip:1104-1112)
extern "C" void orc_silu_mul(const float* gu, float* act, int F) { for (int i = 0; i < F; ++i) act[i] = orc_silu(gu[i]) * gu[F + i]; }
extern "C" void orc_fma_rows(float* acc, const float* v, float w, int n) { for (int i = 0; i < n; ++i) acc[i] = fmaf(w, v[i], acc[i]); }

// ---------------------------------------------------------------- engine (engine/src/qwen35.cpp restated on the CPU)
struct OrcCfg {   // mirrors hp_model_cfg field for field
    int n_embd, n_layer, n_ff, n_vocab, n_head, n_head_kv, n_rot, gdn_qk_heads, gdn_v_heads, attn_every, max_ctx, n_slots;
    int n_expert, n_expert_used, expert_ff, gdn_sigmoid_gate, has_mtp, ep_rank, ep_world, synth_router_logits; float rms_eps, rope_base; unsigned long long seed;
};
namespace {
struct OLin { std::vector<uint8_t> w; int N = 0, K = 0; };
struct OLayer {
    bool is_attn = false; std::vector<uint16_t> attn_norm, post_norm, dt_bias, a_neg, ssm_norm, q_norm, k_norm; std::vector<float> conv_w;
    OLin in_proj, out_proj, gate_up, down;
    std::vector<float> router; OLin exp_gate_up, exp_down, sh_gate_up, sh_down;
};
enum { TK_ATTN_NORM = 0, TK_POST_NORM, TK_IN_PROJ, TK_OUT_PROJ, TK_GATE_UP, TK_DOWN, TK_CONV_W, TK_DT_BIAS, TK_A_NEG, TK_SSM_NORM, TK_Q_NORM, TK_K_NORM,
       TK_ROUTER, TK_EXP_GATE_UP, TK_EXP_DOWN, TK_SH_GATE_UP, TK_SH_DOWN,
       TK_EMBED = 32, TK_OUTPUT_NORM, TK_LM_HEAD, TK_MTP_ENORM, TK_MTP_HNORM, TK_MTP_EH_PROJ, TK_MTP_HEAD_NORM };
inline uint64_t tensor_id(int layer, int kind) { return (uint64_t)(layer + 1) * 64 + (uint64_t)kind; }
}
struct OrcModel {
    OrcCfg c; std::vector<OLayer> layers; OLayer mtp; std::vector<uint16_t> embed, output_norm, enorm, hnorm, head_norm; OLin lm_head, eh_proj;
    std::vector<float> rope;
    // state per slot, double-buffered (qwen35.h:117-118): [slot*2+buf]
    std::vector<std::vector<float>> gdn_state, conv_state; std::vector<int> cur;
    std::vector<std::vector<uint16_t>> kc, vc, mkc, mvc;   // per slot: [layers][n_kv][max_ctx][256]
    std::vector<float> sv_rows; int ld_in = 0;             // saved GDN inputs of the last pass (replay buffers, qwen35.h:124): [n_gdn][32][ld_in]
    std::vector<int> lr0, lT;
    std::vector<float> logits, h, mlogits, mh;
    int ngdn() const { return c.n_layer - c.n_layer / c.attn_every; }
    void gen_layer(OLayer& L, int il, bool is_attn) {
        const int E = c.n_embd, nv = c.gdn_v_heads, nq = c.gdn_qk_heads;
        L.is_attn = is_attn;
        gen_bf16(L.attn_norm, E, c.seed, tensor_id(il, TK_ATTN_NORM), 1.f, 0.1f); gen_bf16(L.post_norm, E, c.seed, tensor_id(il, TK_POST_NORM), 1.f, 0.1f);
        if (is_attn) {
            L.in_proj.N = c.n_head * 512 + 2 * c.n_head_kv * 256; L.in_proj.K = E; gen_q4k(L.in_proj.w, L.in_proj.N, E, c.seed, tensor_id(il, TK_IN_PROJ));
            L.out_proj.N = E; L.out_proj.K = c.n_head * 256; gen_q4k(L.out_proj.w, E, L.out_proj.K, c.seed, tensor_id(il, TK_OUT_PROJ));
            gen_bf16(L.q_norm, 256, c.seed, tensor_id(il, TK_Q_NORM), 1.f, 0.2f); gen_bf16(L.k_norm, 256, c.seed, tensor_id(il, TK_K_NORM), 1.f, 0.2f);
        } else {
            L.in_proj.N = ld_in; L.in_proj.K = E; gen_q4k(L.in_proj.w, ld_in, E, c.seed, tensor_id(il, TK_IN_PROJ));
            L.out_proj.N = E; L.out_proj.K = nv * 128; gen_q4k(L.out_proj.w, E, nv * 128, c.seed, tensor_id(il, TK_OUT_PROJ));
            gen_f32(L.conv_w, (size_t)(2 * nq + nv) * 128 * 4, c.seed, tensor_id(il, TK_CONV_W), 0.f, 0.5f, false);
            gen_bf16(L.dt_bias, nv, c.seed, tensor_id(il, TK_DT_BIAS), 0.f, 0.5f); gen_bf16(L.a_neg, nv, c.seed, tensor_id(il, TK_A_NEG), 0.8f, 0.4f, true);   // never positive (test_fnkernels.cpp:33 draws -|N(0,1)|)
            gen_bf16(L.ssm_norm, 128, c.seed, tensor_id(il, TK_SSM_NORM), 1.f, 0.3f);
        }
        if (c.n_expert == 0) {
            L.gate_up.N = 2 * c.n_ff; L.gate_up.K = E; gen_q4k(L.gate_up.w, 2 * c.n_ff, E, c.seed, tensor_id(il, TK_GATE_UP));
            L.down.N = E; L.down.K = c.n_ff; gen_q4k(L.down.w, E, c.n_ff, c.seed, tensor_id(il, TK_DOWN));
        } else {
            const int F = c.expert_ff;
            gen_f32(L.router, (size_t)(c.n_expert + 1) * E, c.seed, tensor_id(il, TK_ROUTER), 0.f, 1.0f / sqrtf((float)E), false);
            L.exp_gate_up.N = c.n_expert * 2 * F; L.exp_gate_up.K = E; gen_q4k(L.exp_gate_up.w, c.n_expert * 2 * F, E, c.seed, tensor_id(il, TK_EXP_GATE_UP));
            L.exp_down.N = c.n_expert * E; L.exp_down.K = F; gen_q4k(L.exp_down.w, c.n_expert * E, F, c.seed, tensor_id(il, TK_EXP_DOWN));
            L.sh_gate_up.N = 2 * F; L.sh_gate_up.K = E; gen_q4k(L.sh_gate_up.w, 2 * F, E, c.seed, tensor_id(il, TK_SH_GATE_UP));
            L.sh_down.N = E; L.sh_down.K = F; gen_q4k(L.sh_down.w, E, F, c.seed, tensor_id(il, TK_SH_DOWN));
        }
    }
    explicit OrcModel(const OrcCfg& cfg) : c(cfg) {
        const int E = c.n_embd, nv = c.gdn_v_heads, nq = c.gdn_qk_heads;
        ld_in = (2 * nq + nv) * 128 + nv * 128 + 2 * nv;
        layers.resize(c.n_layer);
        for (int il = 0; il < c.n_layer; ++il) gen_layer(layers[il], il, (il + 1) % c.attn_every == 0);
        gen_bf16(embed, (size_t)c.n_vocab * E, c.seed, tensor_id(-1, TK_EMBED), 0.f, 1.f);
        gen_bf16(output_norm, E, c.seed, tensor_id(-1, TK_OUTPUT_NORM), 1.f, 0.1f);
        lm_head.N = c.n_vocab; lm_head.K = E; gen_q4k(lm_head.w, c.n_vocab, E, c.seed, tensor_id(-1, TK_LM_HEAD));
        if (c.has_mtp) {
            gen_layer(mtp, c.n_layer, true);
            gen_bf16(enorm, E, c.seed, tensor_id(-1, TK_MTP_ENORM), 1.f, 0.1f); gen_bf16(hnorm, E, c.seed, tensor_id(-1, TK_MTP_HNORM), 1.f, 0.1f);
            gen_bf16(head_norm, E, c.seed, tensor_id(-1, TK_MTP_HEAD_NORM), 1.f, 0.1f);
            eh_proj.N = E; eh_proj.K = 2 * E; gen_q4k(eh_proj.w, E, 2 * E, c.seed, tensor_id(-1, TK_MTP_EH_PROJ));
        }
        const int half = c.n_rot / 2; rope.resize((size_t)c.max_ctx * half * 2);
        for (int p = 0; p < c.max_ctx; ++p) for (int i = 0; i < half; ++i) {
            const double th = (double)p * std::pow((double)c.rope_base, -2.0 * i / (double)c.n_rot);
            rope[((size_t)p * half + i) * 2] = (float)std::cos(th); rope[((size_t)p * half + i) * 2 + 1] = (float)std::sin(th);
        }
        const size_t st = (size_t)ngdn() * nv * 128 * 128, cs = (size_t)ngdn() * 3 * (2 * nq + nv) * 128;
        gdn_state.assign(c.n_slots * 2, std::vector<float>(st, 0.f)); conv_state.assign(c.n_slots * 2, std::vector<float>(cs, 0.f)); cur.assign(c.n_slots, 0);
        const size_t kvl = (size_t)c.n_head_kv * c.max_ctx * 256, nattn = c.n_layer / c.attn_every;
        kc.assign(c.n_slots, std::vector<uint16_t>(kvl * nattn, 0)); vc = kc;
        mkc.assign(c.n_slots, std::vector<uint16_t>(kvl, 0)); mvc = mkc;
        sv_rows.assign((size_t)ngdn() * 32 * ld_in, 0.f); lr0.assign(c.n_slots, 0); lT.assign(c.n_slots, 0);
        logits.assign((size_t)32 * c.n_vocab, 0.f); mlogits = logits; h.assign((size_t)32 * E, 0.f); mh = h;
    }
    void reset() { for (auto& s : gdn_state) std::fill(s.begin(), s.end(), 0.f); for (auto& s : conv_state) std::fill(s.begin(), s.end(), 0.f); std::fill(cur.begin(), cur.end(), 0); std::fill(lT.begin(), lT.end(), 0); }
    void reset_slot(int s) { for (int b = 0; b < 2; ++b) { std::fill(gdn_state[s * 2 + b].begin(), gdn_state[s * 2 + b].end(), 0.f); std::fill(conv_state[s * 2 + b].begin(), conv_state[s * 2 + b].end(), 0.f); } cur[s] = 0; lT[s] = 0; }

    // shared pieces
    void gemv(const OLin& l, const XQ& xq, float* y, int R, int ldy) { orc_gemv_q4k_q8(l.w.data(), xq.q.data(), xq.d.data(), xq.s.data(), y, l.N, l.K, R, ldy); }
    void norm_in(std::vector<float>& x, const float* y, const std::vector<uint16_t>& w, float* xn, XQ& xq, int R) {
        xq.set(R, c.n_embd);
        orc_add_rmsnorm_quant(x.data(), y, 1, 0, c.n_embd, w.data(), xn, xq.q.data(), xq.d.data(), xq.s.data(), R, c.n_embd, c.rms_eps);
    }
    // qwen35.cpp:247-276 (per-row positions and KV slots)
    void attn_block(const OLayer& L, XQ& xq, std::vector<std::vector<uint16_t>>& K, std::vector<std::vector<uint16_t>>& V, size_t layer_off, const int* pos, const int* slot, int R, std::vector<float>& y) {
        const int ld = L.in_proj.N; std::vector<float> qkv((size_t)R * ld), ao((size_t)R * c.n_head * 256);
        gemv(L.in_proj, xq, qkv.data(), R, ld);
        for (int r = 0; r < R; ++r)
            orc_attn_row(qkv.data() + (size_t)r * ld, c.n_head, c.n_head_kv, c.n_rot, L.q_norm.data(), L.k_norm.data(), rope.data(), pos[r],
                         K[slot[r]].data() + layer_off, V[slot[r]].data() + layer_off, c.max_ctx, ao.data() + (size_t)r * c.n_head * 256, c.rms_eps);
        xq.set(R, c.n_head * 256); orc_quantize_x_q8(ao.data(), R, c.n_head * 256, xq.q.data(), xq.d.data(), xq.s.data());
        y.assign((size_t)R * c.n_embd, 0.f); gemv(L.out_proj, xq, y.data(), R, c.n_embd);
    }
    // qwen35.cpp:278-287
    // Qwen4Exp::moe_layer (qwen4exp.cpp:345-354); xn = the normalised f32 rows the router reads
    void moe_block(const OLayer& L, XQ& xq, const std::vector<float>& xn, int R, std::vector<float>& y, const int* tok, const int* pos, const int* slot, int layer_index) {
        const int E = c.n_embd, F = c.expert_ff, ns = c.n_expert_used + 1, nb = E / 256, nsb = E / 32;
        std::vector<float> lg((size_t)R * (c.n_expert + 1)), w((size_t)R * ns); std::vector<int> ids((size_t)R * ns);
        orc_router_gemv(L.router.data(), xn.data(), lg.data(), c.n_expert + 1, E, R);
        if (c.synth_router_logits) {   // benchmark input control: seeded N(0, 1) expert logits keyed by (layer, slot, token, position, expert)
            const uint64_t key = splitmix64(c.seed ^ 0x726F75746572ull ^ ((uint64_t)layer_index << 40)) | 1ull;
            for (int t = 0; t < R; ++t) for (int e = 0; e < c.n_expert; ++e)
                lg[(size_t)t * (c.n_expert + 1) + e] = irwin(rnd64(key + (uint64_t)slot[t], ((uint64_t)(uint32_t)tok[t] << 32) | (uint32_t)pos[t], (uint64_t)e));
        }
        orc_moe_route(lg.data(), ids.data(), w.data(), R, c.n_expert, c.n_expert_used);
        const size_t eb_up = (size_t)2 * F * nb * 144, eb_dn = (size_t)E * (F / 256) * 144;
        y.assign((size_t)R * E, 0.f);
        std::vector<float> gu(2 * F), act(F), v(E); std::vector<int8_t> aq(F); std::vector<float> ad(F / 32), as(F / 32);
        for (int t = 0; t < R; ++t) {
            std::vector<float> acc(E, 0.f);
            for (int e = 0; e < ns; ++e) {
                const int id = ids[t * ns + e];
                const uint8_t* Wu = id >= 0 ? L.exp_gate_up.w.data() + (size_t)id * eb_up : L.sh_gate_up.w.data();
                const uint8_t* Wd = id >= 0 ? L.exp_down.w.data() + (size_t)id * eb_dn : L.sh_down.w.data();
                orc_gemv_q4k_q8_seq(Wu, xq.q.data() + (size_t)t * E, xq.d.data() + (size_t)t * nsb, xq.s.data() + (size_t)t * nsb, gu.data(), 2 * F, E);
                for (int i = 0; i < F; ++i) act[i] = orc_silu(gu[i]) * gu[F + i];
                orc_quantize_x_q8(act.data(), 1, F, aq.data(), ad.data(), as.data());
                orc_gemv_q4k_q8_seq(Wd, aq.data(), ad.data(), as.data(), v.data(), E, F);
                for (int i = 0; i < E; ++i) acc[i] = fmaf(w[t * ns + e], v[i], acc[i]);   // slot order (gemv.hip:1104-1112)
            }
            memcpy(y.data() + (size_t)t * E, acc.data(), (size_t)E * 4);
        }
    }
    void ffn_block(const OLayer& L, XQ& xq, int R, std::vector<float>& y) {
        const int F = c.n_ff; std::vector<float> gu((size_t)R * 2 * F);
        gemv(L.gate_up, xq, gu.data(), R, 2 * F);
        xq.set(R, F); orc_silu_mul_quant(gu.data(), 2 * F, F, xq.q.data(), xq.d.data(), xq.s.data(), R);
        y.assign((size_t)R * c.n_embd, 0.f); gemv(L.down, xq, y.data(), R, c.n_embd);
    }
    void embed_rows(const int* tok, int R, std::vector<float>& x) {
        x.resize((size_t)R * c.n_embd);
        for (int r = 0; r < R; ++r) { int id = tok[r]; if (id < 0 || id >= c.n_vocab) id = 0; for (int i = 0; i < c.n_embd; ++i) x[(size_t)r * c.n_embd + i] = bf2f(embed[(size_t)id * c.n_embd + i]); }
    }
    // qwen35.cpp:289-381
    void forward(const int* slots, const int* const* toks, const int* Ts, const int* poss, int S) {
        int R = 0; for (int i = 0; i < S; ++i) R += Ts[i];
        std::vector<int> tok(R), pos(R), slot(R); int r0 = 0;
        for (int i = 0; i < S; ++i) { for (int t = 0; t < Ts[i]; ++t) { tok[r0 + t] = toks[i][t]; pos[r0 + t] = poss[i] + t; slot[r0 + t] = slots[i]; } lr0[slots[i]] = r0; lT[slots[i]] = Ts[i]; r0 += Ts[i]; }
        const int E = c.n_embd, nv = c.gdn_v_heads, nq = c.gdn_qk_heads;
        std::vector<float> x, y; XQ xq; embed_rows(tok.data(), R, x);
        const size_t stl = (size_t)nv * 128 * 128, csl = (size_t)3 * (2 * nq + nv) * 128, kvl = (size_t)c.n_head_kv * c.max_ctx * 256;
        int gi = 0, ai = 0; bool have_y = false;
        for (int il = 0; il < c.n_layer; ++il) {
            const OLayer& L = layers[il];
            norm_in(x, have_y ? y.data() : nullptr, L.attn_norm, nullptr, xq, R);
            if (!L.is_attn) {
                float* rows = sv_rows.data() + (size_t)gi * 32 * ld_in;   // raw inputs saved for replay (qwen35.cpp:334-335)
                gemv(L.in_proj, xq, rows, R, ld_in);
                std::vector<float> ao((size_t)R * nv * 128);
                r0 = 0;
                for (int i = 0; i < S; ++i) {
                    const int s = slots[i], in = s * 2 + cur[s], outb = s * 2 + (cur[s] ^ 1);
                    // cur -> nxt (double buffer, qwen35.cpp:303-304): copy then update the copy
                    std::copy(gdn_state[in].begin() + gi * stl, gdn_state[in].begin() + (gi + 1) * stl, gdn_state[outb].begin() + gi * stl);
                    std::copy(conv_state[in].begin() + gi * csl, conv_state[in].begin() + (gi + 1) * csl, conv_state[outb].begin() + gi * csl);
                    orc_gdn_rows(rows + (size_t)r0 * ld_in, ld_in, Ts[i], nq, nv, L.conv_w.data(), L.dt_bias.data(), L.a_neg.data(), L.ssm_norm.data(),
                                 gdn_state[outb].data() + gi * stl, conv_state[outb].data() + gi * csl, ao.data() + (size_t)r0 * nv * 128, nullptr, c.rms_eps, c.gdn_sigmoid_gate);
                    r0 += Ts[i];
                }
                xq.set(R, nv * 128); orc_quantize_x_q8(ao.data(), R, nv * 128, xq.q.data(), xq.d.data(), xq.s.data());
                y.assign((size_t)R * E, 0.f); gemv(L.out_proj, xq, y.data(), R, E);
                ++gi;
            } else {
                attn_block(L, xq, kc, vc, (size_t)ai * kvl, pos.data(), slot.data(), R, y); ++ai;
            }
            if (c.n_expert) { std::vector<float> xn((size_t)R * E); norm_in(x, y.data(), L.post_norm, xn.data(), xq, R); moe_block(L, xq, xn, R, y, tok.data(), pos.data(), slot.data(), il); }
            else { norm_in(x, y.data(), L.post_norm, nullptr, xq, R); ffn_block(L, xq, R, y); }
            have_y = true;
        }
        norm_in(x, y.data(), output_norm, h.data(), xq, R);
        gemv(lm_head, xq, logits.data(), R, c.n_vocab);
    }
    // qwen35.cpp:383-403
    int accept(int slot, int m) {
        if (slot < 0 || slot >= c.n_slots || lT[slot] == 0) return 1;
        const int T = lT[slot], r0 = lr0[slot]; if (m < 1 || m > T) return 1;
        const int nv = c.gdn_v_heads, nq = c.gdn_qk_heads; const size_t stl = (size_t)nv * 128 * 128, csl = (size_t)3 * (2 * nq + nv) * 128;
        const int in = slot * 2 + cur[slot], outb = slot * 2 + (cur[slot] ^ 1);
        if (m < T) {   // replay the first m saved rows from the intact buffer
            int gi = 0;
            for (int il = 0; il < c.n_layer; ++il) {
                const OLayer& L = layers[il]; if (L.is_attn) continue;
                std::copy(gdn_state[in].begin() + gi * stl, gdn_state[in].begin() + (gi + 1) * stl, gdn_state[outb].begin() + gi * stl);
                std::copy(conv_state[in].begin() + gi * csl, conv_state[in].begin() + (gi + 1) * csl, conv_state[outb].begin() + gi * csl);
                orc_gdn_rows(sv_rows.data() + ((size_t)gi * 32 + r0) * ld_in, ld_in, m, nq, nv, L.conv_w.data(), L.dt_bias.data(), L.a_neg.data(), L.ssm_norm.data(),
                             gdn_state[outb].data() + gi * stl, conv_state[outb].data() + gi * csl, nullptr, nullptr, c.rms_eps, c.gdn_sigmoid_gate);
                ++gi;
            }
        }
        cur[slot] ^= 1; lT[slot] = 0; return 0;
    }
    // qwen35.cpp:405-424
    void mtp_forward(int slot, const int* tok, const float* hin, int T, int pos0) {
        const int E = c.n_embd; std::vector<float> e, x((size_t)T * E), y; XQ xq; embed_rows(tok, T, e);
        xq.set(T, 2 * E);
        orc_norm2_concat_quant(e.data(), enorm.data(), hin, E, hnorm.data(), nullptr, xq.q.data(), xq.d.data(), xq.s.data(), T, E, c.rms_eps);
        gemv(eh_proj, xq, x.data(), T, E);
        std::vector<int> pos(T), sl(T, slot); for (int t = 0; t < T; ++t) pos[t] = pos0 + t;
        norm_in(x, nullptr, mtp.attn_norm, nullptr, xq, T);
        attn_block(mtp, xq, mkc, mvc, 0, pos.data(), sl.data(), T, y);
        if (c.n_expert) { std::vector<float> xn((size_t)T * E); norm_in(x, y.data(), mtp.post_norm, xn.data(), xq, T); moe_block(mtp, xq, xn, T, y, tok, pos.data(), sl.data(), c.n_layer); }
        else { norm_in(x, y.data(), mtp.post_norm, nullptr, xq, T); ffn_block(mtp, xq, T, y); }
        norm_in(x, y.data(), head_norm, mh.data(), xq, T);
        gemv(lm_head, xq, mlogits.data(), T, c.n_vocab);
    }
};

extern "C" {
OrcModel* orc_model_create(const OrcCfg* cfg) { try { return new OrcModel(*cfg); } catch (...) { return nullptr; } }
void orc_model_free(OrcModel* m) { delete m; }
void orc_model_reset(OrcModel* m) { m->reset(); }
void orc_model_reset_slot(OrcModel* m, int s) { m->reset_slot(s); }
void orc_model_forward(OrcModel* m, const int* slots, const int* const* toks, const int* Ts, const int* poss, int S) { m->forward(slots, toks, Ts, poss, S); }
int orc_model_accept(OrcModel* m, int slot, int mm) { return m->accept(slot, mm); }
void orc_model_mtp_forward(OrcModel* m, int slot, const int* tok, const float* hin, int T, int pos0) { m->mtp_forward(slot, tok, hin, T, pos0); }
const float* orc_model_logits(OrcModel* m) { return m->logits.data(); }
const float* orc_model_h(OrcModel* m) { return m->h.data(); }
const float* orc_model_mtp_logits(OrcModel* m) { return m->mlogits.data(); }
const float* orc_model_mtp_h(OrcModel* m) { return m->mh.data(); }
const float* orc_model_gdn_state(OrcModel* m, int slot, int gdn_layer) { return m->gdn_state[slot * 2 + m->cur[slot]].data() + (size_t)gdn_layer * m->c.gdn_v_heads * 128 * 128; }
// generated tensor bytes (layer = -1 for model-level tensors); returns size in bytes, 0 if unknown
size_t orc_model_tensor(OrcModel* m, int layer, int kind, const void** ptr) {
    auto v8 = [&](const std::vector<uint8_t>& v) { *ptr = v.data(); return v.size(); };
    auto v16 = [&](const std::vector<uint16_t>& v) { *ptr = v.data(); return v.size() * 2; };
    if (layer < 0) {
        switch (kind) { case TK_EMBED: return v16(m->embed); case TK_OUTPUT_NORM: return v16(m->output_norm); case TK_LM_HEAD: return v8(m->lm_head.w);
                        case TK_MTP_ENORM: return v16(m->enorm); case TK_MTP_HNORM: return v16(m->hnorm); case TK_MTP_HEAD_NORM: return v16(m->head_norm); case TK_MTP_EH_PROJ: return v8(m->eh_proj.w); }
        return 0;
    }
    const OLayer& L = layer == m->c.n_layer ? m->mtp : m->layers[layer];
    switch (kind) { case TK_ATTN_NORM: return v16(L.attn_norm); case TK_POST_NORM: return v16(L.post_norm); case TK_IN_PROJ: return v8(L.in_proj.w); case TK_OUT_PROJ: return v8(L.out_proj.w);
                    case TK_GATE_UP: return v8(L.gate_up.w); case TK_DOWN: return v8(L.down.w); case TK_CONV_W: *ptr = L.conv_w.data(); return L.conv_w.size() * 4;
                    case TK_DT_BIAS: return v16(L.dt_bias); case TK_A_NEG: return v16(L.a_neg); case TK_SSM_NORM: return v16(L.ssm_norm); case TK_Q_NORM: return v16(L.q_norm); case TK_K_NORM: return v16(L.k_norm);
                    case TK_ROUTER: *ptr = L.router.data(); return L.router.size() * 4; case TK_EXP_GATE_UP: return v8(L.exp_gate_up.w); case TK_EXP_DOWN: return v8(L.exp_down.w);
                    case TK_SH_GATE_UP: return v8(L.sh_gate_up.w); case TK_SH_DOWN: return v8(L.sh_down.w); }
    return 0;
}
}
