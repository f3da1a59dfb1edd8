// CPU oracle, part 1: formats, activation quantiser, Q4_K GEMV, argmax/acceptance.
// TEST INFRASTRUCTURE ONLY -- see hp_oracle.h. Build with -ffp-contract=off: every fused
// multiply-add below is an explicit fmaf so that the rounding sequence is fixed by the source.
#include "hp_oracle.h"
#include <cmath>
#include <cstring>
#include <cstdlib>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---------------------------------------------------------------- formats
// engine/src/quant.h:11-17
extern "C" float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {                       // subnormal half: renormalise
            int e = 1;
            while (!(man & 0x400)) { man <<= 1; --e; }
            bits = sign | ((uint32_t)(e + 112) << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f; memcpy(&f, &bits, 4); return f;
}
// engine/src/quant.h:150-155 (round-half-up on the dropped bit, exactly as the reference does)
extern "C" uint16_t orc_f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000; const int e = (int)((x >> 23) & 0xff) - 127 + 15; uint32_t m = x & 0x7fffff;
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000; const uint32_t t = 14 - e; uint32_t r = m >> t; if ((m >> (t - 1)) & 1) r++;
        return (uint16_t)(sign | r);
    }
    if (e >= 31) return (uint16_t)(sign | 0x7c00);
    uint32_t r = sign | ((uint32_t)e << 10) | (m >> 13); if (m & 0x1000) r++;
    return (uint16_t)r;
}
// engine/src/quant.h:37-40
extern "C" void orc_q4k_scale_min(const uint8_t sc12[12], uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 8; ++j) {
        if (j < 4) { sc[j] = sc12[j] & 63; mn[j] = sc12[j + 4] & 63; }
        else { sc[j] = (sc12[j + 4] & 0xF) | ((sc12[j - 4] >> 6) << 4); mn[j] = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4); }
    }
}
// engine/src/quant.h:43-53: element 64g+l = low nibble of byte 32g+l with (scale,min) 2g; 64g+32+l = high nibble with 2g+1
extern "C" void orc_dequant_q4k(const uint8_t* blocks, size_t nblk, float* y) {
    for (size_t b = 0; b < nblk; ++b) {
        const uint8_t* blk = blocks + b * 144;
        uint16_t dh, mh; memcpy(&dh, blk, 2); memcpy(&mh, blk + 2, 2);
        const float d = orc_f16_to_f32(dh), dmin = orc_f16_to_f32(mh);
        uint8_t sc[8], mn[8]; orc_q4k_scale_min(blk + 4, sc, mn);
        const uint8_t* q = blk + 16;
        float* out = y + b * 256;
        for (int g = 0; g < 4; ++g) {
            const float d1 = d * sc[2 * g], m1 = dmin * mn[2 * g], d2 = d * sc[2 * g + 1], m2 = dmin * mn[2 * g + 1];
            for (int l = 0; l < 32; ++l) out[64 * g + l] = d1 * (float)(q[32 * g + l] & 0xF) - m1;
            for (int l = 0; l < 32; ++l) out[64 * g + 32 + l] = d2 * (float)(q[32 * g + l] >> 4) - m2;
        }
    }
}

// ---------------------------------------------------------------- deterministic math
// The reference device code uses the fast intrinsics __expf / log1pf (ops.hip:11-13). This build
// defines exp and log by a fixed sequence of IEEE fp32 operations so that the CUDA kernels and this
// oracle produce the same bits; the definition below is restated (not shared) in the device header.
static inline float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
extern "C" float orc_expf(float x) {
    float xc = x; if (xc > 90.f) xc = 90.f; if (xc < -110.f) xc = -110.f;
    const float fn = rintf(xc * 1.44269504088896341f);
    float r = fmaf(fn, -0.693359375f, xc);
    r = fmaf(fn, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float z = r * r;
    float y = fmaf(p, z, r) + 1.0f;
    const int n = (int)fn, n1 = n >> 1, n2 = n - n1;
    y = y * bits_f((uint32_t)(n1 + 127) << 23);
    return y * bits_f((uint32_t)(n2 + 127) << 23);
}
static float orc_logf_ge1(float x) {   // x >= 1, finite
    const uint32_t ix = f_bits(x);
    int e = (int)(ix >> 23) - 127;
    float m = bits_f((ix & 0x007fffffu) | 0x3f800000u);   // [1, 2)
    if (m > 1.41421356237f) { m = m * 0.5f; e += 1; }
    const float f = m - 1.0f, z = f * f, fe = (float)e;
    float p = 7.0376836292e-2f;
    p = fmaf(p, f, -1.1514610310e-1f);
    p = fmaf(p, f, 1.1676998740e-1f);
    p = fmaf(p, f, -1.2420140846e-1f);
    p = fmaf(p, f, 1.4249322787e-1f);
    p = fmaf(p, f, -1.6668057665e-1f);
    p = fmaf(p, f, 2.0000714765e-1f);
    p = fmaf(p, f, -2.4999993993e-1f);
    p = fmaf(p, f, 3.3333331174e-1f);
    float y = (p * f) * z;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(z, -0.5f, y);
    float r = f + y;
    return fmaf(fe, 0.693359375f, r);
}
extern "C" float orc_log1pf_pos(float e) {
    const float u = 1.0f + e;
    if (u == 1.0f) return e;
    if (!(u < 3.0e38f)) return orc_logf_ge1(3.0e38f);
    const float c = (e - (u - 1.0f)) / u;
    return orc_logf_ge1(u) + c;
}
extern "C" float orc_sigmoid(float x) { return 1.0f / (1.0f + orc_expf(-x)); }          // ops.hip:12
extern "C" float orc_silu(float x) { return x / (1.0f + orc_expf(-x)); }                 // ops.hip:11
extern "C" float orc_softplus(float x) { return x > 20.f ? x : orc_log1pf_pos(orc_expf(x)); }   // ops.hip:13

// ---------------------------------------------------------------- activation quantiser
// gemv.hip:40-50 / bench_gemv.cpp:17-25: amax over 32; d = amax/127; id = 127/amax (two divisions);
// q = round-half-even(x*id); s = d * sum(q).
extern "C" void orc_quantize_x_q8(const float* x, int R, int K, int8_t* q, float* d, float* s) {
    const int nsb = K / 32;
    for (int r = 0; r < R; ++r)
        for (int b = 0; b < nsb; ++b) {
            const float* xb = x + (size_t)r * K + b * 32;
            float amax = 0.f; for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(xb[l]));
            const float dd = amax / 127.f, id = amax > 0.f ? 127.f / amax : 0.f;
            int sum = 0;
            for (int l = 0; l < 32; ++l) { const int qi = (int)nearbyintf(xb[l] * id); q[(size_t)r * K + b * 32 + l] = (int8_t)qi; sum += qi; }
            d[(size_t)r * nsb + b] = dd; s[(size_t)r * nsb + b] = dd * (float)sum;
        }
}

// ---------------------------------------------------------------- Q4_K GEMV, f32 activations
// gemv.hip:1177-1216: lane l of TPR takes blocks l, l+TPR, ...; per 64-group the four running sums over 32
// elements, then acc += d0*s0 - m0*sx0 + d1*s1 - m1*sx1 (left to right); lanes combined by the xor-shuffle
// tree with offsets TPR/2 .. 1 (:1213).
extern "C" void orc_gemv_q4k_f32(const uint8_t* W, const float* x, float* y, int N, int K, int R, int tpr) {
    const int nb = K / 256;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < N; ++row) {
        const uint8_t* wrow = W + (size_t)row * nb * 144;
        std::vector<float> lane(tpr);
        for (int c = 0; c < R; ++c) {
            for (int l = 0; l < tpr; ++l) {
                float acc = 0.f;
                for (int b = l; b < nb; b += tpr) {
                    const uint8_t* blk = wrow + (size_t)b * 144;
                    uint16_t dh, mh; memcpy(&dh, blk, 2); memcpy(&mh, blk + 2, 2);
                    const float d = orc_f16_to_f32(dh), dmin = orc_f16_to_f32(mh);
                    uint8_t sc[8], mn[8]; orc_q4k_scale_min(blk + 4, sc, mn);
                    const float* xb = x + (size_t)c * K + (size_t)b * 256;
                    for (int j = 0; j < 4; ++j) {
                        const float d0 = d * sc[2 * j], m0 = dmin * mn[2 * j], d1 = d * sc[2 * j + 1], m1 = dmin * mn[2 * j + 1];
                        const uint8_t* q = blk + 16 + 32 * j; const float* xc = xb + 64 * j;
                        float s0 = 0.f, s1 = 0.f, sx0 = 0.f, sx1 = 0.f;
                        for (int e = 0; e < 32; ++e) {
                            const float x0 = xc[e], x1 = xc[32 + e];
                            s0 = fmaf(x0, (float)(q[e] & 0xF), s0); s1 = fmaf(x1, (float)(q[e] >> 4), s1);
                            sx0 = sx0 + x0; sx1 = sx1 + x1;
                        }
                        float t = d0 * s0; t = t - m0 * sx0; t = t + d1 * s1; t = t - m1 * sx1;
                        acc = acc + t;
                    }
                }
                lane[l] = acc;
            }
            for (int off = tpr / 2; off > 0; off >>= 1) {
                std::vector<float> nxt(tpr);
                for (int l = 0; l < tpr; ++l) nxt[l] = lane[l] + lane[l ^ off];
                lane.swap(nxt);
            }
            y[(size_t)c * N + row] = lane[0];
        }
    }
}

// ---------------------------------------------------------------- Q4_K GEMV, int8 activations (production numerics)
// gemv.hip:602-672 contract: exact int32 dot over each 32-element sub-block, one fp32 update per sub-block in block
// order, split-K partials summed in a fixed order that depends on the tensor shape only:
//     acc = fmaf((d*sc)*xd, (float)idot, acc);  acc = fmaf(-(dmin*mn), xs, acc);
// The shape-only partition of this build (restated from the kernel's description, not shared with it):
//  - K/256 blocks are cut into P equal parts, P in {1, 2, 4} dividing K/256 with at most 36 blocks per part, chosen to
//    maximise 1000*tiles/(g*ceil(tiles/g)) - 20*log2(P) - (50 if blocks per part is odd), g = 148/P, ties -> smaller P;
//  - the g work groups of a part split the 16-row tiles evenly: group c owns tiles [c*tiles/g, (c+1)*tiles/g);
//  - inside a group the stream of units (tile major, then chunks of cb = 2 (or 1) blocks along the part) is divided
//    evenly over min(12, units) workers: worker w owns units [w*U/We, (w+1)*U/We);
//  - a tile's value for a part is the sum, in worker order, of each worker's partial sum over its own blocks;
//  - y is the sum of the part values in part order.
static int orc_num_parts(int N, int nb) {
    const int tiles = (N + 15) / 16; int best = 0, best_score = -1000000;
    for (int lg = 0; lg < 3; ++lg) {
        const int P = 1 << lg; if (nb % P) continue;
        const int nbp = nb / P; if (nbp > 36) continue;
        const int gc = 148 / P, per = (tiles + gc - 1) / gc;
        const int score = (int)((long long)tiles * 1000 / ((long long)gc * per)) - 20 * lg - ((nbp & 1) ? 50 : 0);
        if (score > best_score) { best_score = score; best = P; }
    }
    return best;
}
extern "C" int orc_gemv_parts(int N, int K) { return orc_num_parts(N, K / 256); }
extern "C" void orc_gemv_q4k_q8(const uint8_t* W, const int8_t* q, const float* xd, const float* xs, float* y, int N, int K, int R, int ldy) {
    const int nb = K / 256, nsb = K / 32, tiles = (N + 15) / 16;
    const int P = orc_num_parts(N, nb);
    if (P == 0) return;
    const int nbp = nb / P, cb = (nbp % 2 == 0) ? 2 : 1, C = nbp / cb, gc = 148 / P;
    for (int p = 0; p < P; ++p) {
        const int kb0 = p * nbp;
#pragma omp parallel for schedule(dynamic, 1)
        for (int cg = 0; cg < gc; ++cg) {
            const int t0 = (int)((long long)cg * tiles / gc), t1 = (int)((long long)(cg + 1) * tiles / gc);
            const long long cu = (long long)(t1 - t0) * C; if (cu == 0) continue;
            const long long we = cu < 12 ? cu : 12;
            auto start = [&](long long w) { return w * cu / we; };
            auto owner = [&](long long u) { return ((u + 1) * we - 1) / cu; };
            for (int tile = t0; tile < t1; ++tile) {
                const long long a0 = (long long)(tile - t0) * C, a1 = a0 + C;
                const long long w_first = owner(a0), w_last = owner(a1 - 1);
                for (int rr = 0; rr < 16; ++rr) {
                    const int row = tile * 16 + rr; if (row >= N) break;
                    const uint8_t* wrow = W + (size_t)row * nb * 144;
                    for (int c = 0; c < R; ++c) {
                        const int8_t* xq = q + (size_t)c * K; const float* cd = xd + (size_t)c * nsb; const float* cs = xs + (size_t)c * nsb;
                        float v = 0.f;
                        for (long long ww = w_first; ww <= w_last; ++ww) {
                            const long long ulo = start(ww) > a0 ? start(ww) : a0, uhi = start(ww + 1) < a1 ? start(ww + 1) : a1;
                            float acc = 0.f;
                            for (long long u = ulo; u < uhi; ++u)
                                for (int blk = 0; blk < cb; ++blk) {
                                    const int b = kb0 + (int)(u - a0) * cb + blk;
                                    const uint8_t* bp = wrow + (size_t)b * 144;
                                    uint16_t dh, mh; memcpy(&dh, bp, 2); memcpy(&mh, bp + 2, 2);
                                    const float d = orc_f16_to_f32(dh), dmin = orc_f16_to_f32(mh);
                                    uint8_t sc[8], mn[8]; orc_q4k_scale_min(bp + 4, sc, mn);
                                    for (int sb = 0; sb < 8; ++sb) {
                                        const int grp = sb >> 1, hi = sb & 1;
                                        const uint8_t* qs = bp + 16 + 32 * grp; const int8_t* xe = xq + (size_t)b * 256 + 32 * sb;
                                        int idot = 0;
                                        for (int e = 0; e < 32; ++e) idot += (int)(hi ? (qs[e] >> 4) : (qs[e] & 0xF)) * (int)xe[e];
                                        const float s0 = d * (float)sc[sb], m = dmin * (float)mn[sb];
                                        const float tt = s0 * cd[b * 8 + sb];
                                        acc = fmaf(tt, (float)idot, acc);
                                        acc = fmaf(-m, cs[b * 8 + sb], acc);
                                    }
                                }
                            v = ww == w_first ? acc : v + acc;
                        }
                        float* yp = y + (size_t)c * ldy + row;
                        *yp = p > 0 ? *yp + v : v;
                    }
                }
            }
        }
    }
}

// bench_gemv.cpp:97-104
extern "C" void orc_gemv_q4k_double(const uint8_t* W, const float* x, double* y, double* mag, int N, int K, int R) {
    const int nb = K / 256;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < N; ++row) {
        std::vector<float> w(K);
        orc_dequant_q4k(W + (size_t)row * nb * 144, nb, w.data());
        for (int c = 0; c < R; ++c) {
            double ref = 0, m = 0;
            for (int k = 0; k < K; ++k) { const double p = (double)w[k] * (double)x[(size_t)c * K + k]; ref += p; m += fabs(p); }
            y[(size_t)c * N + row] = ref; if (mag) mag[(size_t)c * N + row] = m;
        }
    }
}

// ---------------------------------------------------------------- argmax + acceptance
// ops.hip:706-713: strict > inside a scan, ties between scanners resolved to the lower index: max value, lowest index.
extern "C" void orc_argmax(const float* logits, int R, int n, int ld, int* ids, float* vals) {
    for (int r = 0; r < R; ++r) {
        const float* x = logits + (size_t)r * ld;
        float bv = -INFINITY; int bi = -1;
        for (int i = 0; i < n; ++i) if (x[i] > bv) { bv = x[i]; bi = i; }
        ids[r] = bi; if (vals) vals[r] = bv;
    }
}
// spec27b.cpp:92-97
// top-k per row: k rounds of a masked arg-max, strict > from the lowest index (ops.hip:702-716: values descending,
// ties -> lower index; an entry equal to -inf is never selected: id -1)
extern "C" void orc_topk(const float* logits, int R, int n, int ld, int k, int* ids, float* vals) {
    std::vector<char> taken(n);
    for (int r = 0; r < R; ++r) {
        std::fill(taken.begin(), taken.end(), 0);
        const float* x = logits + (size_t)r * ld;
        for (int j = 0; j < k; ++j) {
            float bv = -INFINITY; int bi = -1;
            for (int i = 0; i < n; ++i) if (!taken[i] && x[i] > bv) { bv = x[i]; bi = i; }
            ids[(size_t)r * k + j] = bi; vals[(size_t)r * k + j] = bv; if (bi >= 0) taken[bi] = 1;
        }
    }
}
extern "C" int orc_accept(const int* ids, const int* drafts, int n_draft, int* bonus) {
    int mm = 0; while (mm < n_draft && ids[mm] == drafts[mm]) ++mm;
    if (bonus) *bonus = ids[mm];
    return mm;
}
