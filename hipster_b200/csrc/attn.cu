// GQA decode attention over the f16 KV cache for the rows of a verify pass.
//
// Reference: k_qk_norm_rope_kv (engine/kernels/ops.hip:363-411), the scalar decode attention k_attn (:413-465, the
// semantic reference) and the production split-KV structure k_attn_mq + k_attn_mq_merge (:831-948): fixed absolute
// key splits merged in split order, so that a row's result does not depend on the number of rows in the pass.
//
// Here: head_dim 256, NeoX RoPE on the first n_rot = 64 dims from a host-built cos/sin table (double precision,
// rounded to fp32), K and V stored row-major f16 [slot][kv head][position][256]. One CTA per (split of 128 keys,
// kv head, row group <= 8 rows): the K and V tiles are read once for all rows x q-heads of the group. All arithmetic
// is fp32 FMA in a fixed order (scores: fmaf chain over d = 0..255; P.V: fmaf chain over keys in position order;
// merge: splits in order), so the CPU oracle reproduces it bit for bit. KV traffic is ~2 % of a pass's bytes, so SIMT
// fp32 is affordable, and it avoids the tensor-core rounding hazard the reference documents (docs/decode-27b.md:117-126).
#include "hp_common.cuh"
#include "kernels.h"
#include <algorithm>

namespace hp {
namespace {

constexpr int HD = 256, SPL = ATTN_SPLIT, MAXP = ATTN_MAX_PAIRS;   // pairs = rows of the group x q-heads per kv head
constexpr int KSTRIDE = HD + 4;                                     // f16 elements per K/V tile row (520 B: conflict-free)
constexpr int ESTR = MAXP + 4;                                      // floats per key row of the score tile: lanes = keys hit 8 banks (16-way conflicts at 48)

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

// grid: rows * (n_head + n_kv) blocks of 256 threads; row layout: [q_full: n_head x (256 q | 256 gate) | k: n_kv x 256 | v: n_kv x 256]
// planes != nullptr: the projection arrives as P K-part planes ([rows][ld] each, part_stride apart); they are added in
// part order here (q, gate, k and v slices of this block) and q / gate are written to qkv for the attention kernels.
__global__ void __launch_bounds__(256) k_qk_norm_rope_kv(float* __restrict__ qkv, const float* __restrict__ planes, int P, size_t part_stride,
                                                          int ld, int n_head, int n_kv, const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                                                          const float2* __restrict__ rope, int n_rot, const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                                                          uint16_t* __restrict__ kc, uint16_t* __restrict__ vc, size_t kv_stride, int max_ctx, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh[8]; __shared__ float buf[HD];
    const int t = threadIdx.x, hb = blockIdx.x % (n_head + n_kv), r = blockIdx.x / (n_head + n_kv);
    const int pos = row_pos[r], slot = row_slot[r];
    const bool isq = hb < n_head;
    const size_t xoff = (isq ? (size_t)r * ld + hb * 512 : (size_t)r * ld + n_head * 512 + (hb - n_head) * HD) + t;
    // second slice of this block: the gate of a q head, the v of a kv head
    const size_t yoff = isq ? xoff + HD : (size_t)r * ld + n_head * 512 + n_kv * HD + (hb - n_head) * HD + t;
    float* x = qkv + (xoff - t);
    float xv, yv;
    if (planes) {
        xv = planes[xoff]; yv = planes[yoff];
        for (int p = 1; p < P; ++p) { xv = xv + planes[(size_t)p * part_stride + xoff]; yv = yv + planes[(size_t)p * part_stride + yoff]; }
        if (isq) qkv[yoff] = yv;
    } else { xv = x[t]; yv = qkv[yoff]; }
    const float ss = block_sum_det<8>(xv * xv, sh);
    float n = (xv * (1.0f / sqrtf(ss / (float)HD + eps))) * bf2f((isq ? qw : kw)[t]);
    buf[t] = n;
    __syncthreads();
    const int half = n_rot / 2;
    if (t < n_rot) {
        const int i = t % half; const float2 cs = rope[(size_t)pos * half + i];   // (cos, sin) of pos * base^(-2i/n_rot)
        const float x0 = buf[i], x1 = buf[i + half];
        n = t < half ? fmaf(-x1, cs.y, x0 * cs.x) : fmaf(x1, cs.x, x0 * cs.y);
    }
    x[t] = n;
    if (!isq) {
        const int kh = hb - n_head;
        const float vv = yv;
        const size_t o = (size_t)slot * kv_stride + ((size_t)kh * max_ctx + pos) * HD + t;
        kc[o] = f2h(n); vc[o] = f2h(vv);
    }
}

__device__ __forceinline__ float2 attn_fma2(float2 a, float2 b, float2 c) {   // a * b + c per lane
    float2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(r))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)), "l"(reinterpret_cast<unsigned long long&>(c)));
    return r;
}
struct AttnArgs {
    const float* qkv; int ld, n_head, n_kv;
    const uint16_t* kc; const uint16_t* vc; size_t kv_stride; int max_ctx;
    const int* groups;        // device: per group {r0, T, slot, pos0}
    float* pO; float* pm; float* pl; int nsplit_max;   // partials [group][kv head][split][MAXP] (x 256 for pO)
};
// grid (nsplit_max, n_kv, ngroups), NT threads, dynamic smem. PPT = (row, head) pairs per thread in the score phase
// (warp w takes pairs w*PPT .. w*PPT+PPT-1): 16 warps x 3 cover the 48 pairs of a full verify group, 8 warps x 1 the
// <= 8 pairs of a single-row pass, where the wider tile would spend most warps on absent pairs. The kernel is bound by
// the latency of its fp32 chains at one CTA per SM, so the verify form spreads them over 16 warps. Every score and
// every output element is the same fmaf chain whatever the geometry is.
template <int PPT, int NT>
__global__ void __launch_bounds__(NT) k_attn_split(AttnArgs a) {
    constexpr int NW = NT / 32, NP = NW * PPT;   // pairs this instantiation can hold
    constexpr int PARTS = NT / (HD / 2), PP = NP / PARTS;   // P.V phase: thread = (two dims, part of the pairs)
    static_assert(NT % (HD / 2) == 0 && PP % 4 == 0 && NP <= MAXP, "attention tile geometry");
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t sm_raw[];
    float* sQ = reinterpret_cast<float*>(sm_raw);                                   // [MAXP][256]
    float* sE = sQ + MAXP * HD;                                                     // [SPL][ESTR] scores, then weights
    uint16_t* sK = reinterpret_cast<uint16_t*>(sE + SPL * ESTR);                    // [SPL][KSTRIDE]
    uint16_t* sV = sK + SPL * KSTRIDE;                                              // [SPL][KSTRIDE]
    const int split = blockIdx.x, kh = blockIdx.y, gi = blockIdx.z, tid = threadIdx.x;
    const int r0 = a.groups[gi * 4], T = a.groups[gi * 4 + 1], slot = a.groups[gi * 4 + 2], pos0 = a.groups[gi * 4 + 3];
    const int G = a.n_head / a.n_kv, npairs = T * G;
    const int k_lo = split * SPL;
    const int nkeys = min(SPL, pos0 + T - k_lo);          // keys of this split visible to the last row of the group
    if (nkeys <= 0 || T <= 0) return;
    const size_t pbase = (((size_t)gi * a.n_kv + kh) * a.nsplit_max + split) * MAXP;
    // stage Q (pair = t*G + hh -> row r0+t, head kh*G + hh), K and V tiles
    for (int i = tid; i < npairs * (HD / 4); i += NT) {
        const int p = i / (HD / 4), d4 = i % (HD / 4), tr = p / G, hh = p % G;
        reinterpret_cast<float4*>(sQ)[p * (HD / 4) + d4] = reinterpret_cast<const float4*>(a.qkv + (size_t)(r0 + tr) * a.ld + (kh * G + hh) * 512)[d4];
    }
    const uint16_t* Kg = a.kc + (size_t)slot * a.kv_stride + ((size_t)kh * a.max_ctx + k_lo) * HD;
    const uint16_t* Vg = a.vc + (size_t)slot * a.kv_stride + ((size_t)kh * a.max_ctx + k_lo) * HD;
    for (int i = tid; i < nkeys * (HD / 8); i += NT) {
        const int k = i / (HD / 8), c = i % (HD / 8);
        const uint4 kv = reinterpret_cast<const uint4*>(Kg + (size_t)k * HD)[c], vv = reinterpret_cast<const uint4*>(Vg + (size_t)k * HD)[c];
        uint2* dk = reinterpret_cast<uint2*>(sK + k * KSTRIDE + c * 8); dk[0] = make_uint2(kv.x, kv.y); dk[1] = make_uint2(kv.z, kv.w);
        uint2* dv = reinterpret_cast<uint2*>(sV + k * KSTRIDE + c * 8); dv[0] = make_uint2(vv.x, vv.y); dv[1] = make_uint2(vv.z, vv.w);
    }
    __syncthreads();
    // scores: thread (kq = tid % 32, pq = tid / 32) -> keys kq + 32*i (i < 4), pairs pq*PPT + jx (jx < PPT); fmaf chain over d
    {
        const int kq = tid & 31, pq = tid >> 5;
        float s[4][PPT];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jx = 0; jx < PPT; ++jx) s[i][jx] = 0.f;
        for (int d = 0; d < HD; d += 4) {
            float kf[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint2 kk = *reinterpret_cast<const uint2*>(sK + (kq + 32 * i) * KSTRIDE + d);
                kf[i][0] = h2f((uint16_t)(kk.x & 0xFFFF)); kf[i][1] = h2f((uint16_t)(kk.x >> 16));
                kf[i][2] = h2f((uint16_t)(kk.y & 0xFFFF)); kf[i][3] = h2f((uint16_t)(kk.y >> 16));
            }
#pragma unroll
            for (int jx = 0; jx < PPT; ++jx) {
                const int p = pq * PPT + jx;
                const float4 qv = p < npairs ? *reinterpret_cast<const float4*>(sQ + p * HD + d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[i][jx] = fmaf(qv.x, kf[i][0], s[i][jx]); s[i][jx] = fmaf(qv.y, kf[i][1], s[i][jx]);
                    s[i][jx] = fmaf(qv.z, kf[i][2], s[i][jx]); s[i][jx] = fmaf(qv.w, kf[i][3], s[i][jx]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jx = 0; jx < PPT; ++jx) { const int p = pq * PPT + jx; if (p < MAXP) sE[(kq + 32 * i) * ESTR + p] = s[i][jx] * 0.0625f; }
    }
    __syncthreads();
    // softmax pieces per pair: warp w takes pairs w, w+8, ...; lane l takes keys l, l+32, l+64, l+96. Row t of the group
    // sees keys <= pos0 + t. Maximum: exact in any order. Sum: the lane's keys in ascending order, then the xor tree (16..1).
    {
        const int warp = tid >> 5, lane = tid & 31;
        for (int p = warp; p < npairs; p += NW) {
            const int tr = p / G;
            const int nk = min(nkeys, pos0 + tr + 1 - k_lo);
            float sc[4]; float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 4; ++i) { const int k = lane + 32 * i; sc[i] = k < nk ? sE[k * ESTR + p] : -INFINITY; mx = fmaxf(mx, sc[i]); }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float l = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = lane + 32 * i;
                const float e = k < nk ? expf_det(sc[i] - mx) : 0.f;
                if (k < nkeys) sE[k * ESTR + p] = e;
                l = i == 0 ? e : l + e;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) l = l + __shfl_xor_sync(0xffffffffu, l, off);
            if (lane == 0) { a.pm[pbase + p] = mx; a.pl[pbase + p] = l; }   // nk <= 0: mx = -inf, l = 0 (the merge skips it)
        }
    }
    __syncthreads();
    // o[pair][d] = sum_k e[k][pair] * v[k][d], keys in position order; thread = (dims 2 dq and 2 dq + 1, part of the pairs):
    // a warp's read of four weights serves 64 dims, which halves the shared-memory traffic that bounds this phase
    {
        const int dq = tid % (HD / 2), p_lo = (tid / (HD / 2)) * PP;
        float2 o[PP / 2][2];   // [pairs 2 p, 2 p + 1][dim]: two fp32 fmaf per instruction, each rounded once
#pragma unroll
        for (int p = 0; p < PP / 2; ++p) { o[p][0] = make_float2(0.f, 0.f); o[p][1] = make_float2(0.f, 0.f); }
        for (int k = 0; k < nkeys; ++k) {
            const uint32_t vh = *reinterpret_cast<const uint32_t*>(sV + k * KSTRIDE + 2 * dq);
            const float v0 = h2f((uint16_t)(vh & 0xFFFF)), v1 = h2f((uint16_t)(vh >> 16));
            const float2 vv0 = make_float2(v0, v0), vv1 = make_float2(v1, v1);
#pragma unroll
            for (int p4 = 0; p4 < PP / 4; ++p4) {
                const float4 e = *reinterpret_cast<const float4*>(sE + k * ESTR + p_lo + p4 * 4);
                o[p4 * 2][0] = attn_fma2(make_float2(e.x, e.y), vv0, o[p4 * 2][0]);
                o[p4 * 2][1] = attn_fma2(make_float2(e.x, e.y), vv1, o[p4 * 2][1]);
                o[p4 * 2 + 1][0] = attn_fma2(make_float2(e.z, e.w), vv0, o[p4 * 2 + 1][0]);
                o[p4 * 2 + 1][1] = attn_fma2(make_float2(e.z, e.w), vv1, o[p4 * 2 + 1][1]);
            }
        }
#pragma unroll
        for (int p = 0; p < PP / 2; ++p) {
            if (p_lo + 2 * p < npairs) *reinterpret_cast<float2*>(a.pO + (pbase + p_lo + 2 * p) * HD + 2 * dq) = make_float2(o[p][0].x, o[p][1].x);
            if (p_lo + 2 * p + 1 < npairs) *reinterpret_cast<float2*>(a.pO + (pbase + p_lo + 2 * p + 1) * HD + 2 * dq) = make_float2(o[p][0].y, o[p][1].y);
        }
    }
}

// merge the splits of one (row, q-head) in split order, gate, write f32 + q8. grid rows * n_head, 256 threads
__global__ void __launch_bounds__(256) k_attn_merge(const float* __restrict__ qkv, int ld, int n_head, int n_kv, const int* __restrict__ groups, const int* __restrict__ row_group,
                                                     const float* __restrict__ pO, const float* __restrict__ pm, const float* __restrict__ pl, int nsplit_max,
                                                     float* __restrict__ out, int8_t* __restrict__ oq, float* __restrict__ osc) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x / n_head, head = blockIdx.x % n_head, d = threadIdx.x;
    const int gi = row_group[r];
    const int r0 = groups[gi * 4], pos0 = groups[gi * 4 + 3];
    const int G = n_head / n_kv, kh = head / G, hh = head % G, tr = r - r0, pair = tr * G + hh;
    const int nsplit = (pos0 + tr + 1 + SPL - 1) / SPL;
    const size_t pb = (((size_t)gi * n_kv + kh) * nsplit_max) * MAXP + pair;
    float mx = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, pm[pb + (size_t)s * MAXP]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = pm[pb + (size_t)s * MAXP];
        const float w = expf_det(ms - mx);
        o = fmaf(w, pO[(pb + (size_t)s * MAXP) * HD + d], o);
        l = fmaf(w, pl[pb + (size_t)s * MAXP], l);
    }
    const float gate = qkv[(size_t)r * ld + head * 512 + HD + d];
    const float v = (o / l) * sigmoid_det(gate);
    const size_t oi = (size_t)r * n_head * HD + head * HD + d;
    if (out) out[oi] = v;
    if (oq) warp_quant32_store(v, r, (head * HD + d) >> 5, n_head * HD, oq, osc, d & 31);
}

// descriptors of one sequence of R consecutive rows at pos0.. (slot 0), cut into row groups of gr rows
__global__ void k_attn_desc(int* __restrict__ d, int R, int pos0, int gr) {
    const int t = threadIdx.x; if (t >= R) return;
    d[t] = pos0 + t; d[32 + t] = 0; d[64 + t] = t / gr;
    if (t % gr == 0) { int* g = d + 96 + 4 * (t / gr); g[0] = t; g[1] = min(gr, R - t); g[2] = 0; g[3] = pos0 + t; }
}

}  // namespace

size_t attn_smem_bytes() { return (size_t)MAXP * HD * 4 + (size_t)SPL * ESTR * 4 + 2 * (size_t)SPL * KSTRIDE * 2; }
size_t attn_partial_floats(int ngroups, int n_kv, int nsplit_max) { return (size_t)ngroups * n_kv * nsplit_max * MAXP; }

int attn_rope_kv(const AttnParams& p, int rows, cudaStream_t s) {
    HP_REQUIRE(rows >= 1 && p.n_head % p.n_kv == 0 && p.n_rot % 2 == 0 && p.n_rot <= HD, "attn_rope_kv: bad shape");
    HP_CUDA(launch_pdl<4>(k_qk_norm_rope_kv, dim3(rows * (p.n_head + p.n_kv)), dim3(256), 0, s, p.qkv, p.planes, p.P, p.part_stride, p.ld, p.n_head, p.n_kv, (const uint16_t*)p.q_norm, (const uint16_t*)p.k_norm, (const float2*)p.rope, p.n_rot,
                       p.row_pos, p.row_slot, (uint16_t*)p.kc, (uint16_t*)p.vc, p.kv_stride, p.max_ctx, p.eps));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
int attn_decode(const AttnParams& p, int rows, int ngroups, cudaStream_t s) {
    HP_REQUIRE(rows >= 1 && ngroups >= 1 && p.n_head % p.n_kv == 0 && (p.n_head / p.n_kv) <= MAXP, "attn_decode: at most %d (row, head) pairs per kv head and group", MAXP);
    static bool attr_dev[MAX_DEVICES] = {};   // per device: the opt-in belongs to the device's copy of the kernel
    const int dev = current_device(); if (dev < 0) return HP_ECUDA;
    bool& attr = attr_dev[dev];
    if (!attr) {
        HP_CUDA(cudaFuncSetAttribute(k_attn_split<3, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes()));
        HP_CUDA(cudaFuncSetAttribute(k_attn_split<1, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes()));
        attr = true;
    }
    AttnArgs a; a.qkv = p.qkv; a.ld = p.ld; a.n_head = p.n_head; a.n_kv = p.n_kv; a.kc = (const uint16_t*)p.kc; a.vc = (const uint16_t*)p.vc;
    a.kv_stride = p.kv_stride; a.max_ctx = p.max_ctx; a.groups = p.groups; a.pO = p.pO; a.pm = p.pm; a.pl = p.pl; a.nsplit_max = p.nsplit_max;
    // group sizes live on the device; `rows` bounds the rows of any group, so rows * G <= 8 selects the narrow score tile
    if (rows * (p.n_head / p.n_kv) <= 8) HP_CUDA(launch_pdl<4>(k_attn_split<1, 256>, dim3(p.nsplit_max, p.n_kv, ngroups), dim3(256), attn_smem_bytes(), s, a));
    else HP_CUDA(launch_pdl<4>(k_attn_split<3, 512>, dim3(p.nsplit_max, p.n_kv, ngroups), dim3(512), attn_smem_bytes(), s, a));
    HP_CUDA(launch_pdl<4>(k_attn_merge, dim3(rows * p.n_head), dim3(256), 0, s, p.qkv, p.ld, p.n_head, p.n_kv, p.groups, p.row_group, p.pO, p.pm, p.pl, p.nsplit_max, p.out, (int8_t*)p.xq.q, (float*)p.xq.sc));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

}  // namespace hp

namespace hp {
// Kernel-level form for one sequence: rows r = 0..R-1 at positions pos0 + r. The workspace holds the device-side
// descriptors (256 ints) followed by the split partials.
static int attn_seq_groups(int R, int n_head, int n_kv) { const int gr = std::max(1, std::min(8, ATTN_MAX_PAIRS / (n_head / n_kv))); return (R + gr - 1) / gr; }
size_t attn_seq_workspace_bytes(int R, int n_head, int n_kv, int max_ctx) {
    const size_t np = attn_partial_floats(attn_seq_groups(R, n_head, n_kv), n_kv, (max_ctx + ATTN_SPLIT - 1) / ATTN_SPLIT);
    return 1024 + np * (HD + 2) * sizeof(float);
}
int attn_decode_seq(float* qkv, int ld, int R, int pos0, int n_head, int n_kv, int n_rot, const void* q_norm, const void* k_norm, const void* rope, void* kc, void* vc, int max_ctx,
                    float* out, XQ8F xq, float eps, void* workspace, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && R <= 8 && pos0 >= 0 && pos0 + R <= max_ctx, "attn_decode_seq: 1 <= R <= 8 rows inside the context");
    HP_REQUIRE(n_kv >= 1 && n_head % n_kv == 0 && n_head / n_kv <= ATTN_MAX_PAIRS && ld >= n_head * 512 + 2 * n_kv * HD, "attn_decode_seq: bad head geometry");
    const int gr = std::max(1, std::min(8, ATTN_MAX_PAIRS / (n_head / n_kv))), ng = attn_seq_groups(R, n_head, n_kv);
    int* d = (int*)workspace;
    k_attn_desc<<<1, 32, 0, s>>>(d, R, pos0, gr);
    HP_CUDA(cudaGetLastError());
    AttnParams p; p.qkv = qkv; p.ld = ld; p.n_head = n_head; p.n_kv = n_kv; p.n_rot = n_rot; p.q_norm = q_norm; p.k_norm = k_norm; p.rope = rope;
    p.row_pos = d; p.row_slot = d + 32; p.row_group = d + 64; p.groups = d + 96;
    p.kc = kc; p.vc = vc; p.kv_stride = 0; p.max_ctx = max_ctx; p.nsplit_max = (max_ctx + ATTN_SPLIT - 1) / ATTN_SPLIT;
    const size_t np = attn_partial_floats(ng, n_kv, p.nsplit_max);
    p.pO = (float*)((char*)workspace + 1024); p.pm = p.pO + np * HD; p.pl = p.pm + np;
    p.out = out; p.xq = xq; p.eps = eps;
    const int rc = attn_rope_kv(p, R, s);
    return rc != HP_OK ? rc : attn_decode(p, R, ng, s);
}
}  // namespace hp
