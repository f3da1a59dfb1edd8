// Host engine: see engine.h. Reference: engine/src/qwen35.cpp (constructor :80-153, forward :289-381, accept :383-403,
// mtp_forward :405-424, topk :426-430), MTP driver engine/bench/spec27b.cpp:59-103.
#include "hp_common.cuh"
#include "engine.h"
#include <cmath>
#include <cstring>
#include <algorithm>

namespace hp {

// ------------------------------------------------------------------ seeded weight generation (device)
// Counter-based: value = f(seed, tensor id, index); integer arithmetic plus exactly-rounded float operations only,
// so a CPU regenerates identical tensors. Normal deviates are approximated by the sum of four uniform 16-bit
// integers (Irwin-Hall, sigma = 65536 * sqrt(4/12)), which is bounded by +-3.46 sigma.
__host__ __device__ inline uint16_t f32_to_f16_bits(float f) {   // same rounding as the reference's f32_to_f16 (engine/src/quant.h:150-155)
    const uint32_t x = f_bits(f); const uint32_t sign = (x >> 16) & 0x8000; const int e = (int)((x >> 23) & 0xff) - 127 + 15; uint32_t m = x & 0x7fffff;
    if (e <= 0) { if (e < -10) return (uint16_t)sign; m |= 0x800000; const uint32_t t = 14 - e; uint32_t r = m >> t; if ((m >> (t - 1)) & 1) r++; return (uint16_t)(sign | r); }
    if (e >= 31) return (uint16_t)(sign | 0x7c00);
    uint32_t r = sign | ((uint32_t)e << 10) | (m >> 13); if (m & 0x1000) r++;
    return (uint16_t)r;
}
__host__ __device__ inline uint16_t f32_to_bf16_bits(float f) { uint32_t u = f_bits(f); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }

// Q4_K blocks: quants uniform 0..15, the 6-bit scales/mins uniform 0..63 (any 12 bytes), d and dmin = f16(|N(0, 0.01)|)
__global__ void k_gen_q4k(uint64_t* __restrict__ w, size_t nwords, uint64_t seed, uint64_t tid, size_t word0) {
    const size_t li = (size_t)blockIdx.x * blockDim.x + threadIdx.x; if (li >= nwords) return;
    const size_t i = li + word0;   // global word index of the tensor (a GPU may hold only a slice of it)
    uint64_t v = rnd64(seed, tid, i);
    if (i % 18 == 0) {
        const size_t b = i / 18;
        const uint16_t d = f32_to_f16_bits(fabsf(irwin(rnd64(seed, tid ^ 0xD00Dull, b))) * 0.01f);
        const uint16_t dm = f32_to_f16_bits(fabsf(irwin(rnd64(seed, tid ^ 0xE00Eull, b))) * 0.01f);
        v = (v & 0xFFFFFFFF00000000ull) | (uint64_t)d | ((uint64_t)dm << 16);
    }
    w[li] = v;
}
__global__ void k_gen_bf16(uint16_t* __restrict__ p, size_t n, uint64_t seed, uint64_t tid, float mean, float std, int neg_abs) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; if (i >= n) return;
    float v = mean + std * irwin(rnd64(seed, tid, i)); if (neg_abs) v = -fabsf(v);
    p[i] = f32_to_bf16_bits(v);
}
__global__ void k_gen_f32(float* __restrict__ p, size_t n, uint64_t seed, uint64_t tid, float mean, float std, int neg_abs) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; if (i >= n) return;
    float v = mean + std * irwin(rnd64(seed, tid, i)); if (neg_abs) v = -fabsf(v);
    p[i] = v;
}
__global__ void k_set_ints(int* p, int n, int v) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) p[i] = v; }
__global__ void k_reduce_planes(const float* __restrict__ parts, size_t part_stride, int P, float* __restrict__ y, int N, int ldy) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y; if (n >= N) return;
    float v = parts[(size_t)r * N + n];
    for (int p = 1; p < P; ++p) v = v + parts[(size_t)p * part_stride + (size_t)r * N + n];
    y[(size_t)r * ldy + n] = v;
}

// ---- pass descriptor (ints, device + pinned host copy): per row token / position / slot / attention row group, per
// attention row group {r0, T, slot, pos0}, per sequence {r0, T, slot, -}. A pass has at most MAXR rows, so at most MAXR
// row groups (one per row in the worst head geometry) and MAXS sequences.
enum { D_TOK = 0, D_POS = 32, D_SLOT = 64, D_RGROUP = 96, D_GROUPS = 128, D_SEQS = 256, D_INTS = 320 };
static_assert(D_POS - D_TOK >= Engine::MAXR && D_SLOT - D_POS >= Engine::MAXR && D_RGROUP - D_SLOT >= Engine::MAXR && D_GROUPS - D_RGROUP >= Engine::MAXR, "row tables hold MAXR rows");
static_assert(D_SEQS - D_GROUPS >= 4 * Engine::MAXR && D_INTS - D_SEQS >= 4 * Engine::MAXS, "group / sequence tables hold MAXR groups and MAXS sequences");

// ---- fused speculative round over S slots: device-side bookkeeping (the host loops of engine/bench/spec27b.cpp:77-103
// and engine/bench/batchfn.cpp:96-117). Per-slot state block of SP_INTS ints; the round's inputs (slot list, seeded
// substitutions) arrive in a separate block so that one captured graph serves every round of the same (S, n). ----
enum { SP_ID_LAST = 0, SP_POS = 1, SP_MM = 2, SP_COUNT = 3, SP_POS_OLD = 4, SP_DRAFTS = 8, SP_IDS = 16, SP_OUT = 24, SP_INTS = 32 };
enum { SI_SLOTS = 0, SI_SUBST = 8, SI_INTS = 8 + 8 * 8 };   // inputs: slots[S], subst[request][8]
// Rows of a pass of the round. mode 0: draft step i (one row per slot: the last emitted token or the previous draft, at
// pos + i; spec27b.cpp:81-85); mode 1: verify rows [id_last, d1..dn] at pos.. (spec27b.cpp:88-90); mode 2: MTP catch-up
// rows d1..dn at pos_old + 1.. (spec27b.cpp:99). Request j (slot slots[j]) owns rows j*Tm ..; its rows are cut into
// attention row groups of at most gr rows.
__global__ void k_spec_setup(const int* __restrict__ sp, const int* __restrict__ in, int* __restrict__ d, int mode, int i, int n, int S, int gr) {
    pdl_launch_dependents();
    pdl_wait();
    const int Tm = mode == 0 ? 1 : mode == 1 ? n + 1 : n, gps = (Tm + gr - 1) / gr;
    for (int e = threadIdx.x; e < S * Tm; e += blockDim.x) {
        const int j = e / Tm, t = e - j * Tm, slot = in[SI_SLOTS + j];
        const int* st = sp + slot * SP_INTS;
        int tok, pos;
        if (mode == 0) { tok = i == 0 ? st[SP_ID_LAST] : st[SP_DRAFTS + i - 1]; pos = st[SP_POS] + i; }
        else if (mode == 1) { tok = t == 0 ? st[SP_ID_LAST] : st[SP_DRAFTS + t - 1]; pos = st[SP_POS] + t; }
        else { tok = st[SP_DRAFTS + t]; pos = st[SP_POS_OLD] + 1 + t; }
        d[D_TOK + e] = tok; d[D_POS + e] = pos; d[D_SLOT + e] = slot; d[D_RGROUP + e] = j * gps + t / gr;
        if (t % gr == 0) { int* g = d + D_GROUPS + 4 * (j * gps + t / gr); g[0] = e; g[1] = min(gr, Tm - t); g[2] = slot; g[3] = pos; }
        if (t == 0) { int* q = d + D_SEQS + 4 * j; q[0] = e; q[1] = Tm; q[2] = slot; q[3] = 0; }
    }
}
// rows of hstage (request order) <- per-slot pending hidden rows (draft step 0), or <- rows of the verify pass' h
// (catch-up: rows t < n of each request)
__global__ void __launch_bounds__(256) k_spec_gather_h(const int* __restrict__ in, const float* __restrict__ hpend, const float* __restrict__ h, float* __restrict__ dst, int mode, int n, int E) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x;   // destination row
    const float* src;
    if (mode == 0) src = hpend + (size_t)in[SI_SLOTS + e] * E;
    else { const int j = e / n, t = e - j * n; src = h + (size_t)(j * (n + 1) + t) * E; }
    for (int i = threadIdx.x; i < E; i += 256) dst[(size_t)e * E + i] = src[i];
}
// the draft of request j is the MTP argmax unless the caller substitutes it (seeded acceptance control)
__global__ void k_spec_take(int* __restrict__ sp, const int* __restrict__ in, const int* __restrict__ mids, int i, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = threadIdx.x; if (j >= S) return;
    const int sub = in[SI_SUBST + 8 * j + i];
    sp[in[SI_SLOTS + j] * SP_INTS + SP_DRAFTS + i] = sub >= 0 ? sub : mids[j];
}
// greedy prefix acceptance per slot (spec27b.cpp:92-102): mm accepted drafts, bonus = ids[mm], commit mm+1 rows,
// h_pending = h row mm of the slot. One block per request.
__global__ void __launch_bounds__(256) k_spec_accept(int* __restrict__ sp, const int* __restrict__ in, const int* __restrict__ ids, int* __restrict__ replay_n, int n,
                                                      const float* __restrict__ h, float* __restrict__ hpend, int E) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int smm;
    const int j = blockIdx.x, slot = in[SI_SLOTS + j];
    int* st = sp + slot * SP_INTS; const int* id = ids + j * (n + 1);
    if (threadIdx.x == 0) {
        int mm = 0; while (mm < n && id[mm] == st[SP_DRAFTS + mm]) ++mm;
        for (int i = 0; i <= n; ++i) st[SP_IDS + i] = id[i];
        for (int i = 0; i < mm; ++i) st[SP_OUT + i] = st[SP_DRAFTS + i];
        st[SP_OUT + mm] = id[mm];
        st[SP_MM] = mm; st[SP_COUNT] = mm + 1; st[SP_POS_OLD] = st[SP_POS]; st[SP_POS] = st[SP_POS] + mm + 1; st[SP_ID_LAST] = id[mm];
        replay_n[slot] = mm + 1;
        smm = mm;
    }
    __syncthreads();
    const float* src = h + (size_t)(j * (n + 1) + smm) * E; float* dst = hpend + (size_t)slot * E;
    for (int i = threadIdx.x; i < E; i += 256) dst[i] = src[i];
}

#define HP_TRY(x) do { const int rc_ = (x); if (rc_ != HP_OK) return rc_; } while (0)
// descriptor layout (ints)
Engine::Engine(const hp_model_cfg& cfg) : c_(cfg) {}
Engine::~Engine() {
    ep_destroy();
    for (cudaGraphExec_t g : graphs_) if (g) cudaGraphExecDestroy(g);
    for (auto& v : ep_segs_) for (EpSeg& sg : v) if (sg.g) cudaGraphExecDestroy(sg.g);
    for (void* p : allocs_) cudaFree(p);
    if (h_desc_) cudaFreeHost(h_desc_);
    if (h_spec_) cudaFreeHost(h_spec_);
    if (ev0_) cudaEventDestroy(ev0_); if (ev1_) cudaEventDestroy(ev1_);
    if (s_) cudaStreamDestroy(s_);
}
int Engine::nattn() const { return c_.n_layer / c_.attn_every; }
int Engine::ngdn() const { return c_.n_layer - nattn(); }

int Engine::alloc(void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) { set_error("out of device memory allocating %zu bytes (%s)", bytes, cudaGetErrorString(e)); return HP_ENOMEM; }
    allocs_.push_back(*p); return HP_OK;
}
int Engine::gen_lin(Lin& l, int N, int K, uint64_t tid) {
    l.N = N; l.K = K; l.bytes = (size_t)N * (K / 256) * 144; l.P = gemv_parts(N, K);
    HP_REQUIRE(K % 256 == 0 && l.P > 0, "tensor %d x %d is not a valid Q4_K GEMV shape", N, K);
    if (int rc = alloc((void**)&l.w, l.bytes)) return rc;
    const size_t nwords = l.bytes / 8;
    k_gen_q4k<<<(unsigned)((nwords + 255) / 256), 256, 0, s_>>>((uint64_t*)l.w, nwords, c_.seed, tid, 0);
    HP_CUDA(cudaGetLastError());
    weight_bytes_ += l.bytes;
    if (tiled_) {   // the GEMV streams the tile-major copy; the row-major original is kept only for small (test) models
        HP_TRY(alloc((void**)&l.wt, gemv_tiled_bytes(N, K)));
        HP_TRY(gemv_repack_tiled(l.w, l.wt, N, K, s_));
        if (!keep_rowmajor_) {
            HP_CUDA(cudaStreamSynchronize(s_));
            for (size_t i = 0; i < allocs_.size(); ++i) if (allocs_[i] == l.w) { allocs_.erase(allocs_.begin() + i); break; }
            HP_CUDA(cudaFree(l.w)); l.w = nullptr;
        }
    }
    return HP_OK;
}
int Engine::gen_raw_q4k(Lin& l, size_t rows, int K, uint64_t tid, size_t row0, size_t nrows_local, int interleave_half) {   // expert stacks: no GEMV partition attached
    // rows [row0, row0 + nrows_local) of a tensor of `rows` rows are generated; l.w is offset so that it can be indexed
    // with global row numbers (a GPU that holds a shard of the experts never dereferences the rows of other shards).
    // The grouped expert GEMV streams the tile-major copy l.wt, which holds the local rows only.
    if (nrows_local == (size_t)-1) nrows_local = rows;
    const size_t rb = (size_t)(K / 256) * 144;
    l.N = (int)std::min<size_t>(rows, 0x7fffffff); l.K = K; l.P = 1; l.bytes = nrows_local * rb;
    HP_REQUIRE(K % 256 == 0 && nrows_local % 16 == 0, "expert tensor K=%d must be a multiple of 256 (rows a multiple of 16)", K);
    uint8_t* base = nullptr;
    if (int rc = alloc((void**)&base, l.bytes)) return rc;
    const size_t nwords = l.bytes / 8;
    k_gen_q4k<<<(unsigned)((nwords + 255) / 256), 256, 0, s_>>>((uint64_t*)base, nwords, c_.seed, tid, row0 * rb / 8);
    HP_CUDA(cudaGetLastError());
    l.w = base - row0 * rb;
    weight_bytes_ += l.bytes;
    HP_TRY(alloc((void**)&l.wt, gemv_tiled_bytes(nrows_local, K)));
    HP_TRY(gemv_repack_tiled(base, l.wt, nrows_local, K, s_, interleave_half));
    if (!keep_rowmajor_) {
        HP_CUDA(cudaStreamSynchronize(s_));
        for (size_t i = 0; i < allocs_.size(); ++i) if (allocs_[i] == base) { allocs_.erase(allocs_.begin() + i); break; }
        HP_CUDA(cudaFree(base)); l.w = nullptr;
    }
    return HP_OK;
}
int Engine::gen_bf16(uint16_t** p, size_t n, uint64_t tid, float mean, float std, bool neg_abs) {
    if (int rc = alloc((void**)p, n * 2)) return rc;
    k_gen_bf16<<<(unsigned)((n + 255) / 256), 256, 0, s_>>>(*p, n, c_.seed, tid, mean, std, neg_abs ? 1 : 0);
    HP_CUDA(cudaGetLastError()); weight_bytes_ += n * 2; return HP_OK;
}
int Engine::gen_f32(float** p, size_t n, uint64_t tid, float mean, float std, bool neg_abs) {
    if (int rc = alloc((void**)p, n * 4)) return rc;
    k_gen_f32<<<(unsigned)((n + 255) / 256), 256, 0, s_>>>(*p, n, c_.seed, tid, mean, std, neg_abs ? 1 : 0);
    HP_CUDA(cudaGetLastError()); weight_bytes_ += n * 4; return HP_OK;
}

static inline uint64_t tensor_id(int layer, int kind) { return (uint64_t)(layer + 1) * 64 + (uint64_t)kind; }

int Engine::init() {
    const hp_model_cfg& c = c_;
    HP_REQUIRE(c.n_embd > 0 && c.n_embd % 256 == 0 && c.n_layer >= 1 && c.n_vocab > 0, "bad model shape");
    HP_REQUIRE(c.n_head >= 1 && c.n_head_kv >= 1 && c.n_head % c.n_head_kv == 0 && (c.n_head / c.n_head_kv) <= ATTN_MAX_PAIRS, "bad attention head counts");
    HP_REQUIRE(c.gdn_qk_heads >= 1 && c.gdn_v_heads % c.gdn_qk_heads == 0 && (c.gdn_v_heads * 128) % 256 == 0, "bad GDN head counts");
    HP_REQUIRE(c.attn_every >= 1 && c.n_slots >= 1 && c.n_slots <= MAXS && c.max_ctx >= 16 && c.n_rot % 2 == 0 && c.n_rot <= 256, "bad configuration");
    HP_REQUIRE(c.ep_world <= 1 || (c.n_expert > 0 && c.ep_rank >= 0 && c.ep_rank < c.ep_world && c.n_expert % c.ep_world == 0), "bad expert-parallel configuration");
    HP_REQUIRE(c.n_expert == 0 ? (c.n_ff > 0 && c.n_ff % 256 == 0) : (c.expert_ff % 256 == 0 && c.n_expert_used >= 1 && c.n_expert_used <= 15), "bad FFN shape");
    HP_CUDA(cudaStreamCreateWithFlags(&s_, cudaStreamNonBlocking));
    tiled_ = getenv("HIPSTER_B200_ROWMAJOR") == nullptr;
    // small models keep both layouts (tensor access in tests): dense FFN elements, or routed-expert elements, below 2^28 / 2^30
    keep_rowmajor_ = (size_t)c.n_layer * c.n_embd * (size_t)std::max(c.n_ff, 1) < ((size_t)1 << 28) &&
                     (size_t)c.n_layer * std::max(c.n_expert, 0) * 3 * c.n_embd * (size_t)std::max(c.expert_ff, 0) < ((size_t)1 << 30);
    HP_CUDA(cudaEventCreate(&ev0_)); HP_CUDA(cudaEventCreate(&ev1_));
    const int E = c.n_embd, nv = c.gdn_v_heads, nq = c.gdn_qk_heads;
    const int gdn_in = (2 * nq + nv) * 128 + nv * 128 + 2 * nv, attn_in = c.n_head * 512 + 2 * c.n_head_kv * 256;
    ld_in_ = gdn_in;
    auto gen_layer = [&](LayerW& L, int il, bool is_attn) -> int {
        L.is_attn = is_attn;
        HP_TRY(gen_bf16(&L.attn_norm, E, tensor_id(il, TK_ATTN_NORM), 1.f, 0.1f));
        HP_TRY(gen_bf16(&L.post_norm, E, tensor_id(il, TK_POST_NORM), 1.f, 0.1f));
        if (is_attn) {
            HP_TRY(gen_lin(L.in_proj, attn_in, E, tensor_id(il, TK_IN_PROJ)));
            HP_TRY(gen_lin(L.out_proj, E, c.n_head * 256, tensor_id(il, TK_OUT_PROJ)));
            HP_TRY(gen_bf16(&L.q_norm, 256, tensor_id(il, TK_Q_NORM), 1.f, 0.2f));
            HP_TRY(gen_bf16(&L.k_norm, 256, tensor_id(il, TK_K_NORM), 1.f, 0.2f));
        } else {
            HP_TRY(gen_lin(L.in_proj, gdn_in, E, tensor_id(il, TK_IN_PROJ)));
            HP_TRY(gen_lin(L.out_proj, E, nv * 128, tensor_id(il, TK_OUT_PROJ)));
            HP_TRY(gen_f32(&L.conv_w, (size_t)(2 * nq + nv) * 128 * 4, tensor_id(il, TK_CONV_W), 0.f, 0.5f, false));
            HP_TRY(gen_bf16(&L.dt_bias, nv, tensor_id(il, TK_DT_BIAS), 0.f, 0.5f));
            // the decay exponent must not be positive (a_neg = -exp(A_log) in the model; the reference's kernel test draws
            // -|N(0, 1)|, engine/bench/test_fnkernels.cpp:33): a positive one makes the recurrent state grow without bound
            HP_TRY(gen_bf16(&L.a_neg, nv, tensor_id(il, TK_A_NEG), 0.8f, 0.4f, true));
            HP_TRY(gen_bf16(&L.ssm_norm, 128, tensor_id(il, TK_SSM_NORM), 1.f, 0.3f));
        }
        if (c.n_expert == 0) {
            HP_TRY(gen_lin(L.gate_up, 2 * c.n_ff, E, tensor_id(il, TK_GATE_UP)));
            HP_TRY(gen_lin(L.down, E, c.n_ff, tensor_id(il, TK_DOWN)));
        } else {   // routed experts (contiguous per tensor, qwen4exp weights layout [512*N][K]) + one shared expert + f32 router
            const int F = c.expert_ff;
            HP_TRY(gen_f32(&L.router, (size_t)(c.n_expert + 1) * E, tensor_id(il, TK_ROUTER), 0.f, 1.0f / sqrtf((float)E), false));
            const int w = std::max(1, c.ep_world), elo = (int)((long long)c.ep_rank * c.n_expert / w), ehi = (int)((long long)(c.ep_rank + 1) * c.n_expert / w);
            HP_TRY(gen_raw_q4k(L.exp_gate_up, (size_t)c.n_expert * 2 * F, E, tensor_id(il, TK_EXP_GATE_UP), (size_t)elo * 2 * F, (size_t)(ehi - elo) * 2 * F, F));
            HP_TRY(gen_raw_q4k(L.exp_down, (size_t)c.n_expert * E, F, tensor_id(il, TK_EXP_DOWN), (size_t)elo * E, (size_t)(ehi - elo) * E, 0));
            HP_TRY(gen_raw_q4k(L.sh_gate_up, (size_t)2 * F, E, tensor_id(il, TK_SH_GATE_UP), 0, (size_t)-1, F));
            HP_TRY(gen_raw_q4k(L.sh_down, (size_t)E, F, tensor_id(il, TK_SH_DOWN), 0, (size_t)-1, 0));
        }
        return HP_OK;
    };
    layers_.resize(c.n_layer);
    for (int il = 0; il < c.n_layer; ++il) HP_TRY(gen_layer(layers_[il], il, (il + 1) % c.attn_every == 0));
    HP_TRY(gen_bf16(&embed_, (size_t)c.n_vocab * E, tensor_id(-1, TK_EMBED), 0.f, 1.f));
    HP_TRY(gen_bf16(&output_norm_, E, tensor_id(-1, TK_OUTPUT_NORM), 1.f, 0.1f));
    HP_TRY(gen_lin(lm_head_, c.n_vocab, E, tensor_id(-1, TK_LM_HEAD)));
    if (c.has_mtp) {
        HP_TRY(gen_layer(mtp_, c.n_layer, true));
        HP_TRY(gen_bf16(&mtp_enorm_, E, tensor_id(-1, TK_MTP_ENORM), 1.f, 0.1f));
        HP_TRY(gen_bf16(&mtp_hnorm_, E, tensor_id(-1, TK_MTP_HNORM), 1.f, 0.1f));
        HP_TRY(gen_bf16(&mtp_head_norm_, E, tensor_id(-1, TK_MTP_HEAD_NORM), 1.f, 0.1f));
        HP_TRY(gen_lin(eh_proj_, E, 2 * E, tensor_id(-1, TK_MTP_EH_PROJ)));
    }
    // RoPE table (cos, sin) of pos * base^(-2i/n_rot), computed in double precision on the host
    {
        const int half = c.n_rot / 2; std::vector<float> tab((size_t)c.max_ctx * half * 2);
        for (int p = 0; p < c.max_ctx; ++p)
            for (int i = 0; i < half; ++i) {
                const double th = (double)p * std::pow((double)c.rope_base, -2.0 * i / (double)c.n_rot);
                tab[((size_t)p * half + i) * 2] = (float)std::cos(th); tab[((size_t)p * half + i) * 2 + 1] = (float)std::sin(th);
            }
        HP_TRY(alloc((void**)&rope_, tab.size() * 4));
        HP_CUDA(cudaMemcpyAsync(rope_, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, s_));
        HP_CUDA(cudaStreamSynchronize(s_));
    }
    // state
    st_layer_ = (size_t)nv * 128 * 128; st_stride_ = st_layer_ * ngdn();
    cs_layer_ = (size_t)nv * 3 * 384; cs_stride_ = cs_layer_ * ngdn();
    HP_TRY(alloc((void**)&gdn_state_, st_stride_ * c.n_slots * 4)); HP_TRY(alloc((void**)&conv_state_, cs_stride_ * c.n_slots * 4));
    kv_layer_ = (size_t)c.n_head_kv * c.max_ctx * 256; kv_slot_ = kv_layer_ * nattn();
    HP_TRY(alloc((void**)&kc_, kv_slot_ * c.n_slots * 2)); HP_TRY(alloc((void**)&vc_, kv_slot_ * c.n_slots * 2));
    HP_CUDA(cudaMemsetAsync(kc_, 0, kv_slot_ * c.n_slots * 2, s_)); HP_CUDA(cudaMemsetAsync(vc_, 0, kv_slot_ * c.n_slots * 2, s_));
    if (c.has_mtp) {
        HP_TRY(alloc((void**)&mkc_, kv_layer_ * c.n_slots * 2)); HP_TRY(alloc((void**)&mvc_, kv_layer_ * c.n_slots * 2));
        HP_CUDA(cudaMemsetAsync(mkc_, 0, kv_layer_ * c.n_slots * 2, s_)); HP_CUDA(cudaMemsetAsync(mvc_, 0, kv_layer_ * c.n_slots * 2, s_));
    }
    sv_layer_ = (size_t)nv * 8 * 388; sv_stride_ = sv_layer_ * ngdn();   // raw GDN inputs of the last pass, per slot / layer / head (replay buffers, qwen35.h:124)
    HP_TRY(alloc((void**)&saved_, sv_stride_ * c.n_slots * 4)); HP_CUDA(cudaMemsetAsync(saved_, 0, sv_stride_ * c.n_slots * 4, s_));
    HP_TRY(alloc((void**)&replay_n_, MAXS * 4)); HP_CUDA(cudaMemsetAsync(replay_n_, 0, MAXS * 4, s_));
    pend_.assign(c.n_slots, 0); last_r0_.assign(c.n_slots, 0); last_T_.assign(c.n_slots, 0);
    // work buffers
    const int F = c.n_expert ? c.expert_ff : c.n_ff;
    const size_t bigw = std::max<size_t>({(size_t)gdn_in, (size_t)attn_in, (size_t)2 * F, (size_t)2 * E});
    const size_t kmax = std::max<size_t>({(size_t)2 * E, (size_t)F, (size_t)c.n_head * 256, (size_t)nv * 128});
    HP_TRY(alloc((void**)&x_, (size_t)MAXR * E * 4)); HP_TRY(alloc((void**)&emb_, (size_t)MAXR * E * 4));
    HP_TRY(alloc((void**)&big_, (size_t)MAXR * bigw * 4));
    HP_TRY(alloc((void**)&yparts_, (size_t)4 * MAXR * std::max<size_t>(bigw, E) * 4));
    HP_TRY(alloc((void**)&logits_, (size_t)MAXR * c.n_vocab * 4)); HP_TRY(alloc((void**)&mlogits_, (size_t)MAXR * c.n_vocab * 4));
    HP_TRY(alloc((void**)&h_, (size_t)MAXR * E * 4)); HP_TRY(alloc((void**)&mh_, (size_t)MAXR * E * 4));
    HP_CUDA(cudaMemsetAsync(h_, 0, (size_t)MAXR * E * 4, s_)); HP_CUDA(cudaMemsetAsync(mh_, 0, (size_t)MAXR * E * 4, s_));
    HP_TRY(alloc(&xq_.q, xq_q_bytes(MAXR, (int)kmax))); HP_TRY(alloc(&xq_.sc, xq_sc_floats(MAXR, (int)kmax) * 4));
    HP_CUDA(cudaMemsetAsync(xq_.q, 0, xq_q_bytes(MAXR, (int)kmax), s_)); HP_CUDA(cudaMemsetAsync(xq_.sc, 0, xq_sc_floats(MAXR, (int)kmax) * 4, s_));
    if (c.n_expert) {
        const int ns = c.n_expert_used + 1, pairs = MAXR * ns;
        HP_TRY(alloc((void**)&xn_, (size_t)MAXR * E * 4));
        HP_TRY(alloc((void**)&rlogits_, (size_t)MAXR * (c.n_expert + 1) * 4));
        HP_TRY(alloc((void**)&moe_ids_, (size_t)pairs * 4)); HP_TRY(alloc((void**)&moe_w_, (size_t)pairs * 4));
        HP_TRY(alloc((void**)&route_cnt_, (size_t)MAXR * 4)); HP_CUDA(cudaMemsetAsync(route_cnt_, 0, (size_t)MAXR * 4, s_));
        HP_TRY(alloc((void**)&moe_v_, (size_t)pairs * E * 4));
        HP_TRY(alloc(&moe_segs_, moe_seg_bytes())); HP_TRY(alloc((void**)&moe_ctl_, 16)); HP_TRY(alloc((void**)&moe_touched_, 8));
        HP_CUDA(cudaMemsetAsync(moe_ctl_, 0, 16, s_)); HP_CUDA(cudaMemsetAsync(moe_touched_, 0, 8, s_));
        HP_TRY(alloc(&xq2_.q, xq_q_bytes(pairs, F))); HP_TRY(alloc(&xq2_.sc, xq_sc_floats(pairs, F) * 4));
        HP_CUDA(cudaMemsetAsync(xq2_.q, 0, xq_q_bytes(pairs, F), s_)); HP_CUDA(cudaMemsetAsync(xq2_.sc, 0, xq_sc_floats(pairs, F) * 4, s_));
        moe_out_.N = E; moe_out_.K = F; moe_out_.P = 1;
        { const int w = std::max(1, c.ep_world); e_lo_ = (int)((long long)c.ep_rank * c.n_expert / w); e_hi_ = (int)((long long)(c.ep_rank + 1) * c.n_expert / w); }
    }
    nsplit_max_ = (c.max_ctx + ATTN_SPLIT - 1) / ATTN_SPLIT;
    const size_t np = attn_partial_floats(MAXR, c.n_head_kv, nsplit_max_);
    HP_TRY(alloc((void**)&pO_, np * 256 * 4)); HP_TRY(alloc((void**)&pm_, np * 4)); HP_TRY(alloc((void**)&pl_, np * 4));
    HP_TRY(alloc((void**)&d_desc_, D_INTS * 4)); HP_CUDA(cudaMallocHost((void**)&h_desc_, D_INTS * 4)); memset(h_desc_, 0, D_INTS * 4);
    HP_TRY(alloc((void**)&d_ids_, MAXR * 4)); HP_TRY(alloc((void**)&d_mids_, MAXR * 4)); HP_TRY(alloc((void**)&d_vals_, MAXR * 4)); HP_TRY(alloc((void**)&d_mvals_, MAXR * 4));
    HP_TRY(alloc(&am_scratch_, argmax_scratch_bytes(MAXR, c.n_vocab)));
    HP_TRY(alloc(&topk_scratch_, topk_scratch_bytes(MAXR, c.n_vocab, topk_max_k())));
    HP_TRY(alloc((void**)&d_topk_ids_, (size_t)MAXR * topk_max_k() * 4)); HP_TRY(alloc((void**)&d_topk_vals_, (size_t)MAXR * topk_max_k() * 4));
    HP_TRY(alloc((void**)&prof_kv_, (size_t)2 * nattn() * c.n_head_kv * 8 * 256 * 2 + 16));
    HP_TRY(alloc((void**)&d_spec_, MAXS * SP_INTS * 4)); HP_TRY(alloc((void**)&d_specin_, SI_INTS * 4));
    HP_CUDA(cudaMallocHost((void**)&h_spec_, (SI_INTS + MAXS * SP_INTS) * 4)); memset(h_spec_, 0, (SI_INTS + MAXS * SP_INTS) * 4);
    HP_CUDA(cudaMemsetAsync(d_spec_, 0, MAXS * SP_INTS * 4, s_)); HP_CUDA(cudaMemsetAsync(d_specin_, 0, SI_INTS * 4, s_));
    HP_TRY(alloc((void**)&hpend_, (size_t)MAXS * E * 4)); HP_CUDA(cudaMemsetAsync(hpend_, 0, (size_t)MAXS * E * 4, s_));
    HP_TRY(alloc((void**)&hstage_, (size_t)MAXR * E * 4)); HP_CUDA(cudaMemsetAsync(hstage_, 0, (size_t)MAXR * E * 4, s_));
    HP_TRY(alloc((void**)&hprev_, (size_t)MAXS * E * 4)); HP_CUDA(cudaMemsetAsync(hprev_, 0, (size_t)MAXS * E * 4, s_));
    spec_pos_.assign(c.n_slots, 0); spec_on_.assign(c.n_slots, 0);
    HP_TRY(alloc((void**)&err_, 4)); HP_CUDA(cudaMemsetAsync(err_, 0, 4, s_));
    HP_TRY(reset());
    HP_CUDA(cudaStreamSynchronize(s_));
    return HP_OK;
}

int Engine::reset() {
    HP_CUDA(cudaMemsetAsync(gdn_state_, 0, st_stride_ * c_.n_slots * 4, s_)); HP_CUDA(cudaMemsetAsync(conv_state_, 0, cs_stride_ * c_.n_slots * 4, s_));
    HP_CUDA(cudaMemsetAsync(replay_n_, 0, MAXS * 4, s_));
    for (int s = 0; s < c_.n_slots; ++s) { pend_[s] = 0; last_T_[s] = 0; last_r0_[s] = 0; }
    return HP_OK;
}
int Engine::reset_slot(int slot) {
    HP_REQUIRE(slot >= 0 && slot < c_.n_slots, "reset_slot: bad slot %d", slot);
    HP_CUDA(cudaMemsetAsync(gdn_state_ + (size_t)slot * st_stride_, 0, st_stride_ * 4, s_)); HP_CUDA(cudaMemsetAsync(conv_state_ + (size_t)slot * cs_stride_, 0, cs_stride_ * 4, s_));
    HP_CUDA(cudaMemsetAsync(replay_n_ + slot, 0, 4, s_));
    pend_[slot] = 0; last_T_[slot] = 0; return HP_OK;
}

int Engine::upload_desc() { HP_CUDA(cudaMemcpyAsync(d_desc_, h_desc_, D_INTS * 4, cudaMemcpyHostToDevice, s_)); return HP_OK; }

// profiling only: class bit of a linear by its shape (16 gate|up, 32 down, 64 LM head, 128 input projections, 256 the rest)
static int lin_class_bit(const Lin& l, const hp_model_cfg& c) {
    return l.N == 2 * c.n_ff ? 16 : l.K == c.n_ff ? 32 : l.N == c.n_vocab ? 64 : l.K == c.n_embd ? 128 : 256;
}
int Engine::lin_parts(const Lin& l, int R) {
    if (prof_skip_ & lin_class_bit(l, c_)) return HP_OK;
    return gemv_q4k_q8_parts(l.wt ? l.wt : l.w, xq_, yparts_, l.N, l.K, R, l.N, (size_t)R * l.N, err_, s_, pdl_, l.wt != nullptr);
}
int Engine::lin(const Lin& l, float* out, int ld, int R) {
    if (prof_skip_ & lin_class_bit(l, c_)) return HP_OK;
    if (l.P == 1) return gemv_q4k_q8_parts(l.wt ? l.wt : l.w, xq_, out, l.N, l.K, R, ld, 0, err_, s_, pdl_, l.wt != nullptr);
    HP_TRY(lin_parts(l, R));
    HP_CUDA(launch_pdl<16>(k_reduce_planes, dim3((l.N + 255) / 256, R), dim3(256), 0, s_, yparts_, (size_t)R * l.N, l.P, out, l.N, ld));
    HP_CUDA(cudaGetLastError()); return HP_OK;
}
// residual add of the previous projection's planes + RMSNorm + quantise (qwen35.cpp:311-315)
int Engine::norm_in(const Lin* prev, bool have_y, const uint16_t* w, float* xn, int R) {
    if (gemv_only_ || (prof_skip_ & 2)) return HP_OK;
    if (have_y && prev == &moe_out_)   // the MoE combine runs inside the norm: weighted sum of the per-(row, slot) expert outputs
        return add_rmsnorm_quant(x_, moe_v_, 0, 0, c_.n_embd, w, xn, xq_, R, c_.n_embd, c_.rms_eps, s_, false, moe_w_, c_.n_expert_used + 1);
    return add_rmsnorm_quant(x_, have_y ? yparts_ : nullptr, have_y ? prev->P : 0, have_y ? (size_t)R * prev->N : 0, have_y ? prev->N : 0, w, xn, xq_, R, c_.n_embd, c_.rms_eps, s_);
}
// qwen35.cpp:247-276
int Engine::attn_block(const LayerW& L, uint16_t* kc, uint16_t* vc, size_t kv_stride, int R, int ngroups, bool kv_only) {
    const int ld = L.in_proj.N;
    AttnParams p; p.qkv = big_;
    if (L.in_proj.P > 1 && !(prof_skip_ & 4) && !gemv_only_) {   // the rope kernel adds the K-part planes itself
        HP_TRY(lin_parts(L.in_proj, R));
        p.planes = yparts_; p.P = L.in_proj.P; p.part_stride = (size_t)R * ld;
    } else HP_TRY(lin(L.in_proj, big_, ld, R)); p.ld = ld; p.n_head = c_.n_head; p.n_kv = c_.n_head_kv; p.n_rot = c_.n_rot;
    p.q_norm = L.q_norm; p.k_norm = L.k_norm; p.rope = rope_; p.row_pos = d_desc_ + D_POS; p.row_slot = d_desc_ + D_SLOT; p.row_group = d_desc_ + D_RGROUP; p.groups = d_desc_ + D_GROUPS;
    p.kc = kc; p.vc = vc; p.kv_stride = kv_stride; p.max_ctx = c_.max_ctx; p.pO = pO_; p.pm = pm_; p.pl = pl_; p.nsplit_max = nsplit_max_;
    p.out = nullptr; p.xq = xq_; p.eps = c_.rms_eps;
    if (kv_only) return attn_rope_kv(p, R, s_);   // only this layer's K/V rows are wanted
    if (!gemv_only_ && !(prof_skip_ & 4)) { HP_TRY(attn_rope_kv(p, R, s_)); HP_TRY(attn_decode(p, R, ngroups, s_)); }
    return lin_parts(L.out_proj, R);
}
// qwen35.cpp:278-287
int Engine::ffn_block(const LayerW& L, int R) {
    if (c_.n_expert) return moe_block(L, R);
    const int F = c_.n_ff;
    // The SiLU-gated product keeps a launch of its own between the two GEMVs on purpose. Folding it into the gate|up
    // epilogue and the down projection's staging was measured slower (GEMV launches of a 6-row pass 3.85 -> 4.75 ms): two
    // one-CTA-per-SM GEMVs back to back cannot overlap, while the small kernel between them is the window in which the
    // down projection's CTAs become resident and prime their weight rings.
    HP_TRY(lin(L.gate_up, big_, 2 * F, R));
    if (!gemv_only_ && !(prof_skip_ & 8)) HP_TRY(silu_mul_quant(big_, 2 * F, F, xq_, R, s_));
    return lin_parts(L.down, R);
}

// Qwen4Exp::moe_layer (qwen4exp.cpp:345-354): router -> route -> gate|up for the k+1 slots -> silu*mul+q8 -> down + in-order combine
int Engine::moe_block(const LayerW& L, int R) {
    const hp_model_cfg& c = c_; const int E = c.n_embd, F = c.expert_ff, ns = c.n_expert_used + 1;
    if (gemv_only_) return HP_OK;
    // synthetic routing (see hp_model_cfg.synth_router_logits): the key of a layer's draws; 0 = the router's own logits
    const int lidx = &L == &mtp_ ? c.n_layer : (int)(&L - layers_.data());
    const uint64_t rkey = c.synth_router_logits ? (splitmix64(c.seed ^ 0x726F75746572ull ^ ((uint64_t)lidx << 40)) | 1ull) : 0ull;
    // the (replicated) shared expert is computed by one GPU per layer, in turn, so that no GPU carries all of them
    const int own_sh = c.ep_world > 1 ? (lidx % c.ep_world == c.ep_rank ? 1 : 0) : 1;
    MoeRouteParams rp; rp.W = L.router; rp.x = xn_; rp.logits = rlogits_; rp.E = c.n_expert; rp.K = E; rp.k = c.n_expert_used; rp.T = R;
    rp.ids = moe_ids_; rp.w = moe_w_; rp.ticket = route_cnt_; rp.row_tok = d_desc_ + D_TOK; rp.row_pos = d_desc_ + D_POS; rp.row_slot = d_desc_ + D_SLOT; rp.synth_key = rkey;
    rp.e_lo = e_lo_; rp.e_hi = e_hi_; rp.own_shared = own_sh; rp.segs = moe_segs_; rp.ctl = moe_ctl_; rp.touched = moe_touched_; rp.err = err_;
    HP_TRY(moe_route_group(rp, s_));
    // per-(row, slot) outputs of the experts this GPU owns, grouped by expert so that each touched expert matrix is read
    // once; pairs of experts owned elsewhere stay exact zeros, the exchange fills them in, and the combine runs in slot
    // order (the arithmetic of gemv.hip:1104-1112) on every GPU
    if (c.ep_world > 1) { HP_TRY(ep_ready()); if (!ep_peer_) HP_CUDA(cudaMemsetAsync(moe_v_, 0, (size_t)R * ns * E * 4, s_)); }
    MoeGroupParams g; g.w_gate_up = L.exp_gate_up.wt; g.w_down = L.exp_down.wt; g.sh_gate_up = L.sh_gate_up.wt; g.sh_down = L.sh_down.wt;
    g.E = E; g.F = F; g.nslot = ns; g.T = R; g.e_lo = e_lo_;
    g.xq = xq_; g.xq2 = xq2_; g.v = moe_v_; g.segs = moe_segs_; g.ctl = moe_ctl_; g.err = err_;
    int pushed = 0;
    if (ep_peer_) { g.ep_world = c.ep_world; g.ep_rank = c.ep_rank; g.ep_half = ep_half_; for (int q = 0; q < 8; ++q) { g.ep_x[q] = ep_peer_x_[q]; g.ep_ctl[q] = ep_peer_ctl_[q]; } }
    HP_TRY(moe_experts_grouped(g, s_, &pushed));
    if (c.ep_world > 1) HP_TRY(ep_peer_ ? ep_exchange_peer(R, lidx % c.ep_world, pushed != 0) : ep_exchange(moe_v_, (size_t)R * ns * E));
    return HP_OK;   // combined in slot order by the norm that follows (norm_in)
}

// qwen35.cpp:309-376
int Engine::run_pass(int R, int nseq, int ngroups) {
    const hp_model_cfg& c = c_;
    if (!gemv_only_) HP_TRY(embed_bf16(d_desc_ + D_TOK, embed_, x_, R, c.n_embd, c.n_vocab, s_));
    const Lin* prev = nullptr; int gi = 0, ai = 0;
    for (int il = 0; il < c.n_layer; ++il) {
        const LayerW& L = layers_[il];
        HP_TRY(norm_in(prev, prev != nullptr, L.attn_norm, nullptr, R));
        if (!L.is_attn) {
            HP_TRY(lin(L.in_proj, big_, ld_in_, R));
            GdnParams g; g.rows = big_; g.saved = saved_ + (size_t)gi * sv_layer_; g.saved_stride = sv_stride_; g.ld = ld_in_;
            g.n_qk = c.gdn_qk_heads; g.n_v = c.gdn_v_heads;
            g.off_z = (2 * g.n_qk + g.n_v) * 128; g.off_b = g.off_z + g.n_v * 128; g.off_a = g.off_b + g.n_v;
            g.conv_w = L.conv_w; g.dt_bias = L.dt_bias; g.a_neg = L.a_neg; g.norm_w = L.ssm_norm;
            g.state = gdn_state_ + (size_t)gi * st_layer_; g.conv_state = conv_state_ + (size_t)gi * cs_layer_; g.state_stride = st_stride_; g.conv_stride = cs_stride_;
            g.seq = d_desc_ + D_SEQS; g.replay_n = replay_n_; g.out = nullptr; g.xq = xq_; g.snap = nullptr; g.snap_row_stride = 0; g.eps = c.rms_eps; g.sigmoid_gate = c.gdn_sigmoid_gate;
            if (!gemv_only_ && !(prof_skip_ & 1)) HP_TRY(gdn_forward(g, nseq, s_));
            HP_TRY(lin_parts(L.out_proj, R));
            ++gi;
        } else {
            HP_TRY(attn_block(L, kc_ + (size_t)ai * kv_layer_, vc_ + (size_t)ai * kv_layer_, kv_slot_, R, ngroups));
            ++ai;
        }
        HP_TRY(norm_in(&L.out_proj, true, L.post_norm, c.n_expert ? xn_ : nullptr, R));
        HP_TRY(ffn_block(L, R));
        prev = c.n_expert ? &moe_out_ : &L.down;
    }
    HP_TRY(norm_in(prev, true, output_norm_, h_, R));      // h for all rows (+ q8 of all rows), qwen35.cpp:370
    HP_TRY(lin(lm_head_, logits_, c.n_vocab, R));
    if (gemv_only_) return HP_OK;
    return argmax_rows(logits_, R, c.n_vocab, c.n_vocab, d_ids_, d_vals_, am_scratch_, s_);
}

int Engine::flush_commits() {
    // apply pending accepts: a pass with no new rows (the GDN kernel only replays and writes the state back)
    int n = 0; int* seqs = h_desc_ + D_SEQS;
    // every slot: the replay count lives on the device (the fused round sets it there), 0 means nothing to do
    for (int s = 0; s < c_.n_slots; ++s) { seqs[n * 4] = 0; seqs[n * 4 + 1] = 0; seqs[n * 4 + 2] = s; seqs[n * 4 + 3] = 0; ++n; }
    HP_TRY(upload_desc());
    HP_CUDA(cudaStreamSynchronize(s_));   // the pinned descriptor is rewritten by the caller right after
    int gi = 0;
    for (int il = 0; il < c_.n_layer; ++il) {
        const LayerW& L = layers_[il]; if (L.is_attn) continue;
        GdnParams g; g.rows = big_; g.saved = saved_ + (size_t)gi * sv_layer_; g.saved_stride = sv_stride_; g.ld = ld_in_;
        g.n_qk = c_.gdn_qk_heads; g.n_v = c_.gdn_v_heads; g.off_z = (2 * g.n_qk + g.n_v) * 128; g.off_b = g.off_z + g.n_v * 128; g.off_a = g.off_b + g.n_v;
        g.conv_w = L.conv_w; g.dt_bias = L.dt_bias; g.a_neg = L.a_neg; g.norm_w = L.ssm_norm;
        g.state = gdn_state_ + (size_t)gi * st_layer_; g.conv_state = conv_state_ + (size_t)gi * cs_layer_; g.state_stride = st_stride_; g.conv_stride = cs_stride_;
        g.seq = d_desc_ + D_SEQS; g.replay_n = replay_n_; g.out = nullptr; g.xq = XQ8F{nullptr, nullptr}; g.snap = nullptr; g.snap_row_stride = 0; g.eps = c_.rms_eps; g.sigmoid_gate = c_.gdn_sigmoid_gate;
        HP_TRY(gdn_forward(g, n, s_));
        ++gi;
    }
    HP_CUDA(cudaMemsetAsync(replay_n_, 0, MAXS * 4, s_));
    for (int s = 0; s < c_.n_slots; ++s) pend_[s] = 0;
    return HP_OK;
}

// rows of a pass in request order: per-row tables, attention row groups (rows of one slot, at most ATTN_MAX_PAIRS
// (row, q-head) pairs per kv head) and, for the trunk, the per-sequence table of the GDN kernels
int Engine::fill_desc(const hp_slot_req* reqs, int S, int* rows, int* ngroups, bool with_seqs) {
    int* d = h_desc_; int r0 = 0, ng = 0;
    const int gr = attn_rows_per_group();
    for (int i = 0; i < S; ++i) {
        const hp_slot_req& r = reqs[i];
        if (with_seqs) { d[D_SEQS + i * 4] = r0; d[D_SEQS + i * 4 + 1] = r.T; d[D_SEQS + i * 4 + 2] = r.slot; d[D_SEQS + i * 4 + 3] = 0; }
        for (int t0 = 0; t0 < r.T; t0 += gr) {
            const int tn = std::min(gr, r.T - t0);
            HP_REQUIRE(ng < MAXR, "pass needs more than %d attention row groups", MAXR);   // cannot happen while rows <= MAXR; keeps the table write in bounds
            d[D_GROUPS + ng * 4] = r0 + t0; d[D_GROUPS + ng * 4 + 1] = tn; d[D_GROUPS + ng * 4 + 2] = r.slot; d[D_GROUPS + ng * 4 + 3] = r.pos + t0;
            for (int t = t0; t < t0 + tn; ++t) d[D_RGROUP + r0 + t] = ng;
            ++ng;
        }
        for (int t = 0; t < r.T; ++t) { d[D_TOK + r0 + t] = r.tokens[t]; d[D_POS + r0 + t] = r.pos + t; d[D_SLOT + r0 + t] = r.slot; }
        r0 += r.T;
    }
    *rows = r0; *ngroups = ng;
    return HP_OK;
}

int Engine::forward(const hp_slot_req* reqs, int S, float* ms) {
    HP_REQUIRE(reqs && S >= 1 && S <= c_.n_slots, "bad S");                                  // qwen35.cpp:290
    int T = 0; for (int i = 0; i < S; ++i) T += reqs[i].T > 0 ? reqs[i].T : MAXR + 1;
    HP_REQUIRE(T >= 1 && T <= MAXR, "bad T");                                                // qwen35.cpp:293
    std::vector<char> in_pass(c_.n_slots, 0);
    for (int i = 0; i < S; ++i) {
        const hp_slot_req& r = reqs[i];
        HP_REQUIRE(r.slot >= 0 && r.slot < c_.n_slots && r.T >= 1 && r.T <= 8 && r.pos >= 0 && r.pos + r.T <= c_.max_ctx && r.tokens && !in_pass[r.slot], "bad request");   // qwen35.cpp:298
        in_pass[r.slot] = 1;
    }
    if (c_.ep_world > 1) HP_TRY(ep_ready());
    int ng = 0;
    HP_TRY(fill_desc(reqs, S, &T, &ng, true));
    HP_CUDA(cudaEventRecord(ev0_, s_));
    HP_TRY(upload_desc());
    HP_TRY(run_pass(T, S, ng));
    // the accepted prefixes of the previous pass are now part of the stored state
    int r0 = 0;
    for (int i = 0; i < S; ++i) {
        const hp_slot_req& r = reqs[i];
        HP_CUDA(cudaMemsetAsync(replay_n_ + r.slot, 0, 4, s_)); pend_[r.slot] = 0;
        last_r0_[r.slot] = r0; last_T_[r.slot] = r.T; r0 += r.T;
    }
    HP_CUDA(cudaEventRecord(ev1_, s_)); HP_TRY(sync_stream());
    HP_CUDA(cudaEventElapsedTime(&last_ms_, ev0_, ev1_));
    HP_TRY(check_device_status());
    if (ms) *ms = last_ms_;
    return HP_OK;
}

int Engine::accept(int slot, int m) {
    HP_REQUIRE(slot >= 0 && slot < c_.n_slots && last_T_[slot] > 0, "accept: slot had no rows in the last pass");   // qwen35.cpp:384
    HP_REQUIRE(m >= 1 && m <= last_T_[slot], "bad accept");                                                          // qwen35.cpp:386
    pend_[slot] = m; last_T_[slot] = 0;
    k_set_ints<<<1, 32, 0, s_>>>(replay_n_ + slot, 1, m);
    HP_CUDA(cudaGetLastError()); return HP_OK;
}

// qwen35.cpp:405-424
// kv_only: stop once the block's K/V rows of these positions are in its cache (the catch-up of the fused round needs
// nothing else: the next draft takes its hidden row from the trunk)
int Engine::run_mtp(int R, int ngroups, const float* h_dev, int ldh, bool want_logits, bool kv_only) {
    const hp_model_cfg& c = c_;
    HP_TRY(embed_bf16(d_desc_ + D_TOK, embed_, emb_, R, c.n_embd, c.n_vocab, s_));
    HP_TRY(norm2_concat_quant(emb_, mtp_enorm_, h_dev, ldh, mtp_hnorm_, nullptr, xq_, R, c.n_embd, c.rms_eps, s_));
    HP_TRY(lin_parts(eh_proj_, R));   // x = eh_proj(...) : the norm kernel adds the K-part planes itself
    HP_TRY(add_rmsnorm_quant(x_, yparts_, eh_proj_.P, (size_t)R * eh_proj_.N, eh_proj_.N, mtp_.attn_norm, nullptr, xq_, R, c.n_embd, c.rms_eps, s_, true));
    HP_TRY(attn_block(mtp_, mkc_, mvc_, kv_layer_, R, ngroups, kv_only));
    if (kv_only) return HP_OK;
    HP_TRY(norm_in(&mtp_.out_proj, true, mtp_.post_norm, c.n_expert ? xn_ : nullptr, R));
    HP_TRY(ffn_block(mtp_, R));
    HP_TRY(norm_in(c.n_expert ? &moe_out_ : &mtp_.down, true, mtp_head_norm_, mh_, R));
    if (want_logits) {
        HP_TRY(lin(lm_head_, mlogits_, c.n_vocab, R));
        HP_TRY(argmax_rows(mlogits_, R, c.n_vocab, c.n_vocab, d_mids_, d_mvals_, am_scratch_, s_));
    }
    return HP_OK;
}
int Engine::mtp_forward(const int* tokens, const float* h_dev, int T, int pos0, int slot, bool want_logits) {
    HP_REQUIRE(tokens && T >= 1 && T <= 8, "bad T");                                          // qwen35.cpp:406
    const hp_slot_req r{slot, tokens, T, pos0};
    return mtp_forward_reqs(&r, 1, h_dev, want_logits);
}

int Engine::mtp_forward_reqs(const hp_slot_req* reqs, int S, const float* h_dev, bool want_logits) {
    HP_REQUIRE(c_.has_mtp, "model has no MTP block");
    HP_REQUIRE(reqs && h_dev && S >= 1 && S <= c_.n_slots, "bad S");
    int rows = 0;
    for (int i = 0; i < S; ++i) {
        const hp_slot_req& r = reqs[i];
        HP_REQUIRE(r.slot >= 0 && r.slot < c_.n_slots && r.T >= 1 && r.T <= 8 && r.pos >= 0 && r.pos + r.T <= c_.max_ctx && r.tokens && rows + r.T <= MAXR, "bad request");
        rows += r.T;
    }
    if (c_.ep_world > 1) HP_TRY(ep_ready());
    int ng = 0;
    HP_TRY(fill_desc(reqs, S, &rows, &ng, false));
    HP_TRY(upload_desc());
    HP_TRY(run_mtp(rows, ng, h_dev, c_.n_embd, want_logits));
    HP_TRY(sync_stream());
    return check_device_status();
}

// Qwen35::topk (qwen35.cpp:426-430): ids / vals [T][k], values descending, ties -> lower index
int Engine::topk(int which, int T, int k, int* ids, float* vals) {
    HP_REQUIRE(T >= 1 && T <= MAXR && ids && k >= 1 && k <= topk_max_k() && k <= c_.n_vocab, "topk: bad arguments (1 <= T <= %d, 1 <= k <= %d)", MAXR, topk_max_k());
    if (k == 1) {   // the arg-max of every row was taken on the device at the end of the pass
        HP_TRY(sync_stream());
        HP_CUDA(cudaMemcpy(ids, which ? d_mids_ : d_ids_, T * 4, cudaMemcpyDeviceToHost));
        if (vals) HP_CUDA(cudaMemcpy(vals, which ? d_mvals_ : d_vals_, T * 4, cudaMemcpyDeviceToHost));
        return HP_OK;
    }
    HP_TRY(topk_rows(which ? mlogits_ : logits_, T, c_.n_vocab, c_.n_vocab, k, d_topk_ids_, d_topk_vals_, topk_scratch_, s_));
    HP_TRY(sync_stream());
    HP_CUDA(cudaMemcpy(ids, d_topk_ids_, (size_t)T * k * 4, cudaMemcpyDeviceToHost));
    if (vals) HP_CUDA(cudaMemcpy(vals, d_topk_vals_, (size_t)T * k * 4, cudaMemcpyDeviceToHost));
    return HP_OK;
}

// Prompt ingestion for one slot (Qwen4Exp::prefill + mtp_catchup, qwen4exp.h:57-60,72-74; Backend::prefill,
// front/serve.cpp:29): n tokens at positions pos0.., committed. This build runs them through the verify path in chunks
// of 8 rows; with_mtp also runs the MTP block over the same rows, row p paired with the trunk's hidden row of position
// p - 1 (zeros at position 0; the last row of the previous chunk / call otherwise), so that the draft block's KV cache
// covers the prompt (spec27b.cpp:62-71). Afterwards row 0 of logits / h_nextn / the arg-max ids holds the LAST prompt row.
// ---- expert-parallel exchange over peer memory -------------------------------------------------------------------------
// After the down projection a rank holds the output rows of the (row, slot) pairs whose expert it owns. k_ep_push copies
// them into the other ranks' exchange buffers (plain stores through the NVLink mapping), makes them visible system-wide
// and then, from the CTA that finishes last, stores the number of this exchange into its flag word on every rank.
// k_ep_gather waits (bounded) until every other rank's flag has reached that number and copies the rows it does not own
// from its own exchange buffer into the pair buffer. Exchange n uses half n & 1 of the buffers: a rank can be at most one
// exchange ahead of another (it cannot pass gather n before every rank has pushed n), so two halves never collide.
struct EpXArgs {
    float* v; const int* ids; int npairs, E, n_expert, world, rank, sh_owner;   // pair buffer [npairs][E], expert id per pair (-1 = shared)
    float* x[8]; unsigned* ctl[8]; size_t half; int* err;
};
__device__ __forceinline__ int ep_owner(int id, const EpXArgs& a) {
    if (id < 0) return a.sh_owner;
    return ep_owner_of(id, a.n_expert, a.world);
}
__global__ void __launch_bounds__(256) k_ep_push(EpXArgs a) {
    unsigned* ctl = a.ctl[a.rank];
    const unsigned e = __ldcg(ctl + 8) + 1u;   // number of this exchange (the counter moves when every CTA is done)
    const size_t off = (size_t)(e & 1u) * a.half;
    const int e4 = a.E >> 2, items = a.npairs * e4;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < items; i += gridDim.x * 256) {
        const int pair = i / e4, c = i - pair * e4;
        if (ep_owner(__ldcg(a.ids + pair), a) != a.rank) continue;
        const float4 val = __ldcg(reinterpret_cast<const float4*>(a.v + (size_t)pair * a.E) + c);
        for (int q = 0; q < a.world; ++q)
            if (q != a.rank) reinterpret_cast<float4*>(a.x[q] + off + (size_t)pair * a.E)[c] = val;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(ctl + 9, 1u) == gridDim.x - 1) {
        __threadfence_system();
        for (int q = 0; q < a.world; ++q)
            if (q != a.rank) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.ctl[q] + a.rank), "r"(e) : "memory");
        ctl[9] = 0u; __threadfence();
        atomicExch(ctl + 8, e);
    }
}
// Bounded wait of thread q < world (q != rank) for flags[q] to reach exchange number e: 2^22 polls, then the device status
// word is set (and once it is set, later waits give up at once: a lost peer costs one limit, not one per exchange).
__device__ __forceinline__ void ep_wait_flags(const unsigned* flags, int world, int rank, unsigned e, int* err) {
    if (threadIdx.x < world && (int)threadIdx.x != rank && __ldcg(err) == 0) {
        unsigned f = 0u; int it = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(flags + threadIdx.x) : "memory");
            if ((int)(f - e) >= 0 || ++it >= (1 << 22)) break;
            __nanosleep(64);
        }
        if ((int)(f - e) < 0) atomicExch(err, HP_ETIMEOUT);   // a peer did not deliver: reported through the device status word
    }
    __syncthreads();
}
__global__ void k_ep_wait_probe(const unsigned* flags, int world, int rank, unsigned e, int* err) { ep_wait_flags(flags, world, rank, e, err); }
__global__ void __launch_bounds__(256) k_ep_gather(EpXArgs a) {
    unsigned* ctl = a.ctl[a.rank];
    const unsigned e = __ldcg(ctl + 8);        // the exchange k_ep_push has just sent
    ep_wait_flags(ctl, a.world, a.rank, e, a.err);
    const float* x = a.x[a.rank] + (size_t)(e & 1u) * a.half;
    const int e4 = a.E >> 2, items = a.npairs * e4;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < items; i += gridDim.x * 256) {
        const int pair = i / e4, c = i - pair * e4;
        const int o = ep_owner(__ldcg(a.ids + pair), a);
        if (o == a.rank || o < 0 || o >= a.world) continue;
        reinterpret_cast<float4*>(a.v + (size_t)pair * a.E)[c] = __ldcg(reinterpret_cast<const float4*>(x + (size_t)pair * a.E) + c);
    }
}

__global__ void k_prefill_shift(const float* __restrict__ h, const float* __restrict__ hprev, float* __restrict__ dst, int E, int zero_first) {
    const int t = blockIdx.x;   // dst row t = h row t - 1, row 0 = the remembered row (or zeros at position 0)
    const float* src = t == 0 ? hprev : h + (size_t)(t - 1) * E;
    for (int i = threadIdx.x; i < E; i += 256) dst[(size_t)t * E + i] = (t == 0 && zero_first) ? 0.f : src[i];
}
__global__ void k_prefill_remember(const float* __restrict__ h, float* __restrict__ hprev, int T, int E) {
    for (int i = threadIdx.x; i < E; i += 256) hprev[i] = h[(size_t)(T - 1) * E + i];
}
__global__ void k_prefill_last(float* __restrict__ logits, float* __restrict__ h, int* __restrict__ ids, float* __restrict__ vals, int last, int V, int E) {
    for (int i = blockIdx.x * 256 + threadIdx.x; i < V; i += gridDim.x * 256) logits[i] = logits[(size_t)last * V + i];
    if (blockIdx.x == 0) { for (int i = threadIdx.x; i < E; i += 256) h[i] = h[(size_t)last * E + i]; if (threadIdx.x == 0) { ids[0] = ids[last]; vals[0] = vals[last]; } }
}
int Engine::prefill(int slot, const int* tokens, int n, int pos0, int with_mtp) {
    HP_REQUIRE(slot >= 0 && slot < c_.n_slots && tokens && n >= 1 && pos0 >= 0 && pos0 + n <= c_.max_ctx, "prefill: bad arguments (slot %d, n %d, pos0 %d)", slot, n, pos0);
    HP_REQUIRE(!with_mtp || c_.has_mtp, "model has no MTP block");
    const int E = c_.n_embd;
    int T = 0;
    for (int p = 0; p < n; p += T) {
        T = std::min(8, n - p);
        const hp_slot_req r{slot, tokens + p, T, pos0 + p};
        HP_TRY(forward(&r, 1, nullptr));
        HP_TRY(accept(slot, T));
        if (with_mtp) {
            float* hp = hprev_ + (size_t)slot * E;
            k_prefill_shift<<<T, 256, 0, s_>>>(h_, hp, hstage_, E, pos0 + p == 0 ? 1 : 0);
            k_prefill_remember<<<1, 256, 0, s_>>>(h_, hp, T, E);   // after the shift (stream order): this chunk's last row pairs with the next chunk's first token
            HP_CUDA(cudaGetLastError());
            HP_TRY(mtp_forward_reqs(&r, 1, hstage_, false));
        }
    }
    if (T > 1) {
        k_prefill_last<<<64, 256, 0, s_>>>(logits_, h_, d_ids_, d_vals_, T - 1, c_.n_vocab, E);
        HP_CUDA(cudaGetLastError());
    }
    HP_TRY(sync_stream());
    last_T_[slot] = 0;
    return HP_OK;
}

int Engine::tensor(int layer, int kind, void** ptr, size_t* bytes) const {
    const hp_model_cfg& c = c_; const int E = c.n_embd;
    auto set = [&](const void* p, size_t b) { *ptr = (void*)p; *bytes = b; return HP_OK; };
    if (layer < 0) {
        switch (kind) {
            case TK_EMBED: return set(embed_, (size_t)c.n_vocab * E * 2);
            case TK_OUTPUT_NORM: return set(output_norm_, (size_t)E * 2);
            case TK_LM_HEAD: return set(lm_head_.w, lm_head_.bytes);
            case TK_MTP_ENORM: return set(mtp_enorm_, (size_t)E * 2);
            case TK_MTP_HNORM: return set(mtp_hnorm_, (size_t)E * 2);
            case TK_MTP_HEAD_NORM: return set(mtp_head_norm_, (size_t)E * 2);
            case TK_MTP_EH_PROJ: return set(eh_proj_.w, eh_proj_.bytes);
        }
        set_error("unknown model-level tensor %d", kind); return HP_EINVAL;
    }
    HP_REQUIRE(layer <= c.n_layer && (layer < c.n_layer || c.has_mtp), "bad layer %d", layer);
    const LayerW& L = layer == c.n_layer ? mtp_ : layers_[layer];
    const int nv = c.gdn_v_heads, nq = c.gdn_qk_heads;
    switch (kind) {
        case TK_ATTN_NORM: return set(L.attn_norm, (size_t)E * 2);
        case TK_POST_NORM: return set(L.post_norm, (size_t)E * 2);
        case TK_IN_PROJ: HP_REQUIRE(L.in_proj.w, "the row-major copy of this tensor was released after repacking"); return set(L.in_proj.w, L.in_proj.bytes);
        case TK_OUT_PROJ: return set(L.out_proj.w, L.out_proj.bytes);
        case TK_GATE_UP: return set(L.gate_up.w, L.gate_up.bytes);
        case TK_DOWN: return set(L.down.w, L.down.bytes);
        case TK_CONV_W: return set(L.conv_w, (size_t)(2 * nq + nv) * 128 * 4 * 4);
        case TK_DT_BIAS: return set(L.dt_bias, (size_t)nv * 2);
        case TK_A_NEG: return set(L.a_neg, (size_t)nv * 2);
        case TK_SSM_NORM: return set(L.ssm_norm, 256);
        case TK_Q_NORM: return set(L.q_norm, 512);
        case TK_K_NORM: return set(L.k_norm, 512);
        case TK_ROUTER: return set(L.router, (size_t)(c.n_expert + 1) * E * 4);
        case TK_EXP_GATE_UP: HP_REQUIRE(L.exp_gate_up.w, "the row-major copy of this tensor was released after repacking");
                             return set(L.exp_gate_up.w + (size_t)e_lo_ * 2 * c.expert_ff * (E / 256) * 144, L.exp_gate_up.bytes);   // this GPU's shard
        case TK_EXP_DOWN: HP_REQUIRE(L.exp_down.w, "the row-major copy of this tensor was released after repacking");
                          return set(L.exp_down.w + (size_t)e_lo_ * E * (c.expert_ff / 256) * 144, L.exp_down.bytes);
        case TK_SH_GATE_UP: return set(L.sh_gate_up.w, L.sh_gate_up.bytes);
        case TK_SH_DOWN: return set(L.sh_down.w, L.sh_down.bytes);
    }
    set_error("unknown layer tensor %d", kind); return HP_EINVAL;
}
int Engine::gdn_state(int slot, int gdn_layer, float** ptr, size_t* bytes) {
    HP_REQUIRE(slot >= 0 && slot < c_.n_slots && gdn_layer >= 0 && gdn_layer < ngdn(), "gdn_state: bad index");
    HP_TRY(flush_commits());
    HP_CUDA(cudaStreamSynchronize(s_));
    *ptr = gdn_state_ + (size_t)slot * st_stride_ + (size_t)gdn_layer * st_layer_; *bytes = st_layer_ * 4;
    return HP_OK;
}

size_t Engine::pass_weight_bytes(bool mtp, bool with_head) const {
    size_t b = 0;
    // dense part only; routed-expert bytes depend on the routing (count the distinct (layer, expert) pairs touched)
    if (!mtp) for (const LayerW& L : layers_) b += L.in_proj.bytes + L.out_proj.bytes + L.gate_up.bytes + L.down.bytes + L.sh_gate_up.bytes + L.sh_down.bytes;
    else b += eh_proj_.bytes + mtp_.in_proj.bytes + mtp_.out_proj.bytes + mtp_.gate_up.bytes + mtp_.down.bytes + mtp_.sh_gate_up.bytes + mtp_.sh_down.bytes;
    if (with_head) b += lm_head_.bytes;
    return b;
}

// Diagnostic: device time of `reps` back-to-back verify passes of R rows (what = 0), of only the GEMV launches of such
// passes (what = 1), or of passes that leave out kernel classes (what = 16 + mask: 1 GDN, 2 norms, 4 attention, 8 SiLU,
// 16 gate|up, 32 down, 64 LM head, 128 input projections, 256 other GEMVs; results are then meaningless, only the time is).
// The passes run on slot 0 at its current position (the position of a running speculative stream, else 0). The context
// survives: pending accepts are applied to the stored state first, so that the passes replay nothing and leave the
// recurrent state alone (a pass never advances it), and the K/V rows the passes write are saved before and put back
// afterwards. What does not survive is the right to accept the pass that came before the call: its saved inputs are
// overwritten, so hp_accept for slot 0 is refused until the next hp_forward.
int Engine::profile_pass(int R, int what, int reps, float* ms) {
    HP_REQUIRE(R >= 1 && R <= 8 && reps >= 1 && ms, "profile_pass: bad arguments");
    HP_REQUIRE(c_.ep_world <= 1, "profile_pass: not available on an expert-parallel engine");
    HP_TRY(flush_commits());
    const int pos0 = std::max(0, std::min(spec_on_[0] ? spec_pos_[0] : 0, c_.max_ctx - R));
    // K/V rows [pos0, pos0 + R) of slot 0 in every attention layer and kv head: one strided copy each way
    const size_t row_b = 256 * 2, pitch = (size_t)c_.max_ctx * row_b, height = (size_t)nattn() * c_.n_head_kv, width = (size_t)R * row_b;
    uint16_t* sk = prof_kv_; uint16_t* sv = prof_kv_ + height * 8 * 256;
    if (height) {
        HP_CUDA(cudaMemcpy2DAsync(sk, width, kc_ + (size_t)pos0 * 256, pitch, width, height, cudaMemcpyDeviceToDevice, s_));
        HP_CUDA(cudaMemcpy2DAsync(sv, width, vc_ + (size_t)pos0 * 256, pitch, width, height, cudaMemcpyDeviceToDevice, s_));
    }
    int* d = h_desc_;
    for (int t = 0; t < R; ++t) d[D_TOK + t] = (t * 7919 + 13) % c_.n_vocab;
    std::vector<int> toks(d + D_TOK, d + D_TOK + R);
    const hp_slot_req rq{0, toks.data(), R, pos0};
    int rows = 0, ng = 0;
    HP_TRY(fill_desc(&rq, 1, &rows, &ng, true));
    HP_TRY(upload_desc());
    gemv_only_ = what == 1; prof_skip_ = what >= 16 ? what - 16 : 0;
    int rc = run_pass(R, 1, ng);                     // warm-up (also sets kernel attributes)
    HP_CUDA(cudaEventRecord(ev0_, s_));
    for (int i = 0; i < reps && rc == HP_OK; ++i) rc = run_pass(R, 1, ng);
    HP_CUDA(cudaEventRecord(ev1_, s_));
    gemv_only_ = false; prof_skip_ = 0;
    if (height) {
        HP_CUDA(cudaMemcpy2DAsync(kc_ + (size_t)pos0 * 256, pitch, sk, width, width, height, cudaMemcpyDeviceToDevice, s_));
        HP_CUDA(cudaMemcpy2DAsync(vc_ + (size_t)pos0 * 256, pitch, sv, width, width, height, cudaMemcpyDeviceToDevice, s_));
    }
    HP_CUDA(cudaStreamSynchronize(s_));
    last_T_[0] = 0;
    if (rc != HP_OK) return rc;
    float t = 0; HP_CUDA(cudaEventElapsedTime(&t, ev0_, ev1_)); *ms = t / reps;
    return check_device_status();
}

static int count_kernel_nodes(cudaGraph_t g, int* out) {
    size_t nn = 0; HP_CUDA(cudaGraphGetNodes(g, nullptr, &nn));
    std::vector<cudaGraphNode_t> nodes(nn); if (nn) HP_CUDA(cudaGraphGetNodes(g, nodes.data(), &nn));
    int nk = 0; for (size_t i = 0; i < nn; ++i) { cudaGraphNodeType ty; if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) ++nk; }
    *out += nk; return HP_OK;
}
// Expert-parallel exchange of the per-(row, slot) expert outputs. Every element of the buffer is produced by exactly one
// GPU (the owner of that slot's expert) and is an exact zero on the others, so the result is the owner's value bit for
// bit whatever order the library adds in: an all-gather of a permuted buffer expressed as one NCCL call.
int Engine::ep_exchange(float* buf, size_t n) {
    if (ep_world_ <= 1) return HP_OK;
    if (!seg_out_) return ep_allreduce(buf, n);
    // a round is being captured in segments: close the stretch that ends here, remember the exchange, open the next one
    cudaGraph_t g = nullptr; cudaGraphExec_t ex = nullptr;
    HP_CUDA(cudaStreamEndCapture(s_, &g));
    int nk = 0; const int rc = count_kernel_nodes(g, &nk);
    const cudaError_t ce = rc == HP_OK ? cudaGraphInstantiate(&ex, g, 0) : cudaErrorUnknown;
    cudaGraphDestroy(g);
    if (rc != HP_OK) return rc;
    HP_CUDA(ce);
    seg_out_->push_back(EpSeg{ex, buf, n});
    for (int k = 0; k < 64; ++k) if (seg_out_ == &ep_segs_[k]) graph_kernels_[k] += nk;
    HP_CUDA(cudaStreamBeginCapture(s_, cudaStreamCaptureModeThreadLocal));
    return HP_OK;
}

// ------------------------------------------------------------------ fused device-side round
int Engine::spec_begin(int slot, int id_last, int pos, const float* h_pending_dev) {
    HP_REQUIRE(c_.has_mtp, "model has no MTP block");
    HP_REQUIRE(slot >= 0 && slot < c_.n_slots && pos >= 0 && pos < c_.max_ctx && h_pending_dev, "spec_begin: bad arguments");
    h_spec_[0] = id_last; h_spec_[1] = pos;
    HP_CUDA(cudaMemcpyAsync(d_spec_ + slot * SP_INTS, h_spec_, 8, cudaMemcpyHostToDevice, s_));
    HP_CUDA(cudaMemcpyAsync(hpend_ + (size_t)slot * c_.n_embd, h_pending_dev, (size_t)c_.n_embd * 4, cudaMemcpyDeviceToDevice, s_));
    HP_CUDA(cudaStreamSynchronize(s_));
    spec_pos_[slot] = pos; spec_on_[slot] = 1; last_T_[slot] = 0;
    return HP_OK;
}
int Engine::attn_rows_per_group() const { return std::max(1, std::min(8, ATTN_MAX_PAIRS / (c_.n_head / c_.n_head_kv))); }
int Engine::enqueue_round(int S, int n) {
    const int E = c_.n_embd, gr = attn_rows_per_group();
    auto groups = [&](int Tm) { return S * ((Tm + gr - 1) / gr); };
    HP_CUDA(cudaMemcpyAsync(d_specin_, h_spec_, SI_INTS * 4, cudaMemcpyHostToDevice, s_));
    for (int i = 0; i < n; ++i) {   // draft, chained on the MTP's own h (spec27b.cpp:81-85, batchfn.cpp:98-104)
        HP_CUDA(launch_pdl<2>(k_spec_setup, dim3(1), dim3(32), 0, s_, d_spec_, d_specin_, d_desc_, 0, i, n, S, gr));
        if (i == 0) HP_CUDA(launch_pdl<2>(k_spec_gather_h, dim3(S), dim3(256), 0, s_, d_specin_, hpend_, h_, hstage_, 0, n, E));
        HP_TRY(run_mtp(S, groups(1), i == 0 ? hstage_ : mh_, E, true));
        HP_CUDA(launch_pdl<2>(k_spec_take, dim3(1), dim3(32), 0, s_, d_spec_, d_specin_, d_mids_, i, S));
    }
    HP_CUDA(launch_pdl<2>(k_spec_setup, dim3(1), dim3(32), 0, s_, d_spec_, d_specin_, d_desc_, 1, 0, n, S, gr));
    HP_TRY(run_pass(S * (n + 1), S, groups(n + 1)));
    HP_CUDA(launch_pdl<2>(k_spec_accept, dim3(S), dim3(256), 0, s_, d_spec_, d_specin_, d_ids_, replay_n_, n, h_, hpend_, E));
    // MTP catch-up over the drafts with the target's h rows. All n rows of every slot run; rows beyond a slot's accepted
    // prefix only write KV entries that the next round rewrites before reading them.
    HP_CUDA(launch_pdl<2>(k_spec_setup, dim3(1), dim3(32), 0, s_, d_spec_, d_specin_, d_desc_, 2, 0, n, S, gr));
    const float* hc = h_;
    if (S > 1) { HP_CUDA(launch_pdl<2>(k_spec_gather_h, dim3(S * n), dim3(256), 0, s_, d_specin_, hpend_, h_, hstage_, 1, n, E)); hc = hstage_; }
    HP_TRY(run_mtp(S * n, groups(n), hc, E, false, true));
    HP_CUDA(cudaMemcpyAsync(h_spec_ + SI_INTS, d_spec_, MAXS * SP_INTS * 4, cudaMemcpyDeviceToHost, s_));
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int Engine::spec_round(const int* slots, int S, int n, const int* subst, int* out_tokens, int* out_counts) {
    HP_REQUIRE(c_.has_mtp, "model has no MTP block");
    HP_REQUIRE(slots && S >= 1 && S <= c_.n_slots && n >= 1 && n <= 7 && out_tokens && out_counts, "spec_round: bad arguments (1 <= S <= n_slots, 1 <= n_draft <= 7)");
    HP_REQUIRE(S * (n + 1) <= MAXR, "spec_round: %d slots x %d rows exceed %d rows per pass", S, n + 1, MAXR);
    for (int j = 0; j < S; ++j) {
        const int sl = slots[j];
        HP_REQUIRE(sl >= 0 && sl < c_.n_slots && spec_on_[sl], "spec_round: slot %d was not started with hp_spec_begin", sl);
        for (int q = 0; q < j; ++q) HP_REQUIRE(slots[q] != sl, "spec_round: slot %d listed twice", sl);
        HP_REQUIRE(spec_pos_[sl] + 2 * n + 2 <= c_.max_ctx, "spec_round: context of slot %d exhausted", sl);
    }
    if (c_.ep_world > 1) HP_TRY(ep_ready());
    for (int j = 0; j < 8; ++j) {
        h_spec_[SI_SLOTS + j] = j < S ? slots[j] : 0;
        for (int i = 0; i < 8; ++i) h_spec_[SI_SUBST + 8 * j + i] = (subst && j < S && i < n) ? subst[j * n + i] : -1;
    }
    // A round that carries collectives is replayed as the graphs of the stretches between two exchanges, with the
    // exchanges themselves enqueued by the host in between: capturing the collectives into the graph hung on 2 GPUs
    // (NCCL 2.28.9), and this way the host also stays able to watch the communicator (sync_stream).
    static const bool no_graph = getenv("HIPSTER_B200_NO_GRAPH") != nullptr;
    const int key = (S - 1) * 8 + n;
    HP_CUDA(cudaEventRecord(ev0_, s_));
    if (no_graph) HP_TRY(enqueue_round(S, n));
    else if (c_.ep_world > 1 && !ep_peer_) {
        if (!warmed_[key]) { HP_TRY(enqueue_round(S, n)); HP_TRY(sync_stream()); warmed_[key] = true; goto done; }   // first call: eager
        if (ep_segs_[key].empty()) HP_TRY(capture_segments(key, S, n));
        for (const EpSeg& sg : ep_segs_[key]) {
            HP_CUDA(cudaGraphLaunch(sg.g, s_));
            if (sg.n) HP_TRY(ep_allreduce(sg.buf, sg.n));
        }
        last_round_kernels_ = graph_kernels_[key];
    } else {
        if (!graphs_[key]) {
            if (!warmed_[key]) { HP_TRY(enqueue_round(S, n)); HP_TRY(sync_stream()); warmed_[key] = true; goto done; }   // first call: eager (sets kernel attributes)
            cudaGraph_t g = nullptr;
            HP_CUDA(cudaStreamBeginCapture(s_, cudaStreamCaptureModeThreadLocal));
            const int rc = enqueue_round(S, n);
            const cudaError_t ce = cudaStreamEndCapture(s_, &g);
            if (rc != HP_OK) { if (g) cudaGraphDestroy(g); return rc; }
            HP_CUDA(ce);
            {   // kernels of one round: counted from the captured graph
                size_t nn = 0; HP_CUDA(cudaGraphGetNodes(g, nullptr, &nn));
                std::vector<cudaGraphNode_t> nodes(nn); if (nn) HP_CUDA(cudaGraphGetNodes(g, nodes.data(), &nn));
                int nk = 0; for (size_t i = 0; i < nn; ++i) { cudaGraphNodeType ty; if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) ++nk; }
                graph_kernels_[key] = nk;
            }
            HP_CUDA(cudaGraphInstantiate(&graphs_[key], g, 0));
            HP_CUDA(cudaGraphDestroy(g));
        }
        HP_CUDA(cudaGraphLaunch(graphs_[key], s_));
        last_round_kernels_ = graph_kernels_[key];
    }
done:
    HP_CUDA(cudaEventRecord(ev1_, s_));
    HP_TRY(sync_stream());
    HP_CUDA(cudaEventElapsedTime(&last_ms_, ev0_, ev1_));
    HP_TRY(check_device_status());
    for (int j = 0; j < S; ++j) {
        const int* r = h_spec_ + SI_INTS + slots[j] * SP_INTS;
        out_counts[j] = r[SP_COUNT];
        for (int i = 0; i < r[SP_COUNT]; ++i) out_tokens[j * (n + 1) + i] = r[SP_OUT + i];
        spec_pos_[slots[j]] = r[SP_POS]; last_T_[slots[j]] = 0; pend_[slots[j]] = r[SP_COUNT];
    }
    return HP_OK;
}
// capture one round as segments: ep_exchange() closes the running capture at every exchange and opens the next one
int Engine::capture_segments(int key, int S, int n) {
    std::vector<EpSeg>& segs = ep_segs_[key];
    graph_kernels_[key] = 0;
    HP_CUDA(cudaStreamBeginCapture(s_, cudaStreamCaptureModeThreadLocal));
    seg_out_ = &segs;
    const int rc = enqueue_round(S, n);
    seg_out_ = nullptr;
    cudaGraph_t g = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(s_, &g);
    int rc2 = rc;
    if (rc2 == HP_OK && ce != cudaSuccess) rc2 = cuda_fail(ce, "cudaStreamEndCapture", __FILE__, __LINE__);
    if (rc2 == HP_OK) {
        cudaGraphExec_t ex = nullptr;
        rc2 = count_kernel_nodes(g, &graph_kernels_[key]);
        if (rc2 == HP_OK && cudaGraphInstantiate(&ex, g, 0) != cudaSuccess) { set_error("cannot instantiate a round segment"); rc2 = HP_ECUDA; }
        if (rc2 == HP_OK) segs.push_back(EpSeg{ex, nullptr, 0});
    }
    if (g) cudaGraphDestroy(g);
    if (rc2 != HP_OK) { for (EpSeg& sg : segs) cudaGraphExecDestroy(sg.g); segs.clear(); }
    return rc2;
}
int Engine::check_device_status() {
    int herr = 0; HP_CUDA(cudaMemcpy(&herr, err_, 4, cudaMemcpyDeviceToHost));
    if (herr) { cudaMemset(err_, 0, 4); set_error("a kernel gave up a bounded wait (device status %d)", herr); return herr; }
    return HP_OK;
}

}  // namespace hp

// ------------------------------------------------------------------ NCCL (loaded at run time; only the expert-parallel path needs it)
#include <dlfcn.h>
#include <chrono>
#include <thread>
namespace hp {
namespace {
struct NcclId { char b[128]; };   // ncclUniqueId is 128 opaque bytes, passed by value
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*CommAbort)(void*) = nullptr;
    int (*CommGetAsyncError)(void*, int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;
int nccl_load() {
    if (g_nccl.lib) return HP_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { set_error("cannot load libnccl.so.2: %s", dlerror()); return HP_ECOMM; }
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(h, "ncclAllReduce");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))dlsym(h, "ncclAllGather");
    g_nccl.ReduceScatter = (decltype(g_nccl.ReduceScatter))dlsym(h, "ncclReduceScatter");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort))dlsym(h, "ncclCommAbort");
    g_nccl.CommGetAsyncError = (decltype(g_nccl.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.AllGather || !g_nccl.ReduceScatter || !g_nccl.CommDestroy || !g_nccl.CommAbort || !g_nccl.CommGetAsyncError) {
        set_error("libnccl lacks a required symbol"); return HP_ECOMM;
    }
    g_nccl.lib = h; return HP_OK;
}
int nccl_check(int rc, const char* what) {
    if (rc == 0) return HP_OK;
    set_error("NCCL error %d (%s) in %s", rc, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?", what); return HP_ECOMM;
}
}  // namespace

// The engine's wait for a stream that carries collectives: instead of blocking in the driver without a limit, poll the
// stream and the communicator's asynchronous error state until the work is done, an error shows, or limit_ms passed.
// stream_query: 0 = done, 1 = still running, anything else = failed; comm_error: 0 = healthy (or still in progress),
// anything else = the communicator reports a failure. Returns HP_OK, HP_ECOMM (failure) or HP_ETIMEOUT.
int ep_wait_poll(int (*stream_query)(void*), int (*comm_error)(void*), void* ctx, int limit_ms) {
    HP_REQUIRE(stream_query && limit_ms >= 0, "ep_wait_poll: bad arguments");
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned it = 0;; ++it) {
        const int q = stream_query(ctx);
        if (q == 0) return HP_OK;
        if (q != 1) { set_error("the stream failed while waiting for a collective (status %d)", q); return HP_ECOMM; }
        if (comm_error) { const int ce = comm_error(ctx); if (ce != 0) { set_error("the communicator reported asynchronous error %d while waiting", ce); return HP_ECOMM; } }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > limit_ms) { set_error("no progress on the collective stream after %d ms: a peer has stopped taking part", limit_ms); return HP_ETIMEOUT; }
        if (it > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50)); else std::this_thread::yield();
    }
}
namespace {
struct WaitCtx { cudaStream_t s; void* comm; };
int wait_stream_query(void* p) { const cudaError_t e = cudaStreamQuery(((WaitCtx*)p)->s); return e == cudaSuccess ? 0 : e == cudaErrorNotReady ? 1 : 2 + (int)e; }
int wait_comm_error(void* p) { int st = 0; if (g_nccl.CommGetAsyncError(((WaitCtx*)p)->comm, &st) != 0) return -1; return (st == 0 || st == 7 /* ncclInProgress */) ? 0 : st; }
}
// stream synchronisation of an engine: plain when no communicator is attached, bounded polling otherwise. After a
// failure the communicator is aborted (its kernels are torn down) and the engine refuses further expert-parallel work.
int Engine::sync_stream() {
    if (!nccl_comm_) { HP_CUDA(cudaStreamSynchronize(s_)); return HP_OK; }
    static const int limit = [] { const char* e = getenv("HIPSTER_B200_EP_TIMEOUT_MS"); return e ? atoi(e) : 30000; }();
    WaitCtx c{s_, nccl_comm_};
    const int rc = ep_wait_poll(wait_stream_query, wait_comm_error, &c, limit);
    if (rc != HP_OK) { g_nccl.CommAbort(nccl_comm_); nccl_comm_ = nullptr; ep_failed_ = true; }
    return rc;
}
int Engine::moe_touched(unsigned long long* n) {
    HP_REQUIRE(n && moe_touched_, "moe_touched: not a mixture-of-experts engine");
    HP_TRY(sync_stream());
    HP_CUDA(cudaMemcpy(n, moe_touched_, 8, cudaMemcpyDeviceToHost)); HP_CUDA(cudaMemset(moe_touched_, 0, 8));
    return HP_OK;
}
int Engine::ep_exchange_us(int R, int reps, float* us) {
    HP_REQUIRE(c_.n_expert > 0 && R >= 1 && R <= MAXR && reps >= 1 && us, "ep_exchange_us: bad arguments");
    *us = 0.f;
    if (c_.ep_world <= 1) return HP_OK;
    HP_TRY(ep_ready());
    const size_t n = (size_t)R * (c_.n_expert_used + 1) * c_.n_embd;
    if (!ep_peer_) HP_CUDA(cudaMemsetAsync(moe_v_, 0, n * 4, s_));
    HP_TRY(ep_peer_ ? ep_exchange_peer(R, 0, false) : ep_exchange(moe_v_, n));   // warm-up
    HP_CUDA(cudaEventRecord(ev0_, s_));
    for (int i = 0; i < reps; ++i) HP_TRY(ep_peer_ ? ep_exchange_peer(R, 0, false) : ep_exchange(moe_v_, n));
    HP_CUDA(cudaEventRecord(ev1_, s_));
    HP_TRY(sync_stream());
    float ms = 0; HP_CUDA(cudaEventElapsedTime(&ms, ev0_, ev1_)); *us = ms * 1000.f / reps;
    return HP_OK;
}
int Engine::ep_unique_id(void* id128) { HP_TRY(nccl_load()); return nccl_check(g_nccl.GetUniqueId(id128), "ncclGetUniqueId"); }
int Engine::ep_init(const void* id128) {
    HP_REQUIRE(c_.n_expert > 0 && c_.ep_world > 1, "ep_init: the model was not loaded with ep_world > 1");
    HP_REQUIRE(!nccl_comm_, "ep_init: already initialised");
    HP_TRY(nccl_load());
    NcclId id; memcpy(id.b, id128, 128);
    HP_TRY(nccl_check(g_nccl.CommInitRank(&nccl_comm_, c_.ep_world, id, c_.ep_rank), "ncclCommInitRank"));
    ep_world_ = c_.ep_world; ep_failed_ = false;
    // the peer-memory exchange when every rank can map every other rank's buffers; the NCCL collective otherwise
    static const bool want_peer = getenv("HIPSTER_B200_EP_NCCL") == nullptr;
    if (want_peer) HP_TRY(ep_peer_setup());
    return HP_OK;
}
// Exchange buffers and flag words of this rank, exported through CUDA IPC handles that travel in one all-gather; the mode
// is taken only if EVERY rank mapped every peer (agreed by an all-reduce of the outcome), so that no rank waits for flags
// that another one will never write.
int Engine::ep_peer_setup() {
    struct Handles { cudaIpcMemHandle_t x, c; };
    static_assert(sizeof(Handles) == 128, "two IPC handles");
    const int W = c_.ep_world, me = c_.ep_rank;
    HP_REQUIRE(W <= 8, "ep_peer_setup: at most 8 ranks");
    ep_half_ = (size_t)MAXR * (c_.n_expert_used + 1) * c_.n_embd;
    int okv = 1;
    if (cudaMalloc((void**)&ep_xbuf_, 2 * ep_half_ * 4) != cudaSuccess || cudaMalloc((void**)&ep_ctl_, 64) != cudaSuccess) { cudaGetLastError(); okv = 0; }
    Handles mine; memset(&mine, 0, sizeof(mine));
    if (okv) {
        HP_CUDA(cudaMemset(ep_ctl_, 0, 64));
        if (cudaIpcGetMemHandle(&mine.x, ep_xbuf_) != cudaSuccess || cudaIpcGetMemHandle(&mine.c, ep_ctl_) != cudaSuccess) { cudaGetLastError(); okv = 0; }
    }
    char* d_h = nullptr; HP_CUDA(cudaMalloc((void**)&d_h, (size_t)128 * (W + 1) + 16));
    struct Free { char* p; ~Free() { cudaFree(p); } } free_d_h{d_h};   // scratch of this function, released on every path
    HP_CUDA(cudaMemcpy(d_h, &mine, 128, cudaMemcpyHostToDevice));
    int rc = nccl_check(g_nccl.AllGather(d_h, d_h + 128, 128, /* ncclChar */ 0, nccl_comm_, s_), "ncclAllGather");
    if (rc == HP_OK) rc = sync_stream();
    std::vector<Handles> all(W);
    if (rc == HP_OK && cudaMemcpy(all.data(), d_h + 128, (size_t)128 * W, cudaMemcpyDeviceToHost) != cudaSuccess) rc = HP_ECUDA;
    if (rc != HP_OK) return rc;
    for (int q = 0; q < W && okv; ++q) {
        if (q == me) { ep_peer_x_[q] = ep_xbuf_; ep_peer_ctl_[q] = ep_ctl_; continue; }
        void *px = nullptr, *pc = nullptr;
        if (cudaIpcOpenMemHandle(&px, all[q].x, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); okv = 0; break; }
        ep_peer_x_[q] = (float*)px;
        if (cudaIpcOpenMemHandle(&pc, all[q].c, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); okv = 0; break; }
        ep_peer_ctl_[q] = (unsigned*)pc;
    }
    // agreement: the minimum of the ranks' outcomes
    float* d_ok = (float*)(d_h + 128 * (W + 1)); const float fok = (float)okv; float agreed = 0.f;
    HP_CUDA(cudaMemcpy(d_ok, &fok, 4, cudaMemcpyHostToDevice));
    rc = nccl_check(g_nccl.AllReduce(d_ok, d_ok, 1, /* ncclFloat32 */ 7, /* ncclMin */ 3, nccl_comm_, s_), "ncclAllReduce");
    if (rc == HP_OK) rc = sync_stream();
    if (rc == HP_OK && cudaMemcpy(&agreed, d_ok, 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = HP_ECUDA;
    if (rc != HP_OK) return rc;
    ep_peer_ = agreed > 0.5f;
    if (!ep_peer_) ep_peer_teardown();
    return HP_OK;
}
void Engine::ep_peer_teardown() {
    for (int q = 0; q < 8; ++q) {
        if (q != c_.ep_rank) { if (ep_peer_x_[q]) cudaIpcCloseMemHandle(ep_peer_x_[q]); if (ep_peer_ctl_[q]) cudaIpcCloseMemHandle(ep_peer_ctl_[q]); }
        ep_peer_x_[q] = nullptr; ep_peer_ctl_[q] = nullptr;
    }
    if (ep_xbuf_) cudaFree(ep_xbuf_);
    if (ep_ctl_) cudaFree(ep_ctl_);
    ep_xbuf_ = nullptr; ep_ctl_ = nullptr; ep_peer_ = false;
}
// the gather kernel's wait alone, on caller-provided flag words (one per rank): what a rank does while a peer is silent
int ep_wait_probe(const unsigned* flags_dev, int world, int rank, unsigned expect, int* err, cudaStream_t s) {
    HP_REQUIRE(flags_dev && err && world >= 1 && world <= 8 && rank >= 0 && rank < world, "ep_wait_probe: bad arguments");
    k_ep_wait_probe<<<1, 32, 0, s>>>(flags_dev, world, rank, expect, err);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int Engine::ep_exchange_peer(int R, int sh_owner, bool pushed) {
    HP_TRY(ep_ready());
    EpXArgs a; a.v = moe_v_; a.ids = moe_ids_; a.npairs = R * (c_.n_expert_used + 1); a.E = c_.n_embd; a.n_expert = c_.n_expert; a.world = c_.ep_world; a.rank = c_.ep_rank;
    a.sh_owner = sh_owner; a.half = ep_half_; a.err = err_;
    for (int q = 0; q < 8; ++q) { a.x[q] = ep_peer_x_[q]; a.ctl[q] = ep_peer_ctl_[q]; }
    const int items = a.npairs * (a.E >> 2), grid = std::max(1, std::min(64, (items + 2047) / 2048));
    if (!pushed) k_ep_push<<<grid, 256, 0, s_>>>(a);   // the quad form of the down projection has delivered its outputs itself
    k_ep_gather<<<grid, 256, 0, s_>>>(a);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
// a model loaded as one shard of an expert-parallel group must not run a pass before (or after a failure of) its
// communicator: the experts it does not hold would silently contribute zeros
int Engine::ep_ready() {
    if (c_.ep_world <= 1 || nccl_comm_) return HP_OK;
    set_error(ep_failed_ ? "expert parallelism: the communicator failed earlier; reload the engine" : "expert parallelism is not initialised: call hp_ep_init on every rank before the first pass");
    return HP_ESTATE;
}
void Engine::ep_destroy() {
    if (ep_peer_ && nccl_comm_) {
        // nobody may still be pushing into this rank's exchange buffer when it is freed: one collective as a barrier
        // (bounded like every other wait on this stream)
        if (ep_ctl_ && g_nccl.AllReduce(ep_ctl_ + 12, ep_ctl_ + 12, 1, 7, 0, nccl_comm_, s_) == 0) sync_stream();
    }
    if (ep_xbuf_ || ep_ctl_) { cudaStreamSynchronize(s_); ep_peer_teardown(); }
    if (nccl_comm_ && g_nccl.CommDestroy) { cudaStreamSynchronize(s_); g_nccl.CommDestroy(nccl_comm_); }
    nccl_comm_ = nullptr;
}
int Engine::ep_allreduce(float* buf, size_t n) {
    HP_TRY(ep_ready());
    return nccl_check(g_nccl.AllReduce(buf, buf, n, /* ncclFloat32 */ 7, /* ncclSum */ 0, nccl_comm_, s_), "ncclAllReduce");
}
}
