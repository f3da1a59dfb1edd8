// Internal C++ launchers of the CUDA kernels (device pointers + stream), the layer the reference calls
// "kernels" (engine/kernels/gemv.h, ops.h, fn.h). The C ABI in capi.cu and the engine sit on top of these.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace hp {

// Quantised activations in the fragment-major layout described in hp_common.cuh (reference: struct XQ8, gemv.h:8).
struct XQ8F { void* q; void* sc; };

// Per-device library state is kept in tables indexed by the device ordinal (a process may drive several GPUs).
constexpr int MAX_DEVICES = 64;
inline int current_device() { int d = -1; return (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < MAX_DEVICES) ? d : -1; }
// device status word of the current device (set by kernels whose bounded waits gave up); nullptr if it cannot be allocated
int* device_err_flag();

// ---- gemv_q4k.cu ----
// Work partition of the tensor-core GEMV. It is part of the numerics contract (it fixes the fp32 summation order)
// and depends on the tensor shape only.
constexpr int GEMV_NCTA = 148, GEMV_WARPS = 12, GEMV_STAGES = 2;
constexpr int GEMV_SMEM_LIMIT = 227 * 1024, GEMV_MAX_PART_BLOCKS = 36;
// number of K parts: P in {1, 2, 4} dividing K/256 with at most 36 blocks per part, maximising
//   1000 * tiles / (ctas_per_part * ceil(tiles / ctas_per_part)) - 20 * log2(P) - (50 if K/256/P is odd)
// (ties -> smaller P); 0 when no P qualifies.
__host__ __device__ inline int gemv_num_parts(int N, int nb) {
    const int tiles = (N + 15) / 16; int best = 0, best_score = -1000000;
    for (int lg = 0; lg < 3; ++lg) {
        const int P = 1 << lg; if (nb % P) continue;
        const int nbp = nb / P; if (nbp > GEMV_MAX_PART_BLOCKS) continue;
        const int gc = GEMV_NCTA / P, per = (tiles + gc - 1) / gc;
        const int score = (int)((long long)tiles * 1000 / ((long long)gc * per)) - 20 * lg - ((nbp & 1) ? 50 : 0);
        if (score > best_score) { best_score = score; best = P; }
    }
    return best;
}
// CTA c works on K part c / (148/P) and on tiles [t0, t1): the tiles are split evenly over the CTAs of the part
struct GemvCta { int part, t0, t1; };
__host__ __device__ inline GemvCta gemv_cta(int N, int nb, int P, int c) {
    const int tiles = (N + 15) / 16, gc = GEMV_NCTA / P, cg = c % gc;
    GemvCta r; r.part = c / gc; r.t0 = (int)((long long)cg * tiles / gc); r.t1 = (int)((long long)(cg + 1) * tiles / gc); return r;
}
// inside a CTA the cu units are split evenly and contiguously over weff = min(12, cu) warps
// (cu < 2^20 units per CTA, so 32-bit arithmetic is exact)
__host__ __device__ inline int gemv_warp_start(int cu, int weff, int w) { return (int)((unsigned)w * (unsigned)cu / (unsigned)weff); }
__host__ __device__ inline int gemv_warp_owner(int cu, int weff, int u) { return (int)((((unsigned)u + 1u) * (unsigned)weff - 1u) / (unsigned)cu); }
// scratch for the K-part planes of the public (single-output) entry point
struct GemvWorkspace { float* part; size_t part_bytes; int* err; };
int gemv_parts(int N, int K);
// raw form: part p of the K split writes plane yparts + p * part_stride ([R][ldy] each); the caller adds the planes in order
// tiled = true: W is in the tile-major layout produced by gemv_repack_tiled (gemv_tiled_bytes(N, K) bytes)
int gemv_q4k_q8_parts(const void* W, const XQ8F& x, float* yparts, int N, int K, int R, int ldy, size_t part_stride, int* err, cudaStream_t s, bool pdl, bool tiled);
size_t gemv_tiled_bytes(size_t N, int K);
// interleave_half = F > 0: src is a stack of [gate F rows | up F rows] matrices; gate and up rows of a feature share a tile
int gemv_repack_tiled(const void* src, void* dst, size_t N, int K, cudaStream_t s, int interleave_half = 0);
int gemv_q4k_q8(const void* W, const XQ8F& x, float* y, int N, int K, int R, int ldy, const GemvWorkspace& ws, cudaStream_t s, bool pdl);
int gemv_q4k_f32(const void* W, const float* x, float* y, int N, int K, int R, int* err, cudaStream_t s);

// ---- quant_ops.cu ----
int quantize_x_q8(const float* x, int ldx, XQ8F out, int R, int K, cudaStream_t s);
int xq8_unpack(XQ8F in, int R, int K, int8_t* q, float* d, float* sm, cudaStream_t s);
int dequant_q4k(const void* W, size_t nblk, float* out, cudaStream_t s);

// ---- ops.cu ----
int embed_bf16(const int* tok, const void* table_bf16, float* out, int R, int E, int V, cudaStream_t s);
// x += sum_p y_p (nullable y); xn = rmsnorm(x) * w; xq = q8(xn)   (reference add_rmsnorm_quant, ops.h:14)
int add_rmsnorm_quant(float* x, const float* y, int P, size_t part_stride, int ldy, const void* w_bf16, float* xn, XQ8F xq, int R, int n, float eps, cudaStream_t s, bool assign = false,
                      const float* slotw = nullptr, int nslot = 0);   // assign: x = sum_p y_p instead of x += ...; slotw: y = [R * nslot][ldy] expert outputs, x += sum_e fmaf(slotw, y) in slot order
// out[r] = [rmsnorm(a[r]) * wa | rmsnorm(b[r]) * wb] quantised   (reference norm2_concat_quant, ops.h:16)
int norm2_concat_quant(const float* a, const void* wa, const float* b, int ldb, const void* wb, float* out, XQ8F xq, int R, int n, float eps, cudaStream_t s);
// xq = q8(silu(gu[:, :F]) * gu[:, F:2F])   (reference silu_mul_quant, ops.h:25)
int silu_mul_quant(const float* gu, int ldg, int F, XQ8F xq, int R, cudaStream_t s);
// Gated DeltaNet conv + recurrent step with deferred commit (reference gdn_conv + gdn_step, ops.h:41-51, and the
// replay of Qwen35::accept, qwen35.cpp:383-403)
struct GdnParams {
    const float* rows; float* saved; size_t saved_stride; int ld, off_z, off_b, off_a, n_qk, n_v;
    const float* conv_w; const void* dt_bias; const void* a_neg; const void* norm_w;
    float* state; float* conv_state; size_t state_stride, conv_stride;
    const int* seq; const int* replay_n;                 // device descriptors; seq == nullptr: one sequence {r0 = 0, T = imm_T, slot 0} with imm_replay rows to commit
    int imm_T = 0, imm_replay = 0;
    float* out; XQ8F xq; float* snap; size_t snap_row_stride; float eps; int sigmoid_gate;
};
int gdn_forward(const GdnParams& p, int nseq, cudaStream_t s);

// ---- attn.cu ----
constexpr int ATTN_SPLIT = 128, ATTN_MAX_PAIRS = 48;   // keys per split; (row, q-head) pairs per kv head and row group
struct AttnParams {
    float* qkv; int ld, n_head, n_kv, n_rot;            // rows [q_full n_head x 512 | k n_kv x 256 | v n_kv x 256]
    const float* planes = nullptr; int P = 0; size_t part_stride = 0;   // optional: the projection as K-part planes, summed by the rope kernel into qkv
    const void* q_norm; const void* k_norm; const void* rope;   // bf16 [256] x 2; float2 (cos, sin) [max_ctx][n_rot/2]
    const int* row_pos; const int* row_slot; const int* row_group; const int* groups;   // device descriptors; group = {r0, T, slot, pos0}
    void* kc; void* vc; size_t kv_stride; int max_ctx;   // f16 [slot][n_kv][max_ctx][256] for this layer
    float* pO; float* pm; float* pl; int nsplit_max;     // split partials
    float* out; XQ8F xq; float eps;
};
size_t attn_smem_bytes();
size_t attn_partial_floats(int ngroups, int n_kv, int nsplit_max);
int attn_rope_kv(const AttnParams& p, int rows, cudaStream_t s);          // reference k_qk_norm_rope_kv (ops.hip:363-411)
int attn_decode(const AttnParams& p, int rows, int ngroups, cudaStream_t s);   // reference attn_decode_mq (ops.h:72)

// one sequence of R <= 8 rows at positions pos0.., descriptors and partials in caller-provided workspace
size_t attn_seq_workspace_bytes(int R, int n_head, int n_kv, int max_ctx);
int attn_decode_seq(float* qkv, int ld, int R, int pos0, int n_head, int n_kv, int n_rot, const void* q_norm, const void* k_norm, const void* rope, void* kc, void* vc, int max_ctx,
                    float* out, XQ8F xq, float eps, void* workspace, cudaStream_t s);

// ---- moe.cu ----
// router (reference f32_gemv, fn.hip:252-277), routing (k_moe_route, fn.hip:167-205) and the grouping of the (row, slot)
// pairs by expert, in one launch
constexpr int MOE_MAX_PAIRS = 32 * 16;
struct MoeRouteParams {
    const float* W; const float* x; float* logits; int E, K, k, T;   // router [E + 1][K] f32, rows x [T][K], logits [T][E + 1]
    int* ids; float* w;                                               // [T][k + 1]: expert ids (-1 = shared) and combine weights
    int* ticket;                                                      // five zero-initialised ints (left zero)
    const int* row_tok = nullptr; const int* row_pos = nullptr; const int* row_slot = nullptr; unsigned long long synth_key = 0;   // synth_key != 0: seeded N(0,1) expert logits per (slot, token, position)
    int e_lo = 0, e_hi = 0, own_shared = 1;                           // experts this GPU owns
    void* segs = nullptr; int* ctl = nullptr; unsigned long long* touched = nullptr;   // grouping outputs (segs == nullptr: no grouping)
    int* err = nullptr;                                               // device status word (bounded waits)
};
int moe_route_group(const MoeRouteParams& p, cudaStream_t s);
// Routed experts grouped by expert (see moe.cu). Expert tensors tile-major: gate|up repacked with interleave_half = F.
struct MoeGroupParams {
    const void* w_gate_up; const void* w_down; const void* sh_gate_up; const void* sh_down;   // this GPU's experts [e_lo, e_hi) and the shared expert
    int E, F, nslot, T;                                 // hidden, expert FFN, slots per row (k + 1), rows
    int e_lo;                                           // first routed expert this GPU holds (its tensors start there)
    XQ8F xq, xq2;                                       // quantised rows [T] (K = E) in; quantised silu(gate)*up per pair [T * nslot] (K = F) scratch
    float* v;                                           // per-pair outputs [T * nslot][E] (pairs of experts owned elsewhere are not written)
    void* segs; int* ctl;                               // filled by moe_route_group: MOE_MAX_PAIRS segments of 64 bytes, 4 control ints
    int* err;
    // Expert parallelism over peer memory (ep_world > 1, optional): the down projection also stores every output it
    // computes into the other ranks' exchange buffers (half (n & 1) of it for exchange number n) and, when the whole grid
    // is done, raises this rank's flag word there. ep_ctl[q] = rank q's words: [r] = last exchange delivered by rank r,
    // [8] = exchanges this rank has completed, [9] = ticket.
    int ep_world = 1, ep_rank = 0; float* ep_x[8] = {}; unsigned* ep_ctl[8] = {}; size_t ep_half = 0;
};
size_t moe_seg_bytes();
// *pushed (nullable): set to 1 when the down projection delivered its outputs to the peers itself (the quad form), 0 when the
// caller has to send them
int moe_experts_grouped(const MoeGroupParams& p, cudaStream_t s, int* pushed = nullptr);   // reference gemv_moe + moe_silu_quant + gemv_moe_down (gemv.h:43-50, fn.hip:206-211)
// y[t] = sum over slots e in order of fmaf(slotw[t][e], v[(t, e)], acc) (reference combine, gemv.hip:1104-1112)
int moe_combine(const float* v, const float* slotw, float* y, int T, int nslot, int E, cudaStream_t s);

// ---- argmax.cu ----
// per-row argmax (max value, lowest index) of logits [R][ld] -> ids/vals on device
int argmax_rows(const float* logits, int R, int n, int ld, int* ids, float* vals, void* scratch, cudaStream_t s);
size_t argmax_scratch_bytes(int R, int n);
// per-row top-k (values descending, ties -> lower index; reference argmax_topk, ops.h:118) -> ids / vals [R][k] on device
int topk_rows(const float* logits, int R, int n, int ld, int k, int* ids, float* vals, void* scratch, cudaStream_t s);
size_t topk_scratch_bytes(int R, int n, int k);
int topk_max_k();
// allocation-free variant: partials in a static device array of fixed size (see argmax.cu)
int argmax_rows_static(const float* logits, int R, int n, int ld, int* ids, float* vals, cudaStream_t s);
int argmax_static_max_rows();
int argmax_static_max_n();
// greedy prefix acceptance on device: out[0] = accepted drafts mm, out[1] = bonus id ids[mm]
int accept_greedy(const int* ids, const int* drafts, int n_draft, int* out, cudaStream_t s);

}  // namespace hp
