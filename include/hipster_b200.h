/* hipster_b200 -- C ABI of the B200-native MTP speculative-decode path.
 *
 * The reference (dzannotti/hipster) has no C ABI: its engine is a C++ class API (engine/src/qwen35.h:50-98,
 * engine/src/qwen4exp.h:54-90) over free kernel launchers taking device pointers and a stream
 * (engine/kernels/gemv.h, ops.h, fn.h), consumed by the token-level `struct Backend` of the server
 * (front/serve.cpp:28-41) and by the MTP drivers (engine/bench/spec27b.cpp, specfn.cpp, batchfn.cpp).
 * Every entry point below names the reference interface it replaces.
 *
 * Conventions: all functions return 0 on success or an HP_E* code; hp_last_error() gives the message of the
 * last failure on the calling thread's library instance (the reference throws std::runtime_error instead,
 * engine/src/qwen35.cpp:10,290-298). Nothing throws across this boundary. `stream` is a cudaStream_t passed as
 * void* (NULL = default stream). Pointers named *_dev are device memory, *_host host memory.
 * Not thread-safe per handle: one caller thread per engine, like the reference (front/serve.cpp:249).
 */
#ifndef HIPSTER_B200_H
#define HIPSTER_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { HP_OK = 0, HP_EINVAL = 1, HP_ECUDA = 2, HP_ENOMEM = 3, HP_ETIMEOUT = 4, HP_ESTATE = 5, HP_ECOMM = 6 };

const char* hp_last_error(void);
int hp_version(void);
/* Reads (and clears) the device-side status word that kernels set when a bounded wait gave up. */
int hp_device_status(void* stream);

/* ------------------------------------------------------------------ kernel level (engine/kernels/gemv.h, ops.h) */

/* Size of the quantised-activation buffers for R rows of K elements (reference: struct XQ8, gemv.h:8).
 * The layout is private to the library; buffers must be zero-initialised once by the caller. */
size_t hp_xq8_q_bytes(int R, int K);
size_t hp_xq8_sc_bytes(int R, int K);
/* x f32 [R][ldx] -> int8 per 32 elements. Replaces quantize_x_q8 (gemv.h:9, gemv.hip:36-51). */
int hp_quantize_x_q8(const float* x_dev, int ldx, int R, int K, void* xq_q_dev, void* xq_sc_dev, void* stream);
/* Converts the private layout to the reference's XQ8 rows: q [R][K] i8, d [R][K/32], s [R][K/32] (gemv.h:7-8). */
int hp_xq8_unpack(const void* xq_q_dev, const void* xq_sc_dev, int R, int K, int8_t* q_dev, float* d_dev, float* s_dev, void* stream);
/* Dequantise nblk Q4_K blocks to f32. Replaces the device twins of dequant_q4_K (quant.h:43-53; ops.hip:154-171). */
int hp_dequant_q4k(const void* w_dev, size_t nblk, float* out_dev, void* stream);
/* y[r][n] = sum_k W[n][k] x[r][k], W = Q4_K [N][K/256] blocks, x quantised by hp_quantize_x_q8, y f32 [R][ldy].
 * 1 <= R <= 32; the result of a row does not depend on R. Replaces gemv_q8 / gemv_multi / gemv_wmma
 * (gemv.h:23-33, gemv.hip:291-367,602-672,1306-1331). */
int hp_gemv_q4k_q8(const void* w_dev, const void* xq_q_dev, const void* xq_sc_dev, float* y_dev, int N, int K, int R, int ldy, void* stream);
/* Number of K parts (1, 2 or 4) the GEMV splits a [N][K] tensor into; a function of the shape only. It fixes the
 * fp32 summation order, so it is part of the result's definition (reference analogue: the KS split of gemv_wmma,
 * gemv.hip:1315). */
int hp_gemv_parts(int N, int K);
/* f32-activation baseline, R <= 8, y [R][N]. Replaces gemv_q4_K_f32 (gemv.h:57, gemv.hip:1177-1216). */
int hp_gemv_q4k_f32(const void* w_dev, const float* x_dev, float* y_dev, int N, int K, int R, void* stream);
/* Row-wise argmax (maximum value, lowest index on ties) of logits [R][ld] over n entries.
 * Replaces argmax_topk with k = 1 (ops.h:118, ops.hip:702-716). scratch_dev: hp_argmax_scratch_bytes(R, n) bytes. */
size_t hp_argmax_scratch_bytes(int R, int n);
int hp_argmax(const float* logits_dev, int R, int n, int ld, int* ids_dev, float* vals_dev, void* scratch_dev, void* stream);
/* hp_argmax for callers that must not allocate. It has no counterpart in the reference. A serving loop that has sized
 * its weights, KV caches and state to fill the GPU, or that runs its decode steps on a latency-critical thread, cannot
 * afford a cudaMalloc per call: the allocation may fail, and it serialises against everything running on the device.
 * This variant needs no scratch from the caller: its partial results live in a fixed 16 KiB array inside the library
 * image (held by every GPU that loads the library until the process exits). It accepts at most
 * hp_argmax_noalloc_max_rows() rows of hp_argmax_noalloc_max_n() entries and rejects larger shapes with HP_EINVAL.
 * It calls no allocating routine. The first call on each device resolves the array's address; make that call before
 * any stream capture begins. All calls share the one array: nothing in it has to be cleared between calls (every
 * element read is written first by the same call), but two calls that overlap on the GPU race on it. The stream must
 * belong to the current device (a stream of another device is refused). Not thread-safe: the first call on a device
 * records the address without a lock, so it must not run concurrently with another host thread's call. */
int hp_argmax_noalloc(const float* logits_dev, int R, int n, int ld, int* ids_dev, float* vals_dev, void* stream);
int hp_argmax_noalloc_max_rows(void);
int hp_argmax_noalloc_max_n(void);
/* Greedy prefix acceptance on device: out_dev[0] = number of accepted drafts mm, out_dev[1] = ids[mm] (bonus token).
 * ids_dev holds n_draft+1 target argmaxes. Replaces the host loop of engine/bench/spec27b.cpp:92-97. */
int hp_accept_greedy(const int* ids_dev, const int* drafts_dev, int n_draft, int* out_dev, void* stream);

/* x += sum of n_planes planes of y (plane p at y_dev + p * plane_stride, rows of n floats; n_planes = 0: no add);
 * xn = x * rsqrt(mean(x^2) + eps) * w (bf16 weights); xq = int8 quantisation of xn. One call for R rows.
 * Replaces add_rmsnorm_quant (ops.h:14, ops.hip:79-98). xn_dev may be NULL. */
int hp_add_rmsnorm_quant(float* x_dev, const float* y_dev, int n_planes, size_t plane_stride, const void* w_bf16_dev, float* xn_dev, void* xq_q_dev, void* xq_sc_dev, int R, int n, float eps, void* stream);
/* xq = q8(silu(gate) * up), gate = columns [0, F) and up = [F, 2F) of gate_up [R][ld]. Replaces silu_mul_quant (ops.h:25, ops.hip:146-151). */
int hp_silu_mul_quant(const float* gate_up_dev, int ld, int F, void* xq_q_dev, void* xq_sc_dev, int R, void* stream);
/* One Gated-DeltaNet layer step for one sequence: causal 4-tap conv + SiLU and the gated delta rule over T new rows
 * (rows [T][ld] = qkv | z | beta | alpha, the in-projection output), with per-row state snapshots and rollback.
 * First the first n_replay rows of the PREVIOUS call (their raw inputs are kept in saved_dev) are applied to the
 * committed state in state_dev / conv_state_dev and written back: that is "accept n_replay rows" (rollback to that
 * prefix; Qwen35::accept, qwen35.cpp:383-403). Then the T new rows are processed from that state: out [T][n_v*128]
 * (nullable), quantised out (nullable), snap_dev (nullable) = the state after each new row [T][n_v][128][128]. The
 * committed state is not advanced by the new rows until a later call accepts them. T = 0 only commits.
 * conv_state_dev: hp_gdn_conv_state_floats(n_v) floats, [n_v][3 taps][q 128 | k 128 | v 128] (each value head keeps the
 * history of its own q/k head); saved_dev: hp_gdn_saved_floats(n_v) floats. Replaces gdn_conv + gdn_step (ops.h:41-51). */
size_t hp_gdn_conv_state_floats(int n_v);
size_t hp_gdn_saved_floats(int n_v);
int hp_gdn_layer(const float* rows_dev, int ld, int T, int n_replay, int n_qk, int n_v, const float* conv_w_dev, const void* dt_bias_bf16_dev, const void* a_neg_bf16_dev,
                 const void* norm_w_bf16_dev, float* state_dev, float* conv_state_dev, float* saved_dev, float* out_dev, void* xq_q_dev, void* xq_sc_dev,
                 float* snap_dev, float eps, int sigmoid_gate, void* stream);

/* The streaming layout of the engine's GEMVs: the same Q4_K bytes, permuted so that each (16-row tile, 256-element block)
 * is one contiguous 2304-byte chunk in tensor-core fragment order. w_dev: ggml Q4_K [N][K/256 blocks]; w_tiled_dev:
 * hp_q4k_tiled_bytes(N, K) bytes. interleave_half = F > 0 treats the tensor as a stack of [gate F rows | up F rows]
 * matrices and lets gate and up rows of a feature share a tile (the routed experts' gate|up tensors). The reference keeps
 * ggml row order and repacks nothing; its nearest analogue is the SoA repack of other formats at load (qwen35.cpp:128-134). */
size_t hp_q4k_tiled_bytes(size_t N, int K);
int hp_q4k_repack_tiled(const void* w_dev, void* w_tiled_dev, size_t N, int K, int interleave_half, void* stream);
/* GQA decode attention for one sequence, as one call: per-head RMSNorm of q and k, NeoX RoPE on the first n_rot dims,
 * f16 K/V cache write, causal attention over keys 0..pos (fixed 128-key splits merged in split order), sigmoid gate.
 * qkv_dev [R][ld]: per row [n_head x (256 q | 256 gate) | n_kv x 256 k | n_kv x 256 v] (q and k are normalised and
 * rotated in place); rows r = 0..R-1 (R <= 8) sit at positions pos0 + r. rope_dev: float (cos, sin) pairs
 * [max_ctx][n_rot/2] of pos * base^(-2i/n_rot). k_cache_dev / v_cache_dev: f16 [n_kv][max_ctx][256]. out_dev f32
 * [R][n_head*256] and/or its int8 quantisation (either may be NULL). workspace_dev: hp_attn_workspace_bytes(...) bytes.
 * Replaces qk_norm_rope_kv + attn_decode_mq (ops.h:71-72,96; ops.hip:363-465,831-948). */
size_t hp_attn_workspace_bytes(int R, int n_head, int n_kv, int max_ctx);
int hp_attn_decode(float* qkv_dev, int ld, int R, int pos0, int n_head, int n_kv, int n_rot, const void* q_norm_bf16_dev, const void* k_norm_bf16_dev, const float* rope_dev,
                   void* k_cache_dev, void* v_cache_dev, int max_ctx, float* out_dev, void* xq_q_dev, void* xq_sc_dev, float eps, void* workspace_dev, void* stream);
/* One mixture-of-experts FFN for T <= 32 rows: exact f32 router over n_expert + 1 rows (row n_expert = the shared
 * expert's gate), softmax top-k routing (ties -> lower id) renormalised over the k winners, slot k = the shared expert
 * with weight sigmoid(logit[n_expert]); gate|up GEMV per (row, slot), silu * up + int8, down GEMV, and the weighted
 * combine in slot order. xn_dev f32 [T][E] feeds the router, xq_* (hp_quantize_x_q8 of the same rows) the experts.
 * Expert tensors are Q4_K in the library's tile-major layout (hp_q4k_repack_tiled of the ggml tensors, contiguous per
 * tensor: gate|up [n_expert][2F][E/256 blocks] repacked with interleave_half = F, down [n_expert][E][F/256] with 0).
 * The (row, slot) pairs are grouped by expert, so every touched expert matrix is read once per call.
 * Outputs: ids_dev / weights_dev [T][k+1] (id -1 = shared), y_dev f32 [T][E]. workspace_dev: hp_moe_workspace_bytes(...).
 * Replaces f32_gemv + moe_route + gemv_moe + moe_silu_quant + gemv_moe_down (fn.h, gemv.h:43-50; fn.hip:167-277,
 * gemv.hip:1075-1129; Qwen4Exp::moe_layer, qwen4exp.cpp:345-354). */
size_t hp_moe_workspace_bytes(int T, int E, int F, int n_expert, int k);
int hp_moe_layer(const float* xn_dev, const void* xq_q_dev, const void* xq_sc_dev, const float* router_dev, const void* exp_gate_up_tiled_dev, const void* exp_down_tiled_dev,
                 const void* sh_gate_up_tiled_dev, const void* sh_down_tiled_dev, int T, int E, int F, int n_expert, int k, int* ids_dev, float* weights_dev, float* y_dev,
                 void* workspace_dev, void* stream);

/* ------------------------------------------------------------------ engine level (engine/src/qwen35.h, qwen4exp.h) */

/* Shapes of the hybrid Gated-DeltaNet / attention model. The reference fixes them at compile time (struct Qwen35Dims,
 * qwen35.h:15-26; struct FnDims, qwen4exp.h:18-28); here they are run-time so that reduced-depth models can be checked
 * against the CPU oracle. head_dim is 256 and gdn_dim 128 (as in both reference models); conv kernel 4. */
typedef struct hp_model_cfg {
    int n_embd, n_layer, n_ff, n_vocab;
    int n_head, n_head_kv, n_rot;
    int gdn_qk_heads, gdn_v_heads;
    int attn_every;              /* layer il is full attention when (il + 1) % attn_every == 0 (qwen35.h:25) */
    int max_ctx, n_slots;
    int n_expert, n_expert_used, expert_ff;   /* n_expert = 0: dense SwiGLU FFN; else routed experts + 1 shared expert */
    int gdn_sigmoid_gate;        /* GDN output gate: 0 = silu(z) (27B), 1 = sigmoid(z) (Flash-Next) */
    int has_mtp;
    int ep_rank, ep_world;       /* expert parallelism: this GPU holds routed experts [ep_rank*n_expert/ep_world, ...); 0, 1 = all */
    int synth_router_logits;     /* benchmark input control ("router logits N(0,1)"): 1 = the expert logits that enter the routing
                                    softmax are seeded N(0,1) draws keyed by (layer, slot, token, position, expert), so that rows route to
                                    different experts as they do in a trained model; the router GEMV still runs and its last row still
                                    gates the shared expert. 0 = the router's own logits (the reference arithmetic, fn.hip:252-266) */
    float rms_eps, rope_base;
    unsigned long long seed;     /* weights are random-init, generated on the device from this seed */
} hp_model_cfg;
/* One sequence's contribution to a pass: T tokens continuing that slot's sequence at positions pos..pos+T-1
 * (struct SlotReq, engine/kernels/ops.h:40). tokens is a host pointer borrowed for the call. */
typedef struct hp_slot_req { int slot; const int* tokens; int T; int pos; } hp_slot_req;
typedef struct hp_engine hp_engine;

/* preset: "qwen35-27b" (benchmark configuration 3), "flash-next" (configuration 4), "tiny" / "tiny-moe" (reduced models for parity tests) */
int hp_model_preset(const char* preset, hp_model_cfg* out);
/* Replaces Qwen35::Qwen35(path, max_ctx, n_slots) (qwen35.h:53): no checkpoint is read, weights are generated. */
int hp_load(const hp_model_cfg* cfg, hp_engine** out);
int hp_free(hp_engine* e);
int hp_n_slots(const hp_engine* e);                        /* qwen35.h:67 */
size_t hp_weight_bytes(const hp_engine* e);                /* qwen35.h:91 */
float hp_last_ms(const hp_engine* e);                      /* qwen35.h:93 */
int hp_reset(hp_engine* e);                                /* qwen35.h:88 */
int hp_reset_slot(hp_engine* e, int slot);                 /* qwen35.h:89 */
/* A pass over S slots, rows = sum of T <= 32 (8 per slot): logits [rows][n_vocab] and h_nextn [rows][n_embd] stay on the
 * device. Replaces Qwen35::forward(const SlotReq*, int) (qwen35.h:57-62); *ms_out (nullable) = GPU milliseconds. */
int hp_forward(hp_engine* e, const hp_slot_req* reqs, int S, float* ms_out);
/* Commit the first m (1..T) rows of that slot in the last pass; the recurrent state is rolled back to that prefix.
 * Replaces Qwen35::accept (qwen35.h:63-66, qwen35.cpp:383-403). */
int hp_accept(hp_engine* e, int slot, int m);
/* MTP draft block over T (token, h) pairs at positions pos0.. of `slot`; h_dev [T][n_embd] device rows (may alias
 * hp_h_nextn_dev / hp_mtp_h_dev). Replaces Qwen35::mtp_forward (qwen35.h:68-70, qwen35.cpp:405-424). */
int hp_mtp_forward(hp_engine* e, int slot, const int* tokens_host, const float* h_dev, int T, int pos0);
/* Top-k (1 <= k <= 32) of the first T rows of the target (which = 0) or MTP (which = 1) logits -> host arrays
 * ids_host / vals_host [T][k], values descending, ties -> lower id; vals_host may be NULL.
 * Replaces Qwen35::topk (qwen35.h:87, qwen35.cpp:426-430; k_topk, ops.hip:702-716). */
int hp_topk(hp_engine* e, int which, int T, int k, int* ids_host, float* vals_host);
/* Prompt ingestion for one slot: n tokens at positions pos0.., committed (no accept needed). with_mtp != 0 also runs the
 * MTP block over the same rows so that its KV cache covers the prompt; successive calls for one prompt must follow each
 * other. Afterwards row 0 of hp_logits_dev / hp_h_nextn_dev (and hp_topk(0, 1, ...)) is the LAST prompt row.
 * Replaces Qwen4Exp::prefill + mtp_catchup (qwen4exp.h:57-60,72-74) and Backend::prefill (front/serve.cpp:29); this
 * build feeds the prompt through the verify path in chunks of 8 rows (the GEMM prefill path is not part of it). */
int hp_prefill(hp_engine* e, int slot, const int* tokens_host, int n, int pos0, int with_mtp);
const float* hp_logits_dev(const hp_engine* e);            /* qwen35.h:82 */
const float* hp_h_nextn_dev(const hp_engine* e);           /* qwen35.h:83 */
const float* hp_mtp_logits_dev(const hp_engine* e);        /* qwen35.h:84 */
const float* hp_mtp_h_dev(const hp_engine* e);             /* qwen35.h:85 */
/* MTP block over the rows of S slots in one pass (rows in request order, h_dev holds one row of n_embd floats per
 * request row). Replaces Qwen4Exp::mtp_forward(reqs, S, h) (qwen4exp.h:66-70). */
int hp_mtp_forward_slots(hp_engine* e, const hp_slot_req* reqs, int S, const float* h_dev);
/* Expert parallelism for the MoE configuration (no counterpart in the single-GPU reference): the routed experts are
 * sharded over ep_world GPUs of one node (cfg.ep_rank / cfg.ep_world at load), everything else is replicated. Per MoE
 * layer the per-(row, slot) expert outputs are exchanged with one NCCL collective and combined in slot order on every
 * GPU, so each slot's stream stays bit-identical to its single-GPU run. hp_ep_unique_id fills 128 bytes on one rank;
 * the caller distributes them (e.g. through torch.distributed) and every rank calls hp_ep_init with the same bytes. */
int hp_ep_unique_id(void* id128_out);
int hp_ep_init(hp_engine* e, const void* id128);
/* The wait the engine uses at the end of a pass that carries collectives, exposed so that an integrator can drive it with
 * its own probes: polls stream_query(ctx) (0 = done, 1 = still running, else failed) and comm_error(ctx) (0 = healthy)
 * for at most limit_ms, and returns HP_OK, HP_ECOMM (a failure was reported) or HP_ETIMEOUT (a peer stopped taking part).
 * The engine applies it with cudaStreamQuery and ncclCommGetAsyncError (limit: HIPSTER_B200_EP_TIMEOUT_MS, default
 * 30000), aborts its communicator on failure and then refuses further passes with HP_ESTATE. */
int hp_ep_wait_poll(int (*stream_query)(void*), int (*comm_error)(void*), void* ctx, int limit_ms);
/* Test/diagnostic access: device pointer and size of a generated tensor (layer = -1 for model-level tensors) and of a
 * slot's committed GDN state [gdn_v_heads][128][128] (pending accepts are applied first). */
int hp_tensor_dev(const hp_engine* e, int layer, int kind, void** ptr_out, size_t* bytes_out);
int hp_gdn_state_dev(hp_engine* e, int slot, int gdn_layer, float** ptr_out, size_t* bytes_out);
/* Measurement hooks (the reference's HIPSTER_TIMING categories, qwen35.h:95, qwen35.cpp:181-186): mean device time of
 * `reps` verify passes of R rows (what = 0), of only their GEMV launches (what = 1), or of passes that leave kernel
 * classes out to price them in place (what = 16 + mask: 1 GDN, 2 row norms, 4 attention, 8 SiLU, 16 gate|up, 32 down,
 * 64 LM head, 128 input projections, 256 other GEMVs; only the time means anything then).
 * The passes run on slot 0 at its current position; its context survives (pending accepts are applied first, the K/V rows
 * written are put back), but the pass before the call can no longer be accepted.
 * hp_pass_weight_bytes: Q4_K bytes one trunk pass (mtp = 0) or one MTP-block pass (mtp = 1) reads, with or without the
 * LM head: the algorithmic bytes of the roofline. */
int hp_profile_pass(hp_engine* e, int R, int what, int reps, float* ms_out);
/* More measurement hooks: the number of (layer, expert) matrices touched by the passes since the last call (mixture of
 * experts: the unique expert bytes of the roofline = that count x bytes per expert); the mean device time in microseconds
 * of one expert-parallel exchange for R rows (0 on a single GPU); the kernels in the last fused round's graph. */
int hp_moe_touched(hp_engine* e, unsigned long long* n_out);
int hp_ep_exchange_us(hp_engine* e, int R, int reps, float* us_out);
/* 1 when the expert-parallel exchange runs over peer memory (every rank mapped every other rank's exchange buffer through
 * CUDA IPC at hp_ep_init: one process per GPU on one node), 0 when it is the NCCL collective (HIPSTER_B200_EP_NCCL set, or a
 * rank could not map a peer). In the peer form a fused round is one CUDA graph again. No counterpart in the reference. */
int hp_ep_peer(hp_engine* e);
/* Rank that holds routed expert `expert` (contiguous shards [r * n_expert / world, (r + 1) * n_expert / world)); -1 for an id
 * outside [0, n_expert). The rule the peer-memory exchange uses to tell which rows a rank delivers. */
int hp_ep_owner(int expert, int n_expert, int world);
/* The wait of the peer-memory exchange on its own: one launch in which rank `rank` waits until each of the other ranks'
 * flag words flags_dev[q] (unsigned, q < world) has reached `expect`. The wait is bounded (2^22 polls, about a second):
 * when a flag stays behind the launch ends, the device status word is set and hp_device_status returns HP_ETIMEOUT; the
 * context stays usable. For failure-detection tests (a flag that nothing sets). */
int hp_ep_wait_probe(const void* flags_dev, int world, int rank, unsigned expect, void* stream);
int hp_last_round_kernels(const hp_engine* e);
size_t hp_pass_weight_bytes(const hp_engine* e, int mtp, int with_head);
/* The whole MTP round on the device, for S slots in lock step: n_draft draft steps (one row per slot each), one verify
 * pass of S * (n_draft + 1) rows (<= 32), argmax, greedy acceptance per slot, commit and MTP catch-up, with no logits or
 * ids crossing to the host; only the emitted tokens come back. hp_spec_begin seeds a slot with its last emitted token,
 * that token's position and the pending hidden row (device pointer, n_embd floats).
 * slot_ids_host: the S distinct slots taking part. subst_host (nullable, [S][n_draft] ints): >= 0 replaces that draft
 * (seeded acceptance control), -1 keeps the MTP's argmax. out_tokens_host [S][n_draft + 1]: per slot the accepted drafts
 * followed by the bonus token; out_counts_host [S] = their number (mm + 1).
 * Replaces the host loops of engine/bench/spec27b.cpp:77-103 and engine/bench/batchfn.cpp:96-117. */
int hp_spec_begin(hp_engine* e, int slot, int id_last, int pos, const float* h_pending_dev);
int hp_spec_round(hp_engine* e, const int* slot_ids_host, int S, int n_draft, const int* subst_host, int* out_tokens_host, int* out_counts_host);

#ifdef __cplusplus
}
#endif
#endif
