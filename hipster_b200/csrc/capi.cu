// extern "C" boundary: argument checks, status codes, last-error string. No exceptions cross it.
#include "hp_common.cuh"
#include "kernels.h"
#include "engine.h"
#include <cstring>
#include "../../include/hipster_b200.h"
#include <cstdarg>
#include <cstdio>
#include <string>
#include <exception>

namespace hp {
static thread_local std::string g_last_error;
void set_error(const char* fmt, ...) {
    char buf[512]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
    g_last_error = buf;
}
int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) in %s @%s:%d", (int)e, cudaGetErrorString(e), what, file, line);
    return HP_ECUDA;
}
// one status word per device, set by kernels whose bounded waits gave up
static int* g_dev_err[MAX_DEVICES] = {};
int* device_err_flag() {
    const int dev = current_device(); if (dev < 0) return nullptr;
    if (!g_dev_err[dev]) { if (cudaMalloc(&g_dev_err[dev], sizeof(int)) != cudaSuccess) return nullptr; cudaMemset(g_dev_err[dev], 0, sizeof(int)); }
    return g_dev_err[dev];
}
// workspace of the kernel-level GEMV entry point (per device, allocated on first use; the engine owns its own)
static GemvWorkspace g_ws[MAX_DEVICES] = {};
int default_gemv_workspace(GemvWorkspace* out, size_t need) {
    const int dev = current_device();
    HP_REQUIRE(dev >= 0, "no usable current CUDA device");
    GemvWorkspace& ws = g_ws[dev];
    if (need > ws.part_bytes) {
        if (ws.part) HP_CUDA(cudaFree(ws.part));
        ws.part = nullptr; ws.part_bytes = 0;
        HP_CUDA(cudaMalloc(&ws.part, need));
        ws.part_bytes = need;
    }
    ws.err = device_err_flag();
    *out = ws; return HP_OK;
}
}  // namespace hp

#define HP_GUARD_BEGIN try {
#define HP_GUARD_END } catch (const std::exception& e) { hp::set_error("exception: %s", e.what()); return HP_ESTATE; } catch (...) { hp::set_error("unknown exception"); return HP_ESTATE; }

extern "C" {

const char* hp_last_error(void) { return hp::g_last_error.c_str(); }
int hp_version(void) { return 100; }

int hp_device_status(void* stream) {
    HP_GUARD_BEGIN
    int* f = hp::device_err_flag();
    if (!f) { hp::set_error("cannot allocate the device status word"); return HP_ENOMEM; }
    int h = 0;
    HP_CUDA(cudaMemcpyAsync(&h, f, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    HP_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (h != 0) { HP_CUDA(cudaMemsetAsync(f, 0, sizeof(int), (cudaStream_t)stream)); hp::set_error("a kernel gave up a bounded wait (device status %d)", h); return h; }
    return HP_OK;
    HP_GUARD_END
}

size_t hp_xq8_q_bytes(int R, int K) { return hp::xq_q_bytes(R, K); }
size_t hp_xq8_sc_bytes(int R, int K) { return hp::xq_sc_floats(R, K) * sizeof(float); }

int hp_quantize_x_q8(const float* x_dev, int ldx, int R, int K, void* xq_q_dev, void* xq_sc_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(x_dev && xq_q_dev && xq_sc_dev, "hp_quantize_x_q8: null pointer");
    return hp::quantize_x_q8(x_dev, ldx, hp::XQ8F{xq_q_dev, xq_sc_dev}, R, K, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_xq8_unpack(const void* xq_q_dev, const void* xq_sc_dev, int R, int K, int8_t* q_dev, float* d_dev, float* s_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(xq_q_dev && xq_sc_dev && q_dev && d_dev && s_dev, "hp_xq8_unpack: null pointer");
    HP_REQUIRE(R >= 1 && K > 0 && K % 64 == 0, "hp_xq8_unpack: bad shape R=%d K=%d", R, K);
    return hp::xq8_unpack(hp::XQ8F{(void*)xq_q_dev, (void*)xq_sc_dev}, R, K, q_dev, d_dev, s_dev, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_dequant_q4k(const void* w_dev, size_t nblk, float* out_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(w_dev && out_dev, "hp_dequant_q4k: null pointer");
    return hp::dequant_q4k(w_dev, nblk, out_dev, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_gemv_q4k_q8(const void* w_dev, const void* xq_q_dev, const void* xq_sc_dev, float* y_dev, int N, int K, int R, int ldy, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(w_dev && xq_q_dev && xq_sc_dev && y_dev, "hp_gemv_q4k_q8: null pointer");
    HP_REQUIRE(((uintptr_t)w_dev & 15) == 0, "hp_gemv_q4k_q8: weights must be 16-byte aligned");
    HP_REQUIRE(N > 0 && K > 0 && K % 256 == 0 && R >= 1 && R <= 32, "hp_gemv_q4k_q8: bad shape N=%d K=%d R=%d", N, K, R);
    hp::GemvWorkspace ws; { const int rc = hp::default_gemv_workspace(&ws, (size_t)4 * R * N * sizeof(float)); if (rc) return rc; }
    return hp::gemv_q4k_q8(w_dev, hp::XQ8F{(void*)xq_q_dev, (void*)xq_sc_dev}, y_dev, N, K, R, ldy, ws, (cudaStream_t)stream, false);
    HP_GUARD_END
}
int hp_gemv_parts(int N, int K) { return (N > 0 && K > 0 && K % 256 == 0) ? hp::gemv_parts(N, K) : 0; }
int hp_gemv_q4k_f32(const void* w_dev, const float* x_dev, float* y_dev, int N, int K, int R, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(w_dev && x_dev && y_dev, "hp_gemv_q4k_f32: null pointer");
    HP_REQUIRE(((uintptr_t)w_dev & 15) == 0, "hp_gemv_q4k_f32: weights must be 16-byte aligned");
    return hp::gemv_q4k_f32(w_dev, x_dev, y_dev, N, K, R, hp::device_err_flag(), (cudaStream_t)stream);
    HP_GUARD_END
}
size_t hp_argmax_scratch_bytes(int R, int n) { return (R < 1 || n < 1) ? 0 : hp::argmax_scratch_bytes(R, n); }
int hp_argmax(const float* logits_dev, int R, int n, int ld, int* ids_dev, float* vals_dev, void* scratch_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(logits_dev && ids_dev, "hp_argmax: null pointer");
    return hp::argmax_rows(logits_dev, R, n, ld, ids_dev, vals_dev, scratch_dev, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_argmax_noalloc(const float* logits_dev, int R, int n, int ld, int* ids_dev, float* vals_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(logits_dev && ids_dev, "hp_argmax_noalloc: null pointer");
    return hp::argmax_rows_static(logits_dev, R, n, ld, ids_dev, vals_dev, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_argmax_noalloc_max_rows(void) { return hp::argmax_static_max_rows(); }
int hp_argmax_noalloc_max_n(void) { return hp::argmax_static_max_n(); }
int hp_accept_greedy(const int* ids_dev, const int* drafts_dev, int n_draft, int* out_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(ids_dev && out_dev && (drafts_dev || n_draft == 0), "hp_accept_greedy: null pointer");
    return hp::accept_greedy(ids_dev, drafts_dev, n_draft, out_dev, (cudaStream_t)stream);
    HP_GUARD_END
}

// ------------------------------------------------------------------ layer kernels
int hp_add_rmsnorm_quant(float* x_dev, const float* y_dev, int n_planes, size_t plane_stride, const void* w_bf16_dev, float* xn_dev, void* xq_q_dev, void* xq_sc_dev, int R, int n, float eps, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(x_dev && w_bf16_dev && xq_q_dev && xq_sc_dev && (y_dev || n_planes == 0), "hp_add_rmsnorm_quant: null pointer");
    return hp::add_rmsnorm_quant(x_dev, y_dev, n_planes, plane_stride, n, w_bf16_dev, xn_dev, hp::XQ8F{xq_q_dev, xq_sc_dev}, R, n, eps, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_silu_mul_quant(const float* gate_up_dev, int ld, int F, void* xq_q_dev, void* xq_sc_dev, int R, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(gate_up_dev && xq_q_dev && xq_sc_dev, "hp_silu_mul_quant: null pointer");
    return hp::silu_mul_quant(gate_up_dev, ld, F, hp::XQ8F{xq_q_dev, xq_sc_dev}, R, (cudaStream_t)stream);
    HP_GUARD_END
}
size_t hp_gdn_conv_state_floats(int n_v) { return (size_t)n_v * 3 * 384; }
size_t hp_gdn_saved_floats(int n_v) { return (size_t)n_v * 8 * 388; }
int hp_gdn_layer(const float* rows_dev, int ld, int T, int n_replay, int n_qk, int n_v, const float* conv_w_dev, const void* dt_bias_bf16_dev, const void* a_neg_bf16_dev,
                 const void* norm_w_bf16_dev, float* state_dev, float* conv_state_dev, float* saved_dev, float* out_dev, void* xq_q_dev, void* xq_sc_dev,
                 float* snap_dev, float eps, int sigmoid_gate, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(T >= 0 && T <= 8 && n_replay >= 0 && n_replay <= 8 && T + n_replay >= 1, "hp_gdn_layer: 0 <= T, n_replay <= 8 and T + n_replay >= 1");
    HP_REQUIRE((rows_dev || T == 0) && conv_w_dev && dt_bias_bf16_dev && a_neg_bf16_dev && norm_w_bf16_dev && state_dev && conv_state_dev && saved_dev, "hp_gdn_layer: null pointer");
    HP_REQUIRE(n_qk >= 1 && n_v >= n_qk && n_v % n_qk == 0 && ld >= (2 * n_qk + 2 * n_v) * 128 + 2 * n_v, "hp_gdn_layer: bad shape");
    hp::GdnParams g; g.rows = rows_dev ? rows_dev : state_dev; g.saved = saved_dev; g.saved_stride = 0; g.ld = ld; g.n_qk = n_qk; g.n_v = n_v;
    g.off_z = (2 * n_qk + n_v) * 128; g.off_b = g.off_z + n_v * 128; g.off_a = g.off_b + n_v;
    g.conv_w = conv_w_dev; g.dt_bias = dt_bias_bf16_dev; g.a_neg = a_neg_bf16_dev; g.norm_w = norm_w_bf16_dev;
    g.state = state_dev; g.conv_state = conv_state_dev; g.state_stride = 0; g.conv_stride = 0; g.seq = nullptr; g.replay_n = nullptr; g.imm_T = T; g.imm_replay = n_replay;   // one sequence, described by value
    g.out = out_dev; g.xq = hp::XQ8F{xq_q_dev, xq_sc_dev}; g.snap = snap_dev; g.snap_row_stride = (size_t)n_v * 128 * 128; g.eps = eps; g.sigmoid_gate = sigmoid_gate;
    return hp::gdn_forward(g, 1, (cudaStream_t)stream);
    HP_GUARD_END
}

size_t hp_attn_workspace_bytes(int R, int n_head, int n_kv, int max_ctx) {
    return (R < 1 || n_kv < 1 || n_head < n_kv || max_ctx < 1) ? 0 : hp::attn_seq_workspace_bytes(R, n_head, n_kv, max_ctx);
}
int hp_attn_decode(float* qkv_dev, int ld, int R, int pos0, int n_head, int n_kv, int n_rot, const void* q_norm_bf16_dev, const void* k_norm_bf16_dev, const float* rope_dev,
                   void* k_cache_dev, void* v_cache_dev, int max_ctx, float* out_dev, void* xq_q_dev, void* xq_sc_dev, float eps, void* workspace_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(qkv_dev && q_norm_bf16_dev && k_norm_bf16_dev && rope_dev && k_cache_dev && v_cache_dev && workspace_dev && (out_dev || xq_q_dev), "hp_attn_decode: null pointer");
    HP_REQUIRE((xq_q_dev == nullptr) == (xq_sc_dev == nullptr), "hp_attn_decode: give both quantised-output buffers or neither");
    HP_REQUIRE(n_rot >= 2 && n_rot % 2 == 0 && n_rot <= 256 && ld % 4 == 0, "hp_attn_decode: bad n_rot / ld");
    return hp::attn_decode_seq(qkv_dev, ld, R, pos0, n_head, n_kv, n_rot, q_norm_bf16_dev, k_norm_bf16_dev, rope_dev, k_cache_dev, v_cache_dev, max_ctx, out_dev,
                               hp::XQ8F{xq_q_dev, xq_sc_dev}, eps, workspace_dev, (cudaStream_t)stream);
    HP_GUARD_END
}
size_t hp_q4k_tiled_bytes(size_t N, int K) { return (N < 1 || K < 256 || K % 256) ? 0 : hp::gemv_tiled_bytes(N, K); }
int hp_q4k_repack_tiled(const void* w_dev, void* w_tiled_dev, size_t N, int K, int interleave_half, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(w_dev && w_tiled_dev, "hp_q4k_repack_tiled: null pointer");
    HP_REQUIRE(((uintptr_t)w_dev & 3) == 0 && ((uintptr_t)w_tiled_dev & 15) == 0, "hp_q4k_repack_tiled: misaligned tensor");
    return hp::gemv_repack_tiled(w_dev, w_tiled_dev, N, K, (cudaStream_t)stream, interleave_half);
    HP_GUARD_END
}
// workspace of hp_moe_layer: router logits | ticket counters | per-pair outputs | quantised activations of the pairs | segments | control words
namespace {
struct MoeWs { size_t logits, cnt, v, q2, sc2, segs, ctl, total; };
MoeWs moe_ws(int T, int E, int F, int n_expert, int k) {
    auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t pairs = (size_t)T * (k + 1);
    MoeWs w; size_t o = 0;
    w.logits = o; o += al((size_t)T * (n_expert + 1) * 4);
    w.cnt = o; o += al(32 * 4);
    w.v = o; o += al(pairs * E * 4);
    w.q2 = o; o += al(hp::xq_q_bytes((int)pairs, F));
    w.sc2 = o; o += al(hp::xq_sc_floats((int)pairs, F) * 4);
    w.segs = o; o += al(hp::moe_seg_bytes());
    w.ctl = o; o += 256;
    w.total = o; return w;
}
}
size_t hp_moe_workspace_bytes(int T, int E, int F, int n_expert, int k) { return (T < 1 || E < 1 || F < 1 || n_expert < 1 || k < 1) ? 0 : moe_ws(T, E, F, n_expert, k).total; }
int hp_moe_layer(const float* xn_dev, const void* xq_q_dev, const void* xq_sc_dev, const float* router_dev, const void* exp_gate_up_tiled_dev, const void* exp_down_tiled_dev,
                 const void* sh_gate_up_tiled_dev, const void* sh_down_tiled_dev, int T, int E, int F, int n_expert, int k, int* ids_dev, float* weights_dev, float* y_dev,
                 void* workspace_dev, void* stream) {
    HP_GUARD_BEGIN
    HP_REQUIRE(xn_dev && xq_q_dev && xq_sc_dev && router_dev && exp_gate_up_tiled_dev && exp_down_tiled_dev && sh_gate_up_tiled_dev && sh_down_tiled_dev && ids_dev && weights_dev && y_dev && workspace_dev, "hp_moe_layer: null pointer");
    HP_REQUIRE(T >= 1 && T <= 32 && E % 256 == 0 && F % 256 == 0 && n_expert >= k && k >= 1 && k <= 15, "hp_moe_layer: bad shape T=%d E=%d F=%d experts=%d k=%d", T, E, F, n_expert, k);
    cudaStream_t s = (cudaStream_t)stream;
    const MoeWs w = moe_ws(T, E, F, n_expert, k);
    char* ws = (char*)workspace_dev; const int ns = k + 1;
    float* logits = (float*)(ws + w.logits); int* cnt = (int*)(ws + w.cnt); float* v = (float*)(ws + w.v);
    HP_CUDA(cudaMemsetAsync(cnt, 0, 32 * 4, s));
    HP_CUDA(cudaMemsetAsync(ws + w.q2, 0, w.total - w.q2, s));
    hp::MoeRouteParams rp; rp.W = router_dev; rp.x = xn_dev; rp.logits = logits; rp.E = n_expert; rp.K = E; rp.k = k; rp.T = T; rp.ids = ids_dev; rp.w = weights_dev; rp.ticket = cnt;
    rp.e_lo = 0; rp.e_hi = n_expert; rp.own_shared = 1; rp.segs = ws + w.segs; rp.ctl = (int*)(ws + w.ctl); rp.err = hp::device_err_flag();
    { const int rc = hp::moe_route_group(rp, s); if (rc) return rc; }
    hp::MoeGroupParams g; g.w_gate_up = exp_gate_up_tiled_dev; g.w_down = exp_down_tiled_dev; g.sh_gate_up = sh_gate_up_tiled_dev; g.sh_down = sh_down_tiled_dev;
    g.E = E; g.F = F; g.nslot = ns; g.T = T; g.e_lo = 0;
    g.xq = hp::XQ8F{(void*)xq_q_dev, (void*)xq_sc_dev}; g.xq2 = hp::XQ8F{ws + w.q2, ws + w.sc2}; g.v = v;
    g.segs = ws + w.segs; g.ctl = (int*)(ws + w.ctl); g.err = hp::device_err_flag();
    { const int rc = hp::moe_experts_grouped(g, s); if (rc) return rc; }
    return hp::moe_combine(v, weights_dev, y_dev, T, ns, E, s);
    HP_GUARD_END
}

// ------------------------------------------------------------------ engine
struct hp_engine { hp::Engine impl; explicit hp_engine(const hp_model_cfg& c) : impl(c) {} };

int hp_model_preset(const char* preset, hp_model_cfg* o) {
    HP_GUARD_BEGIN
    HP_REQUIRE(preset && o, "hp_model_preset: null pointer");
    memset(o, 0, sizeof *o);
    o->ep_rank = 0; o->ep_world = 1;
    o->rms_eps = 1e-6f; o->rope_base = 1e7f; o->n_rot = 64; o->attn_every = 4; o->has_mtp = 1; o->n_slots = 1;
    if (!strcmp(preset, "qwen35-27b")) {          // struct Qwen35Dims, engine/src/qwen35.h:15-26
        o->n_embd = 5120; o->n_layer = 64; o->n_ff = 17408; o->n_vocab = 248320; o->n_head = 24; o->n_head_kv = 4;
        o->gdn_qk_heads = 16; o->gdn_v_heads = 48; o->max_ctx = 8192; o->seed = 27;
    } else if (!strcmp(preset, "flash-next")) {   // benchmark configuration 4 shape (head geometry from struct FnDims, qwen4exp.h:18-28)
        o->n_embd = 2048; o->n_layer = 48; o->n_ff = 0; o->n_vocab = 248320; o->n_head = 24; o->n_head_kv = 2;
        o->gdn_qk_heads = 16; o->gdn_v_heads = 48; o->max_ctx = 4096; o->n_slots = 8; o->seed = 48;
        o->n_expert = 512; o->n_expert_used = 10; o->expert_ff = 512; o->gdn_sigmoid_gate = 1; o->synth_router_logits = 1;
    } else if (!strcmp(preset, "tiny")) {
        o->n_embd = 512; o->n_layer = 4; o->n_ff = 1024; o->n_vocab = 2048; o->n_head = 4; o->n_head_kv = 2;
        o->gdn_qk_heads = 2; o->gdn_v_heads = 4; o->max_ctx = 512; o->n_slots = 2; o->seed = 7;
    } else if (!strcmp(preset, "tiny-moe")) {
        o->n_embd = 512; o->n_layer = 4; o->n_ff = 0; o->n_vocab = 2048; o->n_head = 4; o->n_head_kv = 2;
        o->gdn_qk_heads = 2; o->gdn_v_heads = 4; o->max_ctx = 512; o->n_slots = 4; o->seed = 9;
        o->n_expert = 16; o->n_expert_used = 4; o->expert_ff = 256; o->gdn_sigmoid_gate = 1;
    } else { hp::set_error("unknown preset '%s'", preset); return HP_EINVAL; }
    return HP_OK;
    HP_GUARD_END
}
int hp_load(const hp_model_cfg* cfg, hp_engine** out) {
    HP_GUARD_BEGIN
    HP_REQUIRE(cfg && out, "hp_load: null pointer");
    hp_engine* e = new hp_engine(*cfg);
    const int rc = e->impl.init();
    if (rc != HP_OK) { delete e; *out = nullptr; return rc; }
    *out = e; return HP_OK;
    HP_GUARD_END
}
int hp_free(hp_engine* e) { delete e; return HP_OK; }
int hp_n_slots(const hp_engine* e) { return e ? e->impl.cfg().n_slots : 0; }
size_t hp_weight_bytes(const hp_engine* e) { return e ? e->impl.weight_bytes() : 0; }
float hp_last_ms(const hp_engine* e) { return e ? e->impl.last_ms() : 0.f; }
#define HP_ENGINE_CALL(expr) HP_GUARD_BEGIN HP_REQUIRE(e, "null engine handle"); return (expr); HP_GUARD_END
int hp_reset(hp_engine* e) { HP_ENGINE_CALL(e->impl.reset()) }
int hp_reset_slot(hp_engine* e, int slot) { HP_ENGINE_CALL(e->impl.reset_slot(slot)) }
int hp_forward(hp_engine* e, const hp_slot_req* reqs, int S, float* ms_out) { HP_ENGINE_CALL(e->impl.forward(reqs, S, ms_out)) }
int hp_accept(hp_engine* e, int slot, int m) { HP_ENGINE_CALL(e->impl.accept(slot, m)) }
int hp_mtp_forward(hp_engine* e, int slot, const int* tokens_host, const float* h_dev, int T, int pos0) { HP_ENGINE_CALL(e->impl.mtp_forward(tokens_host, h_dev, T, pos0, slot, true)) }
int hp_topk(hp_engine* e, int which, int T, int k, int* ids_host, float* vals_host) { HP_ENGINE_CALL(e->impl.topk(which, T, k, ids_host, vals_host)) }
int hp_prefill(hp_engine* e, int slot, const int* tokens_host, int n, int pos0, int with_mtp) { HP_ENGINE_CALL(e->impl.prefill(slot, tokens_host, n, pos0, with_mtp)) }
const float* hp_logits_dev(const hp_engine* e) { return e ? e->impl.logits() : nullptr; }
const float* hp_h_nextn_dev(const hp_engine* e) { return e ? e->impl.h_nextn() : nullptr; }
const float* hp_mtp_logits_dev(const hp_engine* e) { return e ? e->impl.mtp_logits() : nullptr; }
const float* hp_mtp_h_dev(const hp_engine* e) { return e ? e->impl.mtp_h() : nullptr; }
int hp_tensor_dev(const hp_engine* e, int layer, int kind, void** ptr_out, size_t* bytes_out) {
    HP_GUARD_BEGIN HP_REQUIRE(e && ptr_out && bytes_out, "hp_tensor_dev: null pointer"); return e->impl.tensor(layer, kind, ptr_out, bytes_out); HP_GUARD_END
}
int hp_gdn_state_dev(hp_engine* e, int slot, int gdn_layer, float** ptr_out, size_t* bytes_out) {
    HP_GUARD_BEGIN HP_REQUIRE(e && ptr_out && bytes_out, "hp_gdn_state_dev: null pointer"); return e->impl.gdn_state(slot, gdn_layer, ptr_out, bytes_out); HP_GUARD_END
}
int hp_mtp_forward_slots(hp_engine* e, const hp_slot_req* reqs, int S, const float* h_dev) { HP_ENGINE_CALL(e->impl.mtp_forward_reqs(reqs, S, h_dev, true)) }
int hp_ep_unique_id(void* id128_out) { HP_GUARD_BEGIN HP_REQUIRE(id128_out, "hp_ep_unique_id: null pointer"); return hp::Engine::ep_unique_id(id128_out); HP_GUARD_END }
int hp_ep_init(hp_engine* e, const void* id128) { HP_GUARD_BEGIN HP_REQUIRE(e && id128, "hp_ep_init: null pointer"); return e->impl.ep_init(id128); HP_GUARD_END }
int hp_profile_pass(hp_engine* e, int R, int what, int reps, float* ms_out) { HP_ENGINE_CALL(e->impl.profile_pass(R, what, reps, ms_out)) }
int hp_moe_touched(hp_engine* e, unsigned long long* n_out) { HP_ENGINE_CALL(e->impl.moe_touched(n_out)) }
int hp_ep_exchange_us(hp_engine* e, int R, int reps, float* us_out) { HP_ENGINE_CALL(e->impl.ep_exchange_us(R, reps, us_out)) }
int hp_ep_peer(hp_engine* e) { return e && e->impl.ep_peer() ? 1 : 0; }
int hp_ep_owner(int expert, int n_expert, int world) { return hp::ep_owner_of(expert, n_expert, world); }
int hp_ep_wait_probe(const void* flags_dev, int world, int rank, unsigned expect, void* stream) {
    HP_GUARD_BEGIN
    int* f = hp::device_err_flag();
    if (!f) { hp::set_error("cannot allocate the device status word"); return HP_ENOMEM; }
    return hp::ep_wait_probe((const unsigned*)flags_dev, world, rank, expect, f, (cudaStream_t)stream);
    HP_GUARD_END
}
int hp_last_round_kernels(const hp_engine* e) { return e ? e->impl.last_round_kernels() : 0; }
size_t hp_pass_weight_bytes(const hp_engine* e, int mtp, int with_head) { return e ? e->impl.pass_weight_bytes(mtp != 0, with_head != 0) : 0; }
int hp_spec_begin(hp_engine* e, int slot, int id_last, int pos, const float* h_pending_dev) { HP_ENGINE_CALL(e->impl.spec_begin(slot, id_last, pos, h_pending_dev)) }
int hp_spec_round(hp_engine* e, const int* slot_ids_host, int S, int n_draft, const int* subst_host, int* out_tokens_host, int* out_counts_host) {
    HP_ENGINE_CALL(e->impl.spec_round(slot_ids_host, S, n_draft, subst_host, out_tokens_host, out_counts_host))
}
int hp_ep_wait_poll(int (*stream_query)(void*), int (*comm_error)(void*), void* ctx, int limit_ms) {
    HP_GUARD_BEGIN return hp::ep_wait_poll(stream_query, comm_error, ctx, limit_ms); HP_GUARD_END
}

}  // extern "C"
