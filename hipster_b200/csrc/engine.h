// Host engine of the MTP speculative-decode path: weight arena (random-init, generated on device from a seed),
// per-slot recurrent state and KV caches, the verify / decode pass, the MTP draft block, accept with deferred commit,
// and the fused device-side speculative round. C++ inside the library; exported through the C ABI in capi.cu.
//
// Reference: class Qwen35 (engine/src/qwen35.h:50-149, qwen35.cpp) and class Qwen4Exp (engine/src/qwen4exp.h:54-90).
#pragma once
#include "kernels.h"
#include "../../include/hipster_b200.h"
#include <vector>
#include <string>
#include <cstdlib>

namespace hp {

struct Lin { uint8_t* w = nullptr; uint8_t* wt = nullptr; int N = 0, K = 0, P = 1; size_t bytes = 0; };   // merged Q4_K matrix [N][K/256 blocks]; wt = tile-major copy

struct LayerW {
    bool is_attn = false;
    uint16_t *attn_norm = nullptr, *post_norm = nullptr;          // bf16 [E]
    Lin in_proj;      // GDN: qkv | z | beta | alpha rows; attention: q_full | k | v rows
    Lin out_proj;     // GDN: ssm_out; attention: wo
    Lin gate_up, down;                                            // dense FFN (gate rows then up rows)
    float* conv_w = nullptr; uint16_t *dt_bias = nullptr, *a_neg = nullptr, *ssm_norm = nullptr;   // GDN
    uint16_t *q_norm = nullptr, *k_norm = nullptr;                // attention
    // MoE (n_expert > 0): router f32 [n_expert + 1][E]; expert matrices contiguous per tensor
    float* router = nullptr; Lin exp_gate_up, exp_down, sh_gate_up, sh_down;
};

enum TensorKind { TK_ATTN_NORM = 0, TK_POST_NORM, TK_IN_PROJ, TK_OUT_PROJ, TK_GATE_UP, TK_DOWN, TK_CONV_W, TK_DT_BIAS, TK_A_NEG, TK_SSM_NORM,
                  TK_Q_NORM, TK_K_NORM, TK_ROUTER, TK_EXP_GATE_UP, TK_EXP_DOWN, TK_SH_GATE_UP, TK_SH_DOWN,
                  TK_EMBED = 32, TK_OUTPUT_NORM, TK_LM_HEAD, TK_MTP_ENORM, TK_MTP_HNORM, TK_MTP_EH_PROJ, TK_MTP_HEAD_NORM };

class Engine {
public:
    static constexpr int MAXR = 32, MAXS = 8;
    explicit Engine(const hp_model_cfg& cfg);
    ~Engine();
    int init();                                              // allocate + generate weights; HP_* status
    int forward(const hp_slot_req* reqs, int S, float* ms);  // Qwen35::forward(const SlotReq*, int) (qwen35.h:62)
    int accept(int slot, int m);                             // Qwen35::accept (qwen35.h:66)
    int mtp_forward(const int* tokens, const float* h_dev, int T, int pos0, int slot, bool want_logits);   // qwen35.h:70
    int mtp_forward_reqs(const hp_slot_req* reqs, int S, const float* h_dev, bool want_logits);   // qwen4exp.h:66-70
    static int ep_unique_id(void* id128); int ep_init(const void* id128);
    int topk(int which, int T, int k, int* ids, float* vals);   // Qwen35::topk (qwen35.h:87): ids / vals [T][k] on the host
    int prefill(int slot, const int* tokens, int n, int pos0, int with_mtp);   // Qwen4Exp::prefill + mtp_catchup (qwen4exp.h:57-60,72-74)
    int reset(); int reset_slot(int slot);
    int flush_commits();                                     // apply every pending accept to the stored state
    int tensor(int layer, int kind, void** ptr, size_t* bytes) const;
    int gdn_state(int slot, int gdn_layer, float** ptr, size_t* bytes);
    int spec_begin(int slot, int id_last, int pos, const float* h_pending_dev);
    int spec_round(const int* slots, int S, int n_draft, const int* subst_host, int* out_tokens, int* out_counts);
    const hp_model_cfg& cfg() const { return c_; }
    float* logits() const { return logits_; } float* h_nextn() const { return h_; }
    float* mtp_logits() const { return mlogits_; } float* mtp_h() const { return mh_; }
    size_t weight_bytes() const { return weight_bytes_; } float last_ms() const { return last_ms_; }
    size_t pass_weight_bytes(bool mtp, bool with_head) const;
    int moe_touched(unsigned long long* n);                 // touched (layer, expert) matrices since the last call (measurement)
    int ep_exchange_us(int R, int reps, float* us);          // mean device time of one exchange for R rows (measurement)
    bool ep_peer() const { return ep_peer_; }
    int last_round_kernels() const { return last_round_kernels_; }
    int profile_pass(int R, int what, int reps, float* ms);
private:
    struct Desc;   // device-visible pass descriptor (see engine.cu)
    int alloc(void** p, size_t bytes);
    int gen_lin(Lin& l, int N, int K, uint64_t tid);
    int gen_raw_q4k(Lin& l, size_t rows, int K, uint64_t tid, size_t row0 = 0, size_t nrows_local = (size_t)-1, int interleave_half = 0);
    int gen_bf16(uint16_t** p, size_t n, uint64_t tid, float mean, float std, bool neg_abs = false);
    int gen_f32(float** p, size_t n, uint64_t tid, float mean, float std, bool neg_abs);
    int lin(const Lin& l, float* out, int ld, int R);        // GEMV; P > 1 planes are reduced into out
    int lin_parts(const Lin& l, int R);                      // GEMV into the plane buffer yparts_ (consumer adds the planes)
    int norm_in(const Lin* prev, bool have_y, const uint16_t* w, float* xn, int R);
    int attn_block(const LayerW& L, uint16_t* kc, uint16_t* vc, size_t kv_stride, int R, int ngroups, bool kv_only = false);
    int ffn_block(const LayerW& L, int R);
    int moe_block(const LayerW& L, int R);
    int ep_exchange(float* buf, size_t n);
    int ep_allreduce(float* buf, size_t n);
    int run_pass(int R, int nseq, int ngroups);              // trunk over the rows described by desc_ (already uploaded)
    int run_mtp(int R, int ngroups, const float* h_dev, int ldh, bool want_logits, bool kv_only = false);
    int upload_desc();
    int enqueue_round(int S, int n);
    int attn_rows_per_group() const;
    int check_device_status();
    int ep_ready();
    void ep_destroy();
    int sync_stream();                                       // wait for the engine's stream (bounded polling when collectives are in flight)
    int fill_desc(const hp_slot_req* reqs, int S, int* rows, int* ngroups, bool with_seqs);
    int nattn() const; int ngdn() const;
    hp_model_cfg c_;
    std::vector<LayerW> layers_; LayerW mtp_;
    uint16_t *embed_ = nullptr, *output_norm_ = nullptr, *mtp_enorm_ = nullptr, *mtp_hnorm_ = nullptr, *mtp_head_norm_ = nullptr;
    Lin lm_head_, eh_proj_;
    float* rope_ = nullptr;
    // state
    float *gdn_state_ = nullptr, *conv_state_ = nullptr; size_t st_stride_ = 0, cs_stride_ = 0, st_layer_ = 0, cs_layer_ = 0;
    uint16_t *kc_ = nullptr, *vc_ = nullptr, *mkc_ = nullptr, *mvc_ = nullptr; size_t kv_slot_ = 0, kv_layer_ = 0;
    float* saved_ = nullptr; size_t sv_layer_ = 0, sv_stride_ = 0; int ld_in_ = 0;   // raw GDN inputs of the last pass (for the deferred commit)
    int* replay_n_ = nullptr; std::vector<int> pend_, last_r0_, last_T_;
    // work
    float *x_ = nullptr, *xn_ = nullptr, *big_ = nullptr, *yparts_ = nullptr, *logits_ = nullptr, *mlogits_ = nullptr, *h_ = nullptr, *mh_ = nullptr, *emb_ = nullptr;
    float *pO_ = nullptr, *pm_ = nullptr, *pl_ = nullptr; int nsplit_max_ = 0;
    XQ8F xq_{nullptr, nullptr}, xq2_{nullptr, nullptr};
    float *rlogits_ = nullptr, *moe_w_ = nullptr, *moe_v_ = nullptr; void* moe_segs_ = nullptr; int* moe_ctl_ = nullptr; unsigned long long* moe_touched_ = nullptr; int* moe_ids_ = nullptr; int* route_cnt_ = nullptr; Lin moe_out_;
    int e_lo_ = 0, e_hi_ = 0, ep_world_ = 1; void* nccl_comm_ = nullptr; bool ep_failed_ = false;
    // Peer-memory form of the expert-parallel exchange (one process per GPU, buffers mapped through CUDA IPC): every rank
    // pushes the output rows of the experts it owns into the other ranks' exchange buffers and raises a flag there.
    bool ep_peer_ = false;
    float* ep_xbuf_ = nullptr; size_t ep_half_ = 0;             // own exchange buffer: two halves of MAXR * slots * E floats, used in turn
    unsigned* ep_ctl_ = nullptr;                                // own words: [q] = last exchange rank q has delivered, [8] = exchanges done, [9] = ticket
    float* ep_peer_x_[8] = {}; unsigned* ep_peer_ctl_[8] = {};  // the ranks' buffers as mapped here (own rank: the own pointers)
    int ep_peer_setup(); void ep_peer_teardown();
    int ep_exchange_peer(int R, int sh_owner, bool pushed);
    int *d_desc_ = nullptr, *h_desc_ = nullptr;                  // device / pinned host descriptor
    int *d_ids_ = nullptr, *d_mids_ = nullptr; float *d_vals_ = nullptr, *d_mvals_ = nullptr; void* am_scratch_ = nullptr;
    int *d_spec_ = nullptr, *h_spec_ = nullptr;                   // fused round state (device) / results (pinned host)
    int* d_specin_ = nullptr;                                     // the round's inputs: slot list, seeded substitutions
    float *hpend_ = nullptr, *hstage_ = nullptr, *hprev_ = nullptr;   // per-slot pending h rows; gathered MTP inputs; per-slot last prompt h (prefill catch-up)
    std::vector<int> spec_pos_, spec_on_;
    void* topk_scratch_ = nullptr; int *d_topk_ids_ = nullptr; float* d_topk_vals_ = nullptr;
    uint16_t* prof_kv_ = nullptr;                                 // K/V rows saved around profile_pass
    // a round that carries collectives: the stretches between two exchanges as graphs, the exchanges enqueued by the host
    struct EpSeg { cudaGraphExec_t g; float* buf; size_t n; };
    std::vector<EpSeg> ep_segs_[64]; std::vector<EpSeg>* seg_out_ = nullptr;
    int capture_segments(int key, int S, int n);
    cudaGraphExec_t graphs_[64] = {}; bool warmed_[64] = {}; int graph_kernels_[64] = {}; int last_round_kernels_ = 0;
    int* err_ = nullptr;
    cudaStream_t s_ = nullptr; cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    std::vector<void*> allocs_;
    size_t weight_bytes_ = 0; float last_ms_ = 0;
    int prof_skip_ = 0; bool gemv_only_ = false, tiled_ = true, keep_rowmajor_ = true; bool pdl_ = getenv("HIPSTER_B200_NO_PDL") == nullptr;
};

int ep_wait_poll(int (*stream_query)(void*), int (*comm_error)(void*), void* ctx, int limit_ms);
int ep_wait_probe(const unsigned* flags_dev, int world, int rank, unsigned expect, int* err, cudaStream_t s);
// rank that holds routed expert `id` when n_expert experts are cut into `world` contiguous shards [r * n / world,
// (r + 1) * n / world); -1 for an id outside [0, n_expert)
__host__ __device__ inline int ep_owner_of(int id, int n_expert, int world) {
    if (id < 0 || id >= n_expert || world < 1) return -1;
    return (int)(((long long)(id + 1) * world - 1) / n_expert);
}

}  // namespace hp
