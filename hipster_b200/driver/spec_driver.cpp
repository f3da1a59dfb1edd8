// spec_driver [preset] [n_gen] [n_draft] [prompt_len] [accept_rate_percent] [slots] : greedy generation with MTP speculative
// decoding through the C ABI alone (this file includes include/hipster_b200.h and links libhipster_b200.so, nothing else).
//
// It plays the part of the reference's MTP driver (engine/bench/spec27b.cpp:34-110) for this library: the plain T = 1
// greedy stream first, then the same prefix continued (a) by the host-driven draft / verify / accept / catch-up loop over
// hp_mtp_forward, hp_forward, hp_topk and hp_accept, and (b) by the fused device-side round hp_spec_round. Contract, as in
// the reference: both speculative streams must equal the plain stream token for token. Prints EXACT or MISMATCH and
// exits 0 or 1. Weights are the library's seeded random-init tensors and the prompt is a seeded token sequence (no
// checkpoint, no dataset). accept_rate_percent >= 0 replaces each draft of the fused rounds by the plain stream's own
// next token with that probability and by a different token otherwise (seeded acceptance control); -1 keeps the drafts.
// slots > 1 adds the multi-slot contract of engine/bench/batchfn.cpp:96-131: that many sequences with distinct prompts
// advance in lock step through hp_spec_round over all slots, and each slot's stream must equal its solo run.
#include "hipster_b200.h"
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

static double now_ms() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
#define CK(x) do { const int rc_ = (x); if (rc_ != HP_OK) { fprintf(stderr, "%s failed (%d): %s\n", #x, rc_, hp_last_error()); return 2; } } while (0)
struct Lcg { unsigned long long s; unsigned next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (unsigned)(s >> 33); } };

int main(int argc, char** argv) {
    const char* preset = argc > 1 ? argv[1] : "tiny";
    const int n_gen = argc > 2 ? atoi(argv[2]) : 48, n_draft = argc > 3 ? atoi(argv[3]) : 3, n_prompt = argc > 4 ? atoi(argv[4]) : 21;
    const int rate = argc > 5 ? atoi(argv[5]) : 70, n_slots = argc > 6 ? atoi(argv[6]) : 1;
    if (n_gen < 1 || n_draft < 1 || n_draft > 7 || n_prompt < 1) { fprintf(stderr, "usage: %s [preset] [n_gen] [n_draft 1..7] [prompt_len] [accept_rate_percent]\n", argv[0]); return 2; }
    hp_model_cfg cfg; CK(hp_model_preset(preset, &cfg));
    if (n_slots < 1 || n_slots > 8 || n_slots * (n_draft + 1) > 32) { fprintf(stderr, "slots must be 1..8 with slots * (n_draft + 1) <= 32\n"); return 2; }
    cfg.n_slots = n_slots;
    if (n_prompt + n_gen + 3 * n_draft + 8 > cfg.max_ctx) { fprintf(stderr, "prompt + generation exceed max_ctx %d\n", cfg.max_ctx); return 2; }
    hp_engine* m = nullptr; CK(hp_load(&cfg, &m));
    const int E = cfg.n_embd;
    Lcg rng{1234};
    std::vector<int> prompt(n_prompt); for (int& t : prompt) t = (int)(rng.next() % (unsigned)cfg.n_vocab);
    int ids[64]; float vals[64];

    // ---- plain greedy (T = 1) ----
    const int n_plain = n_gen + n_draft + 2;
    std::vector<int> plain; std::vector<float> gap;
    { CK(hp_reset(m)); CK(hp_prefill(m, 0, prompt.data(), n_prompt, 0, 0));
      CK(hp_topk(m, 0, 1, 1, ids, vals)); int cur = ids[0], pos = n_prompt;
      const double t0 = now_ms();
      for (int i = 0; i < n_plain; ++i) {
          plain.push_back(cur);
          hp_slot_req r{0, &cur, 1, pos++}; CK(hp_forward(m, &r, 1, nullptr)); CK(hp_accept(m, 0, 1));
          CK(hp_topk(m, 0, 1, 2, ids, vals)); cur = ids[0]; gap.push_back(vals[0] - vals[1]);
      }
      const double dt = now_ms() - t0;
      printf("plain greedy: %d tokens in %.1f ms = %.1f t/s\n", n_plain, dt, n_plain * 1000.0 / dt); }

    // ---- MTP speculative greedy, host-driven (the reference's loop) ----
    std::vector<int> spec;
    { CK(hp_reset(m)); CK(hp_prefill(m, 0, prompt.data(), n_prompt, 0, 1));
      CK(hp_topk(m, 0, 1, 1, ids, vals)); int id_last = ids[0], pos = n_prompt; spec.push_back(id_last);
      const float* h_pending = hp_h_nextn_dev(m);   // row 0 = the last prompt row; rows of this buffer stay valid until the next trunk pass
      int rounds = 0, accepted = 0;
      const double t0 = now_ms();
      while ((int)spec.size() < n_gen) {
          std::vector<int> drafts; int tok = id_last; const float* h = h_pending;
          for (int i = 0; i < n_draft; ++i) {   // draft with the MTP block, chained on its own hidden row
              CK(hp_mtp_forward(m, 0, &tok, h, 1, pos + i));
              CK(hp_topk(m, 1, 1, 1, ids, vals)); tok = ids[0]; drafts.push_back(tok); h = hp_mtp_h_dev(m);
          }
          std::vector<int> batch{id_last}; batch.insert(batch.end(), drafts.begin(), drafts.end());
          hp_slot_req r{0, batch.data(), (int)batch.size(), pos}; CK(hp_forward(m, &r, 1, nullptr));
          CK(hp_topk(m, 0, n_draft + 1, 1, ids, vals));
          int mm = 0; while (mm < n_draft && ids[mm] == drafts[mm]) ++mm;
          CK(hp_accept(m, 0, mm + 1));
          for (int i = 0; i < mm; ++i) spec.push_back(drafts[i]);
          const int bonus = ids[mm]; spec.push_back(bonus);
          if (mm > 0) CK(hp_mtp_forward(m, 0, drafts.data(), hp_h_nextn_dev(m), mm, pos + 1));   // catch-up with the target's hidden rows
          h_pending = hp_h_nextn_dev(m) + (size_t)mm * E;
          id_last = bonus; pos += mm + 1; ++rounds; accepted += mm;
      }
      const double dt = now_ms() - t0;
      printf("mtp n=%d host loop: %d tokens in %.1f ms = %.1f t/s | %d rounds, %.2f tokens/round\n", n_draft, (int)spec.size(), dt, spec.size() * 1000.0 / dt, rounds, (double)(accepted + rounds) / rounds); }

    // ---- the fused device-side round ----
    std::vector<int> fused;
    { CK(hp_reset(m)); CK(hp_prefill(m, 0, prompt.data(), n_prompt, 0, 1));
      CK(hp_topk(m, 0, 1, 1, ids, vals)); fused.push_back(ids[0]);
      CK(hp_spec_begin(m, 0, ids[0], n_prompt, hp_h_nextn_dev(m)));
      Lcg sr{99}; int rounds = 0; const int slot = 0;
      const double t0 = now_ms();
      while ((int)fused.size() < n_gen) {
          int sub[8], out[8], cnt = 0;
          for (int i = 0; i < n_draft; ++i) {
              const size_t k = fused.size() + i;   // index in `plain` of the token this draft predicts
              if (rate < 0 || k >= plain.size()) { sub[i] = -1; continue; }
              sub[i] = (int)(sr.next() % 100u) < rate ? plain[k] : (plain[k] + 1) % cfg.n_vocab;
          }
          CK(hp_spec_round(m, &slot, 1, n_draft, sub, out, &cnt));
          for (int i = 0; i < cnt; ++i) fused.push_back(out[i]);
          ++rounds;
      }
      const double dt = now_ms() - t0;
      printf("mtp n=%d fused round: %d tokens in %.1f ms = %.1f t/s | %d rounds, %.2f tokens/round\n", n_draft, (int)fused.size(), dt, fused.size() * 1000.0 / dt, rounds, (double)(fused.size() - 1) / rounds); }

    int bad = 0;
    for (int pass = 0; pass < 2; ++pass) {
        const std::vector<int>& s = pass ? fused : spec; int match = 0;
        for (int i = 0; i < n_gen; ++i) {
            if (plain[i] == s[i]) { ++match; continue; }
            printf("%s: first divergence at %d: plain %d, speculative %d; plain top1 - top2 gap at the step that produced it: %.4f\n", pass ? "fused" : "host loop", i, plain[i], s[i], i > 0 ? gap[i - 1] : 0.f);
            break;
        }
        printf("%s %s: %d/%d tokens identical to plain greedy\n", match == n_gen ? "EXACT" : "MISMATCH", pass ? "(fused round)" : "(host loop)", match, n_gen);
        bad |= match != n_gen;
    }
    // ---- S slots in lock step vs each slot alone (the drafts are the MTP block's own: no substitution)
    if (n_slots > 1) {
        const int S = n_slots, rounds = (n_gen + n_draft) / (n_draft + 1);
        std::vector<std::vector<int>> prompts(S), lock(S), solo(S);
        for (int s = 0; s < S; ++s) { Lcg pr{5000ull + (unsigned)s}; prompts[s].resize(n_prompt - (s % 3)); for (int& t : prompts[s]) t = (int)(pr.next() % (unsigned)cfg.n_vocab); }
        auto begin = [&](int s) -> int {
            if (hp_prefill(m, s, prompts[s].data(), (int)prompts[s].size(), 0, 1)) return 1;
            if (hp_topk(m, 0, 1, 1, ids, vals)) return 1;
            return hp_spec_begin(m, s, ids[0], (int)prompts[s].size(), hp_h_nextn_dev(m));
        };
        CK(hp_reset(m));
        std::vector<int> slots(S), out(S * (n_draft + 1)), cnt(S);
        for (int s = 0; s < S; ++s) { slots[s] = s; CK(begin(s)); }
        const double t0 = now_ms(); size_t total = 0;
        for (int r = 0; r < rounds; ++r) {
            CK(hp_spec_round(m, slots.data(), S, n_draft, nullptr, out.data(), cnt.data()));
            for (int s = 0; s < S; ++s) { lock[s].insert(lock[s].end(), out.begin() + s * (n_draft + 1), out.begin() + s * (n_draft + 1) + cnt[s]); total += cnt[s]; }
        }
        const double dt = now_ms() - t0;
        printf("mtp n=%d, %d slots in lock step: %zu tokens in %.1f ms = %.1f t/s aggregate\n", n_draft, S, total, dt, total * 1000.0 / dt);
        int same = 0;
        for (int s = 0; s < S; ++s) {
            CK(hp_reset(m)); CK(begin(s));
            for (int r = 0; r < rounds; ++r) {
                int c1 = 0; CK(hp_spec_round(m, &s, 1, n_draft, nullptr, out.data(), &c1));
                solo[s].insert(solo[s].end(), out.begin(), out.begin() + c1);
            }
            same += solo[s] == lock[s];
        }
        printf("%s (slots): %d/%d slot streams identical to their solo runs\n", same == S ? "EXACT" : "MISMATCH", same, S);
        bad |= same != S;
    }
    hp_free(m);
    return bad ? 1 : 0;
}
