"""The CUDA engine against the CPU restatement at the BENCHMARK widths (no reduced shapes except depth):

* configuration 3 widths (hidden 5120, FFN 17408, 24/4 heads, GDN 16/48 x 128, vocabulary 248320) cut to 4 layers, with a
  context beyond one attention split: verify logits, h_nextn, recurrent state, accept(m) followed by one more pass, the
  MTP block, and one fused device-side round;
* configuration 5: the Flash-Next-shaped MoE model (512 experts top-10 + shared, hidden 2048) cut to 4 layers, 8 slots x 3
  verify rows in one pass equal to each slot's solo run and to the oracle, and one lock-step fused MTP round over the 8
  slots equal to the solo rounds (engine/bench/batchfn.cpp:128-131).
Everything is compared bit for bit."""
import numpy as np
import pytest

import hipster_b200 as hb
from oracle import orc

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def orc_prefill(ref, slot, prompt, with_mtp, E):
    """hp_prefill restated on the oracle model: 8-row chunks, MTP row p paired with the trunk's hidden row of p - 1."""
    prev = np.zeros(E, dtype=np.float32); T = 0
    for p in range(0, len(prompt), 8):
        toks = prompt[p:p + 8]; T = len(toks)
        ref.forward([(slot, toks, p)]); ref.accept(slot, T)
        h = ref.h_nextn(T)
        if with_mtp:
            hin = np.vstack([prev[None, :], h[:T - 1]]) if T > 1 else prev[None, :].copy()
            ref.mtp_forward(slot, toks, hin, p)
        prev = h[T - 1].copy()
    return T


@pytest.fixture(scope="module")
def dense4():
    cfg = hb.ModelCfg.preset("qwen35-27b", n_layer=4, max_ctx=512, n_slots=1)
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    yield cfg, eng, ref
    eng.close()


def test_dense27b_widths_context_beyond_one_split(dense4):
    cfg, eng, ref = dense4
    E = cfg.n_embd
    prompt = [int(x) for x in np.random.default_rng(27).integers(0, cfg.n_vocab, size=133)]   # 133 > 128: two key splits
    eng.reset(); ref.reset()
    eng.prefill(0, prompt, with_mtp=True)
    T_last = orc_prefill(ref, 0, prompt, True, E)
    assert np.array_equal(bits(eng.logits(1)[0]), bits(ref.logits(T_last)[T_last - 1]))
    assert np.array_equal(bits(eng.h_nextn(1)[0]), bits(ref.h_nextn(T_last)[T_last - 1]))
    pos = len(prompt)
    rows = [int(x) for x in np.random.default_rng(3).integers(0, cfg.n_vocab, size=6)]
    for e in (eng, ref):
        e.forward([(0, rows, pos)])
    assert np.isfinite(ref.logits(6)).all()                                   # random-init weights must not blow the model up
    assert np.array_equal(bits(eng.logits(6)), bits(ref.logits(6)))           # P = 4 K parts of `down`, 248320-row LM head
    assert np.array_equal(bits(eng.h_nextn(6)), bits(ref.h_nextn(6)))
    ids, vals = eng.topk(0, 6, k=5)
    oi, ov = orc.topk(ref.logits(6), 5)
    assert np.array_equal(ids, oi) and np.array_equal(bits(vals), bits(ov))
    # the MTP block over 3 (token, h) pairs: 10240-wide norm2_concat, eh_proj, attention with its own cache
    eng.mtp_forward(0, rows[1:4], eng.h_nextn_ptr(), pos + 1)
    ref.mtp_forward(0, rows[1:4], ref.h_nextn(3), pos + 1)
    assert np.array_equal(bits(eng.mtp_logits(3)), bits(ref.mtp_logits(3)))
    assert np.array_equal(bits(eng.mtp_h(3)), bits(ref.mtp_h(3)))
    # accept 3 of the 6 rows (rollback of the recurrent state), then one more pass on top of it
    for e in (eng, ref):
        e.accept(0, 3)
    for gl in range(3):
        assert np.array_equal(bits(eng.gdn_state(0, gl)), bits(ref.gdn_state(0, gl))), gl
    for e in (eng, ref):
        e.forward([(0, [rows[3], 17], pos + 3)])
    assert np.array_equal(bits(eng.logits(2)), bits(ref.logits(2)))


def test_dense27b_widths_fused_round_equals_oracle_host_loop(dense4):
    """One fused device-side round (5 drafts, 6-row verify, accept, catch-up) against the same round driven step by step
    on the CPU model (engine/bench/spec27b.cpp:77-103)."""
    cfg, eng, ref = dense4
    E, n = cfg.n_embd, 5
    prompt = [int(x) for x in np.random.default_rng(5).integers(0, cfg.n_vocab, size=19)]
    eng.reset(); ref.reset()
    eng.prefill(0, prompt, with_mtp=True)
    T_last = orc_prefill(ref, 0, prompt, True, E)
    id_last = int(eng.topk(0, 1)[0][0]); pos = len(prompt)
    assert id_last == int(orc.argmax(ref.logits(T_last))[0][T_last - 1])
    eng.spec_begin(0, id_last, pos, eng.h_nextn_ptr())
    h_pending = ref.h_nextn(T_last)[T_last - 1].copy()
    for rnd in range(2):
        # oracle: draft
        tok, h, drafts = id_last, h_pending[None, :], []
        for i in range(n):
            ref.mtp_forward(0, [tok], h, pos + i)
            tok = int(orc.argmax(ref.mtp_logits(1))[0][0]); drafts.append(tok); h = ref.mtp_h(1)
        if rnd == 1:
            drafts[2] = (drafts[2] + 1) % cfg.n_vocab       # a forced rejection in the middle
        ref.forward([(0, [id_last] + drafts, pos)])
        ids = orc.argmax(ref.logits(n + 1))[0]
        mm = 0
        while mm < n and ids[mm] == drafts[mm]:
            mm += 1
        ref.accept(0, mm + 1)
        want = drafts[:mm] + [int(ids[mm])]
        hn = ref.h_nextn(n + 1)
        if mm > 0:
            ref.mtp_forward(0, drafts[:mm], hn[:mm], pos + 1)
        h_pending = hn[mm].copy()
        got = eng.spec_round(0, n, subst=[-1, -1, drafts[2], -1, -1] if rnd == 1 else None)
        assert got == want, (rnd, got, want)
        id_last = want[-1]; pos += mm + 1
    for gl in range(3):
        assert np.array_equal(bits(eng.gdn_state(0, gl)), bits(ref.gdn_state(0, gl))), gl


@pytest.fixture(scope="module")
def moe4():
    cfg = hb.ModelCfg.preset("flash-next", n_layer=4, max_ctx=256, n_slots=8)
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    yield cfg, eng, ref
    eng.close()


def test_config5_pass_24_rows_equals_solo_and_oracle(moe4):
    cfg, eng, ref = moe4
    S, n = 8, 2
    prompts = [[int(x) for x in np.random.default_rng(100 + s).integers(0, cfg.n_vocab, size=9 + s)] for s in range(S)]
    rows = [[int(x) for x in np.random.default_rng(200 + s).integers(0, cfg.n_vocab, size=n + 1)] for s in range(S)]
    eng.reset()
    for s in range(S):
        eng.prefill(s, prompts[s], with_mtp=False)
    eng.forward([(s, rows[s], len(prompts[s])) for s in range(S)])            # 8 slots x 3 rows = 24 rows, NT = 3 column tiles
    batched = eng.logits(S * (n + 1)).copy(); hb_ = eng.h_nextn(S * (n + 1)).copy()
    assert np.isfinite(batched).all()
    for s in (0, 3, 7):                                                        # solo runs of three slots
        eng.reset_slot(s)
        eng.prefill(s, prompts[s], with_mtp=False)
        eng.forward([(s, rows[s], len(prompts[s]))])
        assert np.array_equal(bits(eng.logits(n + 1)), bits(batched[3 * s:3 * s + 3])), s
    for s in (1, 6):                                                           # and the oracle for two others
        ref.reset()
        orc_prefill(ref, s, prompts[s], False, cfg.n_embd)
        ref.forward([(s, rows[s], len(prompts[s]))])
        assert np.array_equal(bits(ref.logits(n + 1)), bits(batched[3 * s:3 * s + 3])), s
        assert np.array_equal(bits(ref.h_nextn(n + 1)), bits(hb_[3 * s:3 * s + 3])), s


def test_config5_lockstep_fused_round_equals_solo_rounds(moe4):
    cfg, eng, ref = moe4
    S, n, E = 8, 2, cfg.n_embd
    prompts = [[int(x) for x in np.random.default_rng(300 + s).integers(0, cfg.n_vocab, size=7 + 2 * s)] for s in range(S)]
    subs = [[[-1, 5 + s], [7 + s, -1], [-1, -1]][r] for r in range(3) for s in range(S)]   # [round][slot] substitutions
    subs = [subs[r * S:(r + 1) * S] for r in range(3)]

    def start(slots):
        eng.reset()
        for s in slots:
            eng.prefill(s, prompts[s], with_mtp=True)
            eng.spec_begin(s, int(eng.topk(0, 1)[0][0]), len(prompts[s]), eng.h_nextn_ptr())

    start(range(S))
    lock = [[] for _ in range(S)]
    for r in range(3):
        out = eng.spec_round_slots(list(range(S)), n, subs[r])
        for s in range(S):
            lock[s] += out[s]
    for s in (0, 2, 5, 7):
        start([s])
        solo = []
        for r in range(3):
            solo += eng.spec_round(s, n, subs[r][s])
        assert solo == lock[s], (s, solo, lock[s])
