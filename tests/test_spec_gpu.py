"""The fused device-side MTP round (hp_spec_round) against the host-driven loop and the CPU oracle: the speculative
stream must equal the plain greedy stream exactly (engine/bench/spec27b.cpp:108-110), whatever the drafts are."""
import numpy as np
import pytest
import torch

import hipster_b200 as hb
from hipster_b200 import spec
from hipster_b200.engine import _as_tensor
from oracle import orc

pytestmark = pytest.mark.gpu


class GpuAdapter:
    """Engine + device-side construction of the shifted h rows needed by the MTP prompt catch-up."""

    def __init__(self, eng):
        self.e = eng; self.E = eng.cfg.n_embd
        self.buf = torch.zeros((8, self.E), dtype=torch.float32, device="cuda")
        self.h = _as_tensor(eng.h_nextn_ptr(), 32 * self.E * 4).view(torch.float32).view(32, self.E)

    def __getattr__(self, k):
        return getattr(self.e, k)

    def h_shift(self, prev, T):
        torch.cuda.synchronize()
        self.buf[0] = prev if prev is not None else 0
        if T > 1:
            self.buf[1:T] = self.h[0:T - 1]
        last = self.h[T - 1].clone()
        torch.cuda.synchronize()
        return self.buf.data_ptr(), last


class OrcAdapter:
    def __init__(self, m, cfg):
        self.m = m; self.E = cfg.n_embd; self.T = 1

    def forward(self, reqs):
        self.T = len(reqs[0][1]); self.m.forward(reqs)

    def accept(self, s, m):
        self.m.accept(s, m)

    def mtp_forward(self, slot, toks, h, pos):
        self.m.mtp_forward(slot, toks, h, pos)

    def topk(self, which, T):
        lg = self.m.mtp_logits(T) if which else self.m.logits(self.T)[:T] if T <= self.T else None
        ids, vals = orc.argmax(lg)
        return ids, vals

    def h_shift(self, prev, T):
        h = self.m.h_nextn(T)
        buf = np.zeros((T, self.E), dtype=np.float32)
        if prev is not None:
            buf[0] = prev
        buf[1:T] = h[0:T - 1]
        return buf, h[T - 1].copy()


def last_argmax(a, T):
    return int(a.topk(0, T)[0][T - 1])


@pytest.mark.parametrize("n_draft,rate", [(2, 0.7), (5, 0.7), (3, 0.0), (4, 1.0)])
def test_fused_round_stream_equals_plain_greedy(n_draft, rate):
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg); g = GpuAdapter(eng)
    rng = np.random.default_rng(3)
    prompt = [int(x) for x in rng.integers(0, cfg.n_vocab, size=21)]
    n_gen = 24
    # plain greedy on the GPU engine and on the CPU oracle
    pos = spec.prefill(g, prompt, h_shift=g.h_shift)
    first = last_argmax(g, len(prompt) % 8 or 8)
    plain = [first]
    for i in range(n_gen + n_draft + 1):
        eng.forward([(0, [plain[-1]], pos + i)]); eng.accept(0, 1)
        plain.append(int(eng.topk(0, 1)[0][0]))
    ref = orc.Model(cfg); o = OrcAdapter(ref, cfg)
    opos = spec.prefill(o, prompt, h_shift=o.h_shift)
    oplain = [last_argmax(o, len(prompt) % 8 or 8)]
    for i in range(8):
        o.forward([(0, [oplain[-1]], opos + i)]); o.accept(0, 1)
        oplain.append(last_argmax(o, 1))
    assert oplain == plain[:len(oplain)]
    # fused speculative decode from the same prefix
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift)
    T_last = len(prompt) % 8 or 8
    id_last = last_argmax(g, T_last)
    eng.spec_begin(0, id_last, pos, eng.h_nextn_ptr() + (T_last - 1) * cfg.n_embd * 4)
    out = [id_last]; rounds = 0; accepted = 0
    while len(out) < n_gen:
        sub = spec.seeded_substitutions(plain, len(out), n_draft, rate, rng, cfg.n_vocab)
        got = eng.spec_round(0, n_draft, sub)
        assert 1 <= len(got) <= n_draft + 1
        out += got; rounds += 1; accepted += len(got) - 1
    assert out[:n_gen] == plain[:n_gen]
    if rate == 0.0:
        assert accepted == 0
    if rate == 1.0:
        assert accepted == rounds * n_draft
    # the recurrent state after the fused rounds equals the state of a plain run over the same tokens
    st = [eng.gdn_state(0, gl).copy() for gl in range(3)]
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift)
    for i, t in enumerate(out[:-1]):
        eng.forward([(0, [t], pos + i)]); eng.accept(0, 1)
    for gl in range(3):
        assert np.array_equal(eng.gdn_state(0, gl).view(np.uint32), st[gl].view(np.uint32))
    eng.close()


def test_fused_round_without_substitution_uses_the_mtp_drafts():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg); g = GpuAdapter(eng)
    prompt = list(range(40, 51))
    pos = spec.prefill(g, prompt, h_shift=g.h_shift)
    T_last = len(prompt) % 8 or 8
    id_last = last_argmax(g, T_last)
    eng.spec_begin(0, id_last, pos, eng.h_nextn_ptr() + (T_last - 1) * cfg.n_embd * 4)
    out = [id_last]
    for _ in range(6):
        out += eng.spec_round(0, 3, None)
    # host-driven reference loop (spec27b.cpp:77-103) on a fresh run must give the same stream
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift)
    id_last = last_argmax(g, T_last)
    hp = _as_tensor(eng.h_nextn_ptr(), 32 * cfg.n_embd * 4).view(torch.float32).view(32, cfg.n_embd)
    h_pending = hp[T_last - 1].clone()
    ref_out = [id_last]
    for _ in range(6):
        drafts = []; tok = id_last; hptr = h_pending.data_ptr(); p = pos
        for i in range(3):
            eng.mtp_forward(0, [tok], hptr, p)
            tok = int(eng.topk(1, 1)[0][0]); drafts.append(tok); hptr = eng.mtp_h_ptr(); p += 1
        eng.forward([(0, [id_last] + drafts, pos)])
        ids = eng.topk(0, 4)[0]
        mm = 0
        while mm < 3 and ids[mm] == drafts[mm]:
            mm += 1
        eng.accept(0, mm + 1)
        ref_out += drafts[:mm] + [int(ids[mm])]
        if mm > 0:
            eng.mtp_forward(0, drafts[:mm], eng.h_nextn_ptr(), pos + 1)
        torch.cuda.synchronize()
        h_pending = hp[mm].clone()
        id_last = int(ids[mm]); pos += mm + 1
    assert out == ref_out
    eng.close()
