"""Size-independent properties at the full model sizes of the benchmark configurations (no CPU oracle at these sizes):
the speculative stream equals the plain greedy stream (engine/bench/spec27b.cpp:108-110), a verify row's logits do not
depend on how many rows share the pass (README.md:65 of the reference: "T>1 vs T=1 logits difference 0"), and the
recurrent state after accept(m) equals the state of a run that only ever saw the accepted tokens."""
import numpy as np
import pytest
import torch

import hipster_b200 as hb
from hipster_b200 import spec
from hipster_b200.engine import _as_tensor

pytestmark = pytest.mark.gpu


class Adapter:
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


def logits_rows(eng, T):
    V = eng.cfg.n_vocab
    t = _as_tensor(eng.logits_ptr(), T * V * 4).view(torch.float32).view(T, V)
    torch.cuda.synchronize()
    return t.clone()


@pytest.mark.parametrize("preset,n_draft", [("qwen35-27b", 5), ("flash-next", 2)])
def test_full_size_model_properties(preset, n_draft):
    cfg = hb.ModelCfg.preset(preset, n_slots=1)
    eng = hb.Engine(cfg); g = Adapter(eng)
    rng = np.random.default_rng(11)
    prompt = [int(x) for x in rng.integers(0, cfg.n_vocab, size=133)]      # 133 = 16 passes of 8 + one of 5: crosses a 128-key attention split
    T_last = len(prompt) % 8 or 8
    n_gen = 14

    # plain greedy stream; keep the logits of every single-row pass
    pos = spec.prefill(g, prompt, h_shift=g.h_shift, with_mtp=False)
    plain = [int(eng.topk(0, T_last)[0][T_last - 1])]
    single = []
    for i in range(n_gen + n_draft + 1):
        eng.forward([(0, [plain[-1]], pos + i)]); eng.accept(0, 1)
        single.append(logits_rows(eng, 1)[0])
        plain.append(int(eng.topk(0, 1)[0][0]))

    # the same tokens as one 6-row (3-row) verify pass: every row bit-identical to its single-row pass
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift, with_mtp=False)
    T = n_draft + 1
    eng.forward([(0, plain[:T], pos)])
    multi = logits_rows(eng, T)
    for t in range(T):
        assert torch.equal(multi[t].view(torch.int32), single[t].view(torch.int32)), f"row {t} of a {T}-row pass differs from its 1-row pass"
    # accept a strict prefix, continue one token at a time: same stream, same state as the plain run
    m = 2
    eng.accept(0, m)
    for i in range(m, 6):
        eng.forward([(0, [plain[i]], pos + i)]); eng.accept(0, 1)
        assert int(eng.topk(0, 1)[0][0]) == plain[i + 1]
    st_roll = eng.gdn_state(0, 0).copy()
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift, with_mtp=False)
    for i in range(6):
        eng.forward([(0, [plain[i]], pos + i)]); eng.accept(0, 1)
    assert np.array_equal(eng.gdn_state(0, 0).view(np.uint32), st_roll.view(np.uint32))

    # fused speculative rounds with seeded substitution: the emitted stream is the plain stream
    eng.reset()
    pos = spec.prefill(g, prompt, h_shift=g.h_shift, with_mtp=True)
    id_last = int(eng.topk(0, T_last)[0][T_last - 1])
    assert id_last == plain[0]
    eng.spec_begin(0, id_last, pos, eng.h_nextn_ptr() + (T_last - 1) * cfg.n_embd * 4)
    out = [id_last]
    while len(out) < n_gen:
        sub = spec.seeded_substitutions(plain, len(out), n_draft, 0.7, rng, cfg.n_vocab)
        out += eng.spec_round(0, n_draft, sub)
    assert out[:n_gen] == plain[:n_gen]
    eng.close()
