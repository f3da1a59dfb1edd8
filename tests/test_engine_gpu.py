"""The engine (load, forward, accept, mtp_forward, topk, slots) through the C ABI against the CPU restatement of the
reference engine, on a reduced-depth model with the same seeded weights. Everything is compared bit for bit."""
import numpy as np
import pytest

import hipster_b200 as hb
from hipster_b200.engine import TENSOR_KINDS
from oracle import orc

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def pair():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg)
    ref = orc.Model(cfg)
    yield cfg, eng, ref
    eng.close()


def test_generated_weights_identical(pair):
    cfg, eng, ref = pair
    for layer, kind in [(0, "in_proj"), (0, "conv_w"), (0, "a_neg"), (1, "gate_up"), (3, "in_proj"), (3, "q_norm"), (3, "out_proj"),
                        (-1, "embed"), (-1, "lm_head"), (-1, "mtp_eh_proj"), (cfg.n_layer, "in_proj"), (-1, "mtp_hnorm"), (2, "ssm_norm"), (2, "down")]:
        a = eng.tensor(layer, kind); b = ref.tensor(layer, TENSOR_KINDS[kind])
        assert a.size == b.size and np.array_equal(a, b), (layer, kind)


def test_plain_decode_logits_bit_exact(pair):
    cfg, eng, ref = pair
    eng.reset(); ref.reset()
    toks = [5, 77, 1030, 9, 2047, 0, 3]
    for p, t in enumerate(toks):
        eng.forward([(0, [t], p)]); eng.accept(0, 1)
        ref.forward([(0, [t], p)]); ref.accept(0, 1)
        assert np.array_equal(bits(eng.logits(1)), bits(ref.logits(1))), p
        assert np.array_equal(bits(eng.h_nextn(1)), bits(ref.h_nextn(1))), p
    ids, vals = eng.topk(0, 1)
    oi, ov = orc.argmax(ref.logits(1))
    assert ids[0] == oi[0] and bits(vals)[0] == bits(ov)[0]
    for gl in range(3):
        assert np.array_equal(bits(eng.gdn_state(0, gl)), bits(ref.gdn_state(0, gl)))


@pytest.mark.parametrize("m", [1, 2, 4, 6])
def test_verify_rows_accept_rollback(pair, m):
    """n+1 = 6 verify rows, accept m of them, continue: logits of the verify pass and of the following pass (which depends
    on the rolled-back recurrent state) match the CPU engine; and a verify row equals the same row of T = 1 passes."""
    cfg, eng, ref = pair
    eng.reset(); ref.reset()
    prompt = [11, 12, 13, 14, 15]
    for e in (eng, ref):
        e.forward([(0, prompt, 0)]); e.accept(0, len(prompt))
    rows = [100, 200, 300, 400, 500, 600]
    for e in (eng, ref):
        e.forward([(0, rows, 5)])
    assert np.array_equal(bits(eng.logits(6)), bits(ref.logits(6)))
    lg6 = eng.logits(6).copy()
    for e in (eng, ref):
        e.accept(0, m)
        e.forward([(0, [7, 8], 5 + m)])
    assert np.array_equal(bits(eng.logits(2)), bits(ref.logits(2)))
    for e in (eng, ref):
        e.accept(0, 2)
    for gl in range(3):
        assert np.array_equal(bits(eng.gdn_state(0, gl)), bits(ref.gdn_state(0, gl)))
    # T-invariance (reference README.md:65): replay the same tokens one at a time
    eng.reset()
    for p, t in enumerate(prompt):
        eng.forward([(0, [t], p)]); eng.accept(0, 1)
    for i, t in enumerate(rows[:3]):
        eng.forward([(0, [t], 5 + i)]); eng.accept(0, 1)
        assert np.array_equal(bits(eng.logits(1)[0]), bits(lg6[i]))


def test_mtp_forward_and_chained_drafts(pair):
    cfg, eng, ref = pair
    eng.reset(); ref.reset()
    E = cfg.n_embd
    hz = np.zeros((1, E), dtype=np.float32)
    import torch
    hprev = hz.copy()
    for p, t in enumerate([3, 4, 5, 6]):
        for e in (eng, ref):
            e.forward([(0, [t], p)]); e.accept(0, 1)
        hd = torch.from_numpy(hprev).cuda()
        eng.mtp_forward(0, [t], hd.data_ptr(), p)
        ref.mtp_forward(0, [t], hprev, p)
        assert np.array_equal(bits(eng.mtp_logits(1)), bits(ref.mtp_logits(1)))
        assert np.array_equal(bits(eng.mtp_h(1)), bits(ref.mtp_h(1)))
        hprev = ref.h_nextn(1).copy()
    # chained draft: the MTP's own h feeds the next step (spec27b.cpp:81-85); device pointer aliasing mtp_h
    tok = int(eng.topk(1, 1)[0][0])
    eng.mtp_forward(0, [tok], eng.mtp_h_ptr(), 4)
    ref.mtp_forward(0, [tok], ref.mtp_h(1), 4)
    assert np.array_equal(bits(eng.mtp_logits(1)), bits(ref.mtp_logits(1)))
    # catch-up over several rows with the target's h rows
    for e in (eng, ref):
        e.forward([(0, [9, 10, 11], 4)])
    eng.mtp_forward(0, [10, 11], eng.h_nextn_ptr(), 5)
    ref.mtp_forward(0, [10, 11], ref.h_nextn(2), 5)
    assert np.array_equal(bits(eng.mtp_logits(2)), bits(ref.mtp_logits(2)))


def test_two_slots_in_one_pass_match_solo_runs(pair):
    """README.md:61 contract of the reference (batchfn): per-slot results of a batched pass equal each slot's solo run."""
    cfg, eng, ref = pair
    eng.reset(); ref.reset()
    a, b = [21, 22, 23], [31, 32, 33, 34]
    for e in (eng, ref):
        e.forward([(0, a, 0), (1, b, 0)]); e.accept(0, 3); e.accept(1, 2)
        e.forward([(1, [40], 2), (0, [41, 42], 3)])
    assert np.array_equal(bits(eng.logits(3)), bits(ref.logits(3)))
    both = eng.logits(3).copy()
    eng.reset()
    eng.forward([(1, b, 0)]); eng.accept(1, 2); eng.forward([(1, [40], 2)])
    assert np.array_equal(bits(eng.logits(1)[0]), bits(both[0]))
    eng.forward([(0, a, 0)]); eng.accept(0, 3); eng.forward([(0, [41, 42], 3)])
    assert np.array_equal(bits(eng.logits(2)), bits(both[1:3]))


def test_argument_errors_mirror_the_reference(pair):
    cfg, eng, ref = pair
    eng.reset()
    with pytest.raises(hb.HipsterError, match="bad S"):
        eng.forward([(0, [1], 0), (1, [1], 0), (0, [2], 1)])
    with pytest.raises(hb.HipsterError, match="bad request"):
        eng.forward([(0, list(range(9)), 0)])
    with pytest.raises(hb.HipsterError, match="bad request"):
        eng.forward([(5, [1], 0)])
    with pytest.raises(hb.HipsterError, match="accept"):
        eng.accept(0, 1)
    eng.forward([(0, [1, 2], 0)])
    with pytest.raises(hb.HipsterError, match="bad accept"):
        eng.accept(0, 3)
