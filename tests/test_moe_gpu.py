"""MoE FFN (router, top-k routing with shared expert, grouped expert GEMV, in-order combine) through the engine on a
reduced Flash-Next-shaped model, bit for bit against the CPU restatement (reference: engine/kernels/fn.hip:167-277,
engine/kernels/gemv.hip:1075-1129, engine/src/qwen4exp.cpp:345-354), plus the multi-slot contract of batchfn.cpp."""
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
    cfg = hb.ModelCfg.preset("tiny-moe")
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    yield cfg, eng, ref
    eng.close()


def test_moe_weights_identical(pair):
    cfg, eng, ref = pair
    for layer, kind in [(0, "router"), (0, "exp_gate_up"), (1, "exp_down"), (3, "sh_gate_up"), (2, "sh_down"), (cfg.n_layer, "exp_gate_up")]:
        assert np.array_equal(eng.tensor(layer, kind), ref.tensor(layer, TENSOR_KINDS[kind])), (layer, kind)


def test_moe_forward_accept_mtp_bit_exact(pair):
    cfg, eng, ref = pair
    eng.reset(); ref.reset()
    for e in (eng, ref):
        e.forward([(0, [3, 1000, 77, 12, 9], 0)]); e.accept(0, 5)
        e.forward([(0, [500, 600, 700], 5)])
    assert np.array_equal(bits(eng.logits(3)), bits(ref.logits(3)))
    assert np.array_equal(bits(eng.h_nextn(3)), bits(ref.h_nextn(3)))
    for e in (eng, ref):
        e.accept(0, 2); e.forward([(0, [42], 7)])
    assert np.array_equal(bits(eng.logits(1)), bits(ref.logits(1)))
    eng.mtp_forward(0, [42], eng.h_nextn_ptr(), 7)
    ref.mtp_forward(0, [42], ref.h_nextn(1), 7)
    assert np.array_equal(bits(eng.mtp_logits(1)), bits(ref.mtp_logits(1)))


def test_moe_four_slots_batched_equal_solo(pair):
    """engine/bench/batchfn.cpp:128-131: every slot's rows of a lock-step batched pass equal that slot's solo run."""
    cfg, eng, ref = pair
    eng.reset()
    prompts = {s: [int(x) for x in np.random.default_rng(s).integers(0, cfg.n_vocab, size=6)] for s in range(4)}
    eng.forward([(s, prompts[s], 0) for s in range(4)])
    for s in range(4):
        eng.accept(s, 6 - s)              # different accepted lengths per slot
    eng.forward([(s, [10 + s, 20 + s, 30 + s], 6 - s) for s in range(4)])
    batched = eng.logits(12).copy()
    for s in range(4):
        eng.reset_slot(s)
        eng.forward([(s, prompts[s], 0)]); eng.accept(s, 6 - s)
        eng.forward([(s, [10 + s, 20 + s, 30 + s], 6 - s)])
        assert np.array_equal(bits(eng.logits(3)), bits(batched[3 * s:3 * s + 3])), s
    # and against the oracle for one slot
    ref.reset()
    ref.forward([(2, prompts[2], 0)]); ref.accept(2, 4); ref.forward([(2, [12, 22, 32], 4)])
    assert np.array_equal(bits(ref.logits(3)), bits(batched[6:9]))
