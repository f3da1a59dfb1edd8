"""Boundary behaviour of the engine-level C ABI: top-k with k > 1, hp_prefill against the chunked verify path, the
descriptor capacity with many attention row groups, the survival of a stream across hp_profile_pass, the refusal to run
an expert-parallel shard without its communicator, and the C++ driver that links nothing but the library."""
import os
import subprocess

import numpy as np
import pytest

import hipster_b200 as hb
from hipster_b200 import build as hb_build
from oracle import orc

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_topk_k_matches_oracle_including_ties():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    for e in (eng, ref):
        e.forward([(0, [5, 6, 7, 8, 9], 0)])
    lg = ref.logits(5)
    for k in (1, 2, 10, 32):
        ids, vals = eng.topk(0, 5, k=k)
        oi, ov = orc.topk(lg, k)
        assert np.array_equal(np.asarray(ids).reshape(5, k), oi), k
        assert np.array_equal(bits(np.asarray(vals).reshape(5, k)), bits(ov)), k
    with pytest.raises(hb.HipsterError):
        eng.topk(0, 5, k=33)
    eng.close()


def test_prefill_equals_chunked_forward_and_oracle():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    prompt = [int(x) for x in np.random.default_rng(9).integers(0, cfg.n_vocab, size=21)]
    eng.prefill(0, prompt[:10], pos0=0, with_mtp=True)          # two calls for one prompt: the second continues the first
    eng.prefill(0, prompt[10:], pos0=10, with_mtp=True)
    prev = np.zeros(cfg.n_embd, dtype=np.float32)
    for p0, p1 in [(0, 8), (8, 10), (10, 18), (18, 21)]:         # the chunks hp_prefill used
        toks = prompt[p0:p1]; T = len(toks)
        ref.forward([(0, toks, p0)]); ref.accept(0, T)
        h = ref.h_nextn(T)
        ref.mtp_forward(0, toks, np.vstack([prev[None, :], h[:T - 1]]), p0)
        prev = h[T - 1].copy()
    assert np.array_equal(bits(eng.logits(1)[0]), bits(ref.logits(3)[2]))
    assert np.array_equal(bits(eng.h_nextn(1)[0]), bits(ref.h_nextn(3)[2]))
    assert int(eng.topk(0, 1)[0][0]) == int(orc.argmax(ref.logits(3))[0][2])
    # the draft block's cache covers the prompt: a draft step right after the prompt agrees
    tok = int(eng.topk(0, 1)[0][0])
    eng.mtp_forward(0, [tok], eng.h_nextn_ptr(), 21)
    ref.mtp_forward(0, [tok], ref.h_nextn(3)[2:3], 21)
    assert np.array_equal(bits(eng.mtp_logits(1)), bits(ref.mtp_logits(1)))
    with pytest.raises(hb.HipsterError):
        eng.prefill(0, prompt, pos0=cfg.max_ctx - 3)
    eng.close()


def test_many_attention_row_groups_12_heads_per_kv_head():
    """12 q-heads per kv head allow 4 rows per attention row group: 6 slots x 5 rows = 30 rows need 12 groups, more than
    the 8 an earlier descriptor layout could hold (its overflow ran into the per-sequence table of the GDN kernels)."""
    cfg = hb.ModelCfg.preset("tiny-moe", n_head=24, n_head_kv=2, n_slots=6, max_ctx=128)
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    reqs = [(s, [int(x) for x in np.random.default_rng(40 + s).integers(0, cfg.n_vocab, size=5)], 0) for s in range(6)]
    for e in (eng, ref):
        e.forward(reqs)
    assert np.array_equal(bits(eng.logits(30)), bits(ref.logits(30)))
    for e in (eng, ref):
        for s in range(6):
            e.accept(s, 1 + s % 5)
    reqs2 = [(s, [int(x) for x in np.random.default_rng(60 + s).integers(0, cfg.n_vocab, size=5 if s < 4 else 6)], 1 + s % 5) for s in range(6)]
    for e in (eng, ref):
        e.forward(reqs2)                                          # 32 rows, 12 groups, after per-slot rollbacks
    assert np.array_equal(bits(eng.logits(32)), bits(ref.logits(32)))
    eng.close()


def test_stream_continues_bit_exact_after_profile_pass():
    cfg = hb.ModelCfg.preset("tiny")
    n = 3
    prompt = [int(x) for x in np.random.default_rng(2).integers(0, cfg.n_vocab, size=13)]

    def stream(profile_at):
        eng = hb.Engine(cfg)
        eng.prefill(0, prompt, with_mtp=True)
        eng.spec_begin(0, int(eng.topk(0, 1)[0][0]), len(prompt), eng.h_nextn_ptr())
        out = []
        for r in range(6):
            if r == profile_at:
                assert eng.profile_pass(n + 1, 0, 2) > 0
                assert eng.profile_pass(n + 1, 1, 1) > 0
            out += eng.spec_round(0, n, [-1, (7 * r) % cfg.n_vocab, -1])
        eng.close()
        return out
    assert stream(2) == stream(-1)


def test_accept_is_refused_after_profile_pass():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg)
    eng.forward([(0, [1, 2, 3], 0)])
    eng.profile_pass(2, 0, 1)
    with pytest.raises(hb.HipsterError):
        eng.accept(0, 2)
    eng.close()


def test_expert_parallel_shard_refuses_to_run_without_its_communicator():
    cfg = hb.ModelCfg.preset("tiny-moe", ep_rank=0, ep_world=2)
    eng = hb.Engine(cfg)
    with pytest.raises(hb.HipsterError) as ei:
        eng.forward([(0, [1, 2], 0)])
    assert ei.value.code == 5 and "hp_ep_init" in str(ei.value)      # HP_ESTATE, not silent zeros
    eng.close()


def test_cpp_driver_through_the_c_abi_reports_exact():
    """spec_driver.cpp (the reference's spec27b.cpp:59-110 loop for this library) links only libhipster_b200.so."""
    exe = hb_build.build_driver()
    for args, n_exact in ((["tiny", "40", "3", "21", "70"], 2), (["tiny", "24", "5", "9", "-1"], 2), (["tiny-moe", "18", "2", "11", "70", "4"], 3)):
        r = subprocess.run([exe] + args, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        assert r.stdout.count("EXACT") == n_exact and "MISMATCH" not in r.stdout, r.stdout
    deps = subprocess.run(["ldd", exe], capture_output=True, text=True).stdout
    assert "libhipster_b200.so" in deps and "libcudart" not in deps and "libtorch" not in deps


def test_measurement_hooks_and_full_width_lockstep_round():
    """8 slots x (3 drafts + 1) = 32 verify rows, the most a pass can hold, through the fused multi-slot round on the reduced
    MoE model; the kernel count of the round's graph, the touched-expert counter and the exchange timer answer."""
    cfg = hb.ModelCfg.preset("tiny-moe", n_slots=8)
    eng = hb.Engine(cfg)
    S, n = 8, 3
    prompts = [[int(x) for x in np.random.default_rng(500 + s).integers(0, cfg.n_vocab, size=3 + s)] for s in range(S)]
    for s in range(S):
        eng.prefill(s, prompts[s], with_mtp=True)
        eng.spec_begin(s, int(eng.topk(0, 1)[0][0]), len(prompts[s]), eng.h_nextn_ptr())
    eng.moe_touched()
    lock = [[] for _ in range(S)]
    for r in range(3):
        out = eng.spec_round_slots(list(range(S)), n)
        assert all(1 <= len(o) <= n + 1 for o in out)
        for s in range(S):
            lock[s] += out[s]
    assert eng.last_round_kernels() > 100
    assert eng.moe_touched() > 0 and eng.ep_exchange_us(8) == 0.0          # one GPU: nothing to exchange
    with pytest.raises(hb.HipsterError):
        eng.spec_round_slots(list(range(S)), 4)                             # 8 x 5 rows > 32
    with pytest.raises(hb.HipsterError):
        eng.spec_round_slots([0, 0], 2)                                     # a slot listed twice
    # every slot equals its solo run in another order of slots (the row order of a pass has no influence)
    eng.reset()
    for s in (5, 2):
        eng.prefill(s, prompts[s], with_mtp=True)
        eng.spec_begin(s, int(eng.topk(0, 1)[0][0]), len(prompts[s]), eng.h_nextn_ptr())
    two = [[], []]
    for r in range(3):
        out = eng.spec_round_slots([5, 2], n)
        two[0] += out[0]; two[1] += out[1]
    assert two[0] == lock[5] and two[1] == lock[2]
    eng.close()


def test_single_token_prefill_zero_rows_and_reset_slot():
    cfg = hb.ModelCfg.preset("tiny")
    eng = hb.Engine(cfg); ref = orc.Model(cfg)
    eng.prefill(1, [77], with_mtp=True)                                      # one token: no "last row" move is needed
    ref.forward([(1, [77], 0)]); ref.accept(1, 1)
    assert np.array_equal(bits(eng.logits(1)), bits(ref.logits(1)))
    eng.reset_slot(1); ref.reset_slot(1)
    for e in (eng, ref):
        e.forward([(1, [5, 6], 0), (0, [9], 0)])                             # slots in descending order, ragged row counts
    assert np.array_equal(bits(eng.logits(3)), bits(ref.logits(3)))
    for bad in ([], [(0, [], 0)], [(0, [1] * 9, 0)], [(7, [1], 0)], [(0, [1], cfg.max_ctx)]):
        with pytest.raises(hb.HipsterError):
            eng.forward(bad)
    eng.close()


def test_peer_exchange_wait_is_bounded_and_reports_through_the_status_word():
    """The wait of the peer-memory exchange for a flag that nothing sets must run out by itself (about a second), set the
    device status word (HP_ETIMEOUT through hp_device_status) and leave the context usable; flags that are there pass."""
    import ctypes
    import time
    import torch
    from hipster_b200 import kernels as K_
    from hipster_b200._lib import lib, ptr, HipsterError
    L = lib()
    K_.device_status()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags[1] = 5
    st = torch.cuda.current_stream().cuda_stream
    assert L.hp_ep_wait_probe(ptr(flags), 2, 0, ctypes.c_uint(5), ctypes.c_void_p(st)) == 0
    K_.device_status()                                        # rank 1 has delivered exchange 5: no complaint
    assert L.hp_ep_wait_probe(ptr(flags), 2, 0, ctypes.c_uint(4), ctypes.c_void_p(st)) == 0
    K_.device_status()                                        # a peer that is ahead is fine too
    t0 = time.perf_counter()
    assert L.hp_ep_wait_probe(ptr(flags), 3, 0, ctypes.c_uint(5), ctypes.c_void_p(st)) == 0   # rank 2 never delivers
    with pytest.raises(HipsterError) as ei:
        K_.device_status()
    assert ei.value.code == 4 and "bounded wait" in str(ei.value)        # HP_ETIMEOUT
    assert time.perf_counter() - t0 < 30.0
    K_.device_status()                                        # the word was cleared, the context works
    assert int((flags + 1).sum().item()) == 13
