"""Host-side logic that needs no GPU: the K-part rule of the GEMV (library vs the oracle's mirror), model presets, the
seeded draft substitution, the expected tokens per round, and the expert-parallel ownership map."""
import ctypes

import numpy as np
import pytest

import hipster_b200 as hb
from hipster_b200 import ep, spec
from oracle import orc


def test_k_part_rule_matches_the_oracle_mirror_on_many_shapes():
    L = hb.lib(); O = orc.lib()
    for N in (16, 100, 512, 2368, 5120, 14336, 16480, 17408, 34816, 248320):
        for K in (256, 512, 1024, 2048, 5120, 6144, 10240, 17408):
            assert L.hp_gemv_parts(N, K) == O.orc_gemv_parts(N, K), (N, K)
    # the shapes of the dense configuration: down projection in 4 parts of 17 blocks, the big ones unsplit
    assert L.hp_gemv_parts(5120, 17408) == 4 and L.hp_gemv_parts(34816, 5120) == 1 and L.hp_gemv_parts(248320, 5120) == 1


def test_presets_carry_the_benchmark_shapes():
    c = hb.ModelCfg.preset("qwen35-27b")
    assert (c.n_layer, c.n_embd, c.n_ff, c.n_vocab, c.n_head, c.n_head_kv, c.gdn_qk_heads, c.gdn_v_heads) == (64, 5120, 17408, 248320, 24, 4, 16, 48)
    m = hb.ModelCfg.preset("flash-next")
    assert (m.n_layer, m.n_embd, m.n_expert, m.n_expert_used, m.expert_ff) == (48, 2048, 512, 10, 512)
    with pytest.raises(hb.HipsterError):
        hb.ModelCfg.preset("no-such-model")


def test_seeded_substitution_hits_the_requested_rate_exactly_at_the_extremes():
    plain = list(range(100, 200)); rng = np.random.default_rng(0)
    assert spec.seeded_substitutions(plain, 5, 4, 1.0, rng, 1000) == plain[5:9]
    wrong = spec.seeded_substitutions(plain, 5, 4, 0.0, rng, 1000)
    assert all(w != g for w, g in zip(wrong, plain[5:9]))
    hits = sum(a == b for _ in range(2000) for a, b in zip(spec.seeded_substitutions(plain, 5, 5, 0.7, rng, 1000), plain[5:10]))
    assert abs(hits / 10000 - 0.7) < 0.02


def test_expert_ranges_partition_the_experts():
    for world in (1, 2, 4, 8):
        owners = [ep.owner_of(e, world, 512) for e in range(512)]
        for r in range(world):
            lo, hi = ep.expert_range(r, world, 512)
            assert owners[lo:hi] == [r] * (hi - lo)
        assert sorted(set(owners)) == list(range(world))


def test_buffer_size_helpers():
    L = hb.lib()
    L.hp_argmax_scratch_bytes.restype = ctypes.c_size_t
    assert L.hp_xq8_q_bytes(1, 256) == 256 * 8 and L.hp_xq8_q_bytes(9, 256) == 2 * 256 * 8
    assert L.hp_argmax_scratch_bytes(6, 248320) > 0 and L.hp_argmax_scratch_bytes(0, 5) == 0
