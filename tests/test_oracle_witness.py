"""The two CPU checkers against each other, without a GPU: the bit-exact restatement (whose summation orders follow this
build's kernels) and the independent double-precision transcription of the reference's device source must agree within
the tolerances the benchmark configurations state -- 1e-5 relative for the Gated-DeltaNet layer, 1e-3 of the largest
output for attention (the benchmark allows 1e-2), identical expert choices for the router. Also the top-k oracle."""
import numpy as np

from oracle import orc


def bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def test_gdn_restatement_vs_double_precision_transcription():
    n_qk, n_v, T = 2, 4, 6
    rng = np.random.default_rng(0)
    C = (2 * n_qk + n_v) * 128; ld = C + n_v * 128 + 2 * n_v
    rows = rng.normal(0, 1, size=(T, ld)).astype(np.float32)
    conv_w = rng.normal(0, 0.5, size=C * 4).astype(np.float32)
    dt = bf16_bits(rng.normal(0, 0.5, size=n_v)); a_neg = bf16_bits(-np.abs(rng.normal(0, 1, size=n_v))); nw = bf16_bits(1 + 0.3 * rng.normal(size=128))
    st0 = rng.normal(0, 0.1, size=(n_v, 128, 128)).astype(np.float32)
    st = st0.copy(); hist = np.zeros((3, C), dtype=np.float32)
    out, _ = orc.gdn_rows(rows, n_qk, n_v, conv_w, dt, a_neg, nw, st, hist, 1e-6, 0)
    st64 = st0.astype(np.float64); hist64 = np.zeros((3, C), dtype=np.float64)
    out64 = orc.ref64_gdn_rows(rows, n_qk, n_v, conv_w, bf16_to_f32(dt), bf16_to_f32(a_neg), bf16_to_f32(nw), st64, hist64, 1e-6, 0)
    assert np.abs(out - out64).max() <= 1e-5 * np.abs(out64).max()
    assert np.abs(st - st64).max() <= 1e-5 * np.abs(st64).max()
    assert np.array_equal(hist, hist64.astype(np.float32))


def test_attention_restatement_vs_double_precision_transcription():
    n_head, n_kv, max_ctx, pos0 = 8, 2, 512, 300
    rng = np.random.default_rng(1)
    ld = n_head * 512 + 2 * n_kv * 256
    qkv = rng.normal(0, 1, size=(3, ld)).astype(np.float32)
    qw = bf16_bits(1 + 0.2 * rng.normal(size=256)); kw = bf16_bits(1 + 0.2 * rng.normal(size=256))
    kc = rng.normal(0, 1, size=(n_kv, max_ctx, 256)).astype(np.float16); vc = rng.normal(0, 1, size=(n_kv, max_ctx, 256)).astype(np.float16)
    rope = orc.rope_table(max_ctx, 64, 1e7)
    kco = kc.copy().view(np.uint16); vco = vc.copy().view(np.uint16); q2 = qkv.copy()
    kc64 = kc.astype(np.float32); vc64 = vc.astype(np.float32)
    for r in range(3):
        got = orc.attn_row(q2[r], n_head, n_kv, 64, qw, kw, rope, pos0 + r, kco, vco, max_ctx, 1e-6)
        ref = orc.ref64_attn_row(qkv[r], n_head, n_kv, 64, bf16_to_f32(qw), bf16_to_f32(kw), 1e7, pos0 + r, kc64, vc64, max_ctx, 1e-6)
        assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
    # both wrote the same f16 K / V rows except where the fp32 angle of the reference rounds differently (1 ulp of f16)
    a = kco.view(np.float16)[:, pos0:pos0 + 3].astype(np.float32); b = kc64[:, pos0:pos0 + 3]
    assert np.abs(a - b).max() <= 2e-3 * np.abs(b).max()
    assert np.array_equal(vco.view(np.float16)[:, pos0:pos0 + 3].astype(np.float32), vc64[:, pos0:pos0 + 3])


def test_routing_restatement_vs_double_precision_transcription():
    E, k, T = 512, 10, 24
    lg = np.random.default_rng(2).normal(0, 1, size=(T, E + 1)).astype(np.float32)
    ids = np.empty((T, k + 1), dtype=np.int32); w = np.empty((T, k + 1), dtype=np.float32)
    orc.lib().orc_moe_route(orc.P(lg), orc.P(ids), orc.P(w), T, E, k)
    ids64, w64 = orc.ref64_moe_route(lg, E, k)
    assert np.array_equal(ids, ids64)
    assert np.allclose(w, w64, rtol=1e-5, atol=0)
    assert np.all(ids[:, k] == -1) and np.allclose(w[:, :k].sum(axis=1), 1.0, atol=1e-6)


def test_topk_oracle_order_and_ties():
    x = np.array([[1.0, 5.0, 5.0, -np.inf, 3.0, 5.0], [0.0, 0.0, 0.0, 0.0, 0.0, 0.0]], dtype=np.float32)
    ids, vals = orc.topk(x, 4)
    assert ids[0].tolist() == [1, 2, 5, 4] and vals[0].tolist() == [5.0, 5.0, 5.0, 3.0]
    assert ids[1].tolist() == [0, 1, 2, 3]
    ids, _ = orc.topk(x[:1], 6)
    assert ids[0].tolist() == [1, 2, 5, 4, 0, -1]            # an entry equal to -inf is never selected
    assert np.array_equal(orc.topk(x, 1)[0][:, 0], orc.argmax(x)[0])
