"""Parity of the CUDA Q4_K GEMV path (through the C ABI) with the CPU oracle. Bit-exact for the quantised
activations, the dequantised weights, the int8-activation GEMV, the f32-activation GEMV, argmax and acceptance."""
import numpy as np
import pytest
import torch

import hipster_b200 as hb
from hipster_b200 import kernels as K_, synth
from oracle import orc

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_dequant_q4k_bit_exact():
    W = synth.q4k_matrix(64, 1024, seed=11)
    got = K_.dequant_q4k(dev(W), 64 * 4).cpu().numpy()
    assert np.array_equal(bits(got), bits(orc.dequant_q4k(W)))


@pytest.mark.parametrize("R,K", [(1, 256), (3, 5120), (6, 17408), (9, 512), (24, 2048)])
def test_quantize_x_q8_bit_exact(R, K):
    x = synth.activations(R, K, seed=R * 7 + 1)
    x[0, 64:96] = 0.0
    xq = K_.quantize_x_q8(dev(x))
    q, d, s = [t.cpu().numpy() for t in xq.unpack()]
    oq, od, os_ = orc.quantize_x_q8(x)
    assert np.array_equal(q, oq) and np.array_equal(bits(d), bits(od)) and np.array_equal(bits(s), bits(os_))


@pytest.mark.parametrize("N,K,R", [(16, 256, 1), (48, 1024, 3), (512, 5120, 6), (100, 768, 2), (40, 2048, 8),
                                     (64, 1024, 9), (128, 2048, 24), (32, 17408, 6), (7, 512, 5),
                                     (256, 6144, 24), (80, 6144, 12), (48, 9216, 32)])   # the last three: activations read from L2 (too large to stage)
def test_gemv_q8_bit_exact_vs_oracle(N, K, R):
    W = synth.q4k_matrix(N, K, seed=N + K); x = synth.activations(R, K, seed=R)
    xq = K_.quantize_x_q8(dev(x))
    y = K_.gemv_q4k_q8(dev(W), xq, N, K).cpu().numpy()
    K_.device_status()
    q, d, s = orc.quantize_x_q8(x)
    want = orc.gemv_q4k_q8(W, q, d, s, N, K)
    assert np.array_equal(bits(y), bits(want))


def test_gemv_q8_row_result_independent_of_row_count():
    # the reference's T-invariance contract (README.md:65: T>1 vs T=1 logit difference 0.0000)
    N, K = 256, 5120
    W = dev(synth.q4k_matrix(N, K, seed=3)); x = synth.activations(24, K, seed=4)
    y24 = K_.gemv_q4k_q8(W, K_.quantize_x_q8(dev(x)), N, K).cpu().numpy()
    for r in (0, 5, 8, 23):
        y1 = K_.gemv_q4k_q8(W, K_.quantize_x_q8(dev(x[r:r + 1])), N, K).cpu().numpy()
        assert np.array_equal(bits(y1[0]), bits(y24[r]))
    y6 = K_.gemv_q4k_q8(W, K_.quantize_x_q8(dev(x[:6])), N, K).cpu().numpy()
    assert np.array_equal(bits(y6), bits(y24[:6]))


@pytest.mark.parametrize("N,K,R", [(64, 1024, 1), (200, 5120, 3), (33, 768, 8)])
def test_gemv_f32_bit_exact_vs_oracle(N, K, R):
    W = synth.q4k_matrix(N, K, seed=N); x = synth.activations(R, K, seed=R + 100)
    y = K_.gemv_q4k_f32(dev(W), dev(x), N, K).cpu().numpy()
    assert np.array_equal(bits(y), bits(orc.gemv_q4k_f32(W, x, N, K, tpr=4)))


def test_argmax_and_accept():
    rng = np.random.default_rng(0)
    lg = rng.normal(size=(6, 248320)).astype(np.float32)
    lg[1, 100] = lg[1, 200000] = 50.0      # tie across chunks -> lower index
    lg[2, 248319] = 60.0
    lg[3, 0] = 60.0
    ids, vals = K_.argmax(dev(lg))
    oi, ov = orc.argmax(lg)
    assert np.array_equal(ids.cpu().numpy(), oi) and np.array_equal(bits(vals.cpu().numpy()), bits(ov))
    for drafts in ([int(oi[0]), int(oi[1]), 5, int(oi[3]), 7], [1, 2, 3, 4, 5], [int(v) for v in oi[:5]]):
        out = K_.accept_greedy(ids, dev(np.array(drafts, dtype=np.int32))).cpu().numpy()
        assert tuple(out) == orc.accept(oi, drafts)


def test_config1_kernel_check_full_size():
    """Benchmark configuration 1: N=17408 x K=5120 Q4_K, 3 f32 activation rows, seed 0 -> GEMV, per-row argmax, greedy
    acceptance against 2 seeded draft ids; CUDA vs the CPU restatement, plus the reference's own tolerance rule."""
    N, K, R = 17408, 5120, 3
    W = synth.q4k_matrix(N, K, seed=0); x = synth.activations(R, K, seed=0)
    Wd = dev(W)
    xq = K_.quantize_x_q8(dev(x))
    y = K_.gemv_q4k_q8(Wd, xq, N, K)
    ids, _ = K_.argmax(y)
    q, d, s = orc.quantize_x_q8(x)
    want = orc.gemv_q4k_q8(W, q, d, s, N, K)
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))
    oi, _ = orc.argmax(want)
    assert np.array_equal(ids.cpu().numpy(), oi)
    rng = np.random.default_rng(0)
    drafts = np.array([oi[0], oi[1] if rng.random() < 0.5 else (oi[1] + 1) % N], dtype=np.int32)
    assert tuple(K_.accept_greedy(ids, dev(drafts)).cpu().numpy()) == orc.accept(oi, drafts)
    # reference acceptance rule (bench_gemv.cpp:111): maxrel < 1e-5 vs dequantised weights . quantised x in double
    xr = (q.astype(np.float32).reshape(R, -1, 32) * d[:, :, None]).reshape(R, K).astype(np.float32)
    ref, mag = orc.gemv_q4k_double(W, xr, N, K)
    assert np.max(np.abs(ref - y.cpu().numpy()) / (mag + 1e-20)) < 1e-5
    # f32-activation kernel on the same inputs, bit-exact vs its restatement, and argmax agreement is reported
    yf = K_.gemv_q4k_f32(Wd, dev(x), N, K).cpu().numpy()
    assert np.array_equal(bits(yf), bits(orc.gemv_q4k_f32(W, x, N, K, tpr=4)))


def test_bad_arguments_are_rejected_not_launched():
    W = torch.zeros(144 * 16, dtype=torch.uint8, device="cuda")
    xq = K_.XQ8(1, 256)
    with pytest.raises(hb.HipsterError):
        K_.gemv_q4k_q8(W, xq, 16, 100)         # K not a multiple of 256
    with pytest.raises(hb.HipsterError):
        K_.gemv_q4k_q8(W[1:], xq, 16, 256)     # misaligned weights


def test_all_zero_and_tiny_activations():
    """A 32-element sub-block of zeros quantises to d = 0, q = 0 (no 0/0), and a whole zero row gives exact zeros."""
    N, K = 48, 512
    W = synth.q4k_matrix(N, K, seed=3)
    x = synth.activations(3, K, seed=4); x[1] = 0.0; x[2, 64:96] = 0.0; x[0, :32] = 1e-30
    xq = K_.quantize_x_q8(dev(x))
    q, d, s = [t.cpu().numpy() for t in xq.unpack()]
    oq, od, os_ = orc.quantize_x_q8(x)
    assert np.array_equal(q, oq) and np.array_equal(bits(d), bits(od)) and np.array_equal(bits(s), bits(os_))
    y = K_.gemv_q4k_q8(dev(W), xq, N, K).cpu().numpy()
    assert np.array_equal(bits(y), bits(orc.gemv_q4k_q8(W, oq, od, os_, N, K)))
    assert not y[1].any() and np.isfinite(y).all()
