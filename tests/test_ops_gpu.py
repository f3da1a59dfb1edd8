"""Row norm (+ residual add of K-part planes) and SiLU-gated product with q8 quantisation through the C ABI, bit-exact
against the CPU oracle, on shapes that exercise the edges: rows that leave lanes of a warp idle, two 128-bit groups per
thread, every plane count (compile-time 1 / 2 / 4 and the run-time path)."""
import ctypes

import numpy as np
import pytest
import torch

from hipster_b200 import kernels as K_
from hipster_b200._lib import lib, check, ptr
from oracle import orc

pytestmark = pytest.mark.gpu


def _f(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("R,n,P", [(1, 320, 1), (6, 5120, 4), (3, 2048, 2), (2, 10240, 3), (8, 64, 0), (5, 5184, 4)])
def test_add_rmsnorm_quant_bit_exact(R, n, P):
    rng = np.random.default_rng(R * 1000 + n + P)
    x = rng.standard_normal((R, n)).astype(np.float32)
    y = (rng.standard_normal((max(P, 1), R, n)) * 0.5).astype(np.float32)
    w = (rng.standard_normal(n).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)     # bf16 bit patterns
    eps = 1e-6
    # oracle
    xo = x.copy(); xn_o = np.empty((R, n), np.float32)
    q_o = np.empty((R, n), np.int8); d_o = np.empty((R, n // 32), np.float32); s_o = np.empty((R, n // 32), np.float32)
    O = orc.lib()
    O.orc_add_rmsnorm_quant(_f(xo), _f(y) if P else None, P, ctypes.c_size_t(R * n), n, _f(w), _f(xn_o), _f(q_o), _f(d_o), _f(s_o), R, n, ctypes.c_float(eps))
    # device
    xd = torch.from_numpy(x.copy()).cuda(); yd = torch.from_numpy(y).cuda(); wd = torch.from_numpy(w.view(np.int16)).cuda()
    xn_d = torch.empty((R, n), dtype=torch.float32, device="cuda"); xq = K_.XQ8(R, n)
    check(lib().hp_add_rmsnorm_quant(ptr(xd), ptr(yd) if P else None, P, ctypes.c_size_t(R * n), ptr(wd), ptr(xn_d), ptr(xq.q), ptr(xq.sc), R, n, ctypes.c_float(eps), _stream()))
    q, d, s = xq.unpack()
    torch.cuda.synchronize()
    assert np.array_equal(xd.cpu().numpy().view(np.uint32), xo.view(np.uint32))
    assert np.array_equal(xn_d.cpu().numpy().view(np.uint32), xn_o.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), q_o)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), d_o.view(np.uint32))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_o.view(np.uint32))


@pytest.mark.parametrize("R,F", [(1, 64), (6, 17408), (3, 1024), (4, 192)])
def test_silu_mul_quant_bit_exact(R, F):
    rng = np.random.default_rng(R + F)
    gu = (rng.standard_normal((R, 2 * F)) * 3).astype(np.float32)
    q_o = np.empty((R, F), np.int8); d_o = np.empty((R, F // 32), np.float32); s_o = np.empty((R, F // 32), np.float32)
    orc.lib().orc_silu_mul_quant(_f(gu), 2 * F, F, _f(q_o), _f(d_o), _f(s_o), R)
    gd = torch.from_numpy(gu).cuda(); xq = K_.XQ8(R, F)
    check(lib().hp_silu_mul_quant(ptr(gd), 2 * F, F, ptr(xq.q), ptr(xq.sc), R, _stream()))
    q, d, s = xq.unpack()
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), q_o)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), d_o.view(np.uint32))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_o.view(np.uint32))
