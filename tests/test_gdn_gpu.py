"""Benchmark configuration 2: one Gated-DeltaNet layer verify step at full size (hidden 5120 -> 16 key heads, 48 value heads,
dim 128, conv 4), fp32 state ~ N(0, 0.1), 6 bf16-rounded input rows ~ N(0, 1): per-row state snapshots, rollback to
accepted length k in {0..5}, compared with the sequential one-row-at-a-time scan (GPU and CPU oracle).
The stated tolerance is 1e-5 relative; the CUDA kernel and the oracle actually agree bit for bit.
Mirrors engine/bench/test_fnkernels.cpp:28-53 (same generator style: a_neg = -|N(0,1)|, dt ~ N(0,0.5), norm w = 1+N(0,0.3))."""
import ctypes

import numpy as np
import pytest
import torch

import hipster_b200 as hb
from oracle import orc

pytestmark = pytest.mark.gpu

NQK, NV, D = 16, 48, 128
C = (2 * NQK + NV) * D
LD = C + NV * D + 2 * NV


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return u


def bf16_to_f32(u):
    return (u.astype(np.uint32) << 16).view(np.float32)


def private_conv_state(hist):
    """reference layout [3][C] -> this library's per-value-head layout [n_v][3][q | k | v]."""
    out = np.zeros((NV, 3, 384), dtype=np.float32)
    for h in range(NV):
        hk = h % NQK
        out[h, :, 0:128] = hist[:, hk * D:(hk + 1) * D]
        out[h, :, 128:256] = hist[:, NQK * D + hk * D:NQK * D + (hk + 1) * D]
        out[h, :, 256:384] = hist[:, 2 * NQK * D + h * D:2 * NQK * D + (h + 1) * D]
    return out


class Layer:
    def __init__(self, seed, sigmoid_gate=0):
        rng = np.random.default_rng(seed)
        self.rows = bf16_to_f32(bf16_round(rng.normal(0, 1, size=(6, LD)))).astype(np.float32)
        self.conv_w = rng.normal(0, 0.5, size=(C, 4)).astype(np.float32)
        self.dt = bf16_round(rng.normal(0, 0.5, size=NV)); self.an = bf16_round(-np.abs(rng.normal(0, 1, size=NV)))
        self.nw = bf16_round(1 + rng.normal(0, 0.3, size=D))
        self.state0 = rng.normal(0, 0.1, size=(NV, D, D)).astype(np.float32)
        self.hist0 = rng.normal(0, 1, size=(3, C)).astype(np.float32)
        self.gate = sigmoid_gate
        self.eps = 1e-6

    def dev(self):
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        d = dict(rows=t(self.rows), conv_w=t(self.conv_w), dt=t(self.dt.view(np.int16)), an=t(self.an.view(np.int16)), nw=t(self.nw.view(np.int16)),
                 state=t(self.state0), conv=t(private_conv_state(self.hist0)),
                 saved=torch.zeros(hb.lib().hp_gdn_saved_floats(NV), dtype=torch.float32, device="cuda"))
        return d

    def call(self, d, rows, T, n_replay, out=None, snap=None):
        L = hb.lib()
        hb.check(L.hp_gdn_layer(hb.ptr(rows), LD, T, n_replay, NQK, NV, hb.ptr(d["conv_w"]), hb.ptr(d["dt"]), hb.ptr(d["an"]), hb.ptr(d["nw"]),
                                hb.ptr(d["state"]), hb.ptr(d["conv"]), hb.ptr(d["saved"]), hb.ptr(out), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                hb.ptr(snap), ctypes.c_float(self.eps), self.gate, ctypes.c_void_p(0)))
        torch.cuda.synchronize()


@pytest.fixture(scope="module")
def setup():
    hb.lib().hp_gdn_saved_floats.restype = ctypes.c_size_t
    hb.lib().hp_gdn_conv_state_floats.restype = ctypes.c_size_t
    return Layer(seed=2)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_six_row_verify_with_snapshots_matches_sequential_scan(setup):
    Ly = setup
    d = Ly.dev()
    out6 = torch.empty((6, NV * D), dtype=torch.float32, device="cuda"); snap = torch.empty((6, NV, D, D), dtype=torch.float32, device="cuda")
    Ly.call(d, d["rows"], 6, 0, out6, snap)
    # CPU oracle, sequential scan (reference layout of the conv history)
    st = Ly.state0.copy(); hist = Ly.hist0.copy()
    oout, osnap = orc.gdn_rows(Ly.rows, NQK, NV, Ly.conv_w, Ly.dt, Ly.an, Ly.nw, st, hist, Ly.eps, Ly.gate, want_snap=True)
    o = out6.cpu().numpy(); s = snap.cpu().numpy()
    rel = np.max(np.abs(o - oout)) / np.max(np.abs(oout)); rels = np.max(np.abs(s - osnap)) / np.max(np.abs(osnap))
    assert rel < 1e-5 and rels < 1e-5
    assert np.array_equal(bits(o), bits(oout)) and np.array_equal(bits(s), bits(osnap))
    # GPU sequential one-row-at-a-time scan: each call accepts the previous row and processes one new row
    d2 = Ly.dev(); o1 = torch.empty((1, NV * D), dtype=torch.float32, device="cuda")
    for t in range(6):
        Ly.call(d2, d2["rows"][t:t + 1].contiguous(), 1, 1 if t > 0 else 0, o1, None)
        assert np.array_equal(bits(o1.cpu().numpy()[0]), bits(o[t]))
    # the verify pass did not advance the committed state
    assert np.array_equal(bits(d["state"].cpu().numpy()), bits(Ly.state0))


@pytest.mark.parametrize("k", [0, 1, 2, 3, 4, 5])
def test_rollback_to_accepted_length(setup, k):
    """k accepted drafts = the first k+1 of the 6 rows are committed; the committed state must equal snapshot k and the
    state of a sequential scan over k+1 rows; a following row must see exactly that state."""
    Ly = setup
    d = Ly.dev()
    snap = torch.empty((6, NV, D, D), dtype=torch.float32, device="cuda")
    Ly.call(d, d["rows"], 6, 0, None, snap)
    nxt = torch.from_numpy(Ly.rows[5:6].copy()).cuda(); out_next = torch.empty((1, NV * D), dtype=torch.float32, device="cuda")
    Ly.call(d, nxt, 1, k + 1, out_next, None)          # accept k+1 rows, then one more row
    committed = d["state"].cpu().numpy()
    assert np.array_equal(bits(committed), bits(snap[k].cpu().numpy()))
    st = Ly.state0.copy(); hist = Ly.hist0.copy()
    orc.gdn_rows(Ly.rows[:k + 1], NQK, NV, Ly.conv_w, Ly.dt, Ly.an, Ly.nw, st, hist, Ly.eps, Ly.gate)
    assert np.max(np.abs(committed - st)) / np.max(np.abs(st)) < 1e-5
    assert np.array_equal(bits(committed), bits(st))
    assert np.array_equal(bits(d["conv"].cpu().numpy()), bits(private_conv_state(hist)))
    o2, _ = orc.gdn_rows(Ly.rows[5:6], NQK, NV, Ly.conv_w, Ly.dt, Ly.an, Ly.nw, st, hist, Ly.eps, Ly.gate)
    assert np.array_equal(bits(out_next.cpu().numpy()), bits(o2))


def test_commit_only_call_and_sigmoid_gate():
    Ly = Layer(seed=5, sigmoid_gate=1)
    d = Ly.dev()
    out = torch.empty((4, NV * D), dtype=torch.float32, device="cuda")
    Ly.call(d, d["rows"][:4].contiguous(), 4, 0, out, None)
    Ly.call(d, None, 0, 3, None, None)                   # T = 0: commit 3 rows, nothing else
    st = Ly.state0.copy(); hist = Ly.hist0.copy()
    oo, _ = orc.gdn_rows(Ly.rows[:3], NQK, NV, Ly.conv_w, Ly.dt, Ly.an, Ly.nw, st, hist, Ly.eps, 1)
    assert np.array_equal(bits(d["state"].cpu().numpy()), bits(st))
    assert np.array_equal(bits(out.cpu().numpy()[:3]), bits(oo))


@pytest.mark.parametrize("gate", [0, 1])
def test_kernel_within_1e5_of_the_double_precision_transcription(gate):
    """The stated tolerance of configuration 2 against a checker that owes nothing to this build's kernels: the reference's
    conv + step source (engine/kernels/ops.hip:188-256) evaluated in double precision. Outputs of the 6 rows, every
    per-row state snapshot and the committed state agree within 1e-5 of the largest magnitude."""
    lay = Layer(seed=5, sigmoid_gate=gate)
    d = lay.dev()
    out = torch.zeros((6, NV * D), dtype=torch.float32, device="cuda")
    snap = torch.zeros((6, NV, D, D), dtype=torch.float32, device="cuda")
    lay.call(d, d["rows"], 6, 0, out=out, snap=snap)
    lay.call(d, None, 0, 6)                                   # commit all six rows
    st64 = lay.state0.astype(np.float64); hist64 = lay.hist0.astype(np.float64)
    snaps64 = []
    outs64 = []
    for r in range(6):
        outs64.append(orc.ref64_gdn_rows(lay.rows[r:r + 1], NQK, NV, lay.conv_w.reshape(-1), bf16_to_f32(lay.dt), bf16_to_f32(lay.an), bf16_to_f32(lay.nw),
                                         st64, hist64, lay.eps, gate)[0])
        snaps64.append(st64.copy())
    out64 = np.stack(outs64); snap64 = np.stack(snaps64)
    o = out.cpu().numpy().astype(np.float64); sn = snap.cpu().numpy().astype(np.float64); st = d["state"].cpu().numpy().astype(np.float64)
    assert np.abs(o - out64).max() <= 1e-5 * np.abs(out64).max()
    assert np.abs(sn - snap64).max() <= 1e-5 * np.abs(snap64).max()
    assert np.abs(st - st64).max() <= 1e-5 * np.abs(st64).max()
