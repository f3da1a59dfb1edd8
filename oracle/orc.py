"""ctypes loader of the CPU oracle (TEST INFRASTRUCTURE: imported only by tests/, the smoke check and the
CPU-baseline leg of bench.py; the product package never imports this module)."""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhp_oracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libhipster_ref.so")

_lib = None
_ref = None


def build():
    subprocess.run(["make", "-C", HERE, "-s"], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
        for name in ("orc_f16_to_f32", "orc_expf", "orc_log1pf_pos", "orc_sigmoid", "orc_silu", "orc_softplus"):
            getattr(_lib, name).restype = ctypes.c_float
        for name in ("orc_expf", "orc_log1pf_pos", "orc_sigmoid", "orc_silu", "orc_softplus"):
            getattr(_lib, name).argtypes = [ctypes.c_float]
        _lib.orc_f32_to_f16.restype = ctypes.c_uint16
        _lib.orc_f32_to_f16.argtypes = [ctypes.c_float]
    return _lib


def ref():
    """The reference's own host code (None when oracle/_ref was not built)."""
    global _ref
    if _ref is None and os.path.exists(REF_PATH):
        _ref = ctypes.CDLL(REF_PATH)
        _ref.ref_f16_to_f32.restype = ctypes.c_float
        _ref.ref_f32_to_f16.restype = ctypes.c_uint16
        _ref.ref_f32_to_f16.argtypes = [ctypes.c_float]
    return _ref


def P(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def dequant_q4k(blocks):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    nblk = blocks.size // 144
    out = np.empty(nblk * 256, dtype=np.float32)
    lib().orc_dequant_q4k(P(blocks), ctypes.c_size_t(nblk), P(out))
    return out


def quantize_x_q8(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    q = np.empty((R, K), dtype=np.int8); d = np.empty((R, K // 32), dtype=np.float32); s = np.empty_like(d)
    lib().orc_quantize_x_q8(P(x), R, K, P(q), P(d), P(s))
    return q, d, s


def gemv_q4k_f32(W, x, N, K, tpr=4):
    x = np.ascontiguousarray(x, dtype=np.float32); R = x.shape[0]
    y = np.empty((R, N), dtype=np.float32)
    lib().orc_gemv_q4k_f32(P(W), P(x), P(y), N, K, R, tpr)
    return y


def gemv_q4k_q8(W, q, d, s, N, K):
    R = q.shape[0]
    y = np.empty((R, N), dtype=np.float32)
    lib().orc_gemv_q4k_q8(P(W), P(np.ascontiguousarray(q)), P(np.ascontiguousarray(d)), P(np.ascontiguousarray(s)), P(y), N, K, R, N)
    return y


def gemv_q4k_double(W, x, N, K):
    x = np.ascontiguousarray(x, dtype=np.float32); R = x.shape[0]
    y = np.empty((R, N), dtype=np.float64); mag = np.empty((R, N), dtype=np.float64)
    lib().orc_gemv_q4k_double(P(W), P(x), P(y), P(mag), N, K, R)
    return y, mag


def argmax(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32); R, n = logits.shape
    ids = np.empty(R, dtype=np.int32); vals = np.empty(R, dtype=np.float32)
    lib().orc_argmax(P(logits), R, n, n, P(ids), P(vals))
    return ids, vals


def accept(ids, drafts):
    ids = np.ascontiguousarray(ids, dtype=np.int32); drafts = np.ascontiguousarray(drafts, dtype=np.int32)
    bonus = ctypes.c_int(0)
    mm = lib().orc_accept(P(ids), P(drafts), int(drafts.size), ctypes.byref(bonus))
    return mm, bonus.value


# ---------------------------------------------------------------- engine oracle (hp_oracle_model.cpp)
class OrcCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("n_embd", "n_layer", "n_ff", "n_vocab", "n_head", "n_head_kv", "n_rot", "gdn_qk_heads", "gdn_v_heads",
                                             "attn_every", "max_ctx", "n_slots", "n_expert", "n_expert_used", "expert_ff", "gdn_sigmoid_gate", "has_mtp", "ep_rank", "ep_world")] + \
               [("rms_eps", ctypes.c_float), ("rope_base", ctypes.c_float), ("seed", ctypes.c_ulonglong)]


class Model:
    """CPU restatement of the reference engine (engine/src/qwen35.cpp) on the same seeded weights."""

    def __init__(self, cfg):
        L = lib()
        L.orc_model_create.restype = ctypes.c_void_p
        for n in ("orc_model_logits", "orc_model_h", "orc_model_mtp_logits", "orc_model_mtp_h", "orc_model_gdn_state"):
            getattr(L, n).restype = ctypes.POINTER(ctypes.c_float)
        L.orc_model_tensor.restype = ctypes.c_size_t
        c = OrcCfg()
        for f, _ in OrcCfg._fields_:
            setattr(c, f, getattr(cfg, f))
        self.c = c
        self.h = ctypes.c_void_p(L.orc_model_create(ctypes.byref(c)))
        assert self.h

    def __del__(self):
        try:
            lib().orc_model_free(self.h)
        except Exception:
            pass

    def reset(self):
        lib().orc_model_reset(self.h)

    def reset_slot(self, s):
        lib().orc_model_reset_slot(self.h, s)

    def forward(self, reqs):
        S = len(reqs)
        slots = (ctypes.c_int * S)(*[r[0] for r in reqs]); Ts = (ctypes.c_int * S)(*[len(r[1]) for r in reqs]); poss = (ctypes.c_int * S)(*[r[2] for r in reqs])
        bufs = [(ctypes.c_int * len(r[1]))(*[int(x) for x in r[1]]) for r in reqs]
        toks = (ctypes.POINTER(ctypes.c_int) * S)(*[ctypes.cast(b, ctypes.POINTER(ctypes.c_int)) for b in bufs])
        lib().orc_model_forward(self.h, slots, toks, Ts, poss, S)

    def accept(self, slot, m):
        assert lib().orc_model_accept(self.h, slot, m) == 0

    def mtp_forward(self, slot, tokens, h_in, pos0):
        t = (ctypes.c_int * len(tokens))(*[int(x) for x in tokens])
        h_in = np.ascontiguousarray(h_in, dtype=np.float32)
        lib().orc_model_mtp_forward(self.h, slot, t, P(h_in), len(tokens), pos0)

    def _arr(self, fn, n, *a):
        return np.ctypeslib.as_array(getattr(lib(), fn)(self.h, *a), shape=(n,)).copy()

    def logits(self, T):
        return self._arr("orc_model_logits", T * self.c.n_vocab).reshape(T, -1)

    def h_nextn(self, T):
        return self._arr("orc_model_h", T * self.c.n_embd).reshape(T, -1)

    def mtp_logits(self, T):
        return self._arr("orc_model_mtp_logits", T * self.c.n_vocab).reshape(T, -1)

    def mtp_h(self, T):
        return self._arr("orc_model_mtp_h", T * self.c.n_embd).reshape(T, -1)

    def gdn_state(self, slot, gdn_layer):
        return self._arr("orc_model_gdn_state", self.c.gdn_v_heads * 128 * 128, slot, gdn_layer)

    def tensor(self, layer, kind_id):
        p = ctypes.c_void_p()
        n = lib().orc_model_tensor(self.h, layer, kind_id, ctypes.byref(p))
        return np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint8)), shape=(n,)).copy()


def gdn_rows(rows, n_qk, n_v, conv_w, dt_bias, a_neg, norm_w, state, conv_hist, eps, sigmoid_gate, want_snap=False):
    """Sequential conv + delta-rule step over the rows of one sequence (updates state / conv_hist in place)."""
    rows = np.ascontiguousarray(rows, dtype=np.float32); T, ld = rows.shape
    out = np.empty((T, n_v * 128), dtype=np.float32)
    snap = np.empty((T, n_v, 128, 128), dtype=np.float32) if want_snap else None
    lib().orc_gdn_rows(P(rows), ld, T, n_qk, n_v, P(conv_w), P(dt_bias), P(a_neg), P(norm_w), P(state), P(conv_hist), P(out),
                       P(snap) if want_snap else ctypes.c_void_p(0), ctypes.c_float(eps), int(sigmoid_gate))
    return out, snap
