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
                                             "attn_every", "max_ctx", "n_slots", "n_expert", "n_expert_used", "expert_ff", "gdn_sigmoid_gate", "has_mtp", "ep_rank", "ep_world", "synth_router_logits")] + \
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


def topk(logits, k):
    logits = np.ascontiguousarray(logits, dtype=np.float32); R, n = logits.shape
    ids = np.empty((R, k), dtype=np.int32); vals = np.empty((R, k), dtype=np.float32)
    lib().orc_topk(P(logits), R, n, n, k, P(ids), P(vals))
    return ids, vals


def rope_table(max_ctx, n_rot, base):
    """(cos, sin) of pos * base^(-2i/n_rot) computed in double precision and rounded to f32, [max_ctx][n_rot/2][2]."""
    half = n_rot // 2
    p = np.arange(max_ctx, dtype=np.float64)[:, None]
    th = p * np.power(np.float64(np.float32(base)), -2.0 * np.arange(half, dtype=np.float64) / n_rot)[None, :]
    return np.stack([np.cos(th), np.sin(th)], axis=-1).astype(np.float32)


def attn_row(qkv_row, n_head, n_kv, n_rot, qw, kw, rope, pos, kc, vc, max_ctx, eps):
    """Bit-exact restatement of the attention step for one row (updates qkv_row, kc, vc in place) -> out [n_head*256]."""
    out = np.empty(n_head * 256, dtype=np.float32)
    lib().orc_attn_row(P(qkv_row), n_head, n_kv, n_rot, P(qw), P(kw), P(rope), int(pos), P(kc), P(vc), int(max_ctx), P(out), ctypes.c_float(eps))
    return out


def moe_layer(xn, router, exp_gate_up, exp_down, sh_gate_up, sh_down, E, F, n_expert, k):
    """Bit-exact restatement of one MoE FFN (router -> route -> per-(row, slot) expert GEMVs -> combine in slot order).
    -> (ids [T][k+1], w [T][k+1], y [T][E])."""
    L = lib()
    xn = np.ascontiguousarray(xn, dtype=np.float32); T = xn.shape[0]; ns = k + 1
    lg = np.empty((T, n_expert + 1), dtype=np.float32)
    L.orc_router_gemv(P(router), P(xn), P(lg), n_expert + 1, E, T)
    ids = np.empty((T, ns), dtype=np.int32); w = np.empty((T, ns), dtype=np.float32)
    L.orc_moe_route(P(lg), P(ids), P(w), T, n_expert, k)
    q, d, s = quantize_x_q8(xn)
    eb_up = 2 * F * (E // 256) * 144; eb_dn = E * (F // 256) * 144
    y = np.zeros((T, E), dtype=np.float32)
    gu = np.empty(2 * F, dtype=np.float32); v = np.empty(E, dtype=np.float32)
    sil = L.orc_silu
    for t in range(T):
        acc = np.zeros(E, dtype=np.float32)
        for e in range(ns):
            i = int(ids[t, e])
            Wu = exp_gate_up[i * eb_up:(i + 1) * eb_up] if i >= 0 else sh_gate_up
            Wd = exp_down[i * eb_dn:(i + 1) * eb_dn] if i >= 0 else sh_down
            L.orc_gemv_q4k_q8_seq(P(Wu), P(q[t]), P(d[t]), P(s[t]), P(gu), 2 * F, E)
            act = np.empty((1, F), dtype=np.float32)
            L.orc_silu_mul(P(gu), P(act), F)
            aq, ad, as_ = quantize_x_q8(act)
            L.orc_gemv_q4k_q8_seq(P(Wd), P(aq), P(ad), P(as_), P(v), E, F)
            L.orc_fma_rows(P(acc), P(v), ctypes.c_float(float(w[t, e])), E)
        y[t] = acc
    return ids, w, y, lg


# ---- independent double-precision transcriptions of the reference's device source (hp_oracle_ref64.cpp): tolerance checks
def ref64_gdn_rows(rows, n_qk, n_v, conv_w, dt_bias, a_neg, norm_w, state, conv_hist, eps, sigmoid_gate):
    """rows f32 [T][ld]; conv_w / dt_bias / a_neg / norm_w f32; state f64 [n_v][128][128] and conv_hist f64 [3][C] are
    updated in place -> out f64 [T][n_v*128]."""
    rows = np.ascontiguousarray(rows, dtype=np.float32); T, ld = rows.shape
    out = np.empty((T, n_v * 128), dtype=np.float64)
    lib().ref64_gdn_rows(P(rows), ld, T, n_qk, n_v, P(conv_w), P(dt_bias), P(a_neg), P(norm_w), P(state), P(conv_hist), P(out), ctypes.c_double(eps), int(sigmoid_gate))
    return out


def ref64_attn_row(qkv_row, n_head, n_kv, n_rot, qw, kw, base, pos, kc, vc, max_ctx, eps):
    """qkv_row f32 (not modified); qw / kw f32; kc / vc f32 [n_kv][max_ctx][256] holding f16-representable values,
    updated in place -> out f64 [n_head*256]."""
    out = np.empty(n_head * 256, dtype=np.float64)
    lib().ref64_attn_row(P(qkv_row), n_head, n_kv, n_rot, P(qw), P(kw), ctypes.c_float(base), int(pos), P(kc), P(vc), int(max_ctx), P(out), ctypes.c_double(eps))
    return out


def ref64_moe_route(logits, E, k):
    logits = np.ascontiguousarray(logits, dtype=np.float32); T = logits.shape[0]
    ids = np.empty((T, k + 1), dtype=np.int32); w = np.empty((T, k + 1), dtype=np.float64)
    lib().ref64_moe_route(P(logits), P(ids), P(w), T, E, k)
    return ids, w
