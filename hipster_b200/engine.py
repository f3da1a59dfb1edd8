"""Engine-level host API: Python mirror of the reference's engine classes (class Qwen35, engine/src/qwen35.h:50-98;
class Qwen4Exp, engine/src/qwen4exp.h:54-90) over the C ABI. The engine itself is C++/CUDA inside libhipster_b200.so."""
import ctypes

import numpy as np

from ._lib import lib, check

TENSOR_KINDS = dict(attn_norm=0, post_norm=1, in_proj=2, out_proj=3, gate_up=4, down=5, conv_w=6, dt_bias=7, a_neg=8, ssm_norm=9,
                    q_norm=10, k_norm=11, router=12, exp_gate_up=13, exp_down=14, sh_gate_up=15, sh_down=16,
                    embed=32, output_norm=33, lm_head=34, mtp_enorm=35, mtp_hnorm=36, mtp_eh_proj=37, mtp_head_norm=38)


class ModelCfg(ctypes.Structure):
    """struct hp_model_cfg (include/hipster_b200.h)."""
    _fields_ = [(n, ctypes.c_int) for n in ("n_embd", "n_layer", "n_ff", "n_vocab", "n_head", "n_head_kv", "n_rot", "gdn_qk_heads", "gdn_v_heads",
                                             "attn_every", "max_ctx", "n_slots", "n_expert", "n_expert_used", "expert_ff", "gdn_sigmoid_gate", "has_mtp", "ep_rank", "ep_world", "synth_router_logits")] + \
               [("rms_eps", ctypes.c_float), ("rope_base", ctypes.c_float), ("seed", ctypes.c_ulonglong)]

    @classmethod
    def preset(cls, name, **over):
        c = cls()
        check(lib().hp_model_preset(name.encode(), ctypes.byref(c)))
        for k, v in over.items():
            setattr(c, k, v)
        return c


class SlotReq(ctypes.Structure):
    """struct hp_slot_req == the reference's SlotReq (engine/kernels/ops.h:40)."""
    _fields_ = [("slot", ctypes.c_int), ("tokens", ctypes.POINTER(ctypes.c_int)), ("T", ctypes.c_int), ("pos", ctypes.c_int)]


class Engine:
    def __init__(self, cfg):
        L = lib()
        L.hp_weight_bytes.restype = ctypes.c_size_t
        L.hp_last_ms.restype = ctypes.c_float
        for n in ("hp_logits_dev", "hp_h_nextn_dev", "hp_mtp_logits_dev", "hp_mtp_h_dev"):
            getattr(L, n).restype = ctypes.c_void_p
        self.cfg = cfg
        self._h = ctypes.c_void_p()
        check(L.hp_load(ctypes.byref(cfg), ctypes.byref(self._h)))

    def close(self):
        if self._h:
            lib().hp_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- reference API
    def forward(self, reqs):
        """reqs: list of (slot, tokens, pos) -> GPU ms. Qwen35::forward(const SlotReq*, int)."""
        arr = (SlotReq * len(reqs))()
        keep = []
        for i, (slot, toks, pos) in enumerate(reqs):
            t = (ctypes.c_int * len(toks))(*[int(x) for x in toks]); keep.append(t)
            arr[i] = SlotReq(slot, t, len(toks), pos)
        ms = ctypes.c_float(0)
        check(lib().hp_forward(self._h, arr, len(reqs), ctypes.byref(ms)))
        return ms.value

    def accept(self, slot, m):
        check(lib().hp_accept(self._h, slot, m))

    def mtp_forward(self, slot, tokens, h_dev_ptr, pos0):
        t = (ctypes.c_int * len(tokens))(*[int(x) for x in tokens])
        check(lib().hp_mtp_forward(self._h, slot, t, ctypes.c_void_p(h_dev_ptr), len(tokens), pos0))

    def mtp_forward_slots(self, reqs, h_dev_ptr):
        """reqs: list of (slot, tokens, pos); h_dev_ptr: one row of n_embd floats per request row. Qwen4Exp::mtp_forward(reqs, S, h)."""
        arr = (SlotReq * len(reqs))()
        keep = []
        for i, (slot, toks, pos) in enumerate(reqs):
            t = (ctypes.c_int * len(toks))(*[int(x) for x in toks]); keep.append(t)
            arr[i] = SlotReq(slot, t, len(toks), pos)
        check(lib().hp_mtp_forward_slots(self._h, arr, len(reqs), ctypes.c_void_p(h_dev_ptr)))

    def ep_init(self, id128):
        buf = (ctypes.c_char * 128).from_buffer_copy(bytes(id128))
        check(lib().hp_ep_init(self._h, buf))

    def topk(self, which, T, k=1):
        """Qwen35::topk: (ids, vals) of shape [T] for k = 1, [T][k] otherwise (values descending, ties -> lower id)."""
        ids = (ctypes.c_int * (T * k))(); vals = (ctypes.c_float * (T * k))()
        check(lib().hp_topk(self._h, which, T, k, ids, vals))
        i = np.array(ids[:], dtype=np.int32); v = np.array(vals[:], dtype=np.float32)
        return (i, v) if k == 1 else (i.reshape(T, k), v.reshape(T, k))

    def prefill(self, slot, tokens, pos0=0, with_mtp=True):
        """Qwen4Exp::prefill + mtp_catchup: commits the prompt; row 0 of logits / h_nextn / topk is the last prompt row."""
        t = (ctypes.c_int * len(tokens))(*[int(x) for x in tokens])
        check(lib().hp_prefill(self._h, slot, t, len(tokens), pos0, int(with_mtp)))

    def reset(self):
        check(lib().hp_reset(self._h))

    def reset_slot(self, s):
        check(lib().hp_reset_slot(self._h, s))

    def n_slots(self):
        return lib().hp_n_slots(self._h)

    def weight_bytes(self):
        return lib().hp_weight_bytes(self._h)

    def last_ms(self):
        return lib().hp_last_ms(self._h)

    # device pointers (ints)
    def logits_ptr(self):
        return lib().hp_logits_dev(self._h)

    def h_nextn_ptr(self):
        return lib().hp_h_nextn_dev(self._h)

    def mtp_logits_ptr(self):
        return lib().hp_mtp_logits_dev(self._h)

    def mtp_h_ptr(self):
        return lib().hp_mtp_h_dev(self._h)

    # ---- helpers for tests / benchmarks (device -> host through torch)
    def _fetch(self, ptr, nfloat):
        import torch
        out = torch.empty(nfloat, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        _memcpy_d2d(out.data_ptr(), ptr, nfloat * 4)
        return out.cpu().numpy()

    def logits(self, T):
        return self._fetch(self.logits_ptr(), T * self.cfg.n_vocab).reshape(T, self.cfg.n_vocab)

    def h_nextn(self, T):
        return self._fetch(self.h_nextn_ptr(), T * self.cfg.n_embd).reshape(T, self.cfg.n_embd)

    def mtp_logits(self, T):
        return self._fetch(self.mtp_logits_ptr(), T * self.cfg.n_vocab).reshape(T, self.cfg.n_vocab)

    def mtp_h(self, T):
        return self._fetch(self.mtp_h_ptr(), T * self.cfg.n_embd).reshape(T, self.cfg.n_embd)

    def tensor(self, layer, kind):
        p = ctypes.c_void_p(); n = ctypes.c_size_t()
        check(lib().hp_tensor_dev(self._h, layer, TENSOR_KINDS[kind], ctypes.byref(p), ctypes.byref(n)))
        import torch
        out = torch.empty(n.value, dtype=torch.uint8, device="cuda")
        _memcpy_d2d(out.data_ptr(), p.value, n.value)
        return out.cpu().numpy()

    def gdn_state(self, slot, gdn_layer):
        p = ctypes.c_void_p(); n = ctypes.c_size_t()
        check(lib().hp_gdn_state_dev(self._h, slot, gdn_layer, ctypes.byref(p), ctypes.byref(n)))
        return self._fetch(p.value, n.value // 4)

    def profile_pass(self, R, what, reps):
        ms = ctypes.c_float(0)
        check(lib().hp_profile_pass(self._h, R, what, reps, ctypes.byref(ms)))
        return ms.value

    def pass_weight_bytes(self, mtp, with_head):
        lib().hp_pass_weight_bytes.restype = ctypes.c_size_t
        return lib().hp_pass_weight_bytes(self._h, int(mtp), int(with_head))

    def moe_touched(self):
        """(layer, expert) matrices touched by the passes since the last call."""
        n = ctypes.c_ulonglong(0)
        check(lib().hp_moe_touched(self._h, ctypes.byref(n)))
        return n.value

    def ep_exchange_us(self, R, reps=20):
        us = ctypes.c_float(0)
        check(lib().hp_ep_exchange_us(self._h, R, reps, ctypes.byref(us)))
        return us.value

    def ep_peer(self):
        """True when the expert-parallel exchange runs over peer memory, False when it is the NCCL collective."""
        return bool(lib().hp_ep_peer(self._h))

    def last_round_kernels(self):
        return lib().hp_last_round_kernels(self._h)

    # ---- fused device-side round
    def spec_begin(self, slot, id_last, pos, h_pending_ptr):
        check(lib().hp_spec_begin(self._h, slot, int(id_last), int(pos), ctypes.c_void_p(h_pending_ptr)))

    def spec_round(self, slot, n_draft, subst=None):
        """One slot: the emitted tokens of the round."""
        return self.spec_round_slots([slot], n_draft, None if subst is None else [subst])[0]

    def spec_round_slots(self, slots, n_draft, subst=None):
        """S slots in lock step; subst: per slot a list of n_draft substitutions (or None). -> per slot the emitted tokens."""
        S = len(slots)
        sl = (ctypes.c_int * S)(*[int(x) for x in slots])
        out = (ctypes.c_int * (S * (n_draft + 1)))(); cnt = (ctypes.c_int * S)()
        sub = None
        if subst is not None:
            sub = (ctypes.c_int * (S * n_draft))(*[int(x) for row in subst for x in row])
        check(lib().hp_spec_round(self._h, sl, S, n_draft, sub, out, cnt))
        return [list(out[j * (n_draft + 1):j * (n_draft + 1) + cnt[j]]) for j in range(S)]


def _memcpy_d2d(dst, src, nbytes):
    """Device-to-device copy on torch's current stream, followed by a synchronise (test/bench helper)."""
    import torch
    src_t = _as_tensor(src, nbytes)
    dst_t = _as_tensor(dst, nbytes)
    torch.cuda.synchronize()
    dst_t.copy_(src_t)
    torch.cuda.synchronize()


def _as_tensor(ptr, nbytes):
    import torch

    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}
    return torch.as_tensor(h, device="cuda")
