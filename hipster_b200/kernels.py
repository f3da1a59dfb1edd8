"""Kernel-level host API: the Python mirror of the reference's free kernel launchers
(engine/kernels/gemv.h, ops.h). Arguments are torch CUDA tensors; every call goes through the C ABI."""
import ctypes

import torch

from ._lib import lib, check, ptr


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class XQ8:
    """Quantised activations (reference: struct XQ8, engine/kernels/gemv.h:8) in the library's private layout."""

    def __init__(self, R, K, device="cuda"):
        L = lib()
        self.R, self.K = R, K
        self.q = torch.zeros(L.hp_xq8_q_bytes(R, K), dtype=torch.uint8, device=device)
        self.sc = torch.zeros(L.hp_xq8_sc_bytes(R, K), dtype=torch.uint8, device=device)

    def unpack(self):
        """-> (q int8 [R][K], d f32 [R][K/32], s f32 [R][K/32]) in the reference's row layout."""
        q = torch.empty((self.R, self.K), dtype=torch.int8, device=self.q.device)
        d = torch.empty((self.R, self.K // 32), dtype=torch.float32, device=self.q.device)
        s = torch.empty_like(d)
        check(lib().hp_xq8_unpack(ptr(self.q), ptr(self.sc), self.R, self.K, ptr(q), ptr(d), ptr(s), _stream()))
        return q, d, s


def quantize_x_q8(x, xq=None):
    """x f32 [R][K] -> XQ8 (reference quantize_x_q8, gemv.h:9)."""
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    R, K = x.shape
    xq = xq or XQ8(R, K, x.device)
    check(lib().hp_quantize_x_q8(ptr(x), x.stride(0), R, K, ptr(xq.q), ptr(xq.sc), _stream()))
    return xq


def dequant_q4k(w, nblk):
    out = torch.empty(nblk * 256, dtype=torch.float32, device=w.device)
    check(lib().hp_dequant_q4k(ptr(w), ctypes.c_size_t(nblk), ptr(out), _stream()))
    return out


def gemv_q4k_q8(w, xq, N, K, y=None):
    """y [R][N] = W . x for Q4_K W [N][K/256 blocks] (uint8 tensor) and quantised x (reference gemv_wmma, gemv.h:33)."""
    R = xq.R
    if y is None:
        y = torch.empty((R, N), dtype=torch.float32, device=w.device)
    check(lib().hp_gemv_q4k_q8(ptr(w), ptr(xq.q), ptr(xq.sc), ptr(y), N, K, R, y.stride(0), _stream()))
    return y


def gemv_q4k_f32(w, x, N, K):
    """f32-activation baseline (reference gemv_q4_K_f32, gemv.h:57)."""
    R = x.shape[0]
    y = torch.empty((R, N), dtype=torch.float32, device=w.device)
    check(lib().hp_gemv_q4k_f32(ptr(w), ptr(x), ptr(y), N, K, R, _stream()))
    return y


def argmax(logits, n=None):
    """Row-wise argmax (max value, lowest index) -> (ids int32 [R], vals f32 [R]) (reference argmax_topk k=1, ops.h:118)."""
    R, ld = logits.shape[0], logits.stride(0)
    n = n or logits.shape[1]
    ids = torch.empty(R, dtype=torch.int32, device=logits.device)
    vals = torch.empty(R, dtype=torch.float32, device=logits.device)
    scratch = torch.empty(lib().hp_argmax_scratch_bytes(R, n), dtype=torch.uint8, device=logits.device)
    check(lib().hp_argmax(ptr(logits), R, n, ld, ptr(ids), ptr(vals), ptr(scratch), _stream()))
    return ids, vals


def argmax_noalloc(logits, n=None):
    """argmax() for callers that cannot allocate device memory: the library's built-in scratch holds the partial
    results, so the call takes only the input and the two output tensors (created by the caller beforehand)."""
    R, ld = logits.shape[0], logits.stride(0)
    n = n or logits.shape[1]
    ids = torch.empty(R, dtype=torch.int32, device=logits.device)
    vals = torch.empty(R, dtype=torch.float32, device=logits.device)
    check(lib().hp_argmax_noalloc(ptr(logits), R, n, ld, ptr(ids), ptr(vals), _stream()))
    return ids, vals


def accept_greedy(ids, drafts):
    """-> int32 tensor [mm, bonus] on device (reference host loop, engine/bench/spec27b.cpp:92-97)."""
    out = torch.empty(2, dtype=torch.int32, device=ids.device)
    check(lib().hp_accept_greedy(ptr(ids), ptr(drafts), int(drafts.numel()), ptr(out), _stream()))
    return out


def device_status():
    check(lib().hp_device_status(_stream()))


def attn_decode(qkv, pos0, n_head, n_kv, n_rot, q_norm, k_norm, rope, kc, vc, max_ctx, eps=1e-6, want_q8=True):
    """GQA decode attention of one sequence: qkv f32 [R][ld] (normalised / rotated in place), rows at positions pos0 + r;
    q_norm / k_norm bf16 [256] (int16 tensors), rope f32 [max_ctx][n_rot/2][2], kc / vc f16 [n_kv][max_ctx][256] (updated).
    -> (out f32 [R][n_head*256], XQ8 of it or None). Reference: qk_norm_rope_kv + attn_decode_mq (ops.h:71-72,96)."""
    L = lib()
    L.hp_attn_workspace_bytes.restype = ctypes.c_size_t
    R, ld = qkv.shape[0], qkv.stride(0)
    ws = torch.empty(L.hp_attn_workspace_bytes(R, n_head, n_kv, max_ctx), dtype=torch.uint8, device=qkv.device)
    out = torch.empty((R, n_head * 256), dtype=torch.float32, device=qkv.device)
    xq = XQ8(R, n_head * 256, qkv.device) if want_q8 else None
    check(L.hp_attn_decode(ptr(qkv), ld, R, int(pos0), n_head, n_kv, n_rot, ptr(q_norm), ptr(k_norm), ptr(rope), ptr(kc), ptr(vc), int(max_ctx), ptr(out),
                           ptr(xq.q) if xq else None, ptr(xq.sc) if xq else None, ctypes.c_float(eps), ptr(ws), _stream()))
    return out, xq


def repack_tiled(w, N, K, interleave_half=0):
    """ggml Q4_K [N][K/256 blocks] (uint8 tensor) -> the library's tile-major streaming layout (same bytes, permuted)."""
    L = lib()
    L.hp_q4k_tiled_bytes.restype = ctypes.c_size_t
    L.hp_q4k_tiled_bytes.argtypes = [ctypes.c_size_t, ctypes.c_int]
    out = torch.empty(L.hp_q4k_tiled_bytes(N, K), dtype=torch.uint8, device=w.device)
    check(L.hp_q4k_repack_tiled(ptr(w), ptr(out), ctypes.c_size_t(N), K, interleave_half, _stream()))
    return out


def moe_layer(xn, router, exp_gate_up, exp_down, sh_gate_up, sh_down, F, n_expert, k):
    """One mixture-of-experts FFN over the rows of xn f32 [T][E] -> (ids int32 [T][k+1], weights f32 [T][k+1], y f32 [T][E]).
    The expert tensors are given in ggml order and repacked here (an engine does that once at load).
    Reference: Qwen4Exp::moe_layer (qwen4exp.cpp:345-354)."""
    L = lib()
    L.hp_moe_workspace_bytes.restype = ctypes.c_size_t
    T, E = xn.shape
    xq = quantize_x_q8(xn)
    egu = repack_tiled(exp_gate_up, n_expert * 2 * F, E, F); edn = repack_tiled(exp_down, n_expert * E, F, 0)
    sgu = repack_tiled(sh_gate_up, 2 * F, E, F); sdn = repack_tiled(sh_down, E, F, 0)
    ws = torch.empty(L.hp_moe_workspace_bytes(T, E, F, n_expert, k), dtype=torch.uint8, device=xn.device)
    ids = torch.empty((T, k + 1), dtype=torch.int32, device=xn.device)
    w = torch.empty((T, k + 1), dtype=torch.float32, device=xn.device)
    y = torch.empty((T, E), dtype=torch.float32, device=xn.device)
    check(L.hp_moe_layer(ptr(xn), ptr(xq.q), ptr(xq.sc), ptr(router), ptr(egu), ptr(edn), ptr(sgu), ptr(sdn), T, E, F, n_expert, k,
                         ptr(ids), ptr(w), ptr(y), ptr(ws), _stream()))
    return ids, w, y
