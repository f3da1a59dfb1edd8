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
