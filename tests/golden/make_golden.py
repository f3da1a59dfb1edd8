"""Generates tests/golden/q4k_ref.npz from the reference's OWN host code (engine/src/quant.h compiled into
oracle/_ref/libhipster_ref.so by oracle/Makefile). Run in a container that has the reference checkout:

    make -C oracle && python tests/golden/make_golden.py

The fixture pins the oracle's Q4_K dequantisation, 6-bit scale unpack and f16 conversions on machines where
the reference checkout is absent.
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
sys.path.insert(0, ROOT)
from oracle import orc  # noqa: E402


def main():
    ref = orc.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libhipster_ref.so not built (reference checkout missing?)")
    rng = np.random.default_rng(20240)
    nblk = 40
    blocks = rng.integers(0, 256, size=(nblk, 144), dtype=np.uint8)
    # d, dmin: a spread of normal and subnormal halves, zero, and a negative value
    halves = np.array([0x0000, 0x0001, 0x03FF, 0x0400, 0x1C00, 0x2000, 0x211F, 0x3C00, 0x8400, 0x7BFF], dtype=np.uint16)
    for b in range(nblk):
        blocks[b, 0:2] = np.array([halves[b % len(halves)]], dtype=np.uint16).view(np.uint8)
        blocks[b, 2:4] = np.array([halves[(b * 3 + 1) % len(halves)]], dtype=np.uint16).view(np.uint8)
    blocks[0, 4:16] = 0
    blocks[1, 4:16] = 255
    out = np.empty(nblk * 256, dtype=np.float32)
    for b in range(nblk):   # one "row" of 256 elements per call: dequant_row(12, ...), quant.h:185-187
        ref.ref_dequant_row_q4k(blocks[b].ctypes.data_as(ctypes.c_void_p), out[b * 256:].ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(256))
    sc = np.empty((nblk, 8), dtype=np.uint8); mn = np.empty((nblk, 8), dtype=np.uint8)
    for b in range(nblk):
        for j in range(8):
            d = ctypes.c_uint8(0); m = ctypes.c_uint8(0)
            ref.ref_get_scale_min_k4(j, blocks[b, 4:16].ctypes.data_as(ctypes.c_void_p), ctypes.byref(d), ctypes.byref(m))
            sc[b, j] = d.value; mn[b, j] = m.value
    h_in = np.concatenate([np.arange(0, 65536, 37, dtype=np.uint32), np.array([0, 1, 0x3FF, 0x400, 0x7BFF, 0x7C00, 0x8000, 0xFBFF, 0xFC00], dtype=np.uint32)]).astype(np.uint16)
    h_out = np.array([ref.ref_f16_to_f32(ctypes.c_uint16(int(h))) for h in h_in], dtype=np.float32)
    f_in = np.concatenate([rng.normal(0, 1, 600), rng.normal(0, 1e-3, 200), rng.normal(0, 1e-6, 200), rng.normal(0, 3e4, 100),
                           np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5, 1e30])]).astype(np.float32)
    f_out = np.array([ref.ref_f32_to_f16(float(f)) for f in f_in], dtype=np.uint16)
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "q4k_ref.npz"), blocks=blocks, dequant=out, sc=sc, mn=mn,
                        h_in=h_in, h_out=h_out.view(np.uint32), f_in=f_in.view(np.uint32), f_out=f_out)
    print("wrote q4k_ref.npz", out[:4], sc[2], mn[2])


if __name__ == "__main__":
    main()
