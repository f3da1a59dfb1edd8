"""Seeded synthetic inputs with the shapes and value distributions the benchmark configurations state.

They stand in for the reference's real-checkpoint tensors (no checkpoints or datasets are used):
Q4_K super-blocks with uniform 4-bit quants, uniform 6-bit sub-block scales/mins and fp16 d, dmin = |N(0, 0.01)|;
activations N(0, 1).
"""
import numpy as np


def q4k_matrix(N, K, seed):
    """Random Q4_K weight matrix [N][K/256] blocks of 144 bytes -> uint8 array [N, K/256*144]."""
    assert K % 256 == 0
    rng = np.random.default_rng(seed)
    nb = K // 256
    blk = np.empty((N, nb, 144), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, 0.01, size=(N, nb, 2))).astype(np.float16)
    blk[:, :, 0:4] = d.view(np.uint8).reshape(N, nb, 4)
    # 12 bytes of packed 6-bit fields: every bit pattern is a valid, uniform choice of the 8 scales and 8 mins
    blk[:, :, 4:16] = rng.integers(0, 256, size=(N, nb, 12), dtype=np.uint8)
    blk[:, :, 16:144] = rng.integers(0, 256, size=(N, nb, 128), dtype=np.uint8)
    return blk.reshape(N, nb * 144)


def activations(R, K, seed):
    return np.random.default_rng(seed).normal(0.0, 1.0, size=(R, K)).astype(np.float32)
