"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (random BCQ layers stand in for real checkpoints, as
in the reference's own benchmark, tests/opt/fp16/int3_col_wise_matmul_fp16.cu:191-215,
which also draws random planes and scales).

All arrays are numpy, C-contiguous, in the kernel layout:
  bW uint32 [K/32, q, N]; alpha float32 [G, q, N] (exactly representable in fp16);
  q_bias float32 [G, N] or None; x float16 [M, K].
"""
import zlib

import numpy as np


def seed_for(tag, N, K, q, extra=0):
    return zlib.crc32(f"{tag}:{N}:{K}:{q}:{extra}".encode()) & 0x7FFFFFFF


def activations(M, K, seed):
    """fp16 round of N(0, 1)."""
    rng = np.random.default_rng(seed ^ 0x5A5A)
    return rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)


def bcq_layer(N, K, q, group_size, seed, alpha_std=0.02, with_bias=False, signed_alpha=False):
    """Random BCQ layer: fair +-1 planes packed 32 per word along k (bit k%32 set <=> +1),
    alpha = fp16(|N(0, alpha_std)|) per (group, plane, column)."""
    assert K % 32 == 0 and K % group_size == 0
    rng = np.random.default_rng(seed)
    G = K // group_size
    bW = rng.integers(0, 2**32, size=(K // 32, q, N), dtype=np.uint32)
    a = rng.standard_normal((G, q, N), dtype=np.float32) * alpha_std
    if not signed_alpha:
        a = np.abs(a)
    alpha = a.astype(np.float16).astype(np.float32)
    q_bias = None
    if with_bias:
        q_bias = (rng.standard_normal((G, N), dtype=np.float32) * alpha_std).astype(np.float16).astype(np.float32)
    return bW, alpha, q_bias


def uniform_layer(N, K, q, group_size, seed, scale_std=0.01):
    """Uniform (round-to-nearest style) quantised layer in the Python examples' shapes:
    scale float32 [N, G] = fp16(|N(0, scale_std)|), zero float32 [N, G] integer in [0, 2^q - 1],
    code int32 [N, G, g] uniform in [0, 2^q - 1]."""
    rng = np.random.default_rng(seed)
    G = K // group_size
    scale = np.abs(rng.standard_normal((N, G), dtype=np.float32) * scale_std).astype(np.float16).astype(np.float32)
    scale = np.maximum(scale, np.float32(2.0 ** -14))
    zero = rng.integers(0, 2**q, size=(N, G)).astype(np.float32)
    code = rng.integers(0, 2**q, size=(N, G, group_size), dtype=np.int32)
    return scale, zero, code


def algorithmic_bytes(N, K, q, group_size, M=1, with_bias=False):
    """Bytes one matmul must move: packed planes + alpha (+ q_bias) + x + y."""
    G = K // group_size
    return N * K * q // 8 + 2 * G * q * N + (2 * G * N if with_bias else 0) + 2 * M * K + 2 * M * N
