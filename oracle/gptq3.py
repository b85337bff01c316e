"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference's 3-bit uniform (GPTQ-format) matvec.

Follows VecQuant3MatMulKernel (lutGEMM/src/cuda/kernels/gptq_fp16_bias.hpp:27-105): per column,
res += (scale * code - zero) * x[k] over the 32 codes of every three packed words, code j of a group being bits
3j..3j+2 of the little-endian 96-bit string w0 | w1 << 32 | w2 << 64 (the kernel's tmp1 >> 30 | (tmp2 << 2) & 4 and
tmp2 >> 30 | (tmp1 << 1) & 6 are codes 10 and 21, the ones that straddle words).  The reference accumulates in
fp16; this restatement accumulates in float64 and is the value the fp32 kernel is held to.  The reference has no
CPU implementation and no test vectors for this kernel: parity is pinned on the GPU, against the reference's own
kernels compiled into oracle/_ref/libref_gpu.so, at fp16 accuracy.
"""
import numpy as np


def pack(codes):
    """codes int [K, N] in 0..7 -> uint32 [K*3/32, N]."""
    K, N = codes.shape
    assert K % 32 == 0
    c = codes.reshape(K // 32, 32, N).astype(np.uint64)
    lo = np.zeros((K // 32, N), np.uint64)
    hi = np.zeros((K // 32, N), np.uint64)
    for j in range(32):
        bit = 3 * j
        if bit + 3 <= 64:
            lo |= c[:, j] << np.uint64(bit)
        elif bit >= 64:
            hi |= c[:, j] << np.uint64(bit - 64)
        else:                                   # code 21: bits 63..65
            lo |= (c[:, j] & np.uint64(1)) << np.uint64(63)
            hi |= c[:, j] >> np.uint64(1)
    out = np.empty((K // 32, 3, N), np.uint32)
    out[:, 0] = (lo & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    out[:, 1] = (lo >> np.uint64(32)).astype(np.uint32)
    out[:, 2] = (hi & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    return out.reshape(K * 3 // 32, N)


def unpack(mat):
    """uint32 [K*3/32, N] -> codes int32 [K, N], following the kernel's shifts."""
    KP, N = mat.shape
    g = mat.reshape(KP // 3, 3, N).astype(np.uint64)
    lo = g[:, 0] | (g[:, 1] << np.uint64(32))
    hi = g[:, 2]
    codes = np.empty((KP // 3, 32, N), np.int32)
    for j in range(32):
        bit = 3 * j
        if bit + 3 <= 64:
            codes[:, j] = ((lo >> np.uint64(bit)) & np.uint64(7)).astype(np.int32)
        elif bit >= 64:
            codes[:, j] = ((hi >> np.uint64(bit - 64)) & np.uint64(7)).astype(np.int32)
        else:
            codes[:, j] = (((lo >> np.uint64(63)) & np.uint64(1)) | ((hi & np.uint64(3)) << np.uint64(1))).astype(np.int32)
    return codes.reshape(KP // 3 * 32, N)


def matvec(mat, scale_h, zero_h, x_h):
    """fp16 scale, zero [N], x [M, K] -> float64 [M, N] of sum_k (scale * code - zero) * x."""
    codes = unpack(mat).astype(np.float64)
    s = np.asarray(scale_h, np.float16).astype(np.float64)
    z = np.asarray(zero_h, np.float16).astype(np.float64)
    x = np.asarray(x_h, np.float16).astype(np.float64).reshape(-1, codes.shape[0])
    return (x @ codes) * s[None, :] - x.sum(axis=1, keepdims=True) * z[None, :]
