"""The 3-bit uniform comparison rows (matmul_gptq / matmul_gptq_faster)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import gptq3
from parity_utils import MAE, MAX_REL, error_metrics


def _layer(N, K, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 8, (K, N)).astype(np.int32)
    scale = np.abs(rng.normal(0, 0.01, N)).astype(np.float16)
    zero = (scale.astype(np.float32) * rng.uniform(2, 5, N)).astype(np.float16)      # scale * zero point
    return codes, gptq3.pack(codes), scale, zero


def test_pack_unpack_round_trip_and_known_words():
    codes = np.arange(64).reshape(64, 1) % 8
    mat = gptq3.pack(codes)
    assert mat.shape == (6, 1)
    assert (gptq3.unpack(mat) == codes).all()
    # code j at bits 3j..3j+2: codes 0..9 fill bits 0..29 of word 0, code 10 = 2 puts its low two bits at 30, 31
    w0 = sum((j % 8) << (3 * j) for j in range(10)) | ((2 & 3) << 30)
    assert int(mat[0, 0]) == w0
    rng = np.random.default_rng(0)
    c = rng.integers(0, 8, (256, 7))
    assert (gptq3.unpack(gptq3.pack(c)) == c).all()


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,m", [(256, 256, 1), (1000, 4096, 1), (4096, 4096, 3), (12288, 12288, 1), (40, 2080, 2)])
def test_kernel_matches_oracle(N, K, m):
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import synth
    codes, mat, scale, zero = _layer(N, K, N + K)
    x = synth.activations(m, K, seed=3)
    t = lambda a, dt: torch.from_numpy(a).cuda().view(dt)
    y = torch.empty((m, N), dtype=torch.float16, device="cuda")
    L.matmul_gptq(m, N, K * 3 // 32, t(scale.view(np.int16), torch.float16), t(zero.view(np.int16), torch.float16),
                  t(x.view(np.int16), torch.float16), t(mat.view(np.int32), torch.int32), y)
    ref = gptq3.matvec(mat, scale, zero, x)
    rel, mae = error_metrics(y.float().cpu().numpy(), ref.astype(np.float32))
    assert rel <= MAX_REL and mae <= MAE, (rel, mae)


@pytest.mark.gpu
@pytest.mark.parametrize("faster", [0, 1])
def test_against_the_reference_kernels(faster):
    """The reference's own kernels (fp16 arithmetic, fp16 atomics), compiled for sm_100a: agreement at fp16 accuracy."""
    path = os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "libref_gpu.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_gpu.so not built")
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import synth
    ref_lib = C.CDLL(path)
    if not hasattr(ref_lib, "ref_gpu_matmul_gptq"):
        pytest.skip("prebuilt libref_gpu.so predates the GPTQ entry point")
    ref_lib.ref_gpu_matmul_gptq.argtypes = [C.c_int] * 3 + [C.c_void_p] * 5 + [C.c_int]
    N, K = 2048, 2048                                   # multiples of 256: the reference kernels check no bounds
    codes, mat, scale, zero = _layer(N, K, 11)
    x = synth.activations(1, K, seed=5)
    t = lambda a, dt: torch.from_numpy(a).cuda().view(dt)
    d_scale, d_zero = t(scale.view(np.int16), torch.float16), t(zero.view(np.int16), torch.float16)
    d_x, d_mat = t(x.view(np.int16), torch.float16), t(mat.view(np.int32), torch.int32)
    y = torch.empty((1, N), dtype=torch.float16, device="cuda")
    y_ref = torch.empty((1, N), dtype=torch.float16, device="cuda")
    L.matmul_gptq(1, N, K * 3 // 32, d_scale, d_zero, d_x, d_mat, y)
    torch.cuda.synchronize()
    ref_lib.ref_gpu_matmul_gptq(1, N, K * 3 // 32, d_scale.data_ptr(), d_zero.data_ptr(), d_x.data_ptr(), d_mat.data_ptr(),
                                y_ref.data_ptr(), faster)
    torch.cuda.synchronize()
    exact = gptq3.matvec(mat, scale, zero, x).astype(np.float32)
    ours, theirs = y.float().cpu().numpy(), y_ref.float().cpu().numpy()
    rms = np.sqrt((exact ** 2).mean())
    assert np.abs(ours - exact).mean() <= MAE
    # the reference rounds every product and sum to fp16: a few per cent of the rms is what it delivers
    assert np.abs(theirs - exact).mean() <= 0.05 * rms, (np.abs(theirs - exact).mean(), rms)
    assert np.abs(ours - theirs).mean() <= 0.05 * rms
