"""Pins the CPU oracle: against the reference's own dequantize_cpu (fixtures made
by tests/golden/make_golden.py and, when oracle/_ref is present, live), against
the reference's Python converter/packer outputs, and against independent numpy
restatements."""
import os

import numpy as np
import pytest

from lutgemm_b200 import synth
from oracle import oracle


def np_unpack(bW):
    KW, q, N = bW.shape
    bits = (bW[:, None, :, :] >> np.arange(32, dtype=np.uint32)[None, :, None, None]) & 1
    return (bits.reshape(KW * 32, q, N).astype(np.int8) * 2 - 1)


def np_dense(bW, alpha, q_bias, g):
    s = np_unpack(bW).astype(np.float64)
    K = s.shape[0]
    a = np.repeat(alpha.astype(np.float64), g, axis=0)  # [K, q, N]
    W = (s * a).sum(1)
    if q_bias is not None:
        W = W + np.repeat(q_bias.astype(np.float64), g, axis=0)
    return W


def test_dequantize_matches_reference_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "dequantize_cpu_reference.npz"))
    tags = sorted({k.split("_")[0] for k in z.files})
    assert len(tags) == 5
    for t in tags:
        W = oracle.dequantize_cpu(z[f"{t}_bW"], z[f"{t}_alpha"], int(z[f"{t}_g"]), bool(z[f"{t}_row_wise"]))
        assert W.shape == z[f"{t}_W"].shape
        assert np.array_equal(W.view(np.uint16), z[f"{t}_W"].view(np.uint16)), t


@pytest.mark.skipif(oracle.ref_cpu() is None, reason="oracle/_ref not built")
@pytest.mark.parametrize("N,K,q,g", [(64, 256, 3, 128), (128, 128, 5, 32), (30, 512, 4, 64)])
def test_dequantize_matches_reference_live(N, K, q, g):
    bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=7 + N, signed_alpha=True)
    a = alpha.astype(np.float16)
    for row_wise in (False, True):
        ours = oracle.dequantize_cpu(bW, a, g, row_wise)
        ref = oracle.dequantize_cpu(bW, a, g, row_wise, use_reference=True)
        assert np.array_equal(ours.view(np.uint16), ref.view(np.uint16))


def test_pack_unpack_roundtrip_and_bit_convention():
    rng = np.random.default_rng(0)
    K, q, N = 96, 3, 10
    planes = (rng.integers(0, 2, size=(K, q, N)) * 2 - 1).astype(np.int8)
    bW = oracle.pack_planes(planes)
    assert bW.shape == (K // 32, q, N)
    # bit t of word k/32 <=> plane[k + t] == +1
    assert ((bW[1, 2, 3] >> 5) & 1) == (planes[37, 2, 3] > 0)
    assert np.array_equal(oracle.unpack_planes(bW), planes)
    assert np.array_equal(np_unpack(bW), planes)


def test_converter_matches_python_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "converter_reference.npz"))
    for t in ("a", "b", "c"):
        q = int(z[f"{t}_q"])
        scale, zero, code = z[f"{t}_scale"], z[f"{t}_zero"], z[f"{t}_code"]
        N, G, g = code.shape
        alpha, binary, offset = oracle.uniform_to_bcq(scale.reshape(N, G), zero.reshape(N, G), code, q)
        assert np.array_equal(alpha, z[f"{t}_alpha"])            # bit-exact fp32
        assert np.array_equal(binary, z[f"{t}_binary"])
        assert np.array_equal(offset, z[f"{t}_offset"].reshape(N, G))
        # identity scale*(code-zero) == sum_i alpha_i*binary_i + offset, as the reference's decompress computes it
        dense = (binary.astype(np.float32) * alpha[:, :, None, :]).sum(-1) + offset[:, :, None]
        np.testing.assert_allclose(dense.reshape(N, -1), z[f"{t}_dense"], rtol=0, atol=1e-6)
        np.testing.assert_allclose(dense, scale * (code - zero), rtol=0, atol=1e-6)
        # uint8 interchange format
        packed = oracle.packer_pack(binary.reshape(-1))
        assert np.array_equal(packed, z[f"{t}_packed_u8"])
        assert np.array_equal(oracle.packer_unpack(packed, binary.size), binary.reshape(-1))


def test_python_to_kernel_layout_roundtrip(golden_dir):
    z = np.load(os.path.join(golden_dir, "converter_reference.npz"))
    alpha, binary, offset = z["a_alpha"], z["a_binary"], z["a_offset"]
    N, G, g, q = binary.shape
    alpha_k, bW, qb = oracle.python_to_kernel_layout(alpha, binary, offset.reshape(N, G))
    assert alpha_k.shape == (G, q, N) and bW.shape == (G * g // 32, q, N) and qb.shape == (G, N)
    W = oracle.dequantize_from_qw(bW, alpha_k, qb, g)            # [K, N] fp32, test-side semantics
    np.testing.assert_allclose(W.T, z["a_dense"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("N,K,q,g,bias", [(64, 256, 3, 128, False), (32, 128, 4, 32, True), (16, 64, 8, 64, True)])
def test_matmul_ref_vs_f64_and_numpy(N, K, q, g, bias):
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=11 + K, with_bias=bias, signed_alpha=True)
    x = synth.activations(2, K, seed=3)
    a_h = alpha.astype(np.float16)
    qb_h = None if qb is None else qb.astype(np.float16)
    y_ref = oracle.bcq_matmul_ref(x, bW, a_h, qb_h, g)
    y_64 = oracle.bcq_matmul_f64(x, bW, a_h, qb_h, g)
    y_np = x.astype(np.float64) @ np_dense(bW, alpha, qb, g)
    np.testing.assert_allclose(y_64, y_np, rtol=1e-10, atol=1e-10)
    scale = np.sqrt((y_np ** 2).mean())
    assert np.abs(y_ref - y_np).max() <= 2e-3 * scale + 1e-6   # only the fp16 rounding of W separates them
    # composed from the separately restated pieces: dequantize_cpu -> matmul_cpu (+ offset term)
    W_h = oracle.dequantize_cpu(bW, a_h, g).astype(np.float32)
    y_parts = oracle.matmul_cpu(x.astype(np.float32), W_h)
    if bias:
        gs = x.astype(np.float32).reshape(2, K // g, g).sum(-1)
        y_parts = y_parts + gs @ qb
    np.testing.assert_allclose(y_ref, y_parts, rtol=1e-5, atol=1e-5)
    # the fp32 test-side path, composed from its separately restated pieces
    W32 = oracle.dequantize_from_qw(bW, a_h.astype(np.float32), None if qb is None else qb_h.astype(np.float32), g)
    y32 = oracle.bcq_matmul_fp32(x, bW, a_h, qb_h, g)
    assert np.array_equal(y32, oracle.matmul_cpu(x.astype(np.float32), W32))
    assert np.abs(y32 - y_np).max() <= 1e-5 * scale + 1e-6


def test_thread_count_control():
    oracle.set_threads(2)
    assert oracle.num_threads() == 2
    oracle.set_threads(os.cpu_count() or 1)
