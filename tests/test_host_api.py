"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, its host
functions (packer, converter, layout, uint8 format) are bit-exact with the oracle and the
reference fixtures, bad arguments give status codes, and compute fails loudly without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "lutgemm_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(lutgemm_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    lib = capi.lib()
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, missing
    assert declared == set(capi.SYMBOLS)


def test_status_strings():
    lib = capi.lib()
    for s in range(0, 9):
        assert lib.lutgemm_status_string(s)
    assert b"unknown" in lib.lutgemm_status_string(99)


def test_pack_planes_bit_exact():
    rng = np.random.default_rng(5)
    for K, q, N in [(32, 1, 1), (64, 3, 7), (256, 8, 33), (96, 4, 130)]:
        planes = (rng.integers(0, 2, size=(K, q, N)) * 2 - 1).astype(np.int8)
        assert np.array_equal(L.pack_planes(planes), oracle.pack_planes(planes))


def test_pack_planes_rejects_bad_arguments():
    lib = capi.lib()
    buf = np.zeros(64, np.int8)
    out = np.zeros(4, np.uint32)
    p, o = buf.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)
    assert lib.lutgemm_pack_planes(None, 32, 1, 1, o) == capi.ERR_NULL
    assert lib.lutgemm_pack_planes(p, 33, 1, 1, o) == capi.ERR_SHAPE
    assert lib.lutgemm_pack_planes(p, 32, 9, 1, o) == capi.ERR_BITS
    assert lib.lutgemm_pack_planes(p, 32, 0, 1, o) == capi.ERR_BITS


def test_uniform_to_bcq_matches_reference_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "converter_reference.npz"))
    for t in ("a", "b", "c"):
        q = int(z[f"{t}_q"])
        code = z[f"{t}_code"]
        N, G, g = code.shape
        if g % 32:
            continue
        bW, alpha, q_bias = L.uniform_to_bcq(z[f"{t}_scale"].reshape(N, G), z[f"{t}_zero"].reshape(N, G), code, q)
        # the reference's Python outputs, moved to the kernel layout by the oracle
        a_k, bW_k, qb_k = oracle.python_to_kernel_layout(z[f"{t}_alpha"], z[f"{t}_binary"], z[f"{t}_offset"].reshape(N, G))
        assert np.array_equal(bW, bW_k)
        assert np.array_equal(alpha, a_k)
        assert np.array_equal(q_bias, qb_k)
        # and the library's own layout mover agrees
        bW2, a2, qb2 = L.from_python_layout(z[f"{t}_alpha"], z[f"{t}_binary"], z[f"{t}_offset"].reshape(N, G))
        assert np.array_equal(bW2, bW_k) and np.array_equal(a2, a_k) and np.array_equal(qb2, qb_k)


def test_uniform_to_bcq_identity_on_synthetic_llama_like_group():
    scale, zero, code = synth.uniform_layer(24, 256, 4, 128, seed=9)
    bW, alpha, q_bias = L.uniform_to_bcq(scale, zero, code, 4)
    W = oracle.dequantize_from_qw(bW, alpha, q_bias, 128)           # [K, N]
    want = (scale[:, :, None] * (code - zero[:, :, None])).reshape(24, 256).T
    np.testing.assert_allclose(W, want, rtol=0, atol=2e-6)


def test_packer_uint8_format(golden_dir):
    z = np.load(os.path.join(golden_dir, "converter_reference.npz"))
    for t in ("a", "b", "c"):
        flat = z[f"{t}_binary"].reshape(-1)
        packed = L.packer_pack(flat)
        assert np.array_equal(packed, z[f"{t}_packed_u8"])
        assert np.array_equal(L.packer_unpack(packed, flat.size), flat)
    assert capi.lib().lutgemm_packer_pack(flat.ctypes.data_as(C.c_void_p), 7, packed.ctypes.data_as(C.c_void_p)) == capi.ERR_SHAPE


def test_create_rejects_bad_shapes_before_touching_cuda():
    lib = capi.lib()
    h = C.c_void_p()
    w = np.zeros(64, np.uint32).ctypes.data_as(C.c_void_p)
    a = np.zeros(64, np.float32).ctypes.data_as(C.c_void_p)
    assert lib.lutgemm_weight_create(C.byref(h), None, a, 32, 4, 1, 0, 1, None) == capi.ERR_NULL
    assert lib.lutgemm_weight_create(C.byref(h), w, a, 33, 4, 1, 0, 1, None) == capi.ERR_SHAPE     # K % 32
    assert lib.lutgemm_weight_create(C.byref(h), w, a, 64, 4, 1, 0, 3, None) == capi.ERR_SHAPE     # K % groups
    assert lib.lutgemm_weight_create(C.byref(h), w, a, 64, 4, 1, 0, 4, None) == capi.ERR_SHAPE     # group size 16
    assert lib.lutgemm_weight_create(C.byref(h), w, a, 64, 4, 9, 0, 1, None) == capi.ERR_BITS
    assert lib.lutgemm_weight_create(C.byref(h), w, a, 64, 0, 1, 0, 1, None) == capi.ERR_SHAPE
    assert lib.lutgemm_matmul(w, w, None, 1, None) == capi.ERR_NULL
    assert lib.lutgemm_weight_destroy(None) == capi.OK


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure mode")
def test_ordered_setters_reject_null_handles():
    lib = capi.lib()
    assert lib.lutgemm_workspace_set_ordered(None, 1) == capi.ERR_NULL
    assert lib.lutgemm_weight_set_ordered(None, 1) == capi.ERR_NULL


def test_compute_fails_loudly_without_gpu():
    bW, alpha, _ = synth.bcq_layer(8, 64, 2, 32, seed=1)
    with pytest.raises(L.LutGemmError) as e:
        L.nQWeight_fp16(bW, alpha, 64, 8, 2, False, 2)
    assert e.value.status in (capi.ERR_NO_DEVICE, capi.ERR_CUDA)


def test_algorithmic_bytes_match_published_table():
    assert synth.algorithmic_bytes(12288, 12288, 3, 128) == 63750144
    assert synth.algorithmic_bytes(4096, 4096, 3, 128) == 7094272
    assert synth.algorithmic_bytes(8192, 8192, 4, 128, with_bias=True) == 38830080
    assert synth.algorithmic_bytes(8192, 8192, 2, 64) == 21004288
