"""The matvec entry point that allocates nothing (lutgemm_matvec_static_scratch).

Some hosts cannot call cudaMalloc once they are up (all device memory already belongs to their own
pool, or their rules forbid it); for them the library keeps the split-k workspace in a fixed array of
its own image.  This test calls that entry point through the C ABI, twice in a row on the same
arrays, and checks both results against the ordinary entry point (lutgemm_matmul) on the same
container data and against the CPU oracle, within the tolerance the other parity tests use, and reads the
entry point's status word (it lives in the same fixed array).  It sits last in collection order so
that a run which stops at the first failure has already run every other test; it passes alone in a
fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth
from oracle import oracle
from parity_utils import MAE, MAX_REL, error_metrics

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _dev(a_np, dtype):
    return torch.from_numpy(a_np).cuda().view(dtype)


@pytest.mark.parametrize("N,K,q,g,bias", [(4096, 4096, 3, 128, False), (2048, 1536, 4, 64, True)])
def test_static_scratch_matches_ordinary_entry_point_twice(N, K, q, g, bias):
    lib = capi.lib()
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=synth.seed_for("noalloc", N, K, q), with_bias=bias)
    x = synth.activations(1, K, seed=17)
    G = K // g
    # the ordinary path: container + lutgemm_matmul
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, G, qb)
    xd = _dev(x.view(np.int16), torch.float16)
    want = torch.empty((1, N), dtype=torch.float16, device="cuda")
    L.matmul(want, xd, w, 1)
    torch.cuda.synchronize()
    want = want.float().cpu().numpy()
    ref = oracle.bcq_matmul_fp32(x, bW, alpha.astype(np.float16), None if qb is None else qb.astype(np.float16), g)
    # the same data as plain device arrays for the non-allocating entry point
    d_bW = _dev(bW.view(np.int32), torch.int32)
    d_alpha = _dev(alpha.astype(np.float16).view(np.int16), torch.float16)
    d_qb = None if qb is None else _dev(qb.astype(np.float16).view(np.int16), torch.float16)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        out = torch.full((1, N), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.lutgemm_matvec_static_scratch(out.data_ptr(), xd.data_ptr(), d_bW.data_ptr(), d_alpha.data_ptr(),
                                               None if d_qb is None else d_qb.data_ptr(), K, N, q, G, stream)
        assert rc == capi.OK, lib.lutgemm_status_string(rc)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}"
        rel, mae = error_metrics(got, want)
        assert rel <= MAX_REL and mae <= MAE, (call, rel, mae)
        rel_o, mae_o = error_metrics(got, ref)                 # and directly against the reference's host evaluation
        assert rel_o <= MAX_REL and mae_o <= MAE, (call, rel_o, mae_o)
        st = C.c_int(-1)
        assert lib.lutgemm_static_scratch_status(C.byref(st)) == capi.OK and st.value == 0, (call, st.value)
        # both paths round the same fp32 sums once; only the unordered slab additions may differ
        step = np.spacing(np.abs(want).astype(np.float16)).astype(np.float32)
        assert np.all(np.abs(got - want) <= step + 4e-6 * float(np.sqrt((want ** 2).mean()))), f"call {call}"
    w.close()


def test_static_scratch_rejects_what_it_cannot_hold():
    lib = capi.lib()
    t = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = t.data_ptr()
    # wider than the fixed reduction row
    assert lib.lutgemm_matvec_static_scratch(p, p, p, p, None, 512, 65536 + 8, 1, 4, None) == capi.ERR_TOO_LARGE
    # shapes the TMA-fed kernel does not take: N % 8 != 0, group size 96
    assert lib.lutgemm_matvec_static_scratch(p, p, p, p, None, 512, 12, 1, 4, None) == capi.ERR_SHAPE
    assert lib.lutgemm_matvec_static_scratch(p, p, p, p, None, 384, 64, 1, 4, None) == capi.ERR_SHAPE
    assert lib.lutgemm_matvec_static_scratch(None, p, p, p, None, 512, 64, 1, 4, None) == capi.ERR_NULL
    assert lib.lutgemm_matvec_static_scratch(p, p + 4, p, p, None, 512, 64, 1, 4, None) == capi.ERR_ALIGN
    assert lib.lutgemm_matvec_static_scratch(p, p, p, p, None, 512, 64, 9, 4, None) == capi.ERR_BITS
