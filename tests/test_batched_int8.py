"""GPU parity of the integer tensor-core kernel (batches of up to 16 rows, up to 4 planes, tcgen05.mma.kind::i8; opt-in
through lutgemm_set_batched_int8) against the fp32 host reference (oracle.bcq_matmul_fp32) and against the fp16
tensor-core kernel on the same inputs.  Containers with more than 4 planes stay on the fp16 kernel with the knob on."""
import ctypes

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth
from oracle import oracle
from parity_utils import MAE, MAX_REL, error_metrics

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run(bW, alpha, qb, g, x, int8, f32=True):
    lib = capi.lib()
    lib.lutgemm_set_batched_int8(1 if int8 else 0)
    try:
        K = bW.shape[0] * 32
        q, N = bW.shape[1], bW.shape[2]
        w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, qb)
        m = x.shape[0]
        xd = torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16)
        if f32:
            out = torch.empty((m, N), dtype=torch.float32, device="cuda")
            L.matmul_f32(out, xd, w, m)
        else:
            out = torch.empty((m, N), dtype=torch.float16, device="cuda")
            L.matmul(out, xd, w, m)
        torch.cuda.synchronize()
        st = ctypes.c_int(-1)
        capi.check(lib.lutgemm_weight_device_status(w.handle, ctypes.byref(st)), "device_status")
        assert st.value == 0, f"kernel status {st.value}"
        y = out.float().cpu().numpy()
        w.close()
        return y
    finally:
        lib.lutgemm_set_batched_int8(0)                  # the default


def _ref(bW, alpha, qb, g, x):
    return oracle.bcq_matmul_fp32(x, bW, alpha.astype(np.float16), None if qb is None else qb.astype(np.float16), g)


# one / two / four scale units per 128-k step, groups wider than a step, every plane count, tiles with a ragged right edge,
# a k-range that ends inside a step, one and many k-ranges per column tile
@pytest.mark.parametrize("N,K,q,g,m,bias", [
    (256, 128, 1, 128, 16, False), (256, 256, 2, 64, 16, False), (264, 512, 2, 64, 5, True), (512, 1024, 3, 128, 16, True),
    (384, 1024, 4, 32, 8, True), (520, 1184, 4, 32, 13, False), (1024, 4096, 3, 256, 16, True), (136, 8192, 2, 64, 4, True),
    (256, 2048, 5, 64, 9, False), (256, 1024, 6, 128, 16, True), (128, 768, 7, 32, 7, False), (256, 512, 8, 64, 16, True),
    (2048, 1024, 3, 1024, 12, False), (4096, 4096, 3, 128, 16, False)])
def test_int8_batched_parity(N, K, q, g, m, bias):
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=synth.seed_for("i8", N, K, q, m), with_bias=bias, signed_alpha=True)
    x = synth.activations(m, K, seed=m)
    ref = _ref(bW, alpha, qb, g, x)
    y32 = _run(bW, alpha, qb, g, x, True)
    y16 = _run(bW, alpha, qb, g, x, True, f32=False)
    rel32, mae32 = error_metrics(y32, ref)
    rel16, mae16 = error_metrics(y16, ref)
    assert rel32 <= MAX_REL and rel16 <= MAX_REL, (rel32, rel16)
    assert mae32 <= MAE and mae16 <= MAE, (mae32, mae16)
    # and as close to the fp16 tensor-core kernel (exact products, fp32 sums) as fp32 rounding allows
    y_tc = _run(bW, alpha, qb, g, x, False)
    rel_tc, _ = error_metrics(y32, y_tc)
    assert rel_tc <= 1e-3, rel_tc                         # both are fp32-accurate; the floor of the metric is 1e-2 rms
    if q <= 4:
        assert not np.array_equal(y32, y_tc)              # a different kernel did run: the low fp32 bits differ


def test_int8_batched_config4_rows():
    """Config 4 at full size (8192 x 8192, q = 2, g = 64), 4, 8 and 16 rows, sampled columns against the host reference."""
    N = K = 8192
    bW, alpha, _ = synth.bcq_layer(N, K, 2, 64, seed=synth.seed_for("cfg4", N, K, 2))
    cols = np.arange(0, N, 61)
    for m in (4, 8, 16):
        x = synth.activations(m, K, seed=m)
        y = _run(bW, alpha, None, 64, x, True)
        ref = _ref(np.ascontiguousarray(bW[:, :, cols]), np.ascontiguousarray(alpha[:, :, cols]), None, 64, x)
        rel, mae = error_metrics(y[:, cols], ref)
        assert rel <= 1e-3 and mae <= 1e-4, (m, rel, mae)         # fp32 output: far inside the tolerance


def test_int8_activation_range():
    """Activations spanning the whole fp16 range inside one 128-k block (outliers 2^12 times the bulk, subnormals,
    zero rows, a constant positive row): the block-scaled integers keep every value within 2^13 of the block maximum
    exact, so the result stays at fp32 accuracy of the host reference."""
    N, K, q, g, m = 512, 2048, 3, 64, 16
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=11, with_bias=True, signed_alpha=True)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((m, K)).astype(np.float32) * 0.05
    x[0, ::97] *= 4096.0                                   # outliers
    x[1] = 0.0                                             # a zero row
    x[2] = 1.5                                             # constant: the two large terms cancel almost entirely
    x[3] *= 1e-6                                           # fp16 subnormals
    x[4, 5] = 60000.0                                      # near the fp16 maximum
    x = x.astype(np.float16)
    ref = _ref(bW, alpha, qb, g, x)
    y = _run(bW, alpha, qb, g, x, True)
    y_tc = _run(bW, alpha, qb, g, x, False)
    for r in range(m):
        scale = float(np.abs(ref[r]).max()) + 1e-30
        assert float(np.abs(y[r] - ref[r]).max()) <= 2e-4 * scale + 1e-12, (r, float(np.abs(y[r] - ref[r]).max()), scale)
        assert float(np.abs(y[r] - y_tc[r]).max()) <= 2e-4 * scale + 1e-12, r
    assert np.all(y[1] == 0.0)


def test_int8_ordered_mode_is_bit_reproducible():
    lib = capi.lib()
    N, K, q, g, m = 1024, 4096, 3, 128, 16
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=3, with_bias=False)
    x = synth.activations(m, K, seed=2)
    lib.lutgemm_set_ordered_reduction(1)
    try:
        a = _run(bW, alpha, qb, g, x, True)
        b = _run(bW, alpha, qb, g, x, True)
    finally:
        lib.lutgemm_set_ordered_reduction(0)
    assert np.array_equal(a, b)
    rel, mae = error_metrics(a, _ref(bW, alpha, qb, g, x))
    assert rel <= MAX_REL and mae <= MAE
