"""GPU parity tests: the CUDA library, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Integer/bit work (packer, converter, dense dequantisation) is bit-exact; the matmul
is within max-relative-error 1e-2 and mean-absolute-error 1e-3 of the reference's host
dequant-and-matmul result."""
import os

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth
from oracle import oracle
from parity_utils import MAE, MAX_REL, REF16_FLOOR, error_metrics

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev_x(x):
    return torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16)


def run_matmul(bW, alpha, q_bias, g, x, f32=False):
    K = bW.shape[0] * 32
    q, N = bW.shape[1], bW.shape[2]
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, q_bias)
    m = x.shape[0]
    xd = dev_x(x)
    if f32:
        out = torch.empty((m, N), dtype=torch.float32, device="cuda")
        L.matmul_f32(out, xd, w, m)
    else:
        out = torch.empty((m, N), dtype=torch.float16, device="cuda")
        L.matmul(out, xd, w, m)
    torch.cuda.synchronize()
    import ctypes
    st = ctypes.c_int(-1)
    capi.check(capi.lib().lutgemm_weight_device_status(w.handle, ctypes.byref(st)), "device_status")
    assert st.value == 0, f"kernel status {st.value}"
    y = out.float().cpu().numpy()
    w.close()
    return y


@pytest.fixture(params=[(0, 0), (0, 1), (1, 0)], ids=["tma", "tma-ordered", "regstream"])
def gemv_variant(request):
    """Both matvec kernels, and both split-k modes of the TMA-fed one, compute the same function;
    run the shape grid through each."""
    variant, ordered = request.param
    capi.check(capi.lib().lutgemm_set_gemv_variant(variant), "set_gemv_variant")
    capi.check(capi.lib().lutgemm_set_ordered_reduction(ordered), "set_ordered_reduction")
    yield request.param
    capi.lib().lutgemm_set_gemv_variant(0)
    capi.lib().lutgemm_set_ordered_reduction(0)


def oracle_y(bW, alpha, q_bias, g, x):
    """fp32 host dequant-and-matmul (test-side semantics of the reference)."""
    return oracle.bcq_matmul_fp32(x, bW, alpha.astype(np.float16), None if q_bias is None else q_bias.astype(np.float16), g)


def oracle_y_dense16(bW, alpha, q_bias, g, x):
    """Host result through lutGEMM::dequantize_cpu (dense W rounded to fp16) plus the offset term."""
    return oracle.bcq_matmul_ref(x, bW, alpha.astype(np.float16), None if q_bias is None else q_bias.astype(np.float16), g)


def check(y, ref, K, what, fp32_out=False, wide_range=False):
    """The matvec tolerance.  wide_range: shapes outside the configurations' (q, K) range, drawn with the configurations'
    alpha distribution, whose outputs can be several units large: there an exact result rounded to fp16 already has a
    mean absolute error of about 2^-12 of the mean magnitude, which is added to the bound for the fp16 output (the fp32
    output is held to the plain bound everywhere)."""
    rel, mae = error_metrics(y, ref)
    assert rel <= MAX_REL, f"{what}: max rel err {rel:.3e}"
    if fp32_out or K <= 12288:
        bound = MAE if (fp32_out or not wide_range) else MAE + float(np.abs(ref).mean()) * 2.0 ** -12
        assert mae <= bound, f"{what}: MAE {mae:.3e} > {bound:.3e}"
    return rel, mae


# ---- exhaustive small shapes: every q, odd column counts (generic kernel), table kernel with tails
@pytest.mark.parametrize("q", list(range(1, 9)))
@pytest.mark.parametrize("N,K,g", [(2, 32, 32), (6, 64, 32), (10, 96, 32), (33, 128, 64), (64, 256, 128),
                                   (132, 768, 128), (128, 512, 32), (260, 1280, 256), (20, 256, 64),
                                   (516, 2048, 64), (12, 96, 96), (1028, 1152, 192), (300, 3072, 1024)])
def test_small_shapes_all_planes(q, N, K, g, gemv_variant):
    for bias in (False, True):
        bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=synth.seed_for("small", N, K, q, bias), with_bias=bias,
                                        signed_alpha=True, alpha_std=0.02)
        x = synth.activations(1, K, seed=N + K)
        ref = oracle_y(bW, alpha, qb, g, x)
        y16 = run_matmul(bW, alpha, qb, g, x)
        check(y16, ref, K, f"fp16 N={N} K={K} q={q} bias={bias}")
        rel16, _ = error_metrics(y16, oracle_y_dense16(bW, alpha, qb, g, x), floor=REF16_FLOOR)
        assert rel16 <= MAX_REL, (N, K, q, bias, rel16)
        check(run_matmul(bW, alpha, qb, g, x, f32=True), ref, K, f"fp32 N={N} K={K} q={q} bias={bias}", fp32_out=True)


def test_config1_4096_q3_g128():
    N = K = 4096
    bW, alpha, _ = synth.bcq_layer(N, K, 3, 128, seed=synth.seed_for("cfg1", N, K, 3))
    x = synth.activations(1, K, seed=1)
    ref = oracle_y(bW, alpha, None, 128, x)
    y16 = run_matmul(bW, alpha, None, 128, x)
    rel, mae = check(y16, ref, K, "config1")
    rel16, mae16 = error_metrics(y16, oracle_y_dense16(bW, alpha, None, 128, x), floor=REF16_FLOOR)
    assert rel16 <= MAX_REL and mae16 <= MAE
    f64 = oracle.bcq_matmul_f64(x, bW, alpha.astype(np.float16), None, 128)
    rel64, mae64 = error_metrics(run_matmul(bW, alpha, None, 128, x, f32=True), f64)
    assert rel64 < 1e-4 and mae64 < 1e-5      # the fp32 result is essentially exact


def _sampled_columns_check(N, K, q, g, bias, tag, n_cols=192, uniform=False):
    """Full-size layer on the GPU; the oracle recomputes a seeded sample of columns from a column-sliced
    container (columns are independent), so the check runs at the benchmark sizes in seconds."""
    seed = synth.seed_for(tag, N, K, q)
    if uniform:
        scale, zero, code = synth.uniform_layer(N, K, q, g, seed)
        bW, alpha, qb = L.uniform_to_bcq(scale, zero, code, q)
    else:
        bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed, with_bias=bias)
    x = synth.activations(1, K, seed=seed ^ 77)
    y16 = run_matmul(bW, alpha, qb, g, x)
    y32 = run_matmul(bW, alpha, qb, g, x, f32=True)
    cols = np.sort(np.random.default_rng(seed).choice(N, size=n_cols, replace=False))
    ref = oracle_y(np.ascontiguousarray(bW[:, :, cols]), np.ascontiguousarray(alpha[:, :, cols]),
                   None if qb is None else np.ascontiguousarray(qb[:, cols]), g, x)
    rel, mae = error_metrics(y16[:, cols], ref)
    rel32, mae32 = error_metrics(y32[:, cols], ref)
    ref16 = oracle_y_dense16(np.ascontiguousarray(bW[:, :, cols]), np.ascontiguousarray(alpha[:, :, cols]),
                             None if qb is None else np.ascontiguousarray(qb[:, cols]), g, x)
    assert error_metrics(y32[:, cols], ref16, floor=REF16_FLOOR)[0] <= MAX_REL, tag
    assert rel <= MAX_REL and rel32 <= MAX_REL, (tag, rel, rel32)
    assert mae32 <= MAE, (tag, mae32)
    if K <= 12288:
        assert mae <= MAE, (tag, mae)
    # the fp16 output is the fp32 result rounded once; the two runs add their 24+ slab sums in L2 in
    # different orders, which moves the fp32 result by a few 1e-7 of the slab sums' magnitude
    step = np.spacing(np.abs(y32).astype(np.float16)).astype(np.float32)
    assert np.all(np.abs(y16 - y32) <= step + 4e-6 * float(np.sqrt((y32 ** 2).mean())))
    return y32


@pytest.mark.parametrize("N,K", [(12288, 12288), (36864, 12288), (49152, 12288), (12288, 49152)])
@pytest.mark.parametrize("q", [3, 4])
def test_config2_opt175b_linears(N, K, q):
    _sampled_columns_check(N, K, q, 128, False, "cfg2")


@pytest.mark.parametrize("N,K", [(8192, 8192), (28672, 8192), (8192, 28672)])
def test_config3_uniform4bit_llama70b(N, K):
    _sampled_columns_check(N, K, 4, 128, True, "cfg3", uniform=True)


def test_reference_benchmark_shape_7168():
    # the shape of the reference's own benchmark TEST (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:292-314)
    _sampled_columns_check(28672, 7168, 3, 128, True, "ref-bench")


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16, 32, 64, 128])
def test_config4_batch_sweep(m):
    N = K = 8192
    bW, alpha, _ = synth.bcq_layer(N, K, 2, 64, seed=synth.seed_for("cfg4", N, K, 2))
    x = synth.activations(m, K, seed=m)
    y = run_matmul(bW, alpha, None, 64, x)
    cols = np.arange(0, N, 61)
    ref = oracle_y(np.ascontiguousarray(bW[:, :, cols]), np.ascontiguousarray(alpha[:, :, cols]), None, 64, x)
    rel, mae = error_metrics(y[:, cols], ref)
    assert rel <= MAX_REL and mae <= MAE, (m, rel, mae)


@pytest.mark.parametrize("N,K,q,g,m,bias", [
    (256, 256, 3, 128, 2, False), (128, 128, 1, 32, 16, True), (130, 96, 2, 32, 3, True), (520, 1184, 4, 32, 17, False),
    (1024, 2048, 3, 128, 100, True), (384, 4096, 8, 64, 128, False), (640, 1024, 5, 256, 130, True),
    (4096, 4096, 3, 128, 32, False), (136, 8192, 2, 64, 300, True)])
def test_batched_tensor_core_path(N, K, q, g, m, bias):
    """m >= 2 through the tcgen05 kernel, against the fp32 host reference (same tolerance as the matvec: the
    per-plane operands +-alpha_b are exact in fp16 and the accumulation is fp32); also against one matvec per row."""
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=synth.seed_for("tc", N, K, q, m), with_bias=bias, signed_alpha=True)
    x = synth.activations(m, K, seed=m)
    ref = oracle_y(bW, alpha, qb, g, x)
    capi.lib().lutgemm_set_batched_path(2)           # tensor-core kernel from m = 2 (the default starts at m = 4)
    try:
        y16 = run_matmul(bW, alpha, qb, g, x)
        y32 = run_matmul(bW, alpha, qb, g, x, f32=True)
    finally:
        capi.lib().lutgemm_set_batched_path(1)
    rel, mae = error_metrics(y16, ref)
    rel32, mae32 = error_metrics(y32, ref)
    assert rel <= MAX_REL and rel32 <= MAX_REL, (rel, rel32)
    assert mae32 <= MAE and (K > 12288 or mae <= MAE), (mae, mae32)
    capi.lib().lutgemm_set_batched_path(0)
    try:
        y_rows = run_matmul(bW, alpha, qb, g, x, f32=True)
    finally:
        capi.lib().lutgemm_set_batched_path(1)
    rel_rows, _ = error_metrics(y32, y_rows)
    assert rel_rows <= 1e-3, rel_rows                     # both paths are fp32-accurate


def test_linearity_and_determinism_at_full_size():
    capi.lib().lutgemm_set_ordered_reduction(1)      # slabs added in slab order: run-to-run bit identical
    try:
        _linearity_and_determinism()
    finally:
        capi.lib().lutgemm_set_ordered_reduction(0)


def _linearity_and_determinism():
    N, K, q, g = 12288, 12288, 3, 128
    bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=3)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g)
    x1 = synth.activations(1, K, seed=10).astype(np.float32)
    x2 = synth.activations(1, K, seed=11).astype(np.float32)
    xs = [(x1 * 0.5).astype(np.float16), (x2 * 0.25).astype(np.float16), (x1 * 0.5 + x2 * 0.25).astype(np.float16)]
    ys = []
    for x in xs:
        out = torch.empty((1, N), dtype=torch.float32, device="cuda")
        L.matmul_f32(out, dev_x(x), w, 1)
        out2 = torch.empty((1, N), dtype=torch.float32, device="cuda")
        L.matmul_f32(out2, dev_x(x), w, 1)
        torch.cuda.synchronize()
        assert torch.equal(out, out2)               # run-to-run bit identical
        ys.append(out.cpu().numpy().astype(np.float64))
    # x3 = fp16(x1/2 + x2/4) differs from the exact sum by fp16 rounding only
    scale = np.sqrt((ys[2] ** 2).mean())
    assert np.abs(ys[0] + ys[1] - ys[2]).max() <= 5e-3 * scale
    w.close()


@pytest.mark.parametrize("N,K,q,g,row_wise", [(64, 128, 3, 32, False), (48, 256, 4, 128, False), (130, 96, 8, 32, False),
                                              (32, 128, 2, 128, True), (257, 512, 5, 64, True), (4096, 1024, 3, 128, False)])
def test_dequantize_bit_exact(N, K, q, g, row_wise):
    bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=N * 7 + K, signed_alpha=True)
    row, col = (N, K) if row_wise else (K, N)
    w = L.nQWeight_fp16(bW, alpha, row, col, q, row_wise, K // g)
    fW = w.getDequantiedWeight().cpu().numpy()
    ref = oracle.dequantize_cpu(bW, alpha.astype(np.float16), g, row_wise)
    assert fW.shape == ref.shape
    assert np.array_equal(fW.view(np.uint16), ref.view(np.uint16))
    w.close()


def test_dequantize_matches_reference_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "dequantize_cpu_reference.npz"))
    for t in sorted({k.split("_")[0] for k in z.files}):
        bW, a, g, rw = z[f"{t}_bW"], z[f"{t}_alpha"].astype(np.float32), int(z[f"{t}_g"]), bool(z[f"{t}_row_wise"])
        K, q, N = bW.shape[0] * 32, bW.shape[1], bW.shape[2]
        row, col = (N, K) if rw else (K, N)
        w = L.nQWeight_fp16(bW, a, row, col, q, rw, K // g)
        got = w.getDequantiedWeight().cpu().numpy()
        assert np.array_equal(got.view(np.uint16), z[f"{t}_W"].view(np.uint16)), t
        w.close()


def test_device_packer_and_converter_bit_exact():
    rng = np.random.default_rng(2)
    K, q, N = 256, 3, 200
    planes = (rng.integers(0, 2, size=(K, q, N)) * 2 - 1).astype(np.int8)
    got = L.pack_planes_device(torch.from_numpy(planes).cuda()).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, oracle.pack_planes(planes))
    scale, zero, code = synth.uniform_layer(72, 512, 4, 128, seed=4)
    bW_d, a_d, qb_d = L.uniform_to_bcq_device(torch.from_numpy(scale).cuda(), torch.from_numpy(zero).cuda(),
                                              torch.from_numpy(code).cuda(), 4)
    bW_h, a_h, qb_h = L.uniform_to_bcq(scale, zero, code, 4)
    assert np.array_equal(bW_d.cpu().numpy().view(np.uint32), bW_h)
    assert np.array_equal(a_d.cpu().numpy(), a_h.astype(np.float16))
    assert np.array_equal(qb_d.cpu().numpy(), qb_h.astype(np.float16))


def test_host_call_with_page_locked_buffers_reads_fresh_inputs():
    """The host-buffer call with page-locked buffers reused across calls: every call must see what the host wrote just
    before it, and pageable buffers must give the same numbers."""
    N, K, q, g = 2048, 4096, 3, 128
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=21, with_bias=True)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, qb)
    xin = torch.empty((1, K), dtype=torch.float16).pin_memory()
    yout = torch.empty((1, N), dtype=torch.float16).pin_memory()
    for seed in (1, 2, 3):
        x = synth.activations(1, K, seed=seed)
        xin.numpy()[:] = x
        yout.numpy()[:] = 0
        L.matmul_host(yout.numpy(), xin.numpy(), w, 1)
        ref = oracle_y(bW, alpha, qb, g, x)
        check(yout.numpy().astype(np.float32), ref, K, f"pinned matmul_host, input {seed}")
        y_pageable = np.empty((1, N), np.float16)
        L.matmul_host(y_pageable, x.copy(), w, 1)
        assert np.abs(y_pageable.astype(np.float32) - yout.numpy().astype(np.float32)).max() <= 2e-3 * np.abs(ref).max()


def test_host_buffer_call_and_borrowed_device_container():
    N, K, q, g = 1024, 1024, 3, 128
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=8, with_bias=True)
    x = synth.activations(2, K, seed=5)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, qb)
    y = np.empty((2, N), np.float16)
    L.matmul_host(y, x, w, 2)
    ref = oracle_y(bW, alpha, qb, g, x)
    check(y.astype(np.float32), ref, K, "matmul_host")
    # the same container built from device tensors without a copy
    d_bW = torch.from_numpy(bW.view(np.int32)).cuda()
    d_a = torch.from_numpy(alpha.astype(np.float16)).cuda()
    d_qb = torch.from_numpy(qb.astype(np.float16)).cuda()
    w2 = L.nQWeight_fp16.from_device(d_bW, d_a, d_qb, K, N, q, False, K // g, copy=False)
    out = torch.empty((2, N), dtype=torch.float16, device="cuda")
    L.matmul(out, dev_x(x), w2, 2)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()                                  # split-k reductions are unordered: compare to one fp16 step
    assert np.all(np.abs(got - y.astype(np.float32)) <= np.spacing(np.abs(y)).astype(np.float32) + 4e-6 * float(np.sqrt((got ** 2).mean())))
    assert w2.mSize == N and w2.kSize == K and w2.nb == q and w2.num_groups == K // g and w2.group_size == g
    w.close(); w2.close()


def test_bad_runtime_arguments_return_status():
    bW, alpha, _ = synth.bcq_layer(64, 256, 2, 64, seed=1)
    w = L.nQWeight_fp16(bW, alpha, 256, 64, 2, False, 4)
    x = dev_x(synth.activations(1, 256, seed=1))
    out = torch.empty((1, 64), dtype=torch.float16, device="cuda")
    lib = capi.lib()
    assert lib.lutgemm_matmul(out.data_ptr(), x.data_ptr(), w.handle, 0, None) == capi.ERR_BATCH
    assert lib.lutgemm_matmul(out.data_ptr(), x.data_ptr() + 2, w.handle, 1, None) == capi.ERR_ALIGN
    assert lib.lutgemm_matmul(None, x.data_ptr(), w.handle, 1, None) == capi.ERR_NULL
    n0 = lib.lutgemm_kernel_launch_count()
    L.matmul(out, x, w, 1)
    assert lib.lutgemm_kernel_launch_count() == n0 + 1
    w.close()


def _random_config(rng):
    g = int(rng.choice([32, 64, 96, 128, 256, 512, 1024]))
    K = g * int(rng.integers(1, max(2, 6144 // g)))
    N = int(rng.choice([8, 4, 2, 1])) * int(rng.integers(1, 700))
    q = int(rng.integers(1, 9))
    m = int(rng.choice([1, 1, 2, 3, 4, 5, 16, 17, 33, 64, 100, 128, 131]))
    bias = bool(rng.integers(0, 2))
    return N, K, q, g, m, bias


@pytest.mark.parametrize("seed", list(range(32)))
def test_random_configurations(seed):
    """Seeded random (N, K, q, g, m, q_bias): whatever kernel the dispatch picks (TMA-fed or register-fed matvec, generic
    fallback, tensor-core batched kernel with either operand order) must agree with the fp32 host reference."""
    rng = np.random.default_rng(1000 + seed)
    N, K, q, g, m, bias = _random_config(rng)
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=seed, with_bias=bias, signed_alpha=bool(seed & 1))   # alpha ~ |N(0, 0.02)|
    x = synth.activations(m, K, seed=seed + 7)
    ref = oracle_y(bW, alpha, qb, g, x)
    y32 = run_matmul(bW, alpha, qb, g, x, f32=True)
    y16 = run_matmul(bW, alpha, qb, g, x)
    what = f"N={N} K={K} q={q} g={g} m={m} bias={bias}"
    check(y32, ref, K, what + " fp32 out", fp32_out=True)
    check(y16.astype(np.float32), ref, K, what, wide_range=True)


@pytest.mark.parametrize("N,K,q,g,m,bias", [(2048, 4096, 3, 128, 2, False), (1032, 1184, 4, 32, 3, True), (512, 512, 1, 512, 2, True),
                                            (12288, 12288, 3, 128, 2, False), (264, 1536, 8, 64, 3, False), (4096, 3072, 2, 1024, 2, True)])
def test_two_row_matvec_matches_single_rows(N, K, q, g, m, bias):
    """m = 2, 3 through the two-table kernel (weights read once for two rows) against the fp32 host reference and against
    one launch per row."""
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=N + K + m, with_bias=bias, signed_alpha=True)
    x = synth.activations(m, K, seed=m + 40)
    ref = oracle_y(bW, alpha, qb, g, x)
    lib = capi.lib()
    lib.lutgemm_set_batched_path(0)                  # keep the rows on the LUT matvec
    try:
        y_pair = run_matmul(bW, alpha, qb, g, x, f32=True)
        y_pair16 = run_matmul(bW, alpha, qb, g, x)
        lib.lutgemm_set_row_pairs(0)
        y_single = run_matmul(bW, alpha, qb, g, x, f32=True)
    finally:
        lib.lutgemm_set_row_pairs(1)
        lib.lutgemm_set_batched_path(1)
    check(y_pair, ref, K, "two-row kernel, fp32 out", fp32_out=True)
    check(y_pair16.astype(np.float32), ref, K, "two-row kernel", wide_range=True)
    rms = np.sqrt((ref ** 2).mean())
    assert np.abs(y_pair - y_single).max() <= 1e-5 * max(rms, 1e-6) * np.sqrt(K / 512)      # same sums, reduction order aside
