"""Boundary behaviour beyond the plain X.W call: the reference's W.X overload with n > 1, explicit per-stream
workspaces, mode switches on one container, batched calls inside a stream capture, the host-buffer call's replayed
graph, and the device forms of the Python examples' interchange formats.  All GPU results are held to the CPU oracle
or, for bit/byte work, to the fixtures made by the reference's own Python."""
import ctypes as C
import os

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth
from oracle import oracle
from parity_utils import MAE, MAX_REL, assert_parity, error_metrics

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _dev16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.float16)


def _layer(N, K, q, g, seed, bias=False):
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=seed, with_bias=bias)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, qb)
    return bW, alpha.astype(np.float16), None if qb is None else qb.astype(np.float16), w


@pytest.mark.parametrize("n", [1, 3, 16])
def test_wx_overload_takes_activations_as_columns(n):
    """matmul(output, nqW, input, n): input [K][n], output [N][n] (lutGEMM/src/kernels.cu:56-63, 73-75)."""
    N, K, q, g = 1024, 1536, 3, 128
    bW, a16, _, w = _layer(N, K, q, g, seed=21)
    x = synth.activations(n, K, seed=8)                       # rows of the X.W form
    ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)         # [n][N]
    x_cols = _dev16(np.ascontiguousarray(x.T))                # [K][n]
    out = torch.zeros((N, n), dtype=torch.float16, device="cuda")
    L.matmul_wx(out, w, x_cols, n)
    torch.cuda.synchronize()
    assert_parity(out.float().cpu().numpy().T, ref, K, f"n={n}")
    w.close()


def test_modes_may_be_switched_on_one_container():
    """ordered reductions, then the default L2 reductions, then the two-row kernel, all on one workspace."""
    N, K, q, g = 2048, 2048, 3, 128
    bW, a16, _, w = _layer(N, K, q, g, seed=31)
    x = synth.activations(2, K, seed=5)
    ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)
    xd = _dev16(x)
    lib = capi.lib()
    try:
        for ordered, m in [(1, 1), (0, 1), (0, 2), (1, 1), (0, 2)]:
            lib.lutgemm_set_ordered_reduction(ordered)
            y = torch.zeros((m, N), dtype=torch.float16, device="cuda")
            L.matmul(y, xd[:m].contiguous(), w, m)
            torch.cuda.synchronize()
            assert_parity(y.float().cpu().numpy(), ref[:m], K, f"ordered={ordered} m={m}")
    finally:
        lib.lutgemm_set_ordered_reduction(0)
    w.close()


def test_ordered_mode_per_workspace_overrides_the_process_setting():
    """A workspace (or a container's own) fixed to the bit-reproducible mode repeats its result exactly while the
    process-wide setting stays on the default; -1 hands it back to the process-wide setting."""
    N, K, q, g = 4096, 12288, 3, 128
    bW, a16, _, w = _layer(N, K, q, g, seed=33)
    x = synth.activations(1, K, seed=9)
    ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)
    xd = _dev16(x)
    ws = L.Workspace(N, K, 1).set_ordered(1)
    runs = []
    for _ in range(3):
        y = torch.zeros((1, N), dtype=torch.float32, device="cuda")
        L.matmul_f32(y, xd, w, 1, workspace=ws)
        torch.cuda.synchronize()
        runs.append(y.cpu().numpy())
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    assert_parity(runs[0], ref, K, "ordered workspace")
    w.set_ordered(1)
    y1 = torch.zeros((1, N), dtype=torch.float32, device="cuda")
    L.matmul_f32(y1, xd, w, 1)
    torch.cuda.synchronize()
    assert np.array_equal(y1.cpu().numpy(), runs[0])          # the same slab order on the container's own workspace
    w.set_ordered(-1)
    ws.set_ordered(-1)
    y2 = torch.zeros((1, N), dtype=torch.float32, device="cuda")
    L.matmul_f32(y2, xd, w, 1, workspace=ws)
    torch.cuda.synchronize()
    assert_parity(y2.cpu().numpy(), ref, K, "back on the process-wide setting")
    assert capi.lib().lutgemm_workspace_set_ordered(ws.handle, 2) == capi.ERR_SHAPE
    ws.close()
    w.close()


def test_two_streams_share_a_container_through_their_own_workspaces():
    N, K, q, g = 4096, 4096, 3, 128
    bW, a16, _, w = _layer(N, K, q, g, seed=41)
    xs = synth.activations(2, K, seed=6)
    ref = oracle.bcq_matmul_fp32(xs, bW, a16, None, g)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    spaces = [L.Workspace(N, K, 1), L.Workspace(N, K, 1)]
    xd = [_dev16(xs[i:i + 1]) for i in range(2)]
    ys = [torch.zeros((1, N), dtype=torch.float16, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    for rep in range(50):                                     # interleaved: the two streams overlap on the GPU
        for i in range(2):
            L.matmul(ys[i], xd[i], w, 1, stream=streams[i], workspace=spaces[i])
    torch.cuda.synchronize()
    for i in range(2):
        assert spaces[i].status() == 0
        assert_parity(ys[i].float().cpu().numpy(), ref[i:i + 1], K, f"stream {i}")
    # a workspace that is too small for the container is refused, not overrun
    small = L.Workspace(N // 2, K, 1)
    rc = capi.lib().lutgemm_matmul_ws(ys[0].data_ptr(), xd[0].data_ptr(), w.handle, 1, small.handle, None)
    assert rc == capi.ERR_TOO_LARGE
    for s in spaces + [small]:
        s.close()
    w.close()


def test_first_batched_call_inside_a_stream_capture():
    N, K, q, g, m = 2048, 2048, 2, 64, 16
    bW, a16, _, w = _layer(N, K, q, g, seed=51)
    x = synth.activations(m, K, seed=7)
    ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)
    xd = _dev16(x)
    y = torch.zeros((m, N), dtype=torch.float16, device="cuda")
    side = torch.cuda.Stream()
    # not reserved: the call would have to allocate, which a capture cannot hold -> refused with a status, capture intact
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        g0 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g0, stream=side):
            rc = capi.lib().lutgemm_matmul(y.data_ptr(), xd.data_ptr(), w.handle, m, C.c_void_p(side.cuda_stream))
            torch.zeros(1, device="cuda")                      # something to capture so that the graph is not empty
    assert rc in (capi.OK, capi.ERR_BATCH)                    # OK only if the tile count needs no split-k workspace
    del g0
    # reserved: the first-ever batched call may be the captured one
    w2 = L.nQWeight_fp16(bW, a16.astype(np.float32), K, N, q, False, K // g).reserve_batch(m)
    with torch.cuda.stream(side):
        g1 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g1, stream=side):
            L.matmul(y, xd, w2, m, stream=side)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        y.zero_()
        g1.replay()
        torch.cuda.synchronize()
        rel, mae = error_metrics(y.float().cpu().numpy(), ref)
        assert rel <= MAX_REL and mae <= MAE, (rel, mae)
    del g1
    w.close(); w2.close()


def test_host_buffer_call_on_pinned_and_on_pageable_buffers():
    """Page-locked buffers: a fetch kernel, the matvec storing into the host buffer, a completion word the host polls (no
    copy engine, no stream synchronisation).  Pageable buffers: copy-in / kernels / copy-out.  Either way the call is
    replayed as one graph from the second call with the same buffers on."""
    N, K, q, g = 2048, 1024, 3, 128
    bW, a16, _, w = _layer(N, K, q, g, seed=61)
    lib = capi.lib()
    xin = torch.empty((1, K), dtype=torch.int16).pin_memory()
    yout = torch.empty((1, N), dtype=torch.int16).pin_memory()
    n0 = lib.lutgemm_kernel_launch_count()
    for rep in range(4):                                      # new data in the same buffers each time
        x = synth.activations(1, K, seed=100 + rep)
        xin.numpy()[:] = x.view(np.int16)
        yout.zero_()
        capi.check(lib.lutgemm_matmul_host(yout.data_ptr(), xin.data_ptr(), w.handle, 1), "matmul_host")
        ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)
        assert_parity(yout.numpy().view(np.float16).astype(np.float32), ref, K, f"pinned call {rep}")
    assert lib.lutgemm_kernel_launch_count() - n0 == 12       # fetch, matvec, completion word per call; no copies
    xp = np.empty((3, K), np.float16)                         # pageable, three rows
    yp = np.empty((3, N), np.float16)
    for rep in range(3):                                      # call 0: direct; 1..: the recorded graph
        x = synth.activations(3, K, seed=200 + rep)
        xp[:] = x
        L.matmul_host(yp, xp, w, 3)
        ref = oracle.bcq_matmul_fp32(x, bW, a16, None, g)
        assert_parity(yp.astype(np.float32), ref, K, f"pageable call {rep}")
    us = (C.c_float * 4)()
    capi.check(lib.lutgemm_matmul_host_profile(yout.data_ptr(), xin.data_ptr(), w.handle, 1, us), "matmul_host_profile")
    assert all(v > 0 for v in us) and us[3] >= us[1]
    w.close()


def test_device_packer_and_layout_mover_bit_exact(golden_dir):
    """Packer bytes and the quantisers' tensors on the device against the reference's own Python outputs."""
    z = np.load(os.path.join(golden_dir, "converter_reference.npz"))
    for tag in ("a", "b", "c"):
        binary, packed = z[f"{tag}_binary"], z[f"{tag}_packed_u8"]            # [N,G,g,q] int8, uint8 stream
        alpha_py, offset_py = z[f"{tag}_alpha"], z[f"{tag}_offset"]
        N, G, g, q = binary.shape
        K = G * g
        d_bin = torch.from_numpy(binary).cuda()
        got = L.packer_pack_device(d_bin)
        assert np.array_equal(got.cpu().numpy(), packed.reshape(-1)), tag
        back = L.packer_unpack_device(got, binary.size)
        assert np.array_equal(back.cpu().numpy(), binary.reshape(-1)), tag
        want_bW, want_alpha, want_qb = L.from_python_layout(alpha_py, binary, offset_py.reshape(N, G))
        d_alpha = torch.from_numpy(alpha_py).cuda()
        d_off = torch.from_numpy(np.ascontiguousarray(offset_py.reshape(N, G))).cuda()
        for packed_form in (False, True):
            src = got if packed_form else d_bin
            bW, a16, qb16 = L.from_python_layout_device(d_alpha, src, d_off, N, K, g, q, packed=packed_form)
            torch.cuda.synchronize()
            assert np.array_equal(bW.cpu().numpy().view(np.uint32), want_bW), (tag, packed_form)
            assert np.array_equal(a16.cpu().numpy().view(np.uint16), want_alpha.astype(np.float16).view(np.uint16)), (tag, packed_form)
            assert np.array_equal(qb16.cpu().numpy().view(np.uint16), want_qb.astype(np.float16).view(np.uint16)), (tag, packed_form)
