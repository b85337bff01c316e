"""lutgemm_sequence_*: a list of matvecs in one persistent kernel, against the oracle and against the per-call path."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import lutgemm_b200 as L
from lutgemm_b200 import capi, synth, tp_stack
from oracle import oracle
from parity_utils import assert_parity

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _dev16(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.float16)


def test_sequence_arguments_are_checked_without_a_gpu():
    lib = capi.lib()
    h = C.c_void_p()
    ops = (capi.SeqOp * 1)()
    bufs = (capi.SeqBuffer * 1)()
    assert lib.lutgemm_sequence_create(None, ops, 1, bufs, 0, 0, 1) == capi.ERR_NULL
    assert lib.lutgemm_sequence_create(C.byref(h), ops, 0, bufs, 0, 0, 1) == capi.ERR_SHAPE
    assert lib.lutgemm_sequence_create(C.byref(h), ops, 1, bufs, 0, 2, 2) == capi.ERR_SHAPE      # rank outside the group
    bufs[0].kind, bufs[0].n = 3, 16
    assert lib.lutgemm_sequence_create(C.byref(h), ops, 1, bufs, 1, 0, 1) == capi.ERR_SHAPE      # unknown buffer kind
    bufs[0].kind, bufs[0].n = 2, 16
    ops[0].w, ops[0].in_kind, ops[0].out_kind, ops[0].n = None, 1, 0, 16                         # a NULL step adds rows
    assert lib.lutgemm_sequence_create(C.byref(h), ops, 1, bufs, 1, 0, 1) == capi.ERR_SHAPE
    assert lib.lutgemm_sequence_run(None, None) == capi.ERR_NULL
    assert lib.lutgemm_sequence_destroy(None) == capi.OK


@pytest.mark.gpu
@pytest.mark.parametrize("bias", [False, True])
def test_independent_matvecs_match_the_oracle(bias):
    """Three unrelated matvecs (different shapes and plane counts, one group size) in one launch."""
    import torch
    shapes = [(1024, 1536, 3), (2304, 512, 2), (264, 4096, 4)]          # (N, K, q); 264 columns: a ragged tile
    g = 128
    layers, xs, ys, ops = [], [], [], []
    for i, (N, K, q) in enumerate(shapes):
        bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=50 + i, with_bias=bias)
        w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g, qb)
        xh = synth.activations(1, K, seed=70 + i)
        x, y = _dev16(xh), torch.zeros((1, N), dtype=torch.float16, device="cuda")
        layers.append((bW, alpha, qb, w, xh)); xs.append(x); ys.append(y)
        ops.append(dict(w=w, in_kind=0, x_ext=x, out_kind=0, y_ext=y))
    seq = L.MatvecSequence(ops)
    for rep in range(3):                                                 # the step number advances by itself
        for y in ys:
            y.zero_()
        seq.run()
        assert seq.status() == 0
        for (bW, alpha, qb, w, xh), y, (N, K, q) in zip(layers, ys, shapes):
            ref = oracle.bcq_matmul_fp32(xh, bW, alpha.astype(np.float16), None if qb is None else qb.astype(np.float16), g)
            assert_parity(y.float().cpu().numpy(), ref, K)
    seq.close()
    for _, _, _, w, _ in layers:
        w.close()


@pytest.mark.gpu
def test_chained_stack_matches_per_call_stack_and_oracle_and_replays():
    """world = 1: every hand-over of the decoder stack goes through exchange lines (all-gather and all-reduce forms)."""
    import torch
    from lutgemm_b200 import tp_seq
    H, F, Q, G, LAYERS = 512, 1536, 3, 128, 3
    plain = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, device="cuda", seed=1, generate="host")
    seq = tp_seq.SeqTPStack(H, F, Q, G, LAYERS, device="cuda", seed=1, generate="host")
    xh = synth.activations(1, H, seed=4)
    x = _dev16(xh).reshape(-1)
    want = plain.step(x).float().cpu().numpy()
    for rep in range(3):
        got = seq.step(x).float().cpu().numpy()
        assert seq.device_status() == 0
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-4, rep
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        seq.step()
        with torch.cuda.graph(g, stream=side):
            seq.step()
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(3):
        g.replay()
        torch.cuda.synchronize()
        got = seq._y16.float().cpu().numpy()
        assert seq.device_status() == 0
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-4, rep
    del g
    seq.close()


@pytest.mark.gpu
def test_a_wait_that_nothing_satisfies_runs_out_and_is_reported():
    """A matvec whose input buffer no matvec fills: the bounded wait gives up after the limit, the status word says
    so (4), the launch ends by itself and the context keeps working."""
    import torch
    N, K, q, g = 512, 512, 2, 128
    bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=3)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g)
    y = torch.zeros((1, N), dtype=torch.float16, device="cuda")
    seq = L.MatvecSequence([dict(w=w, in_kind=1, in_buf=0, out_kind=0, y_ext=y)], [(1, K)])
    seq.set_wait_limit(20)
    seq.run()
    torch.cuda.synchronize()                                            # returns: the wait is bounded
    assert seq.status() & 4
    seq.clear_status()
    assert seq.status() == 0
    seq.close()
    xh = synth.activations(1, K, seed=1)
    L.matmul(y, _dev16(xh), w, 1)
    torch.cuda.synchronize()
    ref = oracle.bcq_matmul_fp32(xh, bW, alpha.astype(np.float16), None, g)
    assert_parity(y.float().cpu().numpy(), ref, K)
    w.close()


@pytest.mark.gpu
def test_sequence_stack_two_gpus_matches_nccl_stack():
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(ROOT, "tests", "tp_worker.py"), "--seq"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    good = re.findall(r"TPRESULT rank=\d+ ok=True", out.stdout)
    bad = re.findall(r"TPRESULT rank=\d+ ok=False", out.stdout)
    assert out.returncode == 0 and len(good) == 2 and not bad, out.stdout[-2000:] + out.stderr[-2000:]
