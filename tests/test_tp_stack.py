"""Tensor-parallel sharding of the BCQ linears: shard algebra on the host, a world_size-2 run over gloo
on CPU ranks (host stand-ins for the matvec), and the real kernels on one GPU (and on two when present)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from lutgemm_b200 import synth, tp_stack
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_column_and_row_shards_recombine():
    N, K, q, g, P = 64, 512, 3, 128, 4
    bW, alpha, qb = synth.bcq_layer(N, K, q, g, seed=5, with_bias=True)
    x = synth.activations(1, K, seed=2)
    a_h, qb_h = alpha.astype(np.float16), qb.astype(np.float16)
    full = oracle.bcq_matmul_fp32(x, bW, a_h, qb_h, g)
    cols = []
    for r in range(P):
        sb, sa, sq = tp_stack.shard_columns(bW, alpha, qb, P, r)
        cols.append(oracle.bcq_matmul_fp32(x, sb, sa.astype(np.float16), sq.astype(np.float16), g))
    np.testing.assert_allclose(np.concatenate(cols, axis=1), full, rtol=0, atol=0)          # columns are independent
    rows = []
    for r in range(P):
        sb, sa, sq = tp_stack.shard_rows(bW, alpha, qb, g, P, r)
        xs = np.ascontiguousarray(x[:, r * (K // P):(r + 1) * (K // P)])
        rows.append(oracle.bcq_matmul_fp32(xs, sb, sa.astype(np.float16), sq.astype(np.float16), g))
    np.testing.assert_allclose(np.sum(rows, axis=0), full, rtol=1e-5, atol=1e-5)             # the k-sum is associative
    with pytest.raises(ValueError):
        tp_stack.shard_rows(bW, alpha, qb, g, 8, 0)       # K/P = 64 is not a whole group
    with pytest.raises(ValueError):
        tp_stack.shard_columns(bW, alpha, qb, 16, 0)      # N/P = 4 columns


def test_stack_bytes_match_published_figure():
    assert tp_stack.stack_algorithmic_bytes(12288, 49152, 3, 128, 1) == 764805120
    assert tp_stack.stack_algorithmic_bytes(12288, 49152, 3, 128, 96) == 73421291520


WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["LG_ROOT"])
from lutgemm_b200 import synth, tp_stack
from oracle import oracle

def host_container(bW, alpha, n_loc, k_loc):
    return {"bW": bW, "alpha": alpha.astype(np.float16)}
def mv(out, x, w):
    y = oracle.bcq_matmul_fp32(x.numpy().reshape(1, -1), w["bW"], w["alpha"], None, G)
    out.copy_(torch.from_numpy(y.reshape(-1)).to(out.dtype))
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
H, F, Q, G, LAYERS = 256, 512, 2, 64, 2
st = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, rank=rank, world=world, device="cpu", seed=3,
                            matvec=mv, matvec_f32=mv, make_container=host_container, generate="host")
x = torch.from_numpy(synth.activations(1, H, seed=9).reshape(-1).copy())
y = st.step(x).clone()
ref = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, rank=0, world=1, device="cpu", seed=3,
                             matvec=mv, matvec_f32=mv, make_container=host_container, generate="host")
y1 = ref.step(x).clone()
err = float((y.float() - y1.float()).abs().max()); scale = float(y1.float().abs().max())
gathered = [torch.empty_like(y) for _ in range(world)]
dist.all_gather(gathered, y)
same = all(torch.equal(gathered[0], t) for t in gathered)
print(f"RESULT rank={rank} err={err:.3e} scale={scale:.3e} same={same}", flush=True)
dist.destroy_process_group()
'''


def test_two_rank_stack_over_gloo_matches_single_rank(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, LG_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        line = [l for l in o.splitlines() if l.startswith("RESULT")][0]
        f = dict(kv.split("=") for kv in line.split()[1:])
        assert f["same"] == "True"                                  # every rank ends with the same activations
        assert float(f["err"]) <= 2e-3 * float(f["scale"]) + 1e-3   # fp16 roundings of the intermediate vectors only


SEQ_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["LG_ROOT"])
from lutgemm_b200 import synth, tp_stack, tp_seq
from oracle import oracle

# A host model of what lutgemm_sequence_run does with the list tp_seq.stack_program builds: exchange buffers that every
# rank fills on every rank (fp16 vectors, one fp32 row per rank), consumers that add the rows in rank order and round
# once.  The "stores into every rank's copy" are an all_gather of what each rank produced, placed by the PRODUCER's
# out_off (taken from that rank's own program).
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
H, F, Q, G, LAYERS = 256, 512, 2, 64, 2
def host_container(bW, alpha, n_loc, k_loc):
    return {"bW": bW, "alpha": alpha.astype(np.float16)}
def mv(out, x, w):
    y = oracle.bcq_matmul_fp32(x.numpy().reshape(1, -1), w["bW"], w["alpha"], None, G)
    out.copy_(torch.from_numpy(y.reshape(-1)).to(out.dtype))
st = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, rank=rank, world=world, device="cpu", seed=3,
                            matvec=mv, matvec_f32=mv, make_container=host_container, generate="host")
programs = [tp_seq.stack_program(H, F, LAYERS, r, world) for r in range(world)]
buffers, ops = programs[rank]
vec = {b: np.zeros(n, np.float16) for b, (kind, n) in enumerate(buffers) if kind == 1}
rows = {b: np.zeros((world, n), np.float32) for b, (kind, n) in enumerate(buffers) if kind == 2}
x = synth.activations(1, H, seed=9).reshape(-1).copy()
result = None
for i, o in enumerate(ops):
    w = None if o["idx"] is None else st.weights[o["layer"]][o["idx"]]
    K = o["n"] if w is None else w["bW"].shape[0] * 32
    off = o.get("in_off", 0)
    if o["in_kind"] == 0:
        xin = x
    elif o["in_kind"] == 1:
        xin = vec[o["in_buf"]][off:off + K]
    else:
        acc = np.zeros(K, np.float32)
        for r in range(world):                       # rank order, one rounding
            acc += rows[o["in_buf"]][r, off:off + K]
        xin = acc.astype(np.float16)
    if w is None:
        result = xin.copy()
        continue
    y = oracle.bcq_matmul_fp32(xin.reshape(1, -1), w["bW"], w["alpha"], None, G).reshape(-1)
    N = y.size
    if o["out_kind"] == 1:
        mine = torch.from_numpy(y.astype(np.float16).astype(np.float32))     # fp16 values, carried exactly in fp32
        got = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(got, mine)
        for r in range(world):
            ro = programs[r][1][i]["out_off"]
            vec[o["out_buf"]][ro:ro + N] = got[r].numpy().astype(np.float16)
    else:
        mine = torch.from_numpy(y.astype(np.float32).copy())
        got = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(got, mine)
        for r in range(world):
            rows[o["out_buf"]][r, o.get("out_off", 0):o.get("out_off", 0) + N] = got[r].numpy()
want = st.step(torch.from_numpy(x)).numpy()          # the same shards through gloo collectives
err = float(np.abs(result.astype(np.float32) - want.astype(np.float32)).max()); scale = float(np.abs(want.astype(np.float32)).max())
print(f"RESULT rank={rank} err={err:.3e} scale={scale:.3e} ops={len(ops)} buffers={len(buffers)}", flush=True)
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_program_of_the_stack_over_gloo_matches_collectives(tmp_path, world):
    """The list of matvecs and exchange buffers that the one-launch stack hands to lutgemm_sequence_create, executed by a
    host model of the exchange on two and on four CPU ranks, against the same shards run through gloo all-gather /
    all-reduce."""
    script = tmp_path / "seq_worker.py"
    script.write_text(SEQ_WORKER)
    env = dict(os.environ, LG_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29617 + world), WORLD_SIZE=str(world),
               OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        line = [l for l in o.splitlines() if l.startswith("RESULT")][0]
        f = dict(kv.split("=") for kv in line.split()[1:])
        assert f["ops"] == "9" and f["buffers"] == "8"
        assert float(f["err"]) <= 1e-3 * float(f["scale"]) + 1e-4   # same roundings in both; only summation order differs


@pytest.mark.gpu
def test_single_gpu_stack_matches_host_chain():
    torch = pytest.importorskip("torch")
    H, F, Q, G, LAYERS = 512, 1024, 3, 128, 2
    st = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, device="cuda", seed=1, generate="host")
    x = synth.activations(1, H, seed=4)
    y = st.step(torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16).reshape(-1)).float().cpu().numpy()
    # the same chain on the host with the fp32 reference and the same fp16 roundings between linears
    cur = x
    for layer in range(LAYERS):
        outs = {}
        for idx, (name, N, K, mode) in enumerate(st.shapes):
            bW, alpha, _ = synth.bcq_layer(N, K, Q, G, seed=synth.seed_for("stack", N, K, Q, 131 * layer + idx + 1),
                                           alpha_std=1.0 / np.sqrt(K * Q))
            inp = cur if name in ("qkv", "fc1") else outs["prev"]
            if name == "out":
                inp = np.ascontiguousarray(outs["qkv"][:, :H])
            if name == "fc2":
                inp = outs["fc1"]
            yv = oracle.bcq_matmul_fp32(inp, bW, alpha.astype(np.float16), None, G).astype(np.float16)
            outs[name] = yv
            outs["prev"] = yv
            if name == "out":
                cur = yv
        cur = outs["fc2"]
    ref = cur.astype(np.float32).reshape(-1)
    assert np.abs(y - ref).max() <= 1e-2 * np.abs(ref).max() + 1e-3


@pytest.mark.gpu
def test_fused_stack_single_rank_matches_collective_stack_and_replays():
    """world = 1 exercises the whole fused machinery (peer stores to itself, flags, re-arming, graph replay)."""
    torch = pytest.importorskip("torch")
    from lutgemm_b200 import tp_fused
    H, F, Q, G, LAYERS = 512, 1024, 3, 128, 3
    plain = tp_stack.TPLinearStack(H, F, Q, G, LAYERS, device="cuda", seed=1, generate="host")
    fused = tp_fused.FusedTPStack(H, F, Q, G, LAYERS, device="cuda", seed=1, generate="host")
    x = torch.from_numpy(synth.activations(1, H, seed=4).view(np.int16)).cuda().view(torch.float16).reshape(-1)
    want = plain.step(x).float().cpu().numpy()
    for rep in range(3):                                   # the flags must re-arm themselves between steps
        got = fused.step(x).float().cpu().numpy()
        assert fused.device_status() == 0
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-4, rep
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fused.step(x)
        with torch.cuda.graph(g, stream=side):
            fused.step(x)
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(3):
        g.replay()
        torch.cuda.synchronize()
        got = fused._y16.float().cpu().numpy()
        assert fused.device_status() == 0
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max() + 1e-4, rep
    del g
    fused.close()


@pytest.mark.gpu
def test_fused_stack_two_gpus_matches_nccl_stack():
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "tp_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    import re
    # the two ranks write to the same pipe and their lines can run together: count the records, not the lines
    good = re.findall(r"TPRESULT rank=\d+ ok=True", out.stdout)
    bad = re.findall(r"TPRESULT rank=\d+ ok=False", out.stdout)
    assert out.returncode == 0 and len(good) == 2 and not bad, out.stdout[-2000:] + out.stderr[-2000:]


@pytest.mark.gpu
def test_peer_wait_runs_out_and_reports_status():
    """A tensor-parallel input whose flag nobody raises: the kernel's bounded wait gives up, the container's
    status word reports it (4 = peer time-out), nothing hangs, and the context keeps working."""
    import ctypes as C
    torch = pytest.importorskip("torch")
    import lutgemm_b200 as L
    from lutgemm_b200 import capi
    N, K, q, g = 512, 512, 2, 128
    bW, alpha, _ = synth.bcq_layer(N, K, q, g, seed=3)
    w = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g)
    x = torch.from_numpy(synth.activations(1, K, seed=1).view(np.int16)).cuda().view(torch.float16)
    y = torch.zeros((1, N), dtype=torch.float16, device="cuda")
    words = torch.zeros(8, dtype=torch.int32, device="cuda")          # [0] = flag that stays 0, [1] = done counter
    link = capi.TpLink()
    link.world, link.x_mode, link.out_mode = 1, 1, 0
    link.flag_in, link.flag_target, link.done_counter = words.data_ptr(), 1, words.data_ptr() + 4
    lib = capi.lib()
    rc = lib.lutgemm_matvec_tp(x.data_ptr(), w.handle, C.byref(link), y.data_ptr(), None,
                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == capi.OK
    torch.cuda.synchronize()                                          # returns: the wait is bounded
    st = C.c_int(-1)
    capi.check(lib.lutgemm_weight_device_status(w.handle, C.byref(st)), "device_status")
    assert st.value & 4
    assert int(words[0].item()) == 0 and int(words[1].item()) == 0    # the kernel re-armed its words
    # the context is intact: an ordinary matvec on a fresh container is still right
    w2 = L.nQWeight_fp16(bW, alpha, K, N, q, False, K // g)
    L.matmul(y, x, w2, 1)
    torch.cuda.synchronize()
    ref = oracle.bcq_matmul_fp32(synth.activations(1, K, seed=1), bW, alpha.astype(np.float16), None, g)
    assert np.abs(y.float().cpu().numpy() - ref).max() <= 1e-2 * np.abs(ref).max()
    w.close(); w2.close()
