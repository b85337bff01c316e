#!/usr/bin/env python
"""Benchmark of the BCQ LUT matvec hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 GPU): the metric configuration, one m = 1 matvec y = x.W with N = K = 12288, q = 3 bit
planes, group size 128, random BCQ weights.  One "step" is one matvec on each of ROT distinct weight
sets (ROT x 63.75 MB > 4x the 126 MB L2, so every matvec streams its weights from HBM).
`value` is effective GB/s = algorithmic bytes / device time with everything resident in HBM;
`e2e` is the same through the host-buffer C-ABI call (H2D of x and D2H of y inside the timed region).
With N > 1 ranks (one process per GPU) the workload is the tensor-parallel decoder linear stack (96 layers x
{QKV, out-proj, FC1, FC2}, hidden 12288, FFN 49152, q = 3, g = 128, m = 1; column-parallel + all-gather,
row-parallel + all-reduce): strong scaling, value = the stack's algorithmic bytes / step time, max over ranks.
A step is one kernel launch per GPU (lutgemm_sequence_run).  The N = 1 line carries the same stack on one GPU under
"stack_tp1", so that the N-GPU numbers can be divided by a one-GPU number of the same workload.

`--impl reference` times the reference's CPU path for the same matvec on the host cores:
lutGEMM::dequantize_cpu (compiled from the reference sources into oracle/_ref, run on k-slabs by
every host thread) followed by the test's serial fp32 matmul loop (restated in oracle/, OpenMP over
columns); one matvec per step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from lutgemm_b200 import synth  # noqa: E402

METRIC = "bcq_gemv_effective_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE gemv_tma_kernel launch at the default bench shape
# (N = K = 12288, q = 3, g = 128, m = 1), from an ncu capture of this very command; to be captured again
# whenever that kernel changes (a run under ncu is never a bench value, so the figure is carried here).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 64022272      # 63 812 608 read + 209 664 written


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="reference: the reference's CPU path; reference-gpu (helper leg): the reference's own CUDA kernels, "
                         "compiled for sm_100a into oracle/_ref/libref_gpu.so, on the same matvec")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference-CUDA-kernel leg of the default run")
    ap.add_argument("--reference-gpu", action="store_true", help="with --m > 1: also time the reference's batched path (dequantise + cuBLAS)")
    ap.add_argument("--workload", default="auto", choices=["auto", "gemv", "stack", "quantize", "gptq"],
                    help="gemv: the headline matvec; stack: tensor-parallel decoder linear stack; auto: gemv on 1 GPU, stack on more; "
                         "quantize: the BCQ quantiser (greedy + --rounds refinements) on an [n, k] fp32 layer, a side line; "
                         "gptq: the 3-bit uniform comparison matvec (matmul_gptq), with the reference's two kernels beside it")
    ap.add_argument("--rounds", type=int, default=15, help="quantize workload: refinement rounds")
    ap.add_argument("--tp", default="seq", choices=["seq", "fused", "nccl"],
                    help="stack workload: seq = the whole step as one persistent kernel per GPU (exchange lines over NVLink); "
                         "fused = one kernel per matvec with the exchange fused in (peer pushes + flags); nccl = NCCL collectives")
    ap.add_argument("--no-stack-tp1", action="store_true", help="skip the one-GPU stack anchor of the default run")
    ap.add_argument("--layers", type=int, default=96, help="decoder layers of the stack workload")
    ap.add_argument("--hidden", type=int, default=12288)
    ap.add_argument("--ffn", type=int, default=49152)
    ap.add_argument("--n", type=int, default=12288)
    ap.add_argument("--k", type=int, default=12288)
    ap.add_argument("--q", type=int, default=3)
    ap.add_argument("--g", type=int, default=128)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--m", type=int, default=1, help="activation rows per matmul (1 = the headline matvec)")
    ap.add_argument("--rot", type=int, default=8, help="distinct weight sets cycled per step")
    ap.add_argument("--ntile", type=int, default=0, help="columns per CTA of the matvec (0 = automatic)")
    ap.add_argument("--variant", type=int, default=0, help="0 = bulk-copy fed matvec kernel, 1 = register-streaming kernel")
    ap.add_argument("--ordered", action="store_true", help="bit-reproducible split-k (slabs added in order)")
    ap.add_argument("--int8", action="store_true", help="batches of up to 16 rows: the integer tensor-core kernel instead of the fp16 one")
    ap.add_argument("--no-pdl", action="store_true", help="plain launches instead of programmatic dependent launch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every matvec from Python instead of replaying a CUDA graph")
    return ap.parse_args()


def workload_name(a):
    return f"bcq_gemv m={a.m} n={a.n} k={a.k} q={a.q} g={a.g}" + (" +q_bias" if a.bias else "")


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_gemv(a, threads):
    """One matvec of the workload through the reference's CPU path; returns (seconds, kind, y)."""
    from oracle import oracle
    bW, alpha, qb = synth.bcq_layer(a.n, a.k, a.q, a.g, seed=synth.seed_for("bench", a.n, a.k, a.q, 0), with_bias=a.bias)
    x = synth.activations(1, a.k, seed=123)
    a_h = alpha.astype(np.float16)
    oracle.set_threads(threads)
    have_ref = oracle.ref_cpu() is not None
    W = np.empty((a.k, a.n), np.float16)
    t0 = time.perf_counter()
    if have_ref:
        # the reference function, unmodified, on disjoint k-slabs (whole groups) from every host thread
        groups = a.k // a.g
        per = (groups + threads - 1) // threads
        def slab(i):
            g0, g1 = i * per, min(groups, (i + 1) * per)
            if g0 >= g1:
                return
            k0, k1 = g0 * a.g, g1 * a.g
            W[k0:k1] = oracle.dequantize_cpu(bW[k0 // 32:k1 // 32], a_h[g0:g1], a.g, use_reference=True)
        ts = [threading.Thread(target=slab, args=(i,)) for i in range(threads)]
        [t.start() for t in ts]
        [t.join() for t in ts]
    else:
        W[:] = oracle.dequantize_cpu(bW, a_h, a.g)
    Wf = W.astype(np.float32)
    y = oracle.matmul_cpu(x.astype(np.float32), Wf)
    if qb is not None:
        y = y + x.astype(np.float32).reshape(1, -1, a.g).sum(-1) @ qb
    dt = time.perf_counter() - t0
    return dt, ("reference" if have_ref else "port"), y


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    B = synth.algorithmic_bytes(a.n, a.k, a.q, a.g, 1, a.bias)
    steps, warm = max(1, min(a.steps, 5)), min(a.warmup, 1)
    for _ in range(warm):
        cpu_reference_gemv(a, threads)
    times = []
    kind = "port"
    for _ in range(steps):
        dt, kind, _ = cpu_reference_gemv(a, threads)
        times.append(dt)
    t = sum(times) / len(times)
    val = B / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": a.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(a), "matvecs_per_step": 1},
            "steps_requested": a.steps, "warmup_requested": a.warmup, "steps_capped_at": 5, "warmup_capped_at": 1,
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind,
                             "sample": "one full matvec per step: dequantize_cpu on k-slabs + serial-k fp32 matmul"},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_reference_gpu(a):
    """The reference's CUDA path (lutGEMM::matmul -> cudaMemset + _nqmv / _nqmv_bias, lutGEMM/src/kernels.cu:64-71)
    recompiled for sm_100a, timed on the same matvec with the same rotation of weight sets.  Prints one small JSON line."""
    import ctypes as C
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
    if not os.path.exists(so) or (a.m > 1 and a.q > 4):
        print(json.dumps({"reference_gpu": None, "why": "oracle/_ref/libref_gpu.so not built" if a.q <= 4 or a.m == 1 else
                          "the reference's batched path dequantises nothing for q > 4"}))
        return
    R = C.CDLL(so)
    R.ref_gpu_create.restype = C.c_void_p
    R.ref_gpu_create.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    R.ref_gpu_matmul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    torch.cuda.set_device(0)
    rot = max(1, a.rot)
    keep, ws = [], []
    for i in range(rot):
        bW, alpha, qb = synth.bcq_layer(a.n, a.k, a.q, a.g, seed=synth.seed_for("bench", a.n, a.k, a.q, i), with_bias=a.bias)
        keep.append((bW, alpha, qb))
        ws.append(R.ref_gpu_create(bW.ctypes.data, alpha.ctypes.data, None if qb is None else qb.ctypes.data, a.k, a.n, a.q, a.k // a.g))
    x_host = synth.activations(a.m, a.k, seed=123)
    x = torch.from_numpy(x_host.view(np.int16)).cuda().view(torch.float16)
    y = torch.empty((a.m, a.n), dtype=torch.float16, device="cuda")
    for _ in range(3):
        for w in ws:
            R.ref_gpu_matmul(y.data_ptr(), x.data_ptr(), w, a.m)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = max(1, min(a.steps, 20))
    e0.record()
    for _ in range(steps):
        for w in ws:
            R.ref_gpu_matmul(y.data_ptr(), x.data_ptr(), w, a.m)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * rot)
    B = synth.algorithmic_bytes(a.n, a.k, a.q, a.g, a.m, a.bias)
    # accuracy of the reference kernel on the last weight set, against the fp32 host evaluation
    from oracle import oracle
    bW, alpha, qb = keep[-1]
    ref = oracle.bcq_matmul_fp32(x_host, bW, alpha.astype(np.float16), None if qb is None else qb.astype(np.float16), a.g)
    got = y.float().cpu().numpy()
    print(json.dumps({"reference_gpu": {"us_per_matvec": us, "value": B / (us * 1e-6) / 1e9, "unit": UNIT,
                                        "kernel": ("_nqmv_bias<32>" if a.bias else "_nqmv<64>") if a.m == 1 else
                                                  "_dequantize_t + cublasGemmEx (q_bias ignored, two device synchronisations)",
                                        "launches_per_matvec": 2,
                                        "mae_vs_fp32_host": float(np.abs(got - ref).mean())}}), flush=True)


def shutdown_process_group(dist_mod):
    """Leaves the process group without risking a hang at exit: the captured graphs that hold NCCL kernels are
    gone by now (the caller dropped them); if the communicator tear-down still does not finish, the process
    exits anyway (the JSON line has already been flushed)."""
    sys.stdout.flush()
    sys.stderr.flush()
    if dist_mod is None:
        return
    done = threading.Event()

    def _destroy():
        try:
            dist_mod.destroy_process_group()
        except Exception:
            pass
        done.set()

    threading.Thread(target=_destroy, daemon=True).start()
    if not done.wait(30.0):
        os._exit(0)


def time_stack(a, stack, x, rank, world, dist, barrier, tp):
    """Warm-up, CUDA-graph capture and the timed loop of one stack object; returns (seconds per step, launch kind, clocks)."""
    import torch
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if tp == "seq":
        stack.x_in.copy_(x)
        step = lambda: stack.step()
    else:
        step = lambda: stack.step(x)
    for _ in range(max(3, a.warmup)):
        step()
    barrier()
    run_step, graph = step, None
    if not a.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            run_step = graph.replay
            for _ in range(2):
                run_step()
        except Exception as e:          # capture refused: time eager launches instead
            graph, run_step = None, step
            if rank == 0:
                print(f"bench.py: CUDA graph capture failed ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
        barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        run_step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    kind = "python" if graph is None else "cuda graph of one step, replayed"
    graph = None
    run_step = None
    return ms / 1e3 / a.steps, kind, clocks


def make_stack(a, tp, rank, world, local):
    from lutgemm_b200 import tp_stack
    if tp == "seq":
        from lutgemm_b200 import tp_seq
        return tp_seq.SeqTPStack(a.hidden, a.ffn, a.q, a.g, a.layers, rank=rank, world=world, device=f"cuda:{local}", seed=11)
    if tp == "fused":
        from lutgemm_b200 import tp_fused
        return tp_fused.FusedTPStack(a.hidden, a.ffn, a.q, a.g, a.layers, rank=rank, world=world, device=f"cuda:{local}", seed=11)
    return tp_stack.TPLinearStack(a.hidden, a.ffn, a.q, a.g, a.layers, rank=rank, world=world, device=f"cuda:{local}", seed=11)


def run_stack(a):
    """Tensor-parallel decoder linear stack (BASELINE config 5): `layers` x {QKV, out, FC1, FC2} at m = 1, sharded over
    the ranks (column-parallel + all-gather, row-parallel + all-reduce).  Strong scaling: the stack is the same at every N.
    value = algorithmic bytes of the whole stack / step time (max over ranks), i.e. aggregate effective GB/s.
    Before the timed loop one step of the same shards runs through NCCL collectives and is compared with the path that
    is timed (if the default one-launch form fails that check, the one-kernel-per-matvec form is timed instead and the line
    says so); after the timed loop every rank's device status word is read.  A failing check ends the run with a non-zero code."""
    import torch
    import torch.distributed as dist
    from lutgemm_b200 import capi, tp_stack

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    lib = capi.lib()
    lib.lutgemm_set_dependent_launch(0 if a.no_pdl else 1)
    stack = make_stack(a, a.tp, rank, world, local)
    B = tp_stack.stack_algorithmic_bytes(a.hidden, a.ffn, a.q, a.g, a.layers)
    x_host = synth.activations(1, a.hidden, seed=5).reshape(-1)
    x = torch.from_numpy(x_host.view(np.int16).copy()).cuda().view(torch.float16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the same shards through the process group's collectives (the parent class's step) against the timed path
    def check_against_nccl(stk):
        want = tp_stack.TPLinearStack.step(stk, x).float().clone()
        got = stk.step(x).float().clone()
        torch.cuda.synchronize()
        denom = float(want.abs().max().item()) + 1e-9
        rel = float((got - want).abs().max().item()) / denom
        # both paths round to fp16 after each of the 4 x layers matvecs and add their k-slabs in no fixed order, so
        # they drift apart like a random walk: about 1e-3 of the largest output per sqrt(matvec); garbage would be O(1)
        tol = max(2e-3, 1e-3 * (4 * a.layers) ** 0.5)
        dev_ok = (stk.device_status() == 0) if hasattr(stk, "device_status") else True
        flag = torch.tensor([1.0 if (rel <= tol and bool(torch.isfinite(got).all()) and dev_ok) else 0.0], device="cuda")
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item() > 0.5), rel

    matches, max_rel, fell_back = None, None, None
    if a.tp != "nccl":
        matches, max_rel = check_against_nccl(stack)
        if not matches and a.tp == "seq":
            # every rank takes the same branch (the flag is reduced over the ranks): time the one-kernel-per-matvec form,
            # which keeps its own exchange buffers, and say so in the line
            fell_back = f"the one-launch form failed its check against the NCCL step (max relative difference {max_rel:.3g})"
            if rank == 0:
                print("bench.py: " + fell_back + "; timing --tp fused instead", file=sys.stderr, flush=True)
            del stack
            torch.cuda.empty_cache()
            a.tp = "fused"
            stack = make_stack(a, a.tp, rank, world, local)
            matches, max_rel = check_against_nccl(stack)
    sec_per_step, launch_kind, clocks = time_stack(a, stack, x, rank, world, dist if world > 1 else None, barrier, a.tp)
    status = stack.device_status() if hasattr(stack, "device_status") else 0
    st = torch.tensor([float(status)], device="cuda")
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    status = int(st.item())
    # end to end: the step's activation vector comes from pinned host memory and its result goes back every step
    xin = torch.from_numpy(x_host.view(np.int16).copy()).pin_memory()
    yout = torch.empty(a.hidden, dtype=torch.int16).pin_memory()
    xdev = stack.x_in if a.tp == "seq" else torch.empty(a.hidden, dtype=torch.float16, device="cuda")
    barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        xdev.view(torch.int16).copy_(xin, non_blocking=True)
        y = stack.step() if a.tp == "seq" else stack.step(xdev)
        yout.copy_(y.view(torch.int16), non_blocking=True)
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    ok = status == 0 and matches is not False
    if rank == 0:
        peak, peak_kind = measured_peak()
        value = B / sec_per_step / 1e9
        per_gpu = value / world
        how = {"seq": "the whole step is one persistent kernel per GPU; results travel between matvecs and GPUs in 16-byte exchange "
                      "lines that carry the step number (plain peer stores over NVLink)",
               "fused": "one kernel per matvec, exchange fused in (peer stores + flags over NVLink)",
               "nccl": "NCCL collectives"}[a.tp]
        launches = {"seq": 1, "fused": a.layers * 4 + 1, "nccl": a.layers * 4}[a.tp]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": max(3, a.warmup),
            "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"tensor-parallel decoder linear stack, {a.layers} layers, hidden {a.hidden}, ffn {a.ffn}, "
                                   f"q={a.q} g={a.g} m=1", "parallelism": f"tp{world}: QKV/FC1 column-parallel + all-gather, out-proj/FC2 row-parallel + all-reduce; "
                                   + how, "algorithmic_bytes_per_step": B,
                       "l2": f"{B / world / 1e9:.1f} GB of packed weights per GPU per step, far larger than L2",
                       "launch": launch_kind},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_source": peak_kind, "traffic": None,
                         "kernel": ("gemv_seq_kernel" if a.tp == "seq" else "gemv_tma_kernel") + " (per GPU average over the step, exchange included)"},
            "gpu_launches": int(a.steps * launches),
            "device_status": status,
            "matches_nccl": matches, "max_rel_diff_vs_nccl": max_rel, "tp": a.tp, "tp_fallback": fell_back,
            "matches_nccl_tolerance": None if matches is None else max(2e-3, 1e-3 * (4 * a.layers) ** 0.5),
            "clocks": clocks,
            "e2e": {"value": B * a.steps / dt / 1e9, "unit": UNIT, "h2d_bytes_per_step": 2 * a.hidden, "d2h_bytes_per_step": 2 * a.hidden},
        }
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    shutdown_process_group(dist if world > 1 else None)
    if not ok:
        sys.exit(3)


def run_quantize(a):
    """Side line: the device BCQ quantiser on one synthetic fp32 layer [n, k] straight into the container layout,
    against the numpy restatement of the reference's torch code on a few rows (host cores)."""
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import capi
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    w = torch.randn((a.n, a.k), device="cuda", generator=gen) * 0.02
    lib = capi.lib()
    n0 = lib.lutgemm_kernel_launch_count()
    for _ in range(max(a.warmup, 3)):
        L.bcq_quantize_device(w, a.q, a.rounds, a.g)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        L.bcq_quantize_device(w, a.q, a.rounds, a.g)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    weights = a.n * a.k
    g_eff = a.g if a.g > 0 else a.k                       # --g -1: one group per row, the reference's default
    # bytes that have to move: fp32 weights in, packed planes + fp16 scales out
    alg_bytes = 4 * weights + weights * a.q // 8 + 2 * (a.k // g_eff) * a.q * a.n
    line = {"metric": "bcq_quantize_throughput", "value": weights / ms / 1e3, "unit": "Mweights/s", "n_gpus": 1,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"bcq_quantize n={a.n} k={a.k} q={a.q} g={a.g} rounds={a.rounds}",
                       "l2": f"input {4 * weights / 1e6:.0f} MB per step" + (" (larger than L2)" if 4 * weights > 126e6 else " (fits L2: compute-bound kernel)")},
            "roofline": {"bound": "hbm", "achieved": alg_bytes / ms / 1e6, "peak": measured_peak()[0], "unit": "GB/s",
                         "frac": alg_bytes / ms / 1e6 / measured_peak()[0], "peak_source": measured_peak()[1], "traffic": None,
                         "kernel": "bcq_quantize_kernel", "note": "arithmetic-bound (q x q solves and 2^q-level search per group), far below the HBM bound"},
            "gpu_launches": int(lib.lutgemm_kernel_launch_count() - n0) - max(a.warmup, 3), "clocks": clocks}
    if not a.no_cpu_baseline:
        from oracle import bcq_quantizer as bq
        rows = max(1, min(a.n, (1 << 19) // a.k))
        wh = w[:rows].cpu().numpy()
        t0 = time.perf_counter()
        bq.quantize(wh, a.q, a.rounds, a.g)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": rows * a.k / dt / 1e6, "unit": "Mweights/s", "cores": 1, "kind": "port",
                                "sample": f"{rows} of {a.n} rows, numpy restatement of examples/bcq.py, {dt:.1f} s"}
    print(json.dumps(line))


def run_gptq(a):
    """Side line: the 3-bit uniform (GPTQ-format) matvec of the reference's header, ours and (when oracle/_ref holds them)
    the reference's own two kernels, on the same B200; --rot weight sets cycled so that nothing is served from L2."""
    import ctypes as C
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import capi
    torch.cuda.set_device(0)
    N, K, rot = a.n, a.k, a.rot
    kp = K * 3 // 32
    gen = torch.Generator(device="cuda").manual_seed(99)
    mats = [torch.randint(-2**31, 2**31 - 1, (kp, N), dtype=torch.int32, device="cuda", generator=gen) for _ in range(rot)]
    scale = (torch.randn(N, device="cuda", generator=gen).abs() * 0.01).half()
    zero = (scale.float() * 3.5).half()
    x = torch.randn((1, K), device="cuda", generator=gen).half()
    y = torch.empty((1, N), dtype=torch.float16, device="cuda")
    alg_bytes = kp * N * 4 + 4 * N + 2 * K + 2 * N

    def timed(fn):
        for _ in range(max(a.warmup, 3)):
            for m_ in mats:
                fn(m_)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            for m_ in mats:
                fn(m_)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (a.steps * rot)

    lib = capi.lib()
    n0 = lib.lutgemm_kernel_launch_count()
    sampler = ClockSampler(0)
    sampler.start()
    # one step (rot matvecs) captured into a CUDA graph and replayed: the Python call costs more than the kernel
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for m_ in mats:
            L.matmul_gptq(1, N, kp, scale, zero, x, m_, y)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for m_ in mats:
                L.matmul_gptq(1, N, kp, scale, zero, x, m_, y)
    torch.cuda.synchronize()
    for _ in range(max(a.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.steps * rot)
    clocks = sampler.stop()
    launches = a.steps * rot
    peak, src = measured_peak()
    line = {"metric": "gptq3_gemv_effective_bandwidth", "value": alg_bytes / us / 1e3, "unit": "GB/s", "n_gpus": 1,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": us * rot / 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"gptq3_gemv m=1 n={N} k={K}", "matvecs_per_step": rot,
                       "l2": f"{rot} weight sets cycled ({rot * kp * N * 4 / 1e6:.0f} MB per step)",
                       "launch": "cuda graph of one step, replayed (reference kernels: direct calls, they use the legacy stream)"},
            "us_per_matvec": us,
            "roofline": {"bound": "hbm", "achieved": alg_bytes / us / 1e3, "peak": peak, "unit": "GB/s",
                         "frac": alg_bytes / us / 1e3 / peak, "peak_source": src, "traffic": None, "kernel": "gptq3_gemv_kernel"},
            "gpu_launches": launches, "clocks": clocks}
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
    if os.path.exists(ref_path) and N % 256 == 0 and K % 256 == 0:      # the reference kernels check no bounds
        ref = C.CDLL(ref_path)
        if hasattr(ref, "ref_gpu_matmul_gptq"):
            ref.ref_gpu_matmul_gptq.argtypes = [C.c_int] * 3 + [C.c_void_p] * 5 + [C.c_int]
            y2 = torch.empty_like(y)
            for faster, name in ((0, "VecQuant3MatMulKernel"), (1, "VecQuant3MatMulKernelFaster")):
                t = timed(lambda m_: ref.ref_gpu_matmul_gptq(1, N, kp, scale.data_ptr(), zero.data_ptr(), x.data_ptr(),
                                                             m_.data_ptr(), y2.data_ptr(), faster))
                line.setdefault("reference_gpu", {})[name] = {"us_per_matvec": t, "value": alg_bytes / t / 1e3, "unit": "GB/s",
                                                              "launches_per_matvec": 2}
    print(json.dumps(line))


def batched_numbers(local):
    """Config 4's batched corner on this GPU: n = k = 8192, q = 2, g = 64 at m = 2 (the two-row LUT kernel), m = 16 and
    m = 128 (the tcgen05 kernel) through lutgemm_matmul, CUDA-graph replay over 8 weight sets, with the reference's own
    batched path (dequantise + cuBLAS, child process) beside it.  Returns the dict for the bench line's "batched" key."""
    import torch
    import lutgemm_b200 as L
    n = k = 8192
    q, g, rot = 2, 64, 8
    out = {"workload": f"bcq_gemm n={n} k={k} q={q} g={g}", "kernels": {"m2": "gemv_tma2_kernel", "m16": "gemm_tc_kernel", "m128": "gemm_tc_kernel"}}
    ws = []
    for i in range(rot):
        bW, alpha, _ = synth.bcq_layer(n, k, q, g, seed=synth.seed_for("bench", n, k, q, i))
        ws.append(L.nQWeight_fp16(bW, alpha, k, n, q, False, k // g).reserve_batch(128))
    for m in (2, 16, 128):
        xh = synth.activations(m, k, seed=77)
        x = torch.from_numpy(xh.view(np.int16)).cuda().view(torch.float16)
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        def step():
            for w in ws:
                L.matmul(y, x, w, m)
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 50
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * rot)
        flops = 2.0 * m * n * k * q
        row = {"us": us, "plane_wise_TFLOPs": flops / (us * 1e-6) / 1e12,
               "hbm_GBps": synth.algorithmic_bytes(n, k, q, g, m, False) / (us * 1e-6) / 1e9}
        try:
            child = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--n", str(n), "--k", str(k),
                                    "--q", str(q), "--g", str(g), "--m", str(m), "--rot", "4", "--steps", "5"],
                                   capture_output=True, text=True, timeout=180)
            rows = [l for l in child.stdout.splitlines() if l.startswith("{")]
            ref = json.loads(rows[-1])["reference_gpu"] if rows else None
            if ref:
                row["reference_gpu_us"] = ref["us_per_matvec"]
                row["reference_gpu_mae"] = ref["mae_vs_fp32_host"]
        except Exception:
            pass
        del graph
        out[f"m{m}"] = row
    for w in ws:
        w.close()
    return out


def run_ours(a):
    import torch
    import lutgemm_b200 as L
    from lutgemm_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    lib = capi.lib()
    if a.ntile:
        lib.lutgemm_set_gemv_ntile(a.ntile)
    lib.lutgemm_set_gemv_variant(a.variant)
    lib.lutgemm_set_dependent_launch(0 if a.no_pdl else 1)
    lib.lutgemm_set_batched_int8(1 if a.int8 else 0)
    lib.lutgemm_set_ordered_reduction(1 if a.ordered else 0)
    kernel_name = (("gemv_tma_kernel" if a.m == 1 else "gemv_tma2_kernel") if a.variant == 0 else "gemv_reg_kernel") if a.m < 4 else ("gemm_i8_kernel" if a.int8 and a.m <= 16 and a.q <= 4 else "gemm_tc_kernel")

    B = synth.algorithmic_bytes(a.n, a.k, a.q, a.g, a.m, a.bias)
    rot = max(1, a.rot)
    weights = []
    for i in range(rot):
        bW, alpha, qb = synth.bcq_layer(a.n, a.k, a.q, a.g, seed=synth.seed_for("bench", a.n, a.k, a.q, i + 1000 * rank),
                                        with_bias=a.bias)
        weights.append(L.nQWeight_fp16(bW, alpha, a.k, a.n, a.q, False, a.k // a.g, qb))
    x_host = synth.activations(a.m, a.k, seed=123)
    x = torch.from_numpy(x_host.view(np.int16)).cuda().view(torch.float16)
    ys = [torch.empty((a.m, a.n), dtype=torch.float16, device="cuda") for _ in range(rot)]

    def step():
        for w, y in zip(weights, ys):
            L.matmul(y, x, w, a.m)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, a.warmup)):
        step()
    barrier()
    # One step (ROT matvecs) is captured once into a CUDA graph and replayed, so that the timed
    # region measures the device, not the Python launch path.
    run_step = step
    graph = None
    if not a.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        run_step = graph.replay
        for _ in range(3):
            run_step()
        barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = lib.lutgemm_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        run_step()
    e1.record()
    barrier()
    launches = (lib.lutgemm_kernel_launch_count() - n0) if graph is None else a.steps * rot
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    sec = ms / 1e3
    value = world * a.steps * rot * B / sec / 1e9
    us_per_gemv = sec / (a.steps * rot) * 1e6
    # spread of single steps: 200 replays timed one by one (outside the timed region above)
    spread = None
    if rank == 0:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
        for s0, s1 in evs:
            s0.record()
            run_step()
            s1.record()
        torch.cuda.synchronize()
        per = sorted(s0.elapsed_time(s1) * 1e3 / rot for s0, s1 in evs)
        spread = {"median": per[len(per) // 2], "min": per[0], "max": per[-1], "steps_timed_singly": len(per)}

    # the same ROT matvecs as ONE launch (lutgemm_sequence_run: a persistent kernel walks the list); m = 1 only
    sequence = None
    if rank == 0 and a.m == 1 and a.variant == 0 and not a.ordered:
        try:
            ops = [dict(w=w, in_kind=0, x_ext=x, out_kind=0, y_ext=torch.empty((1, a.n), dtype=torch.float16, device="cuda"))
                   for w in weights]
            seq = L.MatvecSequence(ops)
            for _ in range(max(3, a.warmup)):
                seq.run()
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(a.steps):
                seq.run()
            s1.record()
            torch.cuda.synchronize()
            us_seq = s0.elapsed_time(s1) * 1e3 / (a.steps * rot)
            same = all(bool(torch.allclose(o["y_ext"].float(), y.float(), rtol=0, atol=2e-3 * float(y.float().abs().max())))
                       for o, y in zip(ops, ys))
            sequence = {"us_per_matvec": us_seq, "value": B / (us_seq * 1e-6) / 1e9, "unit": UNIT, "matvecs_per_launch": rot,
                        "kernel": "gemv_seq_kernel", "device_status": seq.status(), "matches_per_call_results": same}
            seq.close()
        except Exception as e:
            sequence = {"error": f"{type(e).__name__}: {e}"}

    # end to end through the host-buffer entry point
    e2e = None
    if not a.no_e2e:
        xin = torch.from_numpy(x_host.view(np.int16)).pin_memory()
        yout = torch.empty((a.m, a.n), dtype=torch.int16).pin_memory()
        def e2e_step():
            for w in weights:
                capi.check(lib.lutgemm_matmul_host(yout.data_ptr(), xin.data_ptr(), w.handle, a.m), "matmul_host")
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": world * a.steps * rot * B / dt / 1e9, "unit": UNIT, "h2d_bytes_per_step": rot * 2 * a.k * a.m,
               "d2h_bytes_per_step": rot * 2 * a.n * a.m, "us_per_matvec": dt / (a.steps * rot) * 1e6}
        # where a call's time goes: events between copy-in, kernels and copy-out on the call's own stream (one call,
        # run without the replayed graph), and the host wall clock of the ordinary call around them
        try:
            import ctypes as C
            us4 = (C.c_float * 4)()
            prof = []
            for _ in range(20):
                capi.check(lib.lutgemm_matmul_host_profile(yout.data_ptr(), xin.data_ptr(), weights[-1].handle, a.m, us4), "matmul_host_profile")
                prof.append(list(us4))
            med = [sorted(p[i] for p in prof)[len(prof) // 2] for i in range(4)]
            e2e["breakdown_us"] = {"host_wall_per_call": e2e["us_per_matvec"],
                                   "device_kernel_per_matvec": us_per_gemv,
                                   "launch_fetch_store_and_completion": e2e["us_per_matvec"] - us_per_gemv,
                                   "path": "page-locked buffers: one graph launch = fetch kernel (activations over the bus) + matvec "
                                           "(result stored into the host buffer) + completion word polled by the host; no copy "
                                           "engine, no stream synchronisation",
                                   "copy_engine_path_parts": {"h2d": med[0], "kernels": med[1], "d2h": med[2], "device_total": med[3],
                                                              "note": "the same call through cudaMemcpyAsync + events (what pageable "
                                                                      "buffers get), for comparison"}}
        except Exception as e:
            e2e["breakdown_us"] = {"error": f"{type(e).__name__}: {e}"}
        # the result that came back is the device result (up to one fp16 step: the split-k reductions are unordered)
        got = yout.numpy().view(np.float16).astype(np.float32)
        want = ys[-1].float().cpu().numpy()
        assert np.all(np.abs(got - want) <= np.spacing(np.abs(want).astype(np.float16)).astype(np.float32)
                      + 4e-6 * float(np.sqrt((want ** 2).mean())))

    if rank != 0:
        graph = None
        run_step = None
        torch.cuda.synchronize()
        shutdown_process_group(dist)
        return

    peak, peak_kind = measured_peak()
    achieved = B / (us_per_gemv * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": max(3, a.warmup),
        "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "matvecs_per_step": rot, "l2": f"{rot} distinct weight sets cycled "
                   f"({rot * B / 1e6:.0f} MB per step, larger than L2)", "algorithmic_bytes_per_matvec": B,
                   "parallelism": f"independent layers per rank x{world}",
                   "launch": "python" if graph is None else "cuda graph of one step, replayed"},
        "us_per_matvec": us_per_gemv,
        "us_per_matvec_single_steps": spread,
        "packed_weight_GBps": a.n * a.k * a.q / 8 / (us_per_gemv * 1e-6) / 1e9,
        "pct_of_8TBps_nominal": 100.0 * achieved / 8000.0,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (a.n, a.k, a.q, a.g, a.m, a.bias, a.variant) == (12288, 12288, 3, 128, 1, False, 0) else None,
                     "kernel": kernel_name},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if e2e:
        line["e2e"] = e2e
    if sequence:
        line["sequence"] = sequence
    if a.m > 1:
        line["tensor_flops_per_matmul"] = 2.0 * a.m * a.n * a.k * (a.q + (1 if a.bias else 0))
        line["tensor_TFLOPs"] = line["tensor_flops_per_matmul"] / (us_per_gemv * 1e-6) / 1e12
    if world == 1 and not a.no_reference_gpu and (a.m == 1 and not a.no_cpu_baseline or a.m > 1 and a.reference_gpu):
        # the reference's own CUDA code on the same call, in a child process (a fault there cannot take this run down):
        # m = 1 its LUT kernels, m > 1 (on request, --reference-gpu) its dequantise + cuBLAS path
        try:
            child = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--n", str(a.n), "--k", str(a.k),
                                    "--q", str(a.q), "--g", str(a.g), "--m", str(a.m), "--rot", str(rot), "--steps", "10"] + (["--bias"] if a.bias else []),
                                   capture_output=True, text=True, timeout=180)
            rows = [l for l in child.stdout.splitlines() if l.startswith("{")]
            line["reference_gpu"] = json.loads(rows[-1])["reference_gpu"] if rows else None
        except Exception:
            line["reference_gpu"] = None
    if world == 1 and not a.no_cpu_baseline and a.m == 1:
        threads = 1
        dt, kind, y_cpu = cpu_reference_gemv(a, threads)
        # same seeds as weight set 0 of rank 0: the CPU result doubles as a live parity check
        y_gpu = ys[0].float().cpu().numpy()
        rms = float(np.sqrt((y_cpu ** 2).mean()))
        line["cpu_baseline"] = {"value": B / dt / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
                                "sample": "one full matvec, single thread as the reference is written "
                                          "(dequantize_cpu + serial-k fp32 matmul)", "seconds": dt,
                                "max_abs_diff_vs_gpu_over_rms": float(np.abs(y_cpu - y_gpu).max() / rms)}
    if world == 1 and a.m == 1 and not a.no_stack_tp1 and (a.n, a.k, a.q, a.g, a.bias) == (12288, 12288, 3, 128, False):
        try:
            line["batched"] = batched_numbers(local)
        except Exception as e:
            line["batched"] = {"error": f"{type(e).__name__}: {e}"}
        # the multi-GPU workload (the 96-layer decoder linear stack) on this one GPU: the anchor of the scaling curve
        graph = None
        run_step = None
        for w in weights:
            w.close()
        weights = []
        torch.cuda.synchronize()
        try:
            from lutgemm_b200 import tp_stack
            st = make_stack(a, "seq", 0, 1, local)
            xs_ = torch.from_numpy(synth.activations(1, a.hidden, seed=5).reshape(-1).view(np.int16).copy()).cuda().view(torch.float16)
            st.x_in.copy_(xs_)
            for _ in range(3):
                st.step()
            torch.cuda.synchronize()
            n_st = max(5, min(a.steps, 30))
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(n_st):
                st.step()
            s1.record()
            torch.cuda.synchronize()
            ms_st = s0.elapsed_time(s1) / n_st
            Bst = tp_stack.stack_algorithmic_bytes(a.hidden, a.ffn, a.q, a.g, a.layers)
            line["stack_tp1"] = {"workload": f"decoder linear stack, {a.layers} layers, hidden {a.hidden}, ffn {a.ffn}, q={a.q} g={a.g} m=1, one GPU",
                                 "ms_per_step": ms_st, "value": Bst / ms_st / 1e6, "unit": UNIT, "steps": n_st,
                                 "algorithmic_bytes_per_step": Bst, "launches_per_step": 1, "device_status": st.device_status(),
                                 "frac_of_peak": Bst / ms_st / 1e6 / peak}
            st.close()
        except Exception as e:
            line["stack_tp1"] = {"error": f"{type(e).__name__}: {e}"}
    print(json.dumps(line), flush=True)
    graph = None
    run_step = None
    torch.cuda.synchronize()
    shutdown_process_group(dist)


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        world_size = int(os.environ.get("WORLD_SIZE", "1"))
        workload = args.workload if args.workload != "auto" else ("gemv" if world_size == 1 else "stack")
        if workload == "stack":
            run_stack(args)
        elif workload == "quantize":
            run_quantize(args)
        elif workload == "gptq":
            run_gptq(args)
        else:
            run_ours(args)
