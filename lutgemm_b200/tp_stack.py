"""Tensor-parallel stack of BCQ decoder linears (one process per GPU, torch.distributed).

The reference has no multi-GPU code at all; this module is the sharding its container layout
calls for when a decoder's linears are spread over P GPUs:

  column-parallel (QKV, FC1): rank r owns output columns [r N/P, (r+1) N/P).  Columns are the
      innermost axis of bW [K/32][q][N], alpha [G][q][N] and q_bias [G][N], so a shard is a strided
      slice that is repacked once into a contiguous container; x is replicated; the fp16 output
      shards are all-gathered.
  row-parallel (out-proj, FC2): rank r owns input features [r K/P, (r+1) K/P), i.e. whole outer
      slabs of bW / alpha / q_bias (K/P must be a multiple of the group size); each rank multiplies
      its slice of x, the fp32 partial results are all-reduced (sum) and rounded to fp16 once.

One decode step (m = 1) of an OPT-style layer here is  x -> QKV -> (first `hidden` outputs stand in
for the attention result) -> out-proj -> FC1 -> FC2 -> x', four matvecs and four collectives.  The
matvecs are the library's kernels (lutgemm_matmul / lutgemm_matmul_f32); the collectives are the
process group's (NCCL on GPUs).  `matvec` / `matvec_f32` can be replaced by host functions so that the
sharding and the exchange steps can be tested on CPU ranks with the gloo backend.
"""
import numpy as np


# ----------------------------------------------------------------------------- sharding (numpy, host)
def shard_columns(bW, alpha, q_bias, P, r):
    """Column-parallel shard r of P: contiguous copies of columns [r N/P, (r+1) N/P)."""
    N = bW.shape[2]
    if N % P != 0 or (N // P) % 8 != 0:
        raise ValueError(f"N = {N} cannot be split over {P} ranks in multiples of 8 columns")
    lo, hi = r * (N // P), (r + 1) * (N // P)
    return (np.ascontiguousarray(bW[:, :, lo:hi]), np.ascontiguousarray(alpha[:, :, lo:hi]),
            None if q_bias is None else np.ascontiguousarray(q_bias[:, lo:hi]))


def shard_rows(bW, alpha, q_bias, group_size, P, r):
    """Row-parallel shard r of P: input features [r K/P, (r+1) K/P) (whole groups, whole packed words)."""
    K = bW.shape[0] * 32
    if K % P != 0 or (K // P) % group_size != 0 or (K // P) % 32 != 0:
        raise ValueError(f"K = {K} cannot be split over {P} ranks in whole groups of {group_size}")
    k0, k1 = r * (K // P), (r + 1) * (K // P)
    g0, g1 = k0 // group_size, k1 // group_size
    return (np.ascontiguousarray(bW[k0 // 32:k1 // 32]), np.ascontiguousarray(alpha[g0:g1]),
            None if q_bias is None else np.ascontiguousarray(q_bias[g0:g1]))


def layer_shapes(hidden, ffn):
    """(name, N, K, mode) of the four linears of one decoder layer."""
    return [("qkv", 3 * hidden, hidden, "col"), ("out", hidden, hidden, "row"),
            ("fc1", ffn, hidden, "col"), ("fc2", hidden, ffn, "row")]


def stack_algorithmic_bytes(hidden, ffn, q, group_size, layers):
    from . import synth
    return layers * sum(synth.algorithmic_bytes(N, K, q, group_size) for _, N, K, _ in layer_shapes(hidden, ffn))


# ----------------------------------------------------------------------------- the stack
class TPLinearStack:
    """`layers` decoder layers sharded over the default process group (or a single rank)."""

    def __init__(self, hidden, ffn, q, group_size, layers, rank=0, world=1, device="cuda", seed=0,
                 matvec=None, matvec_f32=None, make_container=None, generate="device"):
        self.hidden, self.ffn, self.q, self.g, self.layers = hidden, ffn, q, group_size, layers
        self.rank, self.world, self.device = rank, world, device
        self.shapes = layer_shapes(hidden, ffn)
        self._matvec, self._matvec_f32, self._make = matvec, matvec_f32, make_container
        self.weights = []        # [layer][4] containers
        for layer in range(layers):
            row = []
            for idx, (name, N, K, mode) in enumerate(self.shapes):
                row.append(self._build_shard(layer, idx, N, K, mode, seed, generate))
            self.weights.append(row)
        self._alloc_buffers()

    # -- weights -------------------------------------------------------------------------------
    def _alpha_std(self, K):
        # keeps |y| ~ |x| through the stack: y = sum_k x_k sum_b +-alpha_b  =>  var(y) = K q E[alpha^2] var(x)
        return 1.0 / np.sqrt(K * self.q)

    def _build_shard(self, layer, idx, N, K, mode, seed, generate):
        P, r = self.world, self.rank
        if generate == "host":
            # full layer from one seed, then sharded: every rank sees the same logical weights
            from . import synth
            bW, alpha, _ = synth.bcq_layer(N, K, self.q, self.g, seed=synth.seed_for("stack", N, K, self.q, 131 * layer + idx + seed),
                                           alpha_std=self._alpha_std(K))
            if mode == "col":
                sb, sa, _ = shard_columns(bW, alpha, None, P, r)
                return self._container_from_host(sb, sa, N // P, K)
            sb, sa, _ = shard_rows(bW, alpha, None, self.g, P, r)
            return self._container_from_host(sb, sa, N, K // P)
        # device generation: each rank draws its own shard directly on its GPU (66 GB of host traffic avoided)
        import torch
        n_loc, k_loc = (N // P, K) if mode == "col" else (N, K // P)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(1_000_003 * (131 * layer + idx) + 7919 * r + seed)
        bW = torch.randint(-2**31, 2**31 - 1, (k_loc // 32, self.q, n_loc), dtype=torch.int32, device=self.device, generator=gen)
        alpha = (torch.randn((k_loc // self.g, self.q, n_loc), device=self.device, generator=gen).abs_() * self._alpha_std(K)).half()
        from .api import nQWeight_fp16
        return nQWeight_fp16.from_device(bW, alpha, None, k_loc, n_loc, self.q, False, k_loc // self.g, copy=False)

    def _container_from_host(self, bW, alpha, n_loc, k_loc):
        if self._make is not None:
            return self._make(bW, alpha, n_loc, k_loc)
        from .api import nQWeight_fp16
        return nQWeight_fp16(bW, alpha, k_loc, n_loc, self.q, False, k_loc // self.g)

    # -- buffers ---------------------------------------------------------------------------------
    def _alloc_buffers(self):
        import torch
        P, h, f, dev = self.world, self.hidden, self.ffn, self.device
        f16, f32 = torch.float16, torch.float32
        self.qkv_local = torch.empty(3 * h // P, dtype=f16, device=dev)
        self.qkv_full = torch.empty(3 * h, dtype=f16, device=dev)
        self.fc1_local = torch.empty(f // P, dtype=f16, device=dev)
        self.fc1_full = torch.empty(f, dtype=f16, device=dev)
        self.part_h = torch.empty(h, dtype=f32, device=dev)
        self.h16 = torch.empty(h, dtype=f16, device=dev)
        self.x16 = torch.empty(h, dtype=f16, device=dev)

    # -- one decode step ---------------------------------------------------------------------------
    def _mv(self, out, x, w):
        if self._matvec is not None:
            return self._matvec(out, x, w)
        from .api import matmul
        return matmul(out.view(1, -1), x.view(1, -1), w, 1)

    def _mv32(self, out, x, w):
        if self._matvec_f32 is not None:
            return self._matvec_f32(out, x, w)
        from .api import matmul_f32
        return matmul_f32(out.view(1, -1), x.view(1, -1), w, 1)

    def _all_gather(self, full, local):
        if self.world == 1:
            full.copy_(local)
            return
        import torch.distributed as dist
        dist.all_gather_into_tensor(full, local)

    def _all_reduce(self, t):
        if self.world == 1:
            return
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.SUM)

    def step(self, x):
        """x: fp16 [hidden] on self.device (replicated on every rank).  Returns the fp16 [hidden] output."""
        P, r, h, f = self.world, self.rank, self.hidden, self.ffn
        cur = x
        for wq, wo, w1, w2 in self.weights:
            self._mv(self.qkv_local, cur, wq)                                  # column-parallel
            self._all_gather(self.qkv_full, self.qkv_local)
            a_slice = self.qkv_full[r * (h // P):(r + 1) * (h // P)]           # this rank's k-range of the "attention" vector
            self._mv32(self.part_h, a_slice, wo)                               # row-parallel, fp32 partial
            self._all_reduce(self.part_h)
            self.h16.copy_(self.part_h)                                        # one fp16 rounding
            self._mv(self.fc1_local, self.h16, w1)                             # column-parallel
            self._all_gather(self.fc1_full, self.fc1_local)
            f_slice = self.fc1_full[r * (f // P):(r + 1) * (f // P)]
            self._mv32(self.part_h, f_slice, w2)                               # row-parallel
            self._all_reduce(self.part_h)
            self.x16.copy_(self.part_h)
            cur = self.x16
        return cur
