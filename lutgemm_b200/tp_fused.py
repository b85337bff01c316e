"""Tensor-parallel decoder linear stack with the exchange steps fused into the matvec kernels.

Same sharding and the same mathematics as tp_stack.TPLinearStack, but no collective library on the data
path: a column-parallel matvec stores its fp16 shard straight into every rank's gathered vector, a
row-parallel matvec stores its fp32 partial row into its slot on every rank, and the next matvec — which
has already started streaming its weights — waits for a flag before it builds its tables, adding the
partial rows in rank order (a one-shot all-reduce with a fixed summation order).  Four kernel launches per
decoder layer, nothing else.  The buffers are ordinary device allocations shared between the processes of
one node through CUDA IPC (plain peer loads/stores over NVLink; no multicast, no NVLS).

torch.distributed is used once, at set-up, to exchange the 64-byte IPC handles.
"""
import ctypes as C

import numpy as np

from . import capi
from .tp_stack import TPLinearStack


def _align(n, a=256):
    return (n + a - 1) // a * a


class FusedTPStack(TPLinearStack):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._setup_links()

    # ------------------------------------------------------------------ peer-visible buffers and flags
    def _setup_links(self):
        import torch
        lib = capi.lib()
        P, r, h, f, L = self.world, self.rank, self.hidden, self.ffn, self.layers
        # per-layer layout, identical on every rank
        o_qkv = 0
        o_out = _align(o_qkv + 3 * h * 2)
        o_fc1 = _align(o_out + P * h * 4)
        o_fc2 = _align(o_fc1 + f * 2)
        o_flag = _align(o_fc2 + P * h * 4)
        o_done = o_flag + 64
        layer_bytes = _align(o_done + 64)
        total = layer_bytes * L
        local = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        capi.check(lib.lutgemm_ipc_alloc(total, C.byref(local), handle), "ipc_alloc")
        self._local = local.value
        self._peer_ptrs = []
        base = [None] * P
        base[r] = local.value
        if P > 1:
            import torch.distributed as dist
            handles = [None] * P
            dist.all_gather_object(handles, bytes(handle))
            for q in range(P):
                if q == r:
                    continue
                hb = (C.c_ubyte * 64).from_buffer_copy(handles[q])
                ptr = C.c_void_p()
                capi.check(lib.lutgemm_ipc_open(hb, C.byref(ptr)), "ipc_open")
                base[q] = ptr.value
                self._peer_ptrs.append(ptr.value)
            dist.barrier()
        self._base = base
        tiles = []
        for w in self.weights[0]:
            t = C.c_int()
            capi.check(lib.lutgemm_matvec_tiles(w.handle, C.byref(t)), "matvec_tiles")
            tiles.append(t.value)
        self._tiles = tiles

        def link(**kw):
            s = capi.TpLink()
            s.world = P
            for k, v in kw.items():
                if k in ("out16", "out32", "flag_out"):
                    arr = getattr(s, k)
                    for i, p in enumerate(v):
                        arr[i] = p
                else:
                    setattr(s, k, v)
            return s

        self._links = []          # [layer] -> list of (in_ptr, TpLink, container)
        self._lay = dict(qkv=o_qkv, out=o_out, fc1=o_fc1, fc2=o_fc2, flag=o_flag, done=o_done, layer=layer_bytes)
        for l in range(L):
            lb = l * layer_bytes
            wq, wo, w1, w2 = self.weights[l]
            me = base[r] + lb
            row = []
            # QKV: input = caller's x (first layer) or the previous layer's all-reduced FC2 rows
            if l == 0:
                k1 = link(x_mode=0)
                in1 = None      # filled per step
            else:
                pb = base[r] + (l - 1) * layer_bytes
                k1 = link(x_mode=2, x_slots=pb + o_fc2, x_slot_stride=h, x_off=0, flag_in=pb + o_flag + 12,
                          flag_target=P * tiles[3], done_counter=pb + o_done + 12)
                in1 = None
            k1.out_mode = 1
            k1.out_off = r * (3 * h // P)
            for q in range(P):
                k1.out16[q] = base[q] + lb + o_qkv
                k1.flag_out[q] = base[q] + lb + o_flag + 0
            row.append((in1, k1, wq))
            # out-proj: input = this rank's k-slice of the gathered vector (first `hidden` entries stand in for attention)
            k2 = link(x_mode=1, flag_in=me + o_flag + 0, flag_target=P * tiles[0], done_counter=me + o_done + 0, out_mode=2)
            for q in range(P):
                k2.out32[q] = base[q] + lb + o_out + r * h * 4
                k2.flag_out[q] = base[q] + lb + o_flag + 4
            row.append((me + o_qkv + r * (h // P) * 2, k2, wo))
            # FC1: input = all-reduced out-proj rows
            k3 = link(x_mode=2, x_slots=me + o_out, x_slot_stride=h, x_off=0, flag_in=me + o_flag + 4,
                      flag_target=P * tiles[1], done_counter=me + o_done + 4, out_mode=1, out_off=r * (f // P))
            for q in range(P):
                k3.out16[q] = base[q] + lb + o_fc1
                k3.flag_out[q] = base[q] + lb + o_flag + 8
            row.append((None, k3, w1))
            # FC2: input = this rank's k-slice of the gathered FC1 vector
            k4 = link(x_mode=1, flag_in=me + o_flag + 8, flag_target=P * tiles[2], done_counter=me + o_done + 8, out_mode=2)
            for q in range(P):
                k4.out32[q] = base[q] + lb + o_fc2 + r * h * 4
                k4.flag_out[q] = base[q] + lb + o_flag + 12
            row.append((me + o_fc1 + r * (f // P) * 2, k4, w2))
            self._links.append(row)
        self._y16 = torch.empty(h, dtype=torch.float16, device=self.device)

    # ------------------------------------------------------------------ one decode step: 4 launches per layer + 1
    def step(self, x):
        import torch
        lib = capi.lib()
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for l, row in enumerate(self._links):
            for i, (in_ptr, lk, w) in enumerate(row):
                if i == 0 and l == 0:
                    in_ptr = x.data_ptr()
                capi.check(lib.lutgemm_matvec_tp(in_ptr, w.handle, C.byref(lk), None, None, stream), "matvec_tp")
        last = self._base[self.rank] + (self.layers - 1) * self._lay["layer"]
        capi.check(lib.lutgemm_tp_finalize(self._y16.data_ptr(), None, last + self._lay["fc2"], self.hidden, self.world,
                                           self.hidden, last + self._lay["flag"] + 12, self.world * self._tiles[3],
                                           self.weights[0][0].handle, stream), "tp_finalize")
        return self._y16

    def device_status(self):
        st = C.c_int(-1)
        worst = 0
        for row in self.weights:
            for w in row:
                capi.check(capi.lib().lutgemm_weight_device_status(w.handle, C.byref(st)), "device_status")
                worst |= st.value
        return worst

    def close(self):
        lib = capi.lib()
        for p in self._peer_ptrs:
            lib.lutgemm_ipc_close(p)
        self._peer_ptrs = []
        if self._local:
            lib.lutgemm_ipc_free(self._local)
            self._local = None
