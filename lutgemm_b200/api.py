"""Python mirror of the reference's C++ interface for the BCQ matmul path, over the C ABI.

Names and argument meaning follow the reference so that a test written against
lutGEMM::nQWeight_fp16 / lutGEMM::matmul reads the same here:

  nQWeight_fp16(bW, A, row, col, num_bits, is_row_wise_quantize, num_alpha_groups=1, q_bias=None)
      lutGEMM/include/nQWeight_fp16.h:41-47, lutGEMM/src/nQWeight_fp16.cu:60-91 (parsing)
  matmul(output, input, nqW, m)          lutGEMM/include/kernels.h:27, lutGEMM/src/kernels.cu:64-71
  matmul_wx(output, nqW, input, n)       lutGEMM/include/kernels.h:26, lutGEMM/src/kernels.cu:56-63
  dequantize_gpu(nqW, d_fW)              lutGEMM/include/nQWeight_fp16.h:24, lutGEMM/src/nQWeight_fp16.cu:29-35

torch is used only to hold device memory and streams.  All arithmetic happens in the CUDA
library; when it cannot run, calls raise LutGemmError.
"""
import ctypes as C

import numpy as np

from . import capi


def _ptr(a):
    """Device/host pointer of a torch tensor or numpy array (None -> NULL)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data_as(C.c_void_p)
    assert a.is_contiguous()
    return C.c_void_p(a.data_ptr())


def _stream_ptr(stream):
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


class nQWeight_fp16:
    """BCQ weight container on the current CUDA device.

    bW: uint32 [K/32, q, N] (numpy);  A: float32 [G, q, N];  q_bias: float32 [G, N] or None.
    Column-wise (is_row_wise_quantize False): K = row, N = col.  Fields keep the reference's names.
    """

    def __init__(self, bW=None, A=None, row=0, col=0, num_bits=0, is_row_wise_quantize=False,
                 num_alpha_groups=1, q_bias=None):
        self._h = C.c_void_p()
        self._keep = None
        if bW is not None:
            self.parsing(bW, A, row, col, num_bits, is_row_wise_quantize, num_alpha_groups, q_bias)

    def parsing(self, bW, A, row, col, num_bits, is_row_wise_quantize, num_alpha_groups=1, q_bias=None):
        self.close()
        bW = np.ascontiguousarray(bW, dtype=np.uint32)
        A = np.ascontiguousarray(A, dtype=np.float32)
        qb = None if q_bias is None else np.ascontiguousarray(q_bias, dtype=np.float32)
        N, K = (row, col) if is_row_wise_quantize else (col, row)
        if bW.size != (K // 32) * num_bits * N or A.size != num_alpha_groups * num_bits * N or \
                (qb is not None and qb.size != num_alpha_groups * N):
            raise ValueError("array sizes do not match (row, col, num_bits, num_alpha_groups)")
        capi.check(capi.lib().lutgemm_weight_create(C.byref(self._h), _ptr(bW), _ptr(A), row, col, num_bits,
                                                    int(bool(is_row_wise_quantize)), num_alpha_groups, _ptr(qb)),
                   "nQWeight_fp16.parsing")
        self._read_fields()
        return self

    @classmethod
    def from_device(cls, d_bW, d_alpha_fp16, d_q_bias_fp16, row, col, num_bits, is_row_wise_quantize=False,
                    num_alpha_groups=1, copy=False):
        """Wraps (copy=False) or copies tensors that already live on the device in their final types."""
        self = cls()
        capi.check(capi.lib().lutgemm_weight_create_device(
            C.byref(self._h), _ptr(d_bW), _ptr(d_alpha_fp16), _ptr(d_q_bias_fp16), row, col, num_bits,
            int(bool(is_row_wise_quantize)), num_alpha_groups, int(bool(copy))), "nQWeight_fp16.from_device")
        if not copy:
            self._keep = (d_bW, d_alpha_fp16, d_q_bias_fp16)
        self._read_fields()
        return self

    def _read_fields(self):
        d = capi.WeightDesc()
        capi.check(capi.lib().lutgemm_weight_describe(self._h, C.byref(d)), "describe")
        self.bWeight, self.alpha, self.q_bias = d.bWeight, d.alpha, d.q_bias
        self.num_groups, self.group_size = d.num_groups, d.group_size
        self.mSize, self.kSize, self.nb = d.mSize, d.kSize, d.nb
        self.is_row_wise_quantize = bool(d.is_row_wise_quantize)
        self.device = d.device

    @property
    def handle(self):
        if not self._h:
            raise ValueError("empty nQWeight_fp16: call parsing() first")
        return self._h

    def reserve_batch(self, m):
        """Sizes the container's scratch for batches of up to m rows so that no later matmul allocates."""
        capi.check(capi.lib().lutgemm_weight_reserve_batch(self.handle, int(m)), "reserve_batch")
        return self

    def set_ordered(self, mode):
        """Split-k mode of calls on this container's own workspace: 0, 1, or -1 = the process-wide setting."""
        capi.check(capi.lib().lutgemm_weight_set_ordered(self.handle, int(mode)), "weight_set_ordered")
        return self

    def getDequantiedWeight(self, onGPU=True):
        """Dense fp16 weight as a torch CUDA tensor: [K, N] column-wise, [N, K] row-wise
        (lutGEMM/src/nQWeight_fp16.cu:93-99).  Only the GPU path exists here."""
        if not onGPU:
            raise NotImplementedError("this library has no CPU path")
        import torch
        shape = (self.mSize, self.kSize) if self.is_row_wise_quantize else (self.kSize, self.mSize)
        fW = torch.empty(shape, dtype=torch.float16, device=f"cuda:{self.device}")
        dequantize_gpu(self, fW)
        return fW

    def close(self):
        if self._h:
            capi.lib().lutgemm_weight_destroy(self._h)
            self._h = C.c_void_p()
            self._keep = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Workspace:
    """Split-k scratch for one stream (lutgemm_workspace_*): pass one per stream to run a container from several
    streams at once.  Serves containers up to max_n x max_k and batches up to max_m; never grows."""

    def __init__(self, max_n, max_k, max_m=1):
        self._h = C.c_void_p()
        capi.check(capi.lib().lutgemm_workspace_create(C.byref(self._h), int(max_n), int(max_k), int(max_m)), "workspace_create")

    @property
    def handle(self):
        return self._h

    def status(self):
        st = C.c_int(-1)
        capi.check(capi.lib().lutgemm_workspace_status(self._h, C.byref(st)), "workspace_status")
        return st.value

    def set_ordered(self, mode):
        """0 = unordered reductions, 1 = bit-reproducible, -1 = follow the process-wide setting (the initial state)."""
        capi.check(capi.lib().lutgemm_workspace_set_ordered(self._h, int(mode)), "workspace_set_ordered")
        return self

    def close(self):
        if self._h:
            capi.lib().lutgemm_workspace_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def matmul(output, input, nqW, m, algo=0, stream=None, workspace=None):
    """output[m, N] (fp16 CUDA tensor) = input[m, K] (fp16 CUDA tensor) x W.  `algo` is accepted and
    ignored, as in the reference (lutGEMM/src/cuda/kernels/mv_fp16.hpp:121-128).  workspace: a Workspace of the
    calling stream's own (None = the container's)."""
    if workspace is None:
        capi.check(capi.lib().lutgemm_matmul(_ptr(output), _ptr(input), nqW.handle, int(m), _stream_ptr(stream)), "matmul")
    else:
        capi.check(capi.lib().lutgemm_matmul_ws(_ptr(output), _ptr(input), nqW.handle, int(m), workspace.handle,
                                                _stream_ptr(stream)), "matmul_ws")
    return output


def matmul_wx(output, nqW, input, n, algo=0, stream=None):
    """The (output, nqW, input, n) overload (lutGEMM/include/kernels.h:26): W . X with the activations as columns,
    input [K, n] and output [N, n] fp16 CUDA tensors."""
    capi.check(capi.lib().lutgemm_matmul_wx(_ptr(output), nqW.handle, _ptr(input), int(n), _stream_ptr(stream)), "matmul_wx")
    return output


def matmul_f32(output_f32, input, nqW, m, stream=None, workspace=None):
    if workspace is None:
        capi.check(capi.lib().lutgemm_matmul_f32(_ptr(output_f32), _ptr(input), nqW.handle, int(m), _stream_ptr(stream)),
                   "matmul_f32")
    else:
        capi.check(capi.lib().lutgemm_matmul_f32_ws(_ptr(output_f32), _ptr(input), nqW.handle, int(m), workspace.handle,
                                                    _stream_ptr(stream)), "matmul_f32_ws")
    return output_f32


def matmul_host(output_np, input_np, nqW, m):
    """Host-buffer form: numpy fp16 in, numpy fp16 out, copies included, synchronous."""
    capi.check(capi.lib().lutgemm_matmul_host(_ptr(output_np), _ptr(input_np), nqW.handle, int(m)), "matmul_host")
    return output_np


def dequantize_gpu(nqW, d_fW, algo=0, stream=None):
    capi.check(capi.lib().lutgemm_dequantize(nqW.handle, _ptr(d_fW), _stream_ptr(stream)), "dequantize_gpu")
    return d_fW


def pack_planes(planes):
    """+-1 planes int8 [K, q, N] (numpy) -> bW uint32 [K/32, q, N]."""
    planes = np.ascontiguousarray(planes, dtype=np.int8)
    K, q, N = planes.shape
    bW = np.empty((K // 32, q, N), np.uint32)
    capi.check(capi.lib().lutgemm_pack_planes(_ptr(planes), K, q, N, _ptr(bW)), "pack_planes")
    return bW


def pack_planes_device(d_planes, stream=None):
    import torch
    K, q, N = d_planes.shape
    bW = torch.empty((K // 32, q, N), dtype=torch.int32, device=d_planes.device)
    capi.check(capi.lib().lutgemm_pack_planes_device(_ptr(d_planes), K, q, N, _ptr(bW), _stream_ptr(stream)),
               "pack_planes_device")
    return bW


def uniform_to_bcq(scale, zero, code, q):
    """scale, zero float32 [N, G]; code int32 [N, G, g] -> (bW [K/32, q, N], alpha [G, q, N], q_bias [G, N])."""
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    zero = np.ascontiguousarray(zero, dtype=np.float32)
    code = np.ascontiguousarray(code, dtype=np.int32)
    N, G, g = code.shape
    bW = np.empty((G * g // 32, q, N), np.uint32)
    alpha = np.empty((G, q, N), np.float32)
    q_bias = np.empty((G, N), np.float32)
    capi.check(capi.lib().lutgemm_uniform_to_bcq(_ptr(scale), _ptr(zero), _ptr(code), N, G, g, q, _ptr(bW), _ptr(alpha),
                                                 _ptr(q_bias)), "uniform_to_bcq")
    return bW, alpha, q_bias


def uniform_to_bcq_device(d_scale, d_zero, d_code, q, stream=None):
    """Same on the device; returns torch tensors (bW int32 view of the uint32 words, alpha fp16, q_bias fp16)."""
    import torch
    N, G, g = d_code.shape
    dev = d_code.device
    bW = torch.empty((G * g // 32, q, N), dtype=torch.int32, device=dev)
    alpha = torch.empty((G, q, N), dtype=torch.float16, device=dev)
    q_bias = torch.empty((G, N), dtype=torch.float16, device=dev)
    capi.check(capi.lib().lutgemm_uniform_to_bcq_device(_ptr(d_scale), _ptr(d_zero), _ptr(d_code), N, G, g, q, _ptr(bW),
                                                        _ptr(alpha), _ptr(q_bias), _stream_ptr(stream)),
               "uniform_to_bcq_device")
    return bW, alpha, q_bias


def from_python_layout(alpha_py, binary_py, offset_py=None):
    """alpha [N,G,q], binary int8 [N,G,g,q], offset [N,G] or None -> (bW, alpha [G,q,N], q_bias [G,N] or None)."""
    alpha_py = np.ascontiguousarray(alpha_py, dtype=np.float32)
    binary_py = np.ascontiguousarray(binary_py, dtype=np.int8)
    off = None if offset_py is None else np.ascontiguousarray(offset_py, dtype=np.float32)
    N, G, g, q = binary_py.shape
    K = G * g
    bW = np.empty((K // 32, q, N), np.uint32)
    alpha = np.empty((G, q, N), np.float32)
    q_bias = None if off is None else np.empty((G, N), np.float32)
    capi.check(capi.lib().lutgemm_from_python_layout(_ptr(alpha_py), _ptr(binary_py), _ptr(off), N, K, g, q, _ptr(bW),
                                                     _ptr(alpha), _ptr(q_bias)), "from_python_layout")
    return bW, alpha, q_bias


def packer_pack(flat_pm1):
    flat = np.ascontiguousarray(flat_pm1, dtype=np.int8).reshape(-1)
    out = np.empty(flat.size // 8, np.uint8)
    capi.check(capi.lib().lutgemm_packer_pack(_ptr(flat), flat.size, _ptr(out)), "packer_pack")
    return out


def packer_unpack(packed, L):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(L, np.int8)
    capi.check(capi.lib().lutgemm_packer_unpack(_ptr(packed), L, _ptr(out)), "packer_unpack")
    return out


def packer_pack_device(d_flat_pm1, stream=None):
    """Packer.pack on the device: int8 +-1 CUDA tensor (any shape, flattened) -> uint8 CUDA tensor of size L / 8."""
    import torch
    flat = d_flat_pm1.contiguous().view(-1)
    out = torch.empty(flat.numel() // 8, dtype=torch.uint8, device=flat.device)
    capi.check(capi.lib().lutgemm_packer_pack_device(_ptr(flat), flat.numel(), _ptr(out), _stream_ptr(stream)), "packer_pack_device")
    return out


def packer_unpack_device(d_packed, L, stream=None):
    import torch
    out = torch.empty(L, dtype=torch.int8, device=d_packed.device)
    capi.check(capi.lib().lutgemm_packer_unpack_device(_ptr(d_packed), L, _ptr(out), _stream_ptr(stream)), "packer_unpack_device")
    return out


def from_python_layout_device(d_alpha_py, d_binary, d_offset_py, N, K, g, q, packed=False, stream=None):
    """The quantisers' tensors on the device (alpha float [N, G, q]; binary int8 [N, G, g, q], or with packed=True the
    Packer's uint8 stream of it; offset float [N, G] or None) -> (bW int32 [K/32, q, N], alpha fp16 [G, q, N],
    q_bias fp16 [G, N] or None) for nQWeight_fp16.from_device."""
    import torch
    dev = d_alpha_py.device
    bW = torch.empty((K // 32, q, N), dtype=torch.int32, device=dev)
    alpha = torch.empty((K // g, q, N), dtype=torch.float16, device=dev)
    q_bias = None if d_offset_py is None else torch.empty((K // g, N), dtype=torch.float16, device=dev)
    capi.check(capi.lib().lutgemm_from_python_layout_device(
        _ptr(d_alpha_py), None if packed else _ptr(d_binary), _ptr(d_binary) if packed else None, _ptr(d_offset_py),
        N, K, g, q, _ptr(bW), _ptr(alpha), _ptr(q_bias), _stream_ptr(stream)), "from_python_layout_device")
    return bW, alpha, q_bias


def bcq_quantize(w, qbits, rounds=15, group_size=-1):
    """The reference's quantize(w, qbits, rounds, group_size) (examples/bcq.py:23-98, unweighted defaults) on the GPU.

    w float32 [N, K] (numpy).  Returns (w_hat [N, K], binary int8 [N, G, g, qbits], alpha float32 [N, G, qbits]) in the
    quantiser's own layout; from_python_layout() turns (alpha, binary) into the container's.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    g = group_size if group_size > 0 else K
    alpha = np.empty((N, K // g, qbits), np.float32)
    binary = np.empty((N, K // g, g, qbits), np.int8)
    capi.check(capi.lib().lutgemm_bcq_quantize(_ptr(w), N, K, qbits, group_size, rounds, _ptr(alpha), _ptr(binary)),
               "bcq_quantize")
    w_hat = np.einsum("ngkq,ngq->ngk", binary.astype(np.float32), alpha).reshape(N, K)
    return w_hat, binary, alpha


def bcq_quantize_device(d_w, qbits, rounds=15, group_size=-1, stream=None):
    """Same, torch tensors on the device, straight into the container layout: returns (bW int32 [K/32, q, N],
    alpha fp16 [G, q, N]) for nQWeight_fp16.from_device; group_size must be a multiple of 32."""
    import torch
    N, K = d_w.shape
    g = group_size if group_size > 0 else K
    bW = torch.empty((K // 32, qbits, N), dtype=torch.int32, device=d_w.device)
    alpha = torch.empty((K // g, qbits, N), dtype=torch.float16, device=d_w.device)
    capi.check(capi.lib().lutgemm_bcq_quantize_device(_ptr(d_w), N, K, qbits, group_size, rounds, None, None, _ptr(bW),
                                                      _ptr(alpha), _stream_ptr(stream)), "bcq_quantize_device")
    return bW, alpha


def matmul_gptq(m, n, k, scale, bias, A, B, C, stream=None):
    """lutGEMM::matmul_gptq / matmul_gptq_faster (lutGEMM/include/kernels.h:28-33), same argument order: k is the
    number of packed rows K * 3 / 32, scale / bias (the zero term) fp16 [n], A fp16 [m, K], B int32 [k, n], C fp16 [m, n]."""
    capi.check(capi.lib().lutgemm_matmul_gptq(int(m), int(n), int(k), _ptr(scale), _ptr(bias), _ptr(A), _ptr(B), _ptr(C),
                                              _stream_ptr(stream)), "matmul_gptq")


matmul_gptq_faster = matmul_gptq


class MatvecSequence:
    """A fixed list of m = 1 matvecs executed by ONE persistent kernel launch (lutgemm_sequence_* in the C ABI).

    ops: dicts with keys  w (nQWeight_fp16 or None), in_kind / in_buf / in_off, out_kind / out_buf / out_off, n,
         x_ext / y_ext (fp16 CUDA tensors; kept alive by this object).  Missing keys are 0 / None.
    buffers: (kind, n) pairs: kind 1 = fp16 vector of n values, kind 2 = `world` fp32 rows of n values.
    With world > 1 the ranks' exchange-memory handles are swapped through torch.distributed (default group).
    """

    def __init__(self, ops, buffers=(), rank=0, world=1):
        lib = capi.lib()
        self._keep = []
        arr = (capi.SeqOp * len(ops))()
        for i, o in enumerate(ops):
            w = o.get("w")
            arr[i].w = w.handle if w is not None else None
            for k in ("in_kind", "in_buf", "in_off", "out_kind", "out_buf", "out_off", "n"):
                setattr(arr[i], k, int(o.get(k, 0)))
            for k in ("x_ext", "y_ext"):
                t = o.get(k)
                if t is not None:
                    self._keep.append(t)
                    setattr(arr[i], k, t.data_ptr())
            self._keep.append(w)
        barr = (capi.SeqBuffer * max(1, len(buffers)))()
        for i, (kind, n) in enumerate(buffers):
            barr[i].kind, barr[i].n = int(kind), int(n)
        self._h = C.c_void_p()
        self.rank, self.world, self.n_ops = rank, world, len(ops)
        capi.check(lib.lutgemm_sequence_create(C.byref(self._h), arr, len(ops), barr, len(buffers), rank, world),
                   "sequence_create")
        if world > 1:
            import torch.distributed as dist
            mine = (C.c_ubyte * 64)()
            capi.check(lib.lutgemm_sequence_export(self._h, mine), "sequence_export")
            handles = [None] * world
            dist.all_gather_object(handles, bytes(mine))
            for r in range(world):
                if r != rank:
                    hb = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                    capi.check(lib.lutgemm_sequence_connect(self._h, r, hb), "sequence_connect")
            capi.check(lib.lutgemm_sequence_commit(self._h), "sequence_commit")
            dist.barrier()

    def run(self, stream=None):
        capi.check(capi.lib().lutgemm_sequence_run(self._h, _stream_ptr(stream)), "sequence_run")

    def status(self):
        st = C.c_int(-1)
        capi.check(capi.lib().lutgemm_sequence_status(self._h, C.byref(st)), "sequence_status")
        return st.value

    def clear_status(self):
        capi.check(capi.lib().lutgemm_sequence_clear_status(self._h), "sequence_clear_status")

    def set_wait_limit(self, milliseconds):
        capi.check(capi.lib().lutgemm_sequence_set_wait_limit(self._h, int(milliseconds)), "sequence_set_wait_limit")

    def trace(self, enable=True):
        """Switches the per-(matvec, CTA) time stamps on (returns the int64 CUDA tensor [n_ops, ctas, 4] they land in,
        device-clock ns; see lutgemm_sequence_set_trace) or off."""
        if not enable:
            capi.check(capi.lib().lutgemm_sequence_set_trace(self._h, None, 0), "sequence_set_trace")
            self._trace = None
            return None
        import torch
        ctas = self.describe()["ctas"]
        self._trace = torch.zeros((self.n_ops, ctas, 4), dtype=torch.int64, device="cuda")
        capi.check(capi.lib().lutgemm_sequence_set_trace(self._h, self._trace.data_ptr(), self._trace.numel()), "sequence_set_trace")
        return self._trace

    def describe(self):
        a, b, c = C.c_int(), C.c_int(), C.c_size_t()
        capi.check(capi.lib().lutgemm_sequence_describe(self._h, C.byref(a), C.byref(b), C.byref(c)), "sequence_describe")
        return {"launches_per_run": a.value, "ctas": b.value, "exchange_bytes": c.value}

    def close(self):
        if self._h:
            capi.lib().lutgemm_sequence_destroy(self._h)
            self._h = C.c_void_p()
            self._keep = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
