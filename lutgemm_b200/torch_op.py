"""torch operator and module over the C ABI: the caller's side of the BCQ matmul path.

The reference has no link between its Python quantisers (examples/rtn_parameter.py:77-96 convert_bcq_format,
examples/bcq_parameter.py:23-63 compress) and its C++ kernel; its model scripts dequantise back to dense
weights (examples/quant_model_rtn.py:67-101).  This module is that link:

  torch.ops.lutgemm_b200.bcq_linear(x, bW, alpha, q_bias) -> y     (registered with torch.library, has a fake
      implementation for shape propagation, CUDA only: there is no CPU kernel behind it)
  BCQLinear            nn.Module holding the container tensors in kernel layout:
                           bW int32 [K/32, q, N] (bit k % 32 set = +1), alpha fp16 [G, q, N], q_bias fp16 [G, N] or None
  BCQLinear.from_python_layout(alpha [N,G,q], binary [N,G,g,q], offset [N,G] or None)   the quantisers' tensors
  BCQLinear.from_uniform(scale [N,G], zero [N,G], code [N,G,g], q)                     RTN codes, converted on the way

torch holds the memory and the stream; the arithmetic is the library's kernels.
"""
from typing import Optional

import numpy as np
import torch

from . import api

import weakref

_containers = {}      # (device index, data pointers, shapes) -> nQWeight_fp16 wrapping the tensors without a copy


def _container(bW, alpha, q_bias, reserve_rows=0):
    key = (bW.device.index, bW.data_ptr(), alpha.data_ptr(), 0 if q_bias is None else q_bias.data_ptr(),
           tuple(bW.shape), tuple(alpha.shape))
    w = _containers.get(key)
    if w is None:
        kw, q, N = bW.shape
        G = alpha.shape[0]
        with torch.cuda.device(bW.device):
            w = api.nQWeight_fp16.from_device(bW, alpha, q_bias, kw * 32, N, q, False, G, copy=False)
        _containers[key] = w
        # the container (and the workspace it allocated) goes when the weight tensor it wraps goes: after module.to(),
        # a reload of the weights or deletion of the module nothing stays behind
        weakref.finalize(bW, _drop, key)
    if reserve_rows > 1:
        with torch.cuda.device(bW.device):
            w.reserve_batch(reserve_rows)
    return w


def _drop(key):
    w = _containers.pop(key, None)
    if w is not None:
        try:
            w._keep = None
            w.close()
        except Exception:
            pass


def release_containers():
    """Drops every cached container now (they are otherwise dropped when their weight tensor is collected)."""
    for key in list(_containers):
        _drop(key)


def _check(x, bW, alpha, q_bias):
    if bW.dim() != 3 or alpha.dim() != 3 or bW.shape[1] != alpha.shape[1] or bW.shape[2] != alpha.shape[2]:
        raise ValueError("bW must be [K/32, q, N] and alpha [G, q, N]")
    if x.shape[-1] != bW.shape[0] * 32:
        raise ValueError(f"x has {x.shape[-1]} input features, the container {bW.shape[0] * 32}")
    if bW.dtype != torch.int32 or alpha.dtype != torch.float16 or x.dtype != torch.float16:
        raise TypeError("bW int32, alpha and x float16")
    if q_bias is not None and (q_bias.dtype != torch.float16 or tuple(q_bias.shape) != (alpha.shape[0], alpha.shape[2])):
        raise ValueError("q_bias must be float16 [G, N]")


@torch.library.custom_op("lutgemm_b200::bcq_linear", mutates_args=(), device_types="cuda")
def bcq_linear(x: torch.Tensor, bW: torch.Tensor, alpha: torch.Tensor, q_bias: Optional[torch.Tensor]) -> torch.Tensor:
    _check(x, bW, alpha, q_bias)
    K, N = bW.shape[0] * 32, bW.shape[2]
    x2 = x.reshape(-1, K).contiguous()
    m = x2.shape[0]
    y = torch.empty((m, N), dtype=torch.float16, device=x.device)
    if m > 0:
        with torch.cuda.device(x.device):
            api.matmul(y, x2, _container(bW, alpha, q_bias), m, stream=torch.cuda.current_stream())
    return y.reshape(*x.shape[:-1], N)


@bcq_linear.register_fake
def _(x, bW, alpha, q_bias):
    return x.new_empty((*x.shape[:-1], bW.shape[2]), dtype=torch.float16)


class BCQLinear(torch.nn.Module):
    """y = x W^T with W [N, K] held as q bit planes and per-group scales (plus an optional per-group offset)."""

    def __init__(self, bW, alpha, q_bias=None, max_batch=0):
        super().__init__()
        self.register_buffer("bW", bW)
        self.register_buffer("alpha", alpha)
        self.register_buffer("q_bias", q_bias)
        self.in_features, self.out_features = bW.shape[0] * 32, bW.shape[2]
        self.num_bits, self.num_groups = bW.shape[1], alpha.shape[0]
        self.max_batch = max_batch

    def reserve(self, rows=None):
        """Sizes the container's scratch for batches of up to `rows` activation rows now, so that no forward call
        allocates (needed before a forward with more than 3 rows is captured into a CUDA graph)."""
        rows = self.max_batch if rows is None else rows
        if self.bW.is_cuda and rows > 1:
            _container(self.bW, self.alpha, self.q_bias, reserve_rows=rows)
        return self

    @classmethod
    def from_kernel_layout(cls, bW_u32, alpha_f32, q_bias_f32=None, device="cuda"):
        """numpy arrays in the container's layout: uint32 [K/32, q, N], float32 [G, q, N], float32 [G, N]."""
        bW = torch.from_numpy(np.ascontiguousarray(bW_u32, dtype=np.uint32).view(np.int32)).to(device)
        alpha = torch.from_numpy(np.ascontiguousarray(alpha_f32, dtype=np.float32)).to(device).half()
        qb = None if q_bias_f32 is None else torch.from_numpy(np.ascontiguousarray(q_bias_f32, dtype=np.float32)).to(device).half()
        return cls(bW, alpha, qb)

    @classmethod
    def from_python_layout(cls, alpha_py, binary_py, offset_py=None, device="cuda"):
        """The quantisers' tensors (in_ch_wise False): alpha [N, G, q], binary +-1 [N, G, g, q], offset [N, G] or [N, G, 1]."""
        to_np = lambda t: t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
        off = None if offset_py is None else to_np(offset_py).reshape(to_np(alpha_py).shape[:2])
        return cls.from_kernel_layout(*api.from_python_layout(to_np(alpha_py), to_np(binary_py), off), device=device)

    @classmethod
    def from_uniform(cls, scale, zero, code, q, device="cuda"):
        """RTN output: scale, zero [N, G], code int [N, G, g] with W = scale (code - zero) -> q planes, alpha, q_bias."""
        to_np = lambda t: t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
        s, z, c = to_np(scale), to_np(zero), to_np(code)
        return cls.from_kernel_layout(*api.uniform_to_bcq(s.reshape(c.shape[:2]), z.reshape(c.shape[:2]), c, q), device=device)

    def forward(self, x):
        return torch.ops.lutgemm_b200.bcq_linear(x, self.bW, self.alpha, self.q_bias)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.num_bits}, "
                f"groups={self.num_groups}, q_bias={self.q_bias is not None}")
