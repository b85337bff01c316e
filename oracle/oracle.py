"""ctypes binding of the CPU oracle (oracle/lutgemm_oracle.c) and of the
reference's own host code compiled into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  Importable from tests/, the smoke check and the
benchmark's CPU-baseline legs; the shipped package never imports it.

Array conventions (numpy, C-contiguous):
  bW      uint32  [K/32, q, N]
  alpha   float16 [G, q, N]      (or float32 where a function says so)
  q_bias  float16 [G, N] or None
  x       float16 [M, K]
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF_CPU = None

_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def _makefile_default_ref():
    """The default of the Makefile's REF variable (one place holds the path)."""
    for line in open(os.path.join(_HERE, "Makefile")):
        if line.startswith("REF") and "?=" in line:
            return line.split("?=", 1)[1].strip()
    return ""


def build(force=False):
    """Compile the C restatement (and oracle/_ref when the reference tree exists)."""
    so = os.path.join(_HERE, "liblutgemm_oracle.so")
    src = os.path.join(_HERE, "lutgemm_oracle.c")
    stale = (not os.path.exists(so)) or os.path.getmtime(so) < os.path.getmtime(src)
    ref = os.environ.get("REF", "")                   # the Makefile's variable: where the reference tree lies (its default otherwise)
    ref_dir = ref or _makefile_default_ref()
    ref_missing = os.path.isdir(os.path.join(ref_dir, "lutGEMM", "src")) and not os.path.exists(
        os.path.join(_HERE, "_ref", "libref_cpu.so"))
    if force or stale or ref_missing:
        subprocess.check_call(["make", "-s", "-C", _HERE] + (["-B"] if force else []) + (["REF=" + ref] if ref else []))
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        vp = C.c_void_p
        L.lgo_float_to_half.argtypes = [_f32p, _u16p, C.c_size_t]
        L.lgo_half_to_float.argtypes = [_u16p, _f32p, C.c_size_t]
        L.lgo_pack_planes.argtypes = [_i8p, C.c_int, C.c_int, C.c_int, _u32p]
        L.lgo_unpack_planes.argtypes = [_u32p, C.c_int, C.c_int, C.c_int, _i8p]
        L.lgo_dequantize_cpu.argtypes = [_u32p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u16p]
        L.lgo_dequantize_from_qw.argtypes = [_u32p, _f32p, vp, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        L.lgo_matmul_cpu.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.lgo_bcq_matmul_ref.argtypes = [_u16p, _u32p, _u16p, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        L.lgo_bcq_matmul_fp32.argtypes = [_u16p, _u32p, _u16p, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        L.lgo_bcq_matmul_f64.argtypes = [_u16p, _u32p, _u16p, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f64p]
        L.lgo_uniform_to_bcq.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _i8p, _f32p]
        L.lgo_python_to_kernel_layout.argtypes = [_f32p, _i8p, vp, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _u32p, vp]
        L.lgo_packer_pack.argtypes = [_i8p, C.c_size_t, _u8p]
        L.lgo_packer_unpack.argtypes = [_u8p, C.c_size_t, _i8p]
        L.lgo_num_threads.restype = C.c_int
        L.lgo_set_num_threads.argtypes = [C.c_int]
        for f in ("lgo_float_to_half", "lgo_half_to_float", "lgo_pack_planes", "lgo_unpack_planes",
                  "lgo_dequantize_cpu", "lgo_dequantize_from_qw", "lgo_matmul_cpu", "lgo_bcq_matmul_ref",
                  "lgo_bcq_matmul_f64", "lgo_bcq_matmul_fp32", "lgo_uniform_to_bcq", "lgo_python_to_kernel_layout",
                  "lgo_packer_pack", "lgo_packer_unpack", "lgo_set_num_threads"):
            getattr(L, f).restype = None
        _LIB = L
    return _LIB


def ref_cpu():
    """The reference's own dequantize_cpu, or None when oracle/_ref was not built."""
    global _REF_CPU
    if _REF_CPU is None:
        p = os.path.join(_HERE, "_ref", "libref_cpu.so")
        if not os.path.exists(p):
            return None
        R = C.CDLL(p)
        R.ref_dequantize_cpu.argtypes = [_u32p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u16p]
        R.ref_dequantize_cpu.restype = None
        _REF_CPU = R
    return _REF_CPU


def _opt(a, dtype):
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=dtype)
    return a.ctypes.data_as(C.c_void_p), a


def _h(a):
    """float16 array -> uint16 view (C-contiguous)."""
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def set_threads(n):
    lib().lgo_set_num_threads(int(n))


def num_threads():
    return int(lib().lgo_num_threads())


def pack_planes(planes):
    """planes int8 [K, q, N] of +-1 -> bW uint32 [K/32, q, N]."""
    planes = np.ascontiguousarray(planes, dtype=np.int8)
    K, q, N = planes.shape
    bW = np.empty((K // 32, q, N), np.uint32)
    lib().lgo_pack_planes(planes, K, q, N, bW)
    return bW


def unpack_planes(bW):
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    out = np.empty((KW * 32, q, N), np.int8)
    lib().lgo_unpack_planes(bW, KW * 32, q, N, out)
    return out


def dequantize_cpu(bW, alpha_h, group_size, row_wise=False, use_reference=False):
    """Dense fp16 weight, no offset: [K, N] (column-wise) or [N, K] (row-wise)."""
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    K = KW * 32
    out = np.empty((N, K) if row_wise else (K, N), np.float16)
    fn = ref_cpu().ref_dequantize_cpu if use_reference else lib().lgo_dequantize_cpu
    fn(bW, _h(alpha_h), K, N, q, int(group_size), int(bool(row_wise)), out.view(np.uint16))
    return out


def dequantize_from_qw(bW, alpha_f32, q_bias_f32, group_size):
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    K = KW * 32
    W = np.empty((K, N), np.float32)
    qb = _opt(q_bias_f32, np.float32)
    lib().lgo_dequantize_from_qw(bW, np.ascontiguousarray(alpha_f32, dtype=np.float32),
                                 qb[0] if qb else None, K, N, q, int(group_size), W)
    return W


def matmul_cpu(x_f32, W_f32):
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    W = np.ascontiguousarray(W_f32, dtype=np.float32)
    M, K = x.shape
    N = W.shape[1]
    out = np.empty((M, N), np.float32)
    lib().lgo_matmul_cpu(x, W, out, M, N, K)
    return out


def bcq_matmul_fp32(x_h, bW, alpha_h, q_bias_h, group_size):
    """The reference's fp32 host result (test-side dequantizeFrom_qW + matmul_cpu), fp32 [M, N]."""
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    K = KW * 32
    x = _h(x_h).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    qb = None if q_bias_h is None else _h(q_bias_h)
    lib().lgo_bcq_matmul_fp32(x, bW, _h(alpha_h), qb.ctypes.data_as(C.c_void_p) if qb is not None else None,
                              M, N, K, q, int(group_size), y)
    return y


def bcq_matmul_ref(x_h, bW, alpha_h, q_bias_h, group_size):
    """The host result through the library's dequantize_cpu (W rounded to fp16) plus the offset term, fp32 [M, N]."""
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    K = KW * 32
    x = _h(x_h).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    qb = None if q_bias_h is None else _h(q_bias_h)
    lib().lgo_bcq_matmul_ref(x, bW, _h(alpha_h), qb.ctypes.data_as(C.c_void_p) if qb is not None else None,
                             M, N, K, q, int(group_size), y)
    return y


def bcq_matmul_f64(x_h, bW, alpha_h, q_bias_h, group_size):
    bW = np.ascontiguousarray(bW, dtype=np.uint32)
    KW, q, N = bW.shape
    K = KW * 32
    x = _h(x_h).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float64)
    qb = None if q_bias_h is None else _h(q_bias_h)
    lib().lgo_bcq_matmul_f64(x, bW, _h(alpha_h), qb.ctypes.data_as(C.c_void_p) if qb is not None else None,
                             M, N, K, q, int(group_size), y)
    return y


def uniform_to_bcq(scale, zero, code, q):
    """scale, zero float32 [N, G]; code int32 [N, G, g] -> alpha [N,G,q], binary int8 [N,G,g,q], offset [N,G]."""
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    zero = np.ascontiguousarray(zero, dtype=np.float32)
    code = np.ascontiguousarray(code, dtype=np.int32)
    N, G, g = code.shape
    alpha = np.empty((N, G, q), np.float32)
    binary = np.empty((N, G, g, q), np.int8)
    offset = np.empty((N, G), np.float32)
    lib().lgo_uniform_to_bcq(scale.reshape(N, G), zero.reshape(N, G), code, N, G, g, q, alpha, binary, offset)
    return alpha, binary, offset


def python_to_kernel_layout(alpha_py, binary_py, offset_py):
    """alpha [N,G,q], binary int8 [N,G,g,q], offset [N,G] or None -> (alpha_k [G,q,N], bW [K/32,q,N], q_bias_k [G,N] or None)."""
    alpha_py = np.ascontiguousarray(alpha_py, dtype=np.float32)
    binary_py = np.ascontiguousarray(binary_py, dtype=np.int8)
    N, G, g, q = binary_py.shape
    K = G * g
    alpha_k = np.empty((G, q, N), np.float32)
    bW = np.empty((K // 32, q, N), np.uint32)
    off = _opt(offset_py, np.float32)
    qb = np.empty((G, N), np.float32) if off else None
    lib().lgo_python_to_kernel_layout(alpha_py, binary_py, off[0] if off else None, N, K, g, q, alpha_k, bW,
                                      qb.ctypes.data_as(C.c_void_p) if qb is not None else None)
    return alpha_k, bW, qb


def packer_pack(flat_pm1):
    flat = np.ascontiguousarray(flat_pm1, dtype=np.int8).reshape(-1)
    out = np.empty(flat.size // 8, np.uint8)
    lib().lgo_packer_pack(flat, flat.size, out)
    return out


def packer_unpack(packed, L):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(L, np.int8)
    lib().lgo_packer_unpack(packed, L, out)
    return out
