"""ctypes binding of liblutgemm_b200.so (the C ABI in include/lutgemm_b200.h).

The library is the product; nothing here computes.  If the shared library is missing it is
built in-tree with nvcc; if that fails, or if a compute call finds no CUDA device, the error is
raised: there is no CPU fallback.
"""
import ctypes as C
import os

from . import _build

OK = 0
ERR_NULL, ERR_SHAPE, ERR_BITS, ERR_BATCH, ERR_CUDA, ERR_NO_DEVICE, ERR_TOO_LARGE, ERR_ALIGN = range(1, 9)

# every symbol include/lutgemm_b200.h declares
SYMBOLS = (
    "lutgemm_weight_create", "lutgemm_weight_create_device", "lutgemm_weight_destroy", "lutgemm_weight_describe",
    "lutgemm_matmul", "lutgemm_matmul_f32", "lutgemm_matmul_host", "lutgemm_matmul_host_profile", "lutgemm_matmul_wx",
    "lutgemm_weight_reserve_batch", "lutgemm_workspace_create", "lutgemm_workspace_destroy", "lutgemm_workspace_status", "lutgemm_workspace_set_ordered", "lutgemm_weight_set_ordered",
    "lutgemm_matmul_ws", "lutgemm_matmul_f32_ws",
    "lutgemm_matvec_static_scratch", "lutgemm_static_scratch_status", "lutgemm_dequantize",
    "lutgemm_matvec_tp", "lutgemm_matvec_tiles", "lutgemm_tp_finalize",
    "lutgemm_sequence_create", "lutgemm_sequence_export", "lutgemm_sequence_connect", "lutgemm_sequence_commit",
    "lutgemm_sequence_run", "lutgemm_sequence_status", "lutgemm_sequence_clear_status", "lutgemm_sequence_set_wait_limit", "lutgemm_sequence_set_trace", "lutgemm_sequence_describe",
    "lutgemm_sequence_destroy",
    "lutgemm_ipc_alloc", "lutgemm_ipc_open", "lutgemm_ipc_close", "lutgemm_ipc_free",
    "lutgemm_pack_planes", "lutgemm_pack_planes_device", "lutgemm_uniform_to_bcq", "lutgemm_uniform_to_bcq_device",
    "lutgemm_from_python_layout", "lutgemm_packer_pack", "lutgemm_packer_unpack",
    "lutgemm_packer_pack_device", "lutgemm_packer_unpack_device", "lutgemm_from_python_layout_device",
    "lutgemm_bcq_quantize", "lutgemm_bcq_quantize_device", "lutgemm_matmul_gptq",
    "lutgemm_status_string", "lutgemm_last_cuda_error", "lutgemm_kernel_launch_count", "lutgemm_set_gemv_ntile",
    "lutgemm_set_gemv_variant", "lutgemm_set_dependent_launch", "lutgemm_set_batched_path", "lutgemm_set_batched_int8", "lutgemm_set_ordered_reduction", "lutgemm_set_row_pairs", "lutgemm_weight_device_status",
)


class WeightDesc(C.Structure):
    _fields_ = [("bWeight", C.c_void_p), ("alpha", C.c_void_p), ("q_bias", C.c_void_p),
                ("num_groups", C.c_int), ("group_size", C.c_int), ("mSize", C.c_int), ("kSize", C.c_int),
                ("nb", C.c_int), ("is_row_wise_quantize", C.c_int), ("device", C.c_int)]


class TpLink(C.Structure):
    _fields_ = [("x_mode", C.c_int), ("out_mode", C.c_int), ("world", C.c_int), ("out_off", C.c_int),
                ("x_slots", C.c_void_p), ("x_slot_stride", C.c_int), ("x_off", C.c_int),
                ("flag_in", C.c_void_p), ("flag_target", C.c_uint), ("done_counter", C.c_void_p),
                ("out16", C.c_void_p * 8), ("out32", C.c_void_p * 8), ("flag_out", C.c_void_p * 8)]


class SeqBuffer(C.Structure):
    _fields_ = [("kind", C.c_int), ("n", C.c_int)]


class SeqOp(C.Structure):
    _fields_ = [("w", C.c_void_p), ("in_kind", C.c_int), ("in_buf", C.c_int), ("in_off", C.c_int),
                ("out_kind", C.c_int), ("out_buf", C.c_int), ("out_off", C.c_int), ("n", C.c_int),
                ("x_ext", C.c_void_p), ("y_ext", C.c_void_p)]


class LutGemmError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = lib().lutgemm_status_string(status).decode()
        cuda = lib().lutgemm_last_cuda_error()
        super().__init__(f"{where}: status {status} ({msg})" + (f", cudaError {cuda}" if status in (ERR_CUDA, ERR_NO_DEVICE) else ""))


_LIB = None


def lib():
    """Loads (building first if needed) the shared library and declares the prototypes."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB
    if _build.needs_build():
        if os.path.exists(_build.NVCC):
            _build.build()
        elif not os.path.exists(path):
            raise RuntimeError("liblutgemm_b200.so is missing and nvcc is not available to build it; "
                               "lutgemm_b200 has no fallback implementation")
    L = C.CDLL(path)
    vp, ip = C.c_void_p, C.c_int
    L.lutgemm_weight_create.argtypes = [C.POINTER(vp), vp, vp, ip, ip, ip, ip, ip, vp]
    L.lutgemm_weight_create_device.argtypes = [C.POINTER(vp), vp, vp, vp, ip, ip, ip, ip, ip, ip]
    L.lutgemm_weight_destroy.argtypes = [vp]
    L.lutgemm_weight_describe.argtypes = [vp, C.POINTER(WeightDesc)]
    L.lutgemm_matmul.argtypes = [vp, vp, vp, ip, vp]
    L.lutgemm_matmul_f32.argtypes = [vp, vp, vp, ip, vp]
    L.lutgemm_matmul_host.argtypes = [vp, vp, vp, ip]
    L.lutgemm_matmul_host_profile.argtypes = [vp, vp, vp, ip, C.POINTER(C.c_float)]
    L.lutgemm_matmul_wx.argtypes = [vp, vp, vp, ip, vp]
    L.lutgemm_weight_reserve_batch.argtypes = [vp, ip]
    L.lutgemm_workspace_create.argtypes = [C.POINTER(vp), ip, ip, ip]
    L.lutgemm_workspace_destroy.argtypes = [vp]
    L.lutgemm_workspace_status.argtypes = [vp, C.POINTER(ip)]
    L.lutgemm_workspace_set_ordered.argtypes = [vp, ip]
    L.lutgemm_weight_set_ordered.argtypes = [vp, ip]
    L.lutgemm_matmul_ws.argtypes = [vp, vp, vp, ip, vp, vp]
    L.lutgemm_matmul_f32_ws.argtypes = [vp, vp, vp, ip, vp, vp]
    L.lutgemm_static_scratch_status.argtypes = [C.POINTER(ip)]
    L.lutgemm_packer_pack_device.argtypes = [vp, C.c_size_t, vp, vp]
    L.lutgemm_packer_unpack_device.argtypes = [vp, C.c_size_t, vp, vp]
    L.lutgemm_from_python_layout_device.argtypes = [vp, vp, vp, vp, ip, ip, ip, ip, vp, vp, vp, vp]
    L.lutgemm_matvec_static_scratch.argtypes = [vp, vp, vp, vp, vp, ip, ip, ip, ip, vp]
    L.lutgemm_dequantize.argtypes = [vp, vp, vp]
    L.lutgemm_matvec_tp.argtypes = [vp, vp, C.POINTER(TpLink), vp, vp, vp]
    L.lutgemm_matvec_tiles.argtypes = [vp, C.POINTER(ip)]
    L.lutgemm_tp_finalize.argtypes = [vp, vp, vp, ip, ip, ip, vp, C.c_uint, vp, vp]
    L.lutgemm_sequence_create.argtypes = [C.POINTER(vp), C.POINTER(SeqOp), ip, C.POINTER(SeqBuffer), ip, ip, ip]
    L.lutgemm_sequence_export.argtypes = [vp, vp]
    L.lutgemm_sequence_connect.argtypes = [vp, ip, vp]
    L.lutgemm_sequence_commit.argtypes = [vp]
    L.lutgemm_sequence_run.argtypes = [vp, vp]
    L.lutgemm_sequence_status.argtypes = [vp, C.POINTER(ip)]
    L.lutgemm_sequence_clear_status.argtypes = [vp]
    L.lutgemm_sequence_set_wait_limit.argtypes = [vp, ip]
    L.lutgemm_sequence_set_trace.argtypes = [vp, vp, C.c_size_t]
    L.lutgemm_sequence_describe.argtypes = [vp, C.POINTER(ip), C.POINTER(ip), C.POINTER(C.c_size_t)]
    L.lutgemm_sequence_destroy.argtypes = [vp]
    L.lutgemm_ipc_alloc.argtypes = [C.c_size_t, C.POINTER(vp), vp]
    L.lutgemm_ipc_open.argtypes = [vp, C.POINTER(vp)]
    L.lutgemm_ipc_close.argtypes = [vp]
    L.lutgemm_ipc_free.argtypes = [vp]
    L.lutgemm_pack_planes.argtypes = [vp, ip, ip, ip, vp]
    L.lutgemm_pack_planes_device.argtypes = [vp, ip, ip, ip, vp, vp]
    L.lutgemm_uniform_to_bcq.argtypes = [vp, vp, vp, ip, ip, ip, ip, vp, vp, vp]
    L.lutgemm_uniform_to_bcq_device.argtypes = [vp, vp, vp, ip, ip, ip, ip, vp, vp, vp, vp]
    L.lutgemm_from_python_layout.argtypes = [vp, vp, vp, ip, ip, ip, ip, vp, vp, vp]
    L.lutgemm_packer_pack.argtypes = [vp, C.c_size_t, vp]
    L.lutgemm_packer_unpack.argtypes = [vp, C.c_size_t, vp]
    L.lutgemm_matmul_gptq.argtypes = [ip, ip, ip, vp, vp, vp, vp, vp, vp]
    L.lutgemm_bcq_quantize.argtypes = [vp, ip, ip, ip, ip, ip, vp, vp]
    L.lutgemm_bcq_quantize_device.argtypes = [vp, ip, ip, ip, ip, ip, vp, vp, vp, vp, vp]
    L.lutgemm_status_string.argtypes = [ip]
    L.lutgemm_status_string.restype = C.c_char_p
    L.lutgemm_last_cuda_error.restype = ip
    L.lutgemm_kernel_launch_count.restype = C.c_ulonglong
    L.lutgemm_set_gemv_ntile.argtypes = [ip]
    L.lutgemm_set_gemv_variant.argtypes = [ip]
    L.lutgemm_set_dependent_launch.argtypes = [ip]
    L.lutgemm_set_batched_path.argtypes = [ip]
    L.lutgemm_set_batched_int8.argtypes = [ip]
    L.lutgemm_set_ordered_reduction.argtypes = [ip]
    L.lutgemm_set_row_pairs.argtypes = [ip]
    L.lutgemm_weight_device_status.argtypes = [vp, C.POINTER(ip)]
    for name in SYMBOLS:
        fn = getattr(L, name)
        if name not in ("lutgemm_status_string", "lutgemm_kernel_launch_count"):
            fn.restype = ip
    _LIB = L
    return L


def check(status, where):
    if status != OK:
        raise LutGemmError(status, where)
