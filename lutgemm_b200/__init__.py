"""lutgemm_b200: B200 (sm_100a) LUT-GEMM for binary-coding-quantised weights.

The product is the CUDA shared library liblutgemm_b200.so behind the C ABI in
include/lutgemm_b200.h; `api` mirrors the reference's C++ interface on top of it.
"""
from . import synth  # noqa: F401
from .api import (nQWeight_fp16, matmul, matmul_wx, matmul_f32, matmul_host, dequantize_gpu,  # noqa: F401
                  pack_planes, pack_planes_device, uniform_to_bcq, uniform_to_bcq_device,
                  from_python_layout, packer_pack, packer_unpack, bcq_quantize, bcq_quantize_device, matmul_gptq, matmul_gptq_faster, MatvecSequence, Workspace,
                  packer_pack_device, packer_unpack_device, from_python_layout_device)
from .capi import LutGemmError  # noqa: F401
