// Small device kernels beside the matmul: dense dequantisation, the bit-plane packer and the
// uniform -> BCQ converter.  All are plain HBM-streaming kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lg {

// W = sum_b +-alpha (fp32 sum in plane order, one fp16 rounding), no q_bias: bit-identical to
// lutGEMM::dequantize_cpu (lutGEMM/src/nQWeight_fp16.cu:38-59).  One thread per (k-word, n):
// the q packed words are read once and expanded to 32 outputs.
// Column-wise output W[k][N]; row-wise output W[n][K].
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ bW, const __half* __restrict__ alpha, __half* __restrict__ W,
                  int N, int K, int q, int g, int row_wise) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kw = blockIdx.y;
    if (n >= N) return;
    const int grp = (kw * 32) / g;
    uint32_t word[8];
    float av[8];
#pragma unroll
    for (int b = 0; b < 8; b++) {
        if (b < q) {
            word[b] = bW[((size_t)kw * q + b) * N + n];
            av[b] = __half2float(alpha[((size_t)grp * q + b) * N + n]);
        } else {
            word[b] = 0u;
            av[b] = 0.f;
        }
    }
    if (!row_wise) {
        for (int t = 0; t < 32; t++) {
            float s = 0.f;
#pragma unroll
            for (int b = 0; b < 8; b++)
                if (b < q) s = ((word[b] >> t) & 1u) ? s + av[b] : s - av[b];
            W[(size_t)(kw * 32 + t) * N + n] = __float2half_rn(s);
        }
    } else {
        __half out[32];
#pragma unroll
        for (int t = 0; t < 32; t++) {
            float s = 0.f;
#pragma unroll
            for (int b = 0; b < 8; b++)
                if (b < q) s = ((word[b] >> t) & 1u) ? s + av[b] : s - av[b];
            out[t] = __float2half_rn(s);
        }
        uint4* dst = reinterpret_cast<uint4*>(W + (size_t)n * K + kw * 32);   // 64 B, 64-B aligned
        const uint4* src = reinterpret_cast<const uint4*>(out);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = src[i];
    }
}

// planes int8 [K][q][N] of +-1 -> bW [K/32][q][N]; bit t of word kw <=> planes[32 kw + t] > 0
// (packing rule of tests/opt/fp16/int3_col_wise_matmul_fp16.cu:200-215).
__global__ void __launch_bounds__(256)
pack_planes_kernel(const int8_t* __restrict__ planes, uint32_t* __restrict__ bW, int K, int q, int N) {
    const size_t col = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // over q*N
    const int kw = blockIdx.y;
    if (col >= (size_t)q * N) return;
    uint32_t s = 0;
#pragma unroll 8
    for (int t = 0; t < 32; t++)
        if (planes[(size_t)(kw * 32 + t) * q * N + col] > 0) s |= 1u << t;
    bW[(size_t)kw * q * N + col] = s;
}

// Uniform (scale, zero, code) -> kernel-layout BCQ with offset, following
// RTNParameter.convert_bcq_format (examples/rtn_parameter.py:77-96):
//   alpha_b = scale/2 * 2^b, plane b = bit b of the code, q_bias = sum_b alpha_b - scale*zero (fp32),
// then rounded to the container's fp16.  One thread per (k-word, n); the 32 codes of a word are
// contiguous in code[n][G][g].
__global__ void __launch_bounds__(256)
uniform_to_bcq_kernel(const float* __restrict__ scale, const float* __restrict__ zero,
                      const int32_t* __restrict__ code, int N, int G, int g, int q,
                      uint32_t* __restrict__ bW, __half* __restrict__ alpha, __half* __restrict__ q_bias) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kw = blockIdx.y;
    if (n >= N) return;
    const int k = kw * 32;
    const int grp = k / g;
    const int32_t* c = code + ((size_t)n * G + grp) * g + (k - grp * g);
    uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int t = 0; t < 32; t++) {
        const int v = c[t];
#pragma unroll
        for (int b = 0; b < 8; b++) words[b] |= (uint32_t)((v >> b) & 1) << t;
    }
    for (int b = 0; b < q; b++) bW[((size_t)kw * q + b) * N + n] = words[b];
    if (k == grp * g) {   // first word of the group writes the group's scales
        const float sc = scale[(size_t)n * G + grp];
        const float z = sc * zero[(size_t)n * G + grp];
        const float half_s = sc / 2.0f;
        float sum = 0.f;
        for (int b = 0; b < q; b++) {
            const float a = half_s * (float)(1u << b);
            alpha[((size_t)grp * q + b) * N + n] = __float2half_rn(a);
            sum += a;
        }
        q_bias[(size_t)grp * N + n] = __float2half_rn(sum - z);
    }
}

// The Python examples' uint8 interchange format (Packer.pack / Packer.unpack, examples/utils.py:162-181):
// L values of +-1, byte j of the L/8 packed bytes = sum_i 2^i [flat[i L/8 + j] > 0].  One thread per byte:
// eight strided reads (or writes), each coalesced across the warp.
__global__ void __launch_bounds__(256)
packer_pack_kernel(const int8_t* __restrict__ flat, size_t cols, uint8_t* __restrict__ packed) {
    const size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    unsigned v = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) v |= (flat[(size_t)i * cols + j] > 0 ? 1u : 0u) << i;
    packed[j] = (uint8_t)v;
}
__global__ void __launch_bounds__(256)
packer_unpack_kernel(const uint8_t* __restrict__ packed, size_t cols, int8_t* __restrict__ flat) {
    const size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    const unsigned v = packed[j];
#pragma unroll
    for (int i = 0; i < 8; i++) flat[(size_t)i * cols + j] = ((v >> i) & 1u) ? 1 : -1;
}

// The quantisers' tensors (alpha float [N][G][q], binary [N][G][g][q] of +-1, offset float [N][G] or null;
// examples/bcq_parameter.py:41-48, examples/rtn_parameter.py:77-96) -> the container layout on the device:
// bW [K/32][q][N], alpha fp16 [G][q][N], q_bias fp16 [G][N].  PACKED: the binary tensor arrives as Packer bytes
// (element e of the flattened tensor is bit e / (L/8) of byte e % (L/8)) and is never expanded in memory.
// One thread per (k-word, n): its 32 q signs are consecutive elements of the flattened tensor.
template <bool PACKED>
__global__ void __launch_bounds__(128)
python_layout_kernel(const float* __restrict__ alpha_py, const void* __restrict__ binary, const float* __restrict__ offset_py,
                     int N, int K, int g, int q, uint32_t* __restrict__ bW, __half* __restrict__ alpha,
                     __half* __restrict__ q_bias) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kw = blockIdx.y;
    if (n >= N) return;
    const int k = kw * 32, G = K / g, grp = k / g;
    const size_t e0 = ((size_t)n * K + k) * q;                 // first element of this thread in the flattened tensor
    const size_t cols = (size_t)N * K * q / 8;                 // PACKED: bytes in the stream
    uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int t = 0; t < 32; t++) {
#pragma unroll
        for (int b = 0; b < 8; b++) {
            if (b < q) {
                const size_t e = e0 + (size_t)t * q + b;
                bool plus;
                if (PACKED) {
                    const size_t i = e / cols, j = e - i * cols;
                    plus = (reinterpret_cast<const uint8_t*>(binary)[j] >> i) & 1u;
                } else {
                    plus = reinterpret_cast<const int8_t*>(binary)[e] > 0;
                }
                words[b] |= (plus ? 1u : 0u) << t;
            }
        }
    }
    for (int b = 0; b < q; b++) bW[((size_t)kw * q + b) * N + n] = words[b];
    if (k == grp * g) {   // first word of the group moves the group's scales
        const size_t ng = (size_t)n * G + grp;
        for (int b = 0; b < q; b++) alpha[((size_t)grp * q + b) * N + n] = __float2half_rn(alpha_py[ng * q + b]);
        if (offset_py) q_bias[(size_t)grp * N + n] = __float2half_rn(offset_py[ng]);
    }
}

}  // namespace lg
