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

}  // namespace lg
