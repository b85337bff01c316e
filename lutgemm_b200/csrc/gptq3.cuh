// 3-bit uniform (GPTQ-format) matvec, the comparison rows of the reference's public header.
//
// Replaces VecQuant3MatMulKernel / VecQuant3MatMulKernelFaster (lutGEMM/src/cuda/kernels/gptq_fp16_bias.hpp:27-105,
// lutGEMM/src/cuda/kernels/gptq_faster_fp16_bias.hpp:22-103) behind lutGEMM::matmul_gptq / matmul_gptq_faster
// (lutGEMM/src/kernels.cu:40-54):   y[n] = sum_k (scale[n] * code[k][n] - zero[n]) * x[k],
// codes 0..7 packed 32 to three uint32 along k (code j of a group = bits 3j..3j+2 of the 96-bit little-endian
// string), mat [K*3/32][N].
//
// Here: y[n] = scale[n] * S[n] - zero[n] * X with S = sum_k code x (fp32) and X = sum_k x, one fp16 rounding.
// CTA = 32 columns x 8 k-parts; the CTA walks k in slabs of 2048, part p takes 256 k of each slab.  A thread owns
// one column of one part: 24 coalesced word loads per slab, issued a slab ahead.  Decoding costs one LOP3 per
// code: the three code bits are OR-ed, where they sit, into the mantissa of 2^23, so that subtracting 2^23 leaves
// code * 2^s exactly, and the activations in shared memory are pre-multiplied by 2^-s for the position they meet
// (both exact); words are used as they are for fields below bit 16 and shifted down by 16 once for the others,
// and the two codes that straddle words come from funnel shifts.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lg {

constexpr int kG3Cols = 32;                   // columns per CTA
constexpr int kG3Parts = 8;                   // k-parts per CTA (one warp each)
constexpr int kG3PartK = 256;                 // k per part and slab: 8 groups of 32 codes = 24 words
constexpr int kG3SlabK = kG3Parts * kG3PartK; // 2048
constexpr int kG3Threads = kG3Cols * kG3Parts;

// bit offset, inside the (possibly shifted) word it is taken from, of code j of a 32-code group; -1: straddles
__host__ __device__ constexpr int g3_offset(int j) {
    const int bit = 3 * j;                    // position in the 96-bit string
    const int o = bit % 32;
    return (o > 29) ? 0 /* straddling codes are moved to bit 0 */ : (o >= 16 ? o - 16 : o);
}

struct G3Params {
    const uint32_t* mat;     // [K*3/32][N]
    const __half* scale;     // [N]
    const __half* zero;      // [N]
    const __half* x;         // [K]
    __half* y;               // [N]
    int N, K;
};

__device__ __forceinline__ float g3_code(uint32_t word, int off) {
    // (word & (7 << off)) | bits of 2^23, as a float, minus 2^23 = code * 2^off
    return __uint_as_float((word & (7u << off)) | 0x4B000000u) - 8388608.f;
}

__global__ void __launch_bounds__(kG3Threads)
gptq3_gemv_kernel(const G3Params p) {
    __shared__ float xs[kG3SlabK];            // activations of the slab, pre-scaled by 2^-offset of their position
    __shared__ float red[kG3Parts][kG3Cols];
    __shared__ float xsum_s[kG3Parts];
    const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
    const int n = blockIdx.x * kG3Cols + lane;
    const bool n_ok = n < p.N;
    const int nslabs = (p.K + kG3SlabK - 1) / kG3SlabK;
    const size_t rowN = (size_t)p.N;

    auto load_words = [&](int slab, uint32_t (&w)[24]) {
        const int k0 = slab * kG3SlabK + part * kG3PartK;
#pragma unroll
        for (int i = 0; i < 24; i++) {
            const int kk = k0 + (i / 3) * 32;                       // first k of the group this word belongs to
            w[i] = (n_ok && kk < p.K) ? __ldg(p.mat + (size_t)((k0 / 32) * 3 + i) * rowN + n) : 0u;
        }
    };

    uint32_t wq[24];
    load_words(0, wq);
    float acc4[4] = {0.f, 0.f, 0.f, 0.f}, xsum = 0.f;       // four independent chains of fused multiply-adds
    for (int slab = 0; slab < nslabs; slab++) {
        __syncthreads();                                            // previous slab's xs no longer read
        for (int i = tid; i < kG3SlabK; i += kG3Threads) {
            const int k = slab * kG3SlabK + i;
            const float xv = k < p.K ? __half2float(p.x[k]) : 0.f;
            xsum += xv;
            xs[i] = xv * __int_as_float((127 - g3_offset(i & 31)) << 23);      // 2^-offset, exact
        }
        __syncthreads();
        uint32_t w[24];
#pragma unroll
        for (int i = 0; i < 24; i++) w[i] = wq[i];
        if (slab + 1 < nslabs) load_words(slab + 1, wq);
        const float* xp = xs + part * kG3PartK;
#pragma unroll
        for (int gidx = 0; gidx < 8; gidx++) {
            const uint32_t w0 = w[3 * gidx], w1 = w[3 * gidx + 1], w2 = w[3 * gidx + 2];
            const uint32_t word[3] = {w0, w1, w2};
            const uint32_t hi[3] = {w0 >> 16, w1 >> 16, w2 >> 16};
            const uint32_t c10 = __funnelshift_r(w0, w1, 30), c21 = __funnelshift_r(w1, w2, 31);
            float xv[32];
#pragma unroll
            for (int v = 0; v < 8; v++) {
                const float4 t = *reinterpret_cast<const float4*>(xp + gidx * 32 + 4 * v);      // same address for the whole warp
                xv[4 * v] = t.x; xv[4 * v + 1] = t.y; xv[4 * v + 2] = t.z; xv[4 * v + 3] = t.w;
            }
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int bit = 3 * j, wi = bit / 32, o = bit % 32;
                float c;
                if (o > 29) c = g3_code(j == 10 ? c10 : c21, 0);
                else if (o >= 16) c = g3_code(hi[wi], o - 16);
                else c = g3_code(word[wi], o);
                acc4[j & 3] = fmaf(c, xv[j], acc4[j & 3]);
            }
        }
    }
    // add the 8 parts; X = sum of the activations (every thread added its share of every slab)
    xsum = xsum + __shfl_xor_sync(0xffffffffu, xsum, 16);
    xsum = xsum + __shfl_xor_sync(0xffffffffu, xsum, 8);
    xsum = xsum + __shfl_xor_sync(0xffffffffu, xsum, 4);
    xsum = xsum + __shfl_xor_sync(0xffffffffu, xsum, 2);
    xsum = xsum + __shfl_xor_sync(0xffffffffu, xsum, 1);
    red[part][lane] = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
    if (lane == 0) xsum_s[part] = xsum;
    __syncthreads();
    if (part == 0 && n_ok) {
        float s = 0.f, X = 0.f;
#pragma unroll
        for (int i = 0; i < kG3Parts; i++) { s += red[i][lane]; X += xsum_s[i]; }
        p.y[n] = __float2half_rn(__half2float(p.scale[n]) * s - __half2float(p.zero[n]) * X);
    }
}

}  // namespace lg
