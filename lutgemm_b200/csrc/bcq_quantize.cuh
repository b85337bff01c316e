// BCQ quantiser on the device: greedy initialisation + alternating refinement, one warp per (row, group).
//
// Replaces quantize() of the reference's examples/bcq.py:23-98 (torch tensors on CUDA, a dozen library kernels per
// round over the whole layer) for its default, unweighted case (exponent 0, clipping 1, pruning 0):
//   greedy       examples/bcq.py:100-128   b_i = sign(r), alpha_i = mean |r|, r -= alpha_i b_i
//   refinement   examples/bcq.py:130-157   alpha from the normal equations (B^T B) alpha = B^T w by q steps of conjugate
//                                          gradient started at the current alpha (examples/bcq.py:190-206, 1e-6 added to
//                                          both denominators), |alpha| sorted descending, then every weight takes the
//                                          nearest of the 2^q levels sum_i +-alpha_i (examples/bcq.py:165-188: levels
//                                          sorted, q bisection steps on midpoints, `w < mid` goes left).
// Here a group never leaves its warp: the weights stay in registers (lane l holds elements l, l + 32, ...), the
// q x q system is accumulated with warp reductions and solved redundantly by every lane, the 2^q levels are rank-sorted
// in shared memory.  Output in the quantiser's layout (alpha [N][G][q] fp32, binary int8 [N][G][g][q]) and/or directly
// in the matmul's container layout (bW uint32 [K/32][q][N] by warp ballots, alpha fp16 [G][q][N]).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lg {

constexpr int kBqMaxQ = 8;
constexpr int kBqWarps = 8;                   // warps (groups) per CTA

struct BqParams {
    const float* w;          // [N][K], groups of g consecutive k
    int N, K, g, q, rounds;
    float* alpha_py;         // [N][G][q] or nullptr
    signed char* binary_py;  // [N][G][g][q] or nullptr
    uint32_t* bW;            // [K/32][q][N] or nullptr (needs g % 32 == 0)
    __half* alpha_k;         // [G][q][N] or nullptr
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// code of one element: bits 0..7 = "+1" per plane, bits 8..15 = "non-zero" per plane
__device__ __forceinline__ float code_sign(uint32_t code, int i) {
    return ((code >> (8 + i)) & 1u) ? (((code >> i) & 1u) ? 1.f : -1.f) : 0.f;
}

template <int E>
__global__ void __launch_bounds__(kBqWarps * 32)
bcq_quantize_kernel(const BqParams p) {
    __shared__ float s_v[kBqWarps][1 << kBqMaxQ];
    __shared__ float s_vs[kBqWarps][1 << kBqMaxQ];
    __shared__ unsigned char s_ind[kBqWarps][1 << kBqMaxQ];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int G = p.K / p.g;
    const long long grp = (long long)blockIdx.x * kBqWarps + wib;
    if (grp >= (long long)p.N * G) return;                 // whole warps leave together
    const int n = (int)(grp / G), gi = (int)(grp % G);
    const int g = p.g, q = p.q;
    const float* wg = p.w + (size_t)n * p.K + (size_t)gi * g;

    float wv[E];
    uint32_t code[E];
#pragma unroll
    for (int e = 0; e < E; e++) {
        const int idx = e * 32 + lane;
        wv[e] = idx < g ? wg[idx] : 0.f;
        code[e] = 0u;
    }
    float alpha[kBqMaxQ];
#pragma unroll
    for (int i = 0; i < kBqMaxQ; i++) alpha[i] = 0.f;

    // ---- greedy ----
    {
        float r[E];
#pragma unroll
        for (int e = 0; e < E; e++) r[e] = wv[e];
        for (int i = 0; i < q; i++) {
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < E; e++) s += fabsf(r[e]);          // padding elements are 0
            float a = warp_sum_f(s) / (float)g;
            if (a != a) a = 0.f;
#pragma unroll
            for (int e = 0; e < E; e++) {
                const float b = r[e] > 0.f ? 1.f : (r[e] < 0.f ? -1.f : 0.f);
                if (b > 0.f) code[e] |= 1u << i;
                if (b != 0.f) code[e] |= 1u << (8 + i);
                r[e] -= b * a;
            }
#pragma unroll
            for (int j = 0; j < kBqMaxQ; j++) if (j == i) alpha[j] = a;
        }
    }

    // ---- alternating refinement ----
    if (q > 1) {
        const int nlev = 1 << q;
        for (int round = 0; round < p.rounds; round++) {
            // normal equations: integer Gram matrix and B^T w
            float A[kBqMaxQ][kBqMaxQ] = {}, btw[kBqMaxQ];
#pragma unroll
            for (int i = 0; i < kBqMaxQ; i++) {
                if (i >= q) { btw[i] = 0.f; continue; }
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < E; e++) s += code_sign(code[e], i) * wv[e];
                btw[i] = warp_sum_f(s);
#pragma unroll
                for (int j = 0; j < kBqMaxQ; j++) {
                    if (j < i || j >= q) continue;
                    int c = 0;
#pragma unroll
                    for (int e = 0; e < E; e++) c += (int)(code_sign(code[e], i) * code_sign(code[e], j));
                    c = __reduce_add_sync(0xffffffffu, c);
                    A[i][j] = (float)c;
                    A[j][i] = (float)c;
                }
            }
            // q steps of conjugate gradient from the current alpha (every lane the same arithmetic)
            float x[kBqMaxQ], r[kBqMaxQ], pp[kBqMaxQ], Ap[kBqMaxQ];
            float rtr_new = 0.f;
#pragma unroll
            for (int i = 0; i < kBqMaxQ; i++) {
                x[i] = alpha[i];
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < kBqMaxQ; j++) if (i < q && j < q) s += A[i][j] * alpha[j];
                r[i] = i < q ? btw[i] - s : 0.f;
                pp[i] = r[i];
                rtr_new += r[i] * r[i];
            }
            for (int it = 0; it < q; it++) {
                const float rtr = rtr_new;
                float pAp = 0.f;
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) {
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < kBqMaxQ; j++) if (i < q && j < q) s += A[i][j] * pp[j];
                    Ap[i] = i < q ? s : 0.f;
                    pAp += pp[i] * Ap[i];
                }
                const float a = rtr / (pAp + 1e-6f);
                rtr_new = 0.f;
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) {
                    x[i] += a * pp[i];
                    r[i] -= a * Ap[i];
                    rtr_new += r[i] * r[i];
                }
                const float beta = rtr_new / (rtr + 1e-6f);
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) pp[i] = r[i] + beta * pp[i];
            }
            // |alpha| descending (insertion sort over the q live entries)
#pragma unroll
            for (int i = 0; i < kBqMaxQ; i++) alpha[i] = i < q ? fabsf(x[i]) : -1.f;
#pragma unroll
            for (int i = 1; i < kBqMaxQ; i++) {
#pragma unroll
                for (int j = i; j > 0; j--) {
                    if (alpha[j] > alpha[j - 1]) { const float t = alpha[j]; alpha[j] = alpha[j - 1]; alpha[j - 1] = t; }
                }
            }
#pragma unroll
            for (int i = 0; i < kBqMaxQ; i++) if (i >= q) alpha[i] = 0.f;

            // the 2^q levels: level c has sign -1 on plane i iff bit q-1-i of c is set (examples/bcq.py:159-163)
            for (int c = lane; c < nlev; c += 32) {
                float v = 0.f;
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) if (i < q) v += ((c >> (q - 1 - i)) & 1) ? -alpha[i] : alpha[i];
                s_v[wib][c] = v;
            }
            __syncwarp();
            for (int c = lane; c < nlev; c += 32) {          // rank sort, ties by index
                const float v = s_v[wib][c];
                int rank = 0;
                for (int d = 0; d < nlev; d++) {
                    const float u = s_v[wib][d];
                    rank += (u < v || (u == v && d < c)) ? 1 : 0;
                }
                s_vs[wib][rank] = v;
                s_ind[wib][rank] = (unsigned char)c;
            }
            __syncwarp();
            // nearest level by bisection on the midpoints
#pragma unroll
            for (int e = 0; e < E; e++) {
                int left = 0, right = nlev - 1;
                for (int it = 0; it < q; it++) {
                    const int ml = (left + right - 1) / 2, mr = ml + 1;
                    const float mid = (s_vs[wib][ml] + s_vs[wib][mr]) / 2.f;
                    if (wv[e] < mid) right = ml; else left = mr;
                }
                const uint32_t c = s_ind[wib][left];
                uint32_t pos = 0u;
                for (int i = 0; i < q; i++) pos |= (((c >> (q - 1 - i)) & 1u) ^ 1u) << i;
                if (e * 32 + lane < g) code[e] = pos | (((1u << q) - 1u) << 8);      // padding keeps code 0: it must not count in B^T B
            }
            __syncwarp();
        }
    }

    // ---- outputs ----
    if (p.alpha_py && lane < q) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < kBqMaxQ; i++) if (i == lane) a = alpha[i];
        p.alpha_py[((size_t)n * G + gi) * q + lane] = a;
    }
    if (p.alpha_k && lane < q) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < kBqMaxQ; i++) if (i == lane) a = alpha[i];
        p.alpha_k[((size_t)gi * q + lane) * p.N + n] = __float2half_rn(a);
    }
#pragma unroll
    for (int e = 0; e < E; e++) {
        const int idx = e * 32 + lane;
        const bool valid = idx < g;
        if (p.binary_py && valid) {
            signed char* dst = p.binary_py + (((size_t)n * G + gi) * g + idx) * q;
            for (int i = 0; i < q; i++) dst[i] = (signed char)code_sign(code[e], i);
        }
        if (p.bW && e * 32 < g) {                          // g % 32 == 0: whole words; a zero code packs as -1
            for (int i = 0; i < q; i++) {
                const uint32_t word = __ballot_sync(0xffffffffu, valid && ((code[e] >> i) & 1u));
                if (lane == 0) p.bW[((size_t)((gi * g) / 32 + e) * q + i) * p.N + n] = word;
            }
        }
    }
}

}  // namespace lg
