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
// Here a group up to 1024 wide never leaves its warp (wider ones take a CTA, see the end of this file): the weights stay in registers (lane l holds elements l, l + 32, ...), the
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

// ---- groups wider than 1024 (the reference's default is one group per row): one CTA per (row, group) ----
// Same arithmetic; the codes live in shared memory (2 bytes per weight), the weights are re-read from global memory
// (L2) twice per round, sums go through warp shuffles and a shared-memory stage, and warp 0 solves for alpha and
// sorts the levels.
constexpr int kBqBlockThreads = 256;

__device__ __forceinline__ float block_sum_f(float v, float* s_stage, int tid) {
    v = warp_sum_f(v);
    __syncthreads();                                   // s_stage free
    if ((tid & 31) == 0) s_stage[tid >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kBqBlockThreads / 32; w++) t += s_stage[w];
    return t;
}

__global__ void __launch_bounds__(kBqBlockThreads)
bcq_quantize_block_kernel(const BqParams p) {
    extern __shared__ unsigned short s_code[];         // [g]: bits 0..7 "+1" per plane, 8..15 "non-zero" per plane
    __shared__ float s_stage[kBqBlockThreads / 32];
    __shared__ float s_acc[kBqMaxQ + kBqMaxQ * kBqMaxQ];
    __shared__ float s_alpha[kBqMaxQ];
    __shared__ float s_v[1 << kBqMaxQ];
    __shared__ float s_vs[1 << kBqMaxQ];
    __shared__ unsigned char s_ind[1 << kBqMaxQ];
    const int tid = threadIdx.x, lane = tid & 31;
    const int G = p.K / p.g, g = p.g, q = p.q;
    const int n = blockIdx.x / G, gi = blockIdx.x % G;
    const float* wg = p.w + (size_t)n * p.K + (size_t)gi * g;
    if (tid < kBqMaxQ) s_alpha[tid] = 0.f;
    for (int idx = tid; idx < g; idx += kBqBlockThreads) s_code[idx] = 0;
    __syncthreads();

    auto residual = [&](int idx, int upto) {           // w - sum_{j < upto} alpha_j b_j
        float r = wg[idx];
        const uint32_t c = s_code[idx];
        for (int j = 0; j < upto; j++) r -= s_alpha[j] * code_sign(c, j);
        return r;
    };
    // ---- greedy ----
    for (int i = 0; i < q; i++) {
        float s = 0.f;
        for (int idx = tid; idx < g; idx += kBqBlockThreads) s += fabsf(residual(idx, i));
        float a = block_sum_f(s, s_stage, tid) / (float)g;
        if (a != a) a = 0.f;
        for (int idx = tid; idx < g; idx += kBqBlockThreads) {
            const float r = residual(idx, i);
            unsigned short c = s_code[idx];
            if (r > 0.f) c |= (unsigned short)(1u << i);
            if (r != 0.f) c |= (unsigned short)(1u << (8 + i));
            s_code[idx] = c;
        }
        __syncthreads();
        if (tid == 0) s_alpha[i] = a;
        __syncthreads();
    }
    // ---- alternating refinement ----
    if (q > 1) {
        const int nlev = 1 << q;
        for (int round = 0; round < p.rounds; round++) {
            // B^T w and the Gram matrix, reduced over the block
            float btw[kBqMaxQ];
            int cov[kBqMaxQ * (kBqMaxQ + 1) / 2];
#pragma unroll
            for (int i = 0; i < kBqMaxQ; i++) btw[i] = 0.f;
#pragma unroll
            for (int i = 0; i < kBqMaxQ * (kBqMaxQ + 1) / 2; i++) cov[i] = 0;
            for (int idx = tid; idx < g; idx += kBqBlockThreads) {
                const float wv = wg[idx];
                const uint32_t c = s_code[idx];
                int t = 0;
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) {
                    const float bi = i < q ? code_sign(c, i) : 0.f;
                    btw[i] += bi * wv;
#pragma unroll
                    for (int j = i; j < kBqMaxQ; j++, t++) cov[t] += (int)(bi * (j < q ? code_sign(c, j) : 0.f));
                }
            }
            {
                int t = 0;
                for (int i = 0; i < kBqMaxQ; i++) {
                    const float sb = block_sum_f(i < q ? btw[i] : 0.f, s_stage, tid);
                    if (tid == 0) s_acc[i] = sb;
                    for (int j = i; j < kBqMaxQ; j++, t++) {
                        if (i < q && j < q) {
                            const float sc = block_sum_f((float)cov[t], s_stage, tid);      // integer counts below 2^24: exact
                            if (tid == 0) { s_acc[kBqMaxQ + i * kBqMaxQ + j] = sc; s_acc[kBqMaxQ + j * kBqMaxQ + i] = sc; }
                        }
                    }
                }
            }
            __syncthreads();
            if (tid < 32) {
                // warp 0: q steps of conjugate gradient from the current alpha, |alpha| descending, levels rank-sorted
                float x[kBqMaxQ], r[kBqMaxQ], pp[kBqMaxQ], Ap[kBqMaxQ], al[kBqMaxQ];
                float rtr_new = 0.f;
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) al[i] = s_alpha[i];
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) {
                    x[i] = al[i];
                    float sdot = 0.f;
#pragma unroll
                    for (int j = 0; j < kBqMaxQ; j++) if (i < q && j < q) sdot += s_acc[kBqMaxQ + i * kBqMaxQ + j] * al[j];
                    r[i] = i < q ? s_acc[i] - sdot : 0.f;
                    pp[i] = r[i];
                    rtr_new += r[i] * r[i];
                }
                for (int it = 0; it < q; it++) {
                    const float rtr = rtr_new;
                    float pAp = 0.f;
#pragma unroll
                    for (int i = 0; i < kBqMaxQ; i++) {
                        float sdot = 0.f;
#pragma unroll
                        for (int j = 0; j < kBqMaxQ; j++) if (i < q && j < q) sdot += s_acc[kBqMaxQ + i * kBqMaxQ + j] * pp[j];
                        Ap[i] = i < q ? sdot : 0.f;
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
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) al[i] = i < q ? fabsf(x[i]) : -1.f;
#pragma unroll
                for (int i = 1; i < kBqMaxQ; i++) {
#pragma unroll
                    for (int j = i; j > 0; j--) {
                        if (al[j] > al[j - 1]) { const float t2 = al[j]; al[j] = al[j - 1]; al[j - 1] = t2; }
                    }
                }
#pragma unroll
                for (int i = 0; i < kBqMaxQ; i++) if (i >= q) al[i] = 0.f;
                __syncwarp();
                if (lane < kBqMaxQ) {
                    float a = 0.f;
#pragma unroll
                    for (int i = 0; i < kBqMaxQ; i++) if (i == lane) a = al[i];
                    s_alpha[lane] = a;
                }
                for (int c = lane; c < nlev; c += 32) {
                    float v = 0.f;
#pragma unroll
                    for (int i = 0; i < kBqMaxQ; i++) if (i < q) v += ((c >> (q - 1 - i)) & 1) ? -al[i] : al[i];
                    s_v[c] = v;
                }
                __syncwarp();
                for (int c = lane; c < nlev; c += 32) {
                    const float v = s_v[c];
                    int rank = 0;
                    for (int d = 0; d < nlev; d++) {
                        const float u = s_v[d];
                        rank += (u < v || (u == v && d < c)) ? 1 : 0;
                    }
                    s_vs[rank] = v;
                    s_ind[rank] = (unsigned char)c;
                }
            }
            __syncthreads();
            for (int idx = tid; idx < g; idx += kBqBlockThreads) {
                const float wv = wg[idx];
                int left = 0, right = nlev - 1;
                for (int it = 0; it < q; it++) {
                    const int ml = (left + right - 1) / 2, mr = ml + 1;
                    const float mid = (s_vs[ml] + s_vs[mr]) / 2.f;
                    if (wv < mid) right = ml; else left = mr;
                }
                const uint32_t c = s_ind[left];
                uint32_t pos = 0u;
                for (int i = 0; i < q; i++) pos |= (((c >> (q - 1 - i)) & 1u) ^ 1u) << i;
                s_code[idx] = (unsigned short)(pos | (((1u << q) - 1u) << 8));
            }
            __syncthreads();
        }
    }
    // ---- outputs ----
    if (tid < q) {
        if (p.alpha_py) p.alpha_py[((size_t)n * G + gi) * q + tid] = s_alpha[tid];
        if (p.alpha_k) p.alpha_k[((size_t)gi * q + tid) * p.N + n] = __float2half_rn(s_alpha[tid]);
    }
    const int g_pad = (g + 31) / 32 * 32;
    for (int idx = tid; idx < g_pad; idx += kBqBlockThreads) {        // whole warps walk whole 32-element words
        const bool valid = idx < g;
        const uint32_t c = valid ? s_code[idx] : 0u;
        if (p.binary_py && valid) {
            signed char* dst = p.binary_py + (((size_t)n * G + gi) * g + idx) * q;
            for (int i = 0; i < q; i++) dst[i] = (signed char)code_sign(c, i);
        }
        if (p.bW) {                                         // g % 32 == 0 here; a zero code packs as -1
            for (int i = 0; i < q; i++) {
                const uint32_t word = __ballot_sync(0xffffffffu, valid && ((c >> i) & 1u));
                if (lane == 0) p.bW[((size_t)((gi * g + idx) / 32) * q + i) * p.N + n] = word;
            }
        }
    }
}

}  // namespace lg
