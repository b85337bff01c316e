// LUT matvec for BCQ weights (m = 1), sm_100a.
//
// Replaces _nqmv / _nqmv_bias of the reference (lutGEMM/src/cuda/kernels/mv_fp16.hpp:25-97,
// lutGEMM/src/cuda/kernels/mv_fp16_bias.hpp:24-118).  Same mathematics — a 2^8-entry table of
// signed partial sums per 8 activations, one table lookup per packed weight byte — with a
// different machine mapping:
//
//  * The table is stored TRANSPOSED in shared memory, lut[idx][slot] (fp32), where slot is the
//    8-activation chunk inside a 512-k slab (64 chunks, 256 B per idx row, 64 KB per CTA).
//    A shared-memory bank is then selected by the chunk, not by the random weight byte.  In every
//    lookup instruction the 32 lanes of a warp address 32 different chunks (8 different packed
//    words x 4 byte positions, the byte position rotated by the lane's column quad), so every
//    lookup is bank-conflict free whatever the weights are.  The reference's lut[chunk][idx] fp16
//    layout takes ~3 wavefronts per lookup on random bytes.
//  * One PRMT builds the whole shared-memory offset (idx << 8 | slot * 4) from the packed word, so
//    a lookup costs three instructions: PRMT, LDS, FADD.
//  * Packed words are streamed with 128-bit non-allocating loads (4 columns per lane), one plane
//    row and eight k-words per warp instruction, prefetched one column block ahead.
//  * Entries and accumulation are fp32; alpha (and q_bias) are applied per 32-k word in fp32.
//  * No atomics and no memset: every CTA writes its slab's partial sums to a workspace and the last
//    CTA to finish a column tile adds the slabs in slab order and rounds to fp16 once, so the
//    result is deterministic (the reference's half2 atomicAdd order is not).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lg {

constexpr int kSlabK = 512;                    // k per CTA slab
constexpr int kSlots = kSlabK / 8;             // 64 chunks of 8 activations
constexpr int kLutBytes = 256 * kSlots * 4;    // 65536
constexpr int kGemvThreads = 256;
constexpr int kWarpCols = 16;                  // columns per warp step (4 per lane x 4 lane quads)
constexpr int kCtaCols = kWarpCols * (kGemvThreads / 32);   // 128

struct GemvParams {
    const uint32_t* bW;      // [K/32][q][N]
    const __half* alpha;     // [G][q][N]
    const __half* q_bias;    // [G][N] or nullptr
    const __half* x;         // [K]
    float* partial;          // [nslabs][N] split-k workspace (unused when nslabs == 1)
    unsigned* counters;      // [gridDim.x], zero between launches
    __half* y16;             // [N] or nullptr
    float* y32;              // [N] or nullptr
    int N, K, q, g;
    int n_tile;              // columns per CTA, multiple of kCtaCols
    int nslabs;              // gridDim.y
};

__device__ __forceinline__ uint4 ldg_stream_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// The table is addressed as bytes from the start of the CTA's dynamic shared memory; plain C++
// accesses let the compiler schedule the lookups freely between barriers.
template <int IMM>
__device__ __forceinline__ float lds_f32(const unsigned char* lut, uint32_t off) {
    return *reinterpret_cast<const float*>(lut + off + IMM);
}
__device__ __forceinline__ void sts_f32(unsigned char* lut, uint32_t off, float v) {
    *reinterpret_cast<float*>(lut + off) = v;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}

// Builds lut[idx][slot] for the 64 chunks of one slab.  Thread t owns chunk (t & 63) and the 64
// entries idx in [64 * (t >> 6), +64), walked in Gray-code order so that each entry is one add away
// from the previous one.  A warp stores 32 consecutive slots of one idx row: conflict free.
__device__ __forceinline__ void build_lut(unsigned char* lut, const __half* x, int k0, int K, int tid) {
    const int j = tid & 63, part = tid >> 6;
    float xv[8];
    {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (k0 + 8 * j < K) raw = *reinterpret_cast<const uint4*>(x + k0 + 8 * j);
        float2 a = h2_to_f2(raw.x), b = h2_to_f2(raw.y), c = h2_to_f2(raw.z), d = h2_to_f2(raw.w);
        xv[0] = a.x; xv[1] = a.y; xv[2] = b.x; xv[3] = b.y; xv[4] = c.x; xv[5] = c.y; xv[6] = d.x; xv[7] = d.y;
    }
    float e = -xv[0] - xv[1] - xv[2] - xv[3] - xv[4] - xv[5];
    e += (part & 1) ? xv[6] : -xv[6];
    e += (part & 2) ? xv[7] : -xv[7];
    const uint32_t base = (uint32_t)part * (64u * 256u) + (uint32_t)j * 4u;
    sts_f32(lut, base, e);
#pragma unroll
    for (int c = 1; c < 64; c++) {
        const int t = (c & 1) ? 0 : (c & 2) ? 1 : (c & 4) ? 2 : (c & 8) ? 3 : (c & 16) ? 4 : 5;   // bit flipped between gray(c-1) and gray(c)
        const int gcode = c ^ (c >> 1);
        const float two_x = 2.0f * xv[t];
        e = ((gcode >> t) & 1) ? e + two_x : e - two_x;
        sts_f32(lut, base + (uint32_t)gcode * 256u, e);
    }
}

// Q: number of planes (compile time).  BIAS: container has q_bias.
template <int Q, bool BIAS>
__global__ void __launch_bounds__(kGemvThreads, (Q <= 4) ? 2 : 1)
gemv_lut_kernel(const GemvParams p) {
    extern __shared__ __align__(1024) unsigned char lut[];
    __shared__ int s_is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int a = lane & 7;      // which of 8 packed words (k) this lane owns in each 256-k block
    const int r = lane >> 3;     // which column quad; also the byte rotation
    const int N = p.N;
    const int slab = blockIdx.y;
    const int k0 = slab * kSlabK;
    const int nblk = (p.K - k0 >= kSlabK) ? 2 : 1;             // 256-k blocks in this slab
    const int n_begin = blockIdx.x * p.n_tile;
    const int n_end = min(N, n_begin + p.n_tile);

    // Per-lane lookup constants: byte beta = (s + r) & 3 of a word goes to slot 4a + beta.
    uint32_t cs = 0, sel[4];
#pragma unroll
    for (int b = 0; b < 4; b++) cs |= (uint32_t)(16 * a + 4 * b) << (8 * b);
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const uint32_t beta = (uint32_t)(s + r) & 3u;
        sel[s] = 0xCC00u | (beta << 4) | (4u + beta);     // {0, 0, w.byte[beta], cs.byte[beta]}
    }

    const size_t rowN = (size_t)N;
    // word row of (block i, plane b): ((slab*16 + 8i + a) * q + b)
    const uint32_t* wrow[2];
    const __half* arow[2];
    const __half* brow[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int kw = slab * (kSlabK / 32) + 8 * i + a;
        const int grp = (kw * 32) / p.g;
        wrow[i] = p.bW + (size_t)kw * Q * rowN;
        arow[i] = p.alpha + (size_t)grp * Q * rowN;
        brow[i] = BIAS ? p.q_bias + (size_t)grp * rowN : nullptr;
    }

    uint4 w[2][Q];
    uint2 al[2][Q];
    uint2 qb[2];
    auto load_block = [&](int n, uint4 (&ww)[2][Q], uint2 (&aa)[2][Q], uint2 (&bb)[2]) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const bool ok = (n < n_end) && (i < nblk);
#pragma unroll
            for (int b = 0; b < Q; b++) {
                ww[i][b] = ok ? ldg_stream_v4(wrow[i] + (size_t)b * rowN + n) : make_uint4(0, 0, 0, 0);
                aa[i][b] = ok ? ldg_v2(arow[i] + (size_t)b * rowN + n) : make_uint2(0, 0);
            }
            if (BIAS) bb[i] = ok ? ldg_v2(brow[i] + n) : make_uint2(0, 0);
        }
    };

    int n = n_begin + warp * kWarpCols + 4 * r;
    load_block(n, w, al, qb);           // in flight while the table is built

    build_lut(lut, p.x, k0, p.K, tid);
    __syncthreads();

    // sum of the 32 activations under each of this lane's words: 4 entries idx = 255
    float xs[2] = {0.f, 0.f};
    if (BIAS) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t ad = 255u * 256u + (uint32_t)(32 * i + 4 * a) * 4u;
            xs[i] = lds_f32<0>(lut, ad) + lds_f32<4>(lut, ad) + lds_f32<8>(lut, ad) + lds_f32<12>(lut, ad);
        }
    }

    float* part_out = p.partial + (size_t)slab * rowN;
    const bool direct = (p.nslabs == 1);

    for (; n - 4 * r < n_end; n += kCtaCols) {   // loop bound is warp-uniform
        uint4 wn[2][Q];
        uint2 aln[2][Q];
        uint2 qbn[2];
        if (Q <= 4) load_block(n + kCtaCols, wn, aln, qbn);

        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; i++) {
#pragma unroll
            for (int b = 0; b < Q; b++) {
                const uint32_t ww[4] = {w[i][b].x, w[i][b].y, w[i][b].z, w[i][b].w};
                const float2 a01 = h2_to_f2(al[i][b].x), a23 = h2_to_f2(al[i][b].y);
                const float av[4] = {a01.x, a01.y, a23.x, a23.y};
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float t;
                    if (i == 0) {
                        t = lds_f32<0>(lut, prmt(ww[c], cs, sel[0]));
                        t += lds_f32<0>(lut, prmt(ww[c], cs, sel[1]));
                        t += lds_f32<0>(lut, prmt(ww[c], cs, sel[2]));
                        t += lds_f32<0>(lut, prmt(ww[c], cs, sel[3]));
                    } else {
                        t = lds_f32<128>(lut, prmt(ww[c], cs, sel[0]));
                        t += lds_f32<128>(lut, prmt(ww[c], cs, sel[1]));
                        t += lds_f32<128>(lut, prmt(ww[c], cs, sel[2]));
                        t += lds_f32<128>(lut, prmt(ww[c], cs, sel[3]));
                    }
                    acc[c] = fmaf(t, av[c], acc[c]);
                }
            }
            if (BIAS) {
                const float2 b01 = h2_to_f2(qb[i].x), b23 = h2_to_f2(qb[i].y);
                acc[0] = fmaf(xs[i], b01.x, acc[0]);
                acc[1] = fmaf(xs[i], b01.y, acc[1]);
                acc[2] = fmaf(xs[i], b23.x, acc[2]);
                acc[3] = fmaf(xs[i], b23.y, acc[3]);
            }
        }
        // add the 8 lanes (k words) that share a column quad
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) {
#pragma unroll
            for (int c = 0; c < 4; c++) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
        }
        if (a == 0 && n < n_end) {
            if (!direct) {
                *reinterpret_cast<float4*>(part_out + n) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            } else {
                if (p.y32) *reinterpret_cast<float4*>(p.y32 + n) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                if (p.y16) {
                    __half2 lo = __floats2half2_rn(acc[0], acc[1]), hi = __floats2half2_rn(acc[2], acc[3]);
                    uint2 o;
                    o.x = *reinterpret_cast<uint32_t*>(&lo);
                    o.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(p.y16 + n) = o;
                }
            }
        }
        if (Q <= 4) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
#pragma unroll
                for (int b = 0; b < Q; b++) { w[i][b] = wn[i][b]; al[i][b] = aln[i][b]; }
                if (BIAS) qb[i] = qbn[i];
            }
        } else {
            load_block(n + kCtaCols, w, al, qb);
        }
    }
    if (direct) return;

    // Split-k finish: the last CTA of this column tile adds the slabs in slab order.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
        s_is_last = (prev == (unsigned)p.nslabs - 1u);
    }
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();
    for (int c = n_begin + 4 * tid; c < n_end; c += 4 * kGemvThreads) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = p.partial + c;
#pragma unroll 8
        for (int sl = 0; sl < p.nslabs; sl++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sl * rowN));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (p.y32) *reinterpret_cast<float4*>(p.y32 + c) = s;
        if (p.y16) {
            __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(p.y16 + c) = o;
        }
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;   // ready for the next launch on this stream
}

// Fallback for shapes the LUT kernel does not take (N % 4 != 0 or K % 256 != 0): one thread per
// column, activations staged in shared memory, signs applied bit by bit.  Correctness path only.
__global__ void __launch_bounds__(128)
gemv_generic_kernel(const uint32_t* __restrict__ bW, const __half* __restrict__ alpha,
                    const __half* __restrict__ q_bias, const __half* __restrict__ x,
                    __half* __restrict__ y16, float* __restrict__ y32, int N, int K, int q, int g) {
    __shared__ float xs[1024];
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    float acc = 0.f;
    for (int kt = 0; kt < K; kt += 1024) {
        const int klen = min(1024, K - kt);
        __syncthreads();
        for (int i = threadIdx.x; i < klen; i += blockDim.x) xs[i] = __half2float(x[kt + i]);
        __syncthreads();
        if (n < N) {
            for (int kw = 0; kw < klen / 32; kw++) {
                const int k = kt + kw * 32;
                const int grp = k / g;
                float xsum = 0.f;
                if (q_bias) {
                    for (int t = 0; t < 32; t++) xsum += xs[kw * 32 + t];
                    acc = fmaf(xsum, __half2float(q_bias[(size_t)grp * N + n]), acc);
                }
                for (int b = 0; b < q; b++) {
                    const uint32_t word = bW[((size_t)(k / 32) * q + b) * N + n];
                    float t_sum = 0.f;
#pragma unroll 8
                    for (int t = 0; t < 32; t++) t_sum += ((word >> t) & 1u) ? xs[kw * 32 + t] : -xs[kw * 32 + t];
                    acc = fmaf(t_sum, __half2float(alpha[((size_t)grp * q + b) * N + n]), acc);
                }
            }
        }
    }
    if (n < N) {
        if (y32) y32[n] = acc;
        if (y16) y16[n] = __float2half_rn(acc);
    }
}

}  // namespace lg
