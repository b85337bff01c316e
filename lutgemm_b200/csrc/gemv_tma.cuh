// LUT matvec for BCQ weights (m = 1), sm_100a: bulk-copy (TMA) fed, one CTA per SM.
//
// Replaces _nqmv / _nqmv_bias of the reference (lutGEMM/src/cuda/kernels/mv_fp16.hpp:25-97,
// lutGEMM/src/cuda/kernels/mv_fp16_bias.hpp:24-118).  Same mathematics — a 2^8-entry table of signed
// partial sums per 8 activations, one lookup per packed weight byte — mapped to the machine as follows.
//
//  CTA = (column tile) x (1024-k slab).  544 threads: 16 consumer warps + 1 producer warp.
//
//  Table.  lut[idx][slot] fp32, TRANSPOSED: the shared-memory bank is chosen by the slot (the
//  8-activation chunk), not by the random weight byte.  128 chunks -> two [256][64] halves of 64 KB.
//  Chunk (word kw = 4a + j, byte beta) lives in slot 32 j + 4 a + beta.  In every lookup instruction
//  the 32 lanes of a warp hold 8 different a and, through a per-quad byte rotation, 4 different beta:
//  32 different banks, so lookups never conflict, whatever the weights are.  One PRMT turns a packed
//  byte into the shared-memory offset (idx << 8 | slot * 4): a lookup is PRMT + LDS + add.
//
//  Weights.  The producer warp streams the packed planes with plain bulk copies (cp.async.bulk,
//  global -> shared, mbarrier completion; no multicast): one stage = one bit plane x 1024 k x 256
//  columns = 32 rows of 1 KB, each row one copy, rows padded to 1040 B so that the consumers'
//  128-bit reads (8 lanes = 8 different k-words per quarter warp) touch 8 different bank groups.
//  Three stages (100 KB) are in flight; a consumer warp releases a stage as soon as its 4 words per
//  lane are in registers.
//
//  Scales.  A lane's four words of a slab are consecutive in k, so with group size >= 128 they share
//  one alpha: 16 lookups are summed, then one FMA (WPG = words per group = 4; 2 and 1 for group
//  sizes 64 and 32).  alpha / q_bias come through ordinary 64-bit loads, issued before the stage wait.
//
//  Result.  fp32 throughout; the 8 lanes that share columns are added with shuffles, each CTA writes
//  its slab's partial sums, and the last CTA of a column tile adds the slabs in slab order and rounds
//  to fp16 once: no atomics on data, no memset, run-to-run identical results.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_async.cuh"

namespace lg {

constexpr int kSlab2 = 1024;                                // k per CTA
constexpr int kStageCols = 256;                             // columns per stage
constexpr int kConsWarps = 16;
constexpr int kGemv2Threads = (kConsWarps + 1) * 32;        // 544
constexpr int kStages = 3;
constexpr int kRowPitch = kStageCols * 4 + 16;              // 1040
constexpr int kStageBytes = 32 * kRowPitch;                 // 33280
constexpr int kLut2Bytes = 2 * 65536;
constexpr int kBarOff = kLut2Bytes + kStages * kStageBytes; // 230912
constexpr int kGemv2Smem = kBarOff + 64;

enum { kStatusOk = 0, kStatusProducerTimeout = 1, kStatusConsumerTimeout = 2 };

struct Gemv2Params {
    const uint32_t* bW;      // [K/32][q][N]
    const __half* alpha;     // [G][q][N]
    const __half* q_bias;    // [G][N] or nullptr
    const __half* x;         // [K]
    float* partial;          // [nslabs][N] split-k workspace (unused when nslabs == 1)
    unsigned* counters;      // [gridDim.x], zero between launches
    int* status;             // device word; set non-zero if a bounded wait ran out
    __half* y16;             // [N] or nullptr
    float* y32;              // [N] or nullptr
    int N, K, q, g;
    int n_tile;              // columns per CTA, multiple of kStageCols
    int nslabs;              // gridDim.y
};

__device__ __forceinline__ uint2 ldg_nc_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}
// Two fp32 adds in one instruction (packed f32x2, new on sm_100).
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rd;\n"
        "mov.b64 ra, {%2, %3};\n"
        "mov.b64 rb, {%4, %5};\n"
        "add.rn.f32x2 rd, ra, rb;\n"
        "mov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// Sum of the four table entries selected by the four bytes of one packed word.  IMM is the
// compile-time part of the slot address (table half and word parity).
template <int IMM>
__device__ __forceinline__ float2 lookup_word(const unsigned char* lut, uint32_t word, uint32_t cs,
                                              const uint32_t (&sel)[4]) {
    const float l0 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[0]) + IMM);
    const float l1 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[1]) + IMM);
    const float l2 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[2]) + IMM);
    const float l3 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[3]) + IMM);
    return add_f32x2(make_float2(l0, l1), make_float2(l2, l3));
}

// Table for the 128 chunks of one slab.  Consumer thread t owns slot (t & 127) and the 64 entries
// idx in [64 (t >> 7), +64), walked in Gray-code order (one add per entry).  A warp stores 32
// consecutive slots of one idx row: conflict free.
__device__ __forceinline__ void build_lut2(unsigned char* lut, const __half* x, int k0, int K, int ctid) {
    const int slot = ctid & 127, part = ctid >> 7;
    const int j = slot >> 5, a = (slot & 31) >> 2, beta = slot & 3;
    const int chunk = 4 * (4 * a + j) + beta;            // 8-activation chunk in natural k order
    float xv[8];
    {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (k0 + 8 * chunk < K) raw = *reinterpret_cast<const uint4*>(x + k0 + 8 * chunk);
        const float2 f0 = half2_bits_to_float2(raw.x), f1 = half2_bits_to_float2(raw.y);
        const float2 f2 = half2_bits_to_float2(raw.z), f3 = half2_bits_to_float2(raw.w);
        xv[0] = f0.x; xv[1] = f0.y; xv[2] = f1.x; xv[3] = f1.y; xv[4] = f2.x; xv[5] = f2.y; xv[6] = f3.x; xv[7] = f3.y;
    }
    float e = -xv[0] - xv[1] - xv[2] - xv[3] - xv[4] - xv[5];
    e += (part & 1) ? xv[6] : -xv[6];
    e += (part & 2) ? xv[7] : -xv[7];
    unsigned char* base = lut + (slot >> 6) * 65536 + part * (64 * 256) + (slot & 63) * 4;
    *reinterpret_cast<float*>(base) = e;
#pragma unroll
    for (int c = 1; c < 64; c++) {
        const int t = (c & 1) ? 0 : (c & 2) ? 1 : (c & 4) ? 2 : (c & 8) ? 3 : (c & 16) ? 4 : 5;   // bit that flips
        const int gcode = c ^ (c >> 1);
        const float two_x = 2.0f * xv[t];
        e = ((gcode >> t) & 1) ? e + two_x : e - two_x;
        *reinterpret_cast<float*>(base + gcode * 256) = e;
    }
}

// WPG: packed words per alpha group inside a lane's four consecutive words (4: g >= 128, 2: g = 64,
// 1: g = 32 or any other multiple of 32).  BIAS: container has q_bias.
template <int WPG, bool BIAS>
__global__ void __launch_bounds__(kGemv2Threads, 1)
gemv_tma_kernel(const Gemv2Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* lut = smem;
    const uint32_t stage0 = smem_u32(smem + kLut2Bytes);
    const uint32_t bar_full = smem_u32(smem + kBarOff);          // kStages x 8 B
    const uint32_t bar_empty = bar_full + 8 * kStages;
    int* s_flag = reinterpret_cast<int*>(smem + kBarOff + 48);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N, q = p.q;
    const int slab = blockIdx.y;
    const int k0 = slab * kSlab2;
    const int kw0 = slab * (kSlab2 / 32);
    const int rows_valid = min(32, p.K / 32 - kw0);              // packed words of this slab that exist
    const int n_begin = blockIdx.x * p.n_tile;
    const int n_end = min(N, n_begin + p.n_tile);
    const int ncg = (n_end - n_begin + kStageCols - 1) / kStageCols;
    const int total_stages = ncg * q;
    const size_t rowN = (size_t)N;

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kConsWarps) {
        // ---------------- producer: one row (one packed k-word, 256 columns) per lane ----------------
        const int a = lane & 7, j = lane >> 3;
        const int kw_local = 4 * a + j;
        const bool row_ok = kw_local < rows_valid;
        const uint32_t* src_row = p.bW + (size_t)(kw0 + kw_local) * q * rowN;
        for (int t = 0; t < total_stages; t++) {
            const int cg = t / q, b = t - cg * q, slot = t % kStages;
            if (t >= kStages) {
                if (!mbar_wait_bounded(bar_empty + 8 * slot, ((t / kStages) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.status, kStatusProducerTimeout);
                    break;
                }
            }
            const int col0 = n_begin + cg * kStageCols;
            const uint32_t bytes = (uint32_t)min(kStageCols, n_end - col0) * 4u;
            if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * slot, bytes * (uint32_t)rows_valid);
            __syncwarp();
            if (row_ok)
                bulk_g2s(stage0 + slot * kStageBytes + lane * kRowPitch, src_row + (size_t)b * rowN + col0, bytes,
                         bar_full + 8 * slot);
        }
    } else {
        // ---------------- consumers ----------------
        const int a = lane & 7;      // this lane's words in the slab: kw = 4a + j, j = 0..3
        const int r = lane >> 3;     // column quad inside the warp's 16 columns; also the byte rotation
        build_lut2(lut, p.x, k0, p.K, tid);
        asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");

        uint32_t cs = 0, sel[4];
#pragma unroll
        for (int b = 0; b < 4; b++) cs |= (uint32_t)(16 * a + 4 * b) << (8 * b);
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const uint32_t beta = (uint32_t)(s + r) & 3u;
            sel[s] = 0xCC00u | (beta << 4) | (4u + beta);     // -> {0, 0, word.byte[beta], cs.byte[beta]}
        }

        constexpr int NG = 4 / WPG;                            // alpha groups among the lane's 4 words
        int grp[NG];
        bool grp_ok[NG];
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            const int kw_local = 4 * a + gi * WPG;
            grp[gi] = (k0 + 32 * kw_local) / p.g;
            grp_ok[gi] = kw_local < rows_valid;
        }
        float xsum[NG];
        if (BIAS) {
            // sum of the activations under each group of words: entries idx = 255 (all signs +)
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                float s = 0.f;
#pragma unroll
                for (int jj = 0; jj < WPG; jj++) {
                    const int j = gi * WPG + jj;
                    const unsigned char* e = lut + (j >> 1) * 65536 + 255 * 256 + ((j & 1) * 32 + 4 * a) * 4;
                    s += *reinterpret_cast<const float*>(e) + *reinterpret_cast<const float*>(e + 4) +
                         *reinterpret_cast<const float*>(e + 8) + *reinterpret_cast<const float*>(e + 12);
                }
                xsum[gi] = s;
            }
        }

        float* part_out = p.partial + (size_t)slab * rowN;
        const bool direct = (p.nslabs == 1);
        const uint32_t my_off = (uint32_t)a * kRowPitch + (uint32_t)(16 * warp + 4 * r) * 4u;
        bool aborted = false;
        int t = 0;
        // alpha is fetched two stages ahead of its use (a stage lasts about as long as one trip to L2/HBM)
        const int col_w = n_begin + 16 * warp + 4 * r;
        int pf_cg = 0, pf_b = 0;
        auto fetch_alpha = [&](uint2 (&dst)[NG]) {
            const int c = col_w + pf_cg * kStageCols;
            const bool ok = (pf_cg < ncg) && (c < n_end);
#pragma unroll
            for (int gi = 0; gi < NG; gi++)
                dst[gi] = (ok && grp_ok[gi]) ? ldg_nc_v2(p.alpha + ((size_t)grp[gi] * q + pf_b) * rowN + c)
                                             : make_uint2(0u, 0u);
            if (++pf_b == q) { pf_b = 0; pf_cg++; }
        };
        uint2 av[NG], av1[NG], av2[NG];
        fetch_alpha(av1);
        fetch_alpha(av2);
        for (int cg = 0; cg < ncg && !aborted; cg++) {
            const int col = n_begin + cg * kStageCols + 16 * warp + 4 * r;
            const bool col_ok = col < n_end;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            uint2 bv[NG];
            if (BIAS) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++)
                    bv[gi] = (col_ok && grp_ok[gi]) ? ldg_nc_v2(p.q_bias + (size_t)grp[gi] * rowN + col) : make_uint2(0u, 0u);
            }
            for (int b = 0; b < q; b++, t++) {
                const int slot = t % kStages;
#pragma unroll
                for (int gi = 0; gi < NG; gi++) { av[gi] = av1[gi]; av1[gi] = av2[gi]; }
                fetch_alpha(av2);
                if (!mbar_wait_bounded(bar_full + 8 * slot, (t / kStages) & 1)) {
                    atomicExch(p.status, kStatusConsumerTimeout);
                    aborted = true;
                    break;
                }
                const unsigned char* st = smem + kLut2Bytes + slot * kStageBytes + my_off;
                uint4 wv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) wv[j] = *reinterpret_cast<const uint4*>(st + j * 8 * kRowPitch);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * slot);   // words are in registers: free the stage

#pragma unroll
                for (int gi = 0; gi < NG; gi++) {
                    float2 s2[4];
#pragma unroll
                    for (int jj = 0; jj < WPG; jj++) {
                        const int j = gi * WPG + jj;
                        const uint32_t ww[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            float2 v;
                            if (j == 0) v = lookup_word<0>(lut, ww[c], cs, sel);
                            else if (j == 1) v = lookup_word<128>(lut, ww[c], cs, sel);
                            else if (j == 2) v = lookup_word<65536>(lut, ww[c], cs, sel);
                            else v = lookup_word<65536 + 128>(lut, ww[c], cs, sel);
                            s2[c] = (jj == 0) ? v : add_f32x2(s2[c], v);
                        }
                    }
                    const float2 a01 = half2_bits_to_float2(av[gi].x), a23 = half2_bits_to_float2(av[gi].y);
                    acc[0] = fmaf(s2[0].x + s2[0].y, a01.x, acc[0]);
                    acc[1] = fmaf(s2[1].x + s2[1].y, a01.y, acc[1]);
                    acc[2] = fmaf(s2[2].x + s2[2].y, a23.x, acc[2]);
                    acc[3] = fmaf(s2[3].x + s2[3].y, a23.y, acc[3]);
                }
            }
            if (aborted) break;
            if (BIAS) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++) {
                    const float2 b01 = half2_bits_to_float2(bv[gi].x), b23 = half2_bits_to_float2(bv[gi].y);
                    acc[0] = fmaf(xsum[gi], b01.x, acc[0]);
                    acc[1] = fmaf(xsum[gi], b01.y, acc[1]);
                    acc[2] = fmaf(xsum[gi], b23.x, acc[2]);
                    acc[3] = fmaf(xsum[gi], b23.y, acc[3]);
                }
            }
            // add the 8 lanes (k words) that share a column quad
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) {
#pragma unroll
                for (int c = 0; c < 4; c++) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
            }
            if (a == 0 && col_ok) {
                if (!direct) {
                    *reinterpret_cast<float4*>(part_out + col) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                } else {
                    if (p.y32) *reinterpret_cast<float4*>(p.y32 + col) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    if (p.y16) {
                        __half2 lo = __floats2half2_rn(acc[0], acc[1]), hi = __floats2half2_rn(acc[2], acc[3]);
                        uint2 o;
                        o.x = *reinterpret_cast<uint32_t*>(&lo);
                        o.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(p.y16 + col) = o;
                    }
                }
            }
        }
    }
    if (p.nslabs == 1) return;

    // Split-k finish: the last CTA of this column tile adds the slabs in slab order.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
        *s_flag = (prev == (unsigned)p.nslabs - 1u);
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    for (int c = n_begin + 4 * tid; c < n_end; c += 4 * kGemv2Threads) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = p.partial + c;
#pragma unroll 4
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

}  // namespace lg
