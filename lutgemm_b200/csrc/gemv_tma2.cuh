// Two-row LUT matvec (m = 2, and the first two of m = 3), sm_100a: one pass over the packed planes serves two
// activation rows.
//
// Same machinery as gemv_tma_kernel (gemv_tma.cuh: CTA = column tile x 512-k slab, tiled TMA ring, transposed
// table, lane mapping, L2 reductions across slabs, programmatic dependent launch) with two 64 KB tables, one per
// row, side by side in shared memory: every packed byte is turned into its table offset once (one PRMT) and looked up
// in both tables (the second at +64 KB, an immediate offset), so the weight stream, its staging and the address
// arithmetic are paid once for two rows.  The ring is 5 stages deep instead of 8 (two tables leave 97 KB).
// No tensor-parallel links and no ordered mode here: callers that need them take one row at a time.
// Replaces two calls of _nqmv / _nqmv_bias (lutGEMM/src/cuda/kernels/mv_fp16.hpp:25-97, mv_fp16_bias.hpp:24-118).
#pragma once
#include "gemv_tma.cuh"

namespace lg {

constexpr int kRows2 = 2;
constexpr int kXchg2Off = kRows2 * kLut2Bytes;                // 131072: half-warp exchange, 1 KB per row
constexpr int kBar2Off = kXchg2Off + kRows2 * 1024;
constexpr int kStage02Off = kBar2Off + 256;
__host__ __device__ constexpr int gemv22_num_stages(int a_rows) {
    return (kSmemLimit - kStage02Off) / gemv2_stage_bytes(a_rows) < kMaxStages
               ? (kSmemLimit - kStage02Off) / gemv2_stage_bytes(a_rows) : kMaxStages;
}
__host__ __device__ constexpr int gemv22_smem_bytes(int a_rows) {
    return kStage02Off + gemv22_num_stages(a_rows) * gemv2_stage_bytes(a_rows);
}

struct Gemv22Params {
    Gemv2Params b;           // x = row 0; y16 / y32 = row 0; partial = reduction row of row 0
    const __half* x1;        // row 1
    __half* y16_1;           // row 1 outputs (or nullptr)
    float* y32_1;
    float* partial1;         // second zeroed reduction row [N]
};

// the four table entries of one packed word, in both tables
template <int IMM>
__device__ __forceinline__ void lookup_word2(const unsigned char* lut, uint32_t word, uint32_t cs, const uint32_t (&sel)[4],
                                             float2& r0, float2& r1) {
    const uint32_t o0 = prmt_b32(word, cs, sel[0]), o1 = prmt_b32(word, cs, sel[1]);
    const uint32_t o2 = prmt_b32(word, cs, sel[2]), o3 = prmt_b32(word, cs, sel[3]);
    const float a0 = *reinterpret_cast<const float*>(lut + o0 + IMM), a1 = *reinterpret_cast<const float*>(lut + o1 + IMM);
    const float a2 = *reinterpret_cast<const float*>(lut + o2 + IMM), a3 = *reinterpret_cast<const float*>(lut + o3 + IMM);
    const float b0 = *reinterpret_cast<const float*>(lut + o0 + IMM + kLut2Bytes), b1 = *reinterpret_cast<const float*>(lut + o1 + IMM + kLut2Bytes);
    const float b2 = *reinterpret_cast<const float*>(lut + o2 + IMM + kLut2Bytes), b3 = *reinterpret_cast<const float*>(lut + o3 + IMM + kLut2Bytes);
    r0 = add_f32x2(make_float2(a0, a1), make_float2(a2, a3));
    r1 = add_f32x2(make_float2(b0, b1), make_float2(b2, b3));
}

// WPG, BIAS, tmW, tmA: as gemv_tma_kernel.
template <int WPG, bool BIAS>
__global__ void __launch_bounds__(kGemv2Threads, 1)
gemv_tma2_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, const Gemv22Params pp) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const Gemv2Params& p = pp.b;
    unsigned char* lut = smem;
    const int stage_bytes = gemv2_stage_bytes(p.a_rows);
    const int nstages = gemv22_num_stages(p.a_rows);
    const uint32_t bar_full = smem_u32(smem + kBar2Off);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    int* s_flag = reinterpret_cast<int*>(smem + kBar2Off + 16 * kMaxStages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N, q = p.q;
    const int slab = blockIdx.y;
    const int k0 = slab * kSlab2;
    const int kw0 = slab * kSlabWords;
    const int n_begin = blockIdx.x * p.n_tile;
    const int n_end = min(N, n_begin + p.n_tile);
    const int ncg = (n_end - n_begin + kStageCols - 1) / kStageCols;
    const int total_stages = ncg * q;
    const size_t rowN = (size_t)N;

    if (tid == 0) {
        for (int s = 0; s < nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsWarps) {
        // ---------------- producer (weights and scales are never written by a kernel: starts before the dependency wait) ----
        if (lane == 0) {
            tma_prefetch_descriptor(&tmW);
            tma_prefetch_descriptor(&tmA);
            const int grp0 = k0 / p.g;
            const uint32_t tx = (uint32_t)stage_bytes;
            int slot = 0, round = 0;
            for (int t = 0; t < total_stages; t++) {
                const int cg = t / q, b = t - cg * q;
                if (round > 0) {
                    if (!mbar_wait_bounded(bar_empty + 8 * slot, (round - 1) & 1)) {
                        atomicExch(p.status, kStatusProducerTimeout);
                        break;
                    }
                }
                const int col0 = n_begin + cg * kStageCols;
                const uint32_t dst = smem_u32(smem + kStage02Off + slot * stage_bytes);
                mbar_arrive_expect_tx(bar_full + 8 * slot, tx);
                tma_load_3d(dst, &tmW, col0, b, kw0, bar_full + 8 * slot);
                tma_load_3d(dst + kWStageBytes, &tmA, col0, b, grp0, bar_full + 8 * slot);
                if (++slot == nstages) { slot = 0; round++; }
            }
        }
        pdl_wait_prior_grids();
    } else {
        // ---------------- consumers ----------------
        const int c8 = lane & 7, rr = lane >> 3;
        const int cb = warp & 7, h = warp >> 3;
        const int jp = (c8 & 1) ^ h;
        uint32_t cs = 0, sel[4];
#pragma unroll
        for (int b = 0; b < 4; b++) cs |= (uint32_t)(32 * rr + 16 * jp + 4 * b) << (8 * b);
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const uint32_t beta = (uint32_t)(s + (c8 >> 1)) & 3u;
            sel[s] = 0xCC00u | (beta << 4) | (4u + beta);
        }
        constexpr int NG = 2 / WPG;
        int arow[NG], grp[NG];
        bool grp_ok[NG];
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            const int kw_local = 4 * rr + jp + 2 * gi * WPG;
            grp[gi] = (k0 + 32 * kw_local) / p.g;
            arow[gi] = grp[gi] - k0 / p.g;
            grp_ok[gi] = (k0 + 32 * kw_local) < p.K;
        }
        pdl_wait_prior_grids();                  // the activations may come from the previous kernel
        const TpLink no_link = {};
        build_lut2(lut, p.x, k0, p.K, tid, no_link);
        build_lut2(lut + kLut2Bytes, pp.x1, k0, p.K, tid, no_link);
        asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");

        float xsum[kRows2][NG];
        if (BIAS) {
#pragma unroll
            for (int r = 0; r < kRows2; r++) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++) {
                    float s = 0.f;
#pragma unroll
                    for (int jj = 0; jj < WPG; jj++) {
                        const int u = gi * WPG + jj;
                        const unsigned char* e = lut + r * kLut2Bytes + 255 * 256 + (32 * u + 8 * rr + 4 * jp) * 4;
                        s += *reinterpret_cast<const float*>(e) + *reinterpret_cast<const float*>(e + 4) +
                             *reinterpret_cast<const float*>(e + 8) + *reinterpret_cast<const float*>(e + 12);
                    }
                    xsum[r][gi] = s;
                }
            }
        }

        float4* xchg0 = reinterpret_cast<float4*>(smem + kXchg2Off) + cb * 8 + c8;
        float4* xchg1 = xchg0 + 64;                                   // second row's exchange slots, 1 KB further
        const int col_in_stage = 32 * cb + 4 * c8;
        const uint32_t w_off = (uint32_t)(4 * rr + jp) * kRowPitch + (uint32_t)col_in_stage * 4u;
        bool aborted = false;
        int slot = 0, round = 0;
        for (int cg = 0; cg < ncg; cg++) {
            const int col = n_begin + cg * kStageCols + col_in_stage;
            const bool col_ok = col < n_end;
            float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            uint2 bv[NG];
            if (BIAS) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++)
                    bv[gi] = (col_ok && grp_ok[gi]) ? ldg_nc_v2(p.q_bias + (size_t)grp[gi] * rowN + col) : make_uint2(0u, 0u);
            }
            for (int b = 0; b < q && !aborted; b++) {
                if (!mbar_wait_bounded(bar_full + 8 * slot, round & 1)) {
                    atomicExch(p.status, kStatusConsumerTimeout);
                    aborted = true;     // keep walking the loops (the pair barriers below must stay matched)
                    break;
                }
                const unsigned char* st = smem + kStage02Off + slot * stage_bytes + w_off;
                const unsigned char* sa = smem + kStage02Off + slot * stage_bytes + kWStageBytes + col_in_stage * 2;
                uint4 wv[2];
#pragma unroll
                for (int u = 0; u < 2; u++) wv[u] = *reinterpret_cast<const uint4*>(st + u * 2 * kRowPitch);
                uint2 av[NG];
#pragma unroll
                for (int gi = 0; gi < NG; gi++) av[gi] = *reinterpret_cast<const uint2*>(sa + arow[gi] * kARowPitch);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * slot);   // words are in registers: free the stage
                if (++slot == nstages) { slot = 0; round++; }

#pragma unroll
                for (int gi = 0; gi < NG; gi++) {
                    float2 s0[4], s1[4];
#pragma unroll
                    for (int jj = 0; jj < WPG; jj++) {
                        const int u = gi * WPG + jj;
                        const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            float2 v0, v1;
                            if (u == 0) lookup_word2<0>(lut, ww[c], cs, sel, v0, v1);
                            else lookup_word2<128>(lut, ww[c], cs, sel, v0, v1);
                            s0[c] = (jj == 0) ? v0 : add_f32x2(s0[c], v0);
                            s1[c] = (jj == 0) ? v1 : add_f32x2(s1[c], v1);
                        }
                    }
                    const float2 a01 = half2_bits_to_float2(av[gi].x), a23 = half2_bits_to_float2(av[gi].y);
                    acc0[0] = fmaf(s0[0].x + s0[0].y, a01.x, acc0[0]);
                    acc0[1] = fmaf(s0[1].x + s0[1].y, a01.y, acc0[1]);
                    acc0[2] = fmaf(s0[2].x + s0[2].y, a23.x, acc0[2]);
                    acc0[3] = fmaf(s0[3].x + s0[3].y, a23.y, acc0[3]);
                    acc1[0] = fmaf(s1[0].x + s1[0].y, a01.x, acc1[0]);
                    acc1[1] = fmaf(s1[1].x + s1[1].y, a01.y, acc1[1]);
                    acc1[2] = fmaf(s1[2].x + s1[2].y, a23.x, acc1[2]);
                    acc1[3] = fmaf(s1[3].x + s1[3].y, a23.y, acc1[3]);
                }
            }
            if (BIAS) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++) {
                    const float2 b01 = half2_bits_to_float2(bv[gi].x), b23 = half2_bits_to_float2(bv[gi].y);
                    acc0[0] = fmaf(xsum[0][gi], b01.x, acc0[0]);
                    acc0[1] = fmaf(xsum[0][gi], b01.y, acc0[1]);
                    acc0[2] = fmaf(xsum[0][gi], b23.x, acc0[2]);
                    acc0[3] = fmaf(xsum[0][gi], b23.y, acc0[3]);
                    acc1[0] = fmaf(xsum[1][gi], b01.x, acc1[0]);
                    acc1[1] = fmaf(xsum[1][gi], b01.y, acc1[1]);
                    acc1[2] = fmaf(xsum[1][gi], b23.x, acc1[2]);
                    acc1[3] = fmaf(xsum[1][gi], b23.y, acc1[3]);
                }
            }
            // add the 4 lanes (128-k runs) that share a column quad
#pragma unroll
            for (int off = 8; off < 32; off <<= 1) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    acc0[c] += __shfl_xor_sync(0xffffffffu, acc0[c], off);
                    acc1[c] += __shfl_xor_sync(0xffffffffu, acc1[c], off);
                }
            }
            // add the two warp halves (the other word parity) through shared memory
            if (h == 1 && rr == 0) {
                *xchg0 = make_float4(acc0[0], acc0[1], acc0[2], acc0[3]);
                *xchg1 = make_float4(acc1[0], acc1[1], acc1[2], acc1[3]);
            }
            asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");
            if (h == 0 && rr == 0 && col_ok) {
                const float4 o0 = *xchg0, o1 = *xchg1;
                red_add_v4(p.partial + col, make_float4(acc0[0] + o0.x, acc0[1] + o0.y, acc0[2] + o0.z, acc0[3] + o0.w));
                red_add_v4(pp.partial1 + col, make_float4(acc1[0] + o1.x, acc1[1] + o1.y, acc1[2] + o1.z, acc1[3] + o1.w));
            }
            asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");   // exchange slots free for the next column group
        }
    }

    // ---- split-k finish: the last CTA of the column tile converts both reduction rows and leaves them zeroed ----
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
#pragma unroll
        for (int r = 0; r < kRows2; r++) {
            float* src = (r == 0 ? p.partial : pp.partial1) + c;
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src));
            __stcg(reinterpret_cast<float4*>(src), make_float4(0.f, 0.f, 0.f, 0.f));
            float* y32 = r == 0 ? p.y32 : pp.y32_1;
            __half* y16 = r == 0 ? p.y16 : pp.y16_1;
            if (y32) *reinterpret_cast<float4*>(y32 + c) = v;
            if (y16) {
                __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&lo);
                o.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(y16 + c) = o;
            }
        }
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;   // ready for the next launch on this stream
}
}  // namespace lg
