// Register-fed variant of the LUT matvec (m = 1), sm_100a, and the any-shape fallback kernel.
//
// gemv_reg_kernel computes exactly what gemv_tma_kernel does (same transposed 64 KB table, same lane
// mapping, same split-k finish and tensor-parallel links; see gemv_tma.cuh) but brings the packed planes
// and alpha straight from global memory into registers: each lane issues two 128-bit non-allocating
// loads per stage, a quarter warp covering 128 consecutive bytes of one packed row, and keeps
// kRegDepth stages in flight in a register queue.  Nothing is staged in shared memory, so the
// shared-memory pipe carries only the lookups and the table build.  It takes any N % 4 == 0 and any
// group size that is a multiple of 32, which makes it the fallback for containers the TMA-fed kernel
// refuses (N % 8 != 0, group sizes that neither divide nor are multiples of 512).
// Replaces _nqmv / _nqmv_bias (lutGEMM/src/cuda/kernels/mv_fp16.hpp:25-97, mv_fp16_bias.hpp:24-118).
#pragma once
#include "gemv_tma.cuh"

namespace lg {

constexpr int kRegThreads = 512;
constexpr int kRegDepth = 4;                                  // stages of words / scales held in registers
constexpr int kRegFlagOff = kXchgOff + 1024;
constexpr int kRegSmemBytes = kRegFlagOff + 64;

__device__ __forceinline__ uint4 ldg_stream_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// WPG: packed words per alpha group among a lane's two words of a stage (2: g % 128 == 0, else 1).
template <int WPG, bool BIAS>
__global__ void __launch_bounds__(kRegThreads, 1)
gemv_reg_kernel(const Gemv2Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* lut = smem;
    int* s_flag = reinterpret_cast<int*>(smem + kRegFlagOff);

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

    const int c8 = lane & 7;                 // 16-byte column chunk inside the warp's 32 columns
    const int rr = lane >> 3;                // which 128-k run of the slab
    const int cb = warp & 7, h = warp >> 3;
    const int jp = (c8 & 1) ^ h;             // this lane's words in the slab: kw = 4 rr + jp + 2 u, u = 0, 1
    const int col_in_stage = 32 * cb + 4 * c8;
    pdl_launch_dependents();

    // ---- register queue of packed words and scales; weights are static, so it fills before the wait ----
    constexpr int NG = 2 / WPG;
    const uint32_t* wrow[2];
    bool row_ok[2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int kw = kw0 + 4 * rr + jp + 2 * u;
        row_ok[u] = kw * 32 < p.K;
        wrow[u] = p.bW + (size_t)kw * q * rowN;
    }
    int grp[NG];
    bool grp_ok[NG];
    const __half* arow[NG];
#pragma unroll
    for (int gi = 0; gi < NG; gi++) {
        const int kw_local = 4 * rr + jp + 2 * gi * WPG;
        grp_ok[gi] = (k0 + 32 * kw_local) < p.K;
        grp[gi] = grp_ok[gi] ? (k0 + 32 * kw_local) / p.g : 0;
        arow[gi] = p.alpha + (size_t)grp[gi] * q * rowN;
    }
    int pf_cg = 0, pf_b = 0;
    auto fetch = [&](uint4 (&w)[2], uint2 (&a)[NG]) {
        const int col = n_begin + pf_cg * kStageCols + col_in_stage;
        const bool ok = (pf_cg < ncg) && (col < n_end);
        const size_t off = (size_t)pf_b * rowN + col;
#pragma unroll
        for (int u = 0; u < 2; u++) w[u] = (ok && row_ok[u]) ? ldg_stream_v4(wrow[u] + off) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int gi = 0; gi < NG; gi++) a[gi] = (ok && grp_ok[gi]) ? ldg_nc_v2(arow[gi] + off) : make_uint2(0u, 0u);
        if (++pf_b == q) { pf_b = 0; pf_cg++; }
    };
    uint4 wq[kRegDepth][2];
    uint2 aq[kRegDepth][NG];
#pragma unroll
    for (int d = 0; d < kRegDepth; d++) fetch(wq[d], aq[d]);

    pdl_wait_prior_grids();                  // the activations may come from the previous kernel
    if (p.tp.x_mode != 0) {
        if (tid == 0) {
            if (!wait_flag_bounded(p.tp.flag_in, p.tp.flag_target)) atomicExch(p.status, kStatusPeerTimeout);
            const unsigned prev = atomicAdd(p.tp.done_counter, 1u);
            if (prev == gridDim.x * gridDim.y - 1u) {
                *reinterpret_cast<volatile unsigned*>(p.tp.flag_in) = 0u;
                *reinterpret_cast<volatile unsigned*>(p.tp.done_counter) = 0u;
            }
        }
        __syncthreads();
    }
    build_lut2(lut, p.x, k0, p.K, tid, p.tp);
    __syncthreads();

    uint32_t cs = 0, sel[4];
#pragma unroll
    for (int b = 0; b < 4; b++) cs |= (uint32_t)(32 * rr + 16 * jp + 4 * b) << (8 * b);
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const uint32_t beta = (uint32_t)(s + (c8 >> 1)) & 3u;
        sel[s] = 0xCC00u | (beta << 4) | (4u + beta);
    }
    float xsum[NG];
    if (BIAS) {
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            float s = 0.f;
#pragma unroll
            for (int jj = 0; jj < WPG; jj++) {
                const int u = gi * WPG + jj;
                const unsigned char* e = lut + 255 * 256 + (32 * u + 8 * rr + 4 * jp) * 4;
                s += *reinterpret_cast<const float*>(e) + *reinterpret_cast<const float*>(e + 4) +
                     *reinterpret_cast<const float*>(e + 8) + *reinterpret_cast<const float*>(e + 12);
            }
            xsum[gi] = s;
        }
    }

    float* part_out = p.partial + (size_t)slab * rowN;
    float4* xchg = reinterpret_cast<float4*>(smem + kXchgOff) + cb * 8 + c8;
    int cg = 0, b = 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    uint2 bv[NG];
    auto fetch_bias = [&]() {
        const int col = n_begin + cg * kStageCols + col_in_stage;
#pragma unroll
        for (int gi = 0; gi < NG; gi++)
            bv[gi] = (BIAS && cg < ncg && col < n_end && grp_ok[gi]) ? ldg_nc_v2(p.q_bias + (size_t)grp[gi] * rowN + col) : make_uint2(0u, 0u);
    };
    fetch_bias();
    for (int t0 = 0; t0 < total_stages; t0 += kRegDepth) {
#pragma unroll
        for (int d = 0; d < kRegDepth; d++) {
            if (t0 + d >= total_stages) break;
            const uint4 w0 = wq[d][0], w1 = wq[d][1];
            uint2 av[NG];
#pragma unroll
            for (int gi = 0; gi < NG; gi++) av[gi] = aq[d][gi];
            fetch(wq[d], aq[d]);                              // refill the slot kRegDepth stages ahead
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                float2 s2[4];
#pragma unroll
                for (int jj = 0; jj < WPG; jj++) {
                    const int u = gi * WPG + jj;
                    const uint4 wv = (u == 0) ? w0 : w1;
                    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float2 v = (u == 0) ? lookup_word<0>(lut, ww[c], cs, sel) : lookup_word<128>(lut, ww[c], cs, sel);
                        s2[c] = (jj == 0) ? v : add_f32x2(s2[c], v);
                    }
                }
                const float2 a01 = half2_bits_to_float2(av[gi].x), a23 = half2_bits_to_float2(av[gi].y);
                acc[0] = fmaf(s2[0].x + s2[0].y, a01.x, acc[0]);
                acc[1] = fmaf(s2[1].x + s2[1].y, a01.y, acc[1]);
                acc[2] = fmaf(s2[2].x + s2[2].y, a23.x, acc[2]);
                acc[3] = fmaf(s2[3].x + s2[3].y, a23.y, acc[3]);
            }
            if (++b == q) {
                // ---- the column group is complete: offset term, cross-lane sums, slab partial out ----
                b = 0;
                const int col = n_begin + cg * kStageCols + col_in_stage;
                const bool col_ok = col < n_end;
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
#pragma unroll
                for (int off = 8; off < 32; off <<= 1) {
#pragma unroll
                    for (int c = 0; c < 4; c++) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
                }
                if (h == 1 && rr == 0) *xchg = make_float4(acc[0], acc[1], acc[2], acc[3]);
                asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");
                if (h == 0 && rr == 0 && col_ok) {
                    const float4 o = *xchg;
                    const float4 r4 = make_float4(acc[0] + o.x, acc[1] + o.y, acc[2] + o.z, acc[3] + o.w);
                    if (p.ordered) *reinterpret_cast<float4*>(part_out + col) = r4;
                    else red_add_v4(p.partial + col, r4);
                }
                asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");
                cg++;
                acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                fetch_bias();
            }
        }
    }
    splitk_finish<kRegThreads>(p, tid, n_begin, n_end, s_flag);
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
