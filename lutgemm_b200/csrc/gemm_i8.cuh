// Batched BCQ matmul for 4 <= m <= 16 rows on the tensor cores' integer path (tcgen05.mma.kind::i8), sm_100a.
//
// The fp16 tensor-core kernel (gemm_tc.cuh) writes every weight as an fp16 value +-alpha into tensor memory: one
// instruction per weight in the expansion warps, which is what bounds it for few rows.  Here the scales stay out of the
// operand.  With s = +-1 the sign of a weight and bit = (s + 1) / 2,
//
//   y[r][n] = sum over groups G of  sum over planes b of  alpha[G][b][n] * sum over k in G of s_b[k][n] * x[r][k]
//           = sum over G, b of alpha[G][b][n] * (2 * D_b[G][r][n] - S[G][r]),       D_b = sum_k bit_b[k][n] * x[r][k],
//                                                                                    S   = sum_k x[r][k],
//
// so the tensor cores only ever multiply the packed BITS (0 / 1 bytes: one shift and one mask turn four weights into
// an operand register) with the activations, and q_bias needs no product at all (its term is q_bias[G][n] * S[G][r]).
// The activations are turned into block-scaled 24-bit integers per 128-k step and row: v = round(x * 2^s) with the
// largest power of two that keeps the block maximum inside the digits' range, so every fp16 input within 2^13 of its
// block's maximum is represented EXACTLY (11 significant bits + 13) and the rest to 2^-24 of that maximum.  v is
// written as three signed int8 digits, v = 65536 d2 + 256 d1 + d0, which ride as the 3 x 16 rows of the MMA's B
// operand.  Every product and sum is an exact integer; the accumulators are int32, one per (scale group, plane), and a set of epilogue warps
// applies alpha, the activation scale and the S terms in fp32 while the next groups are being multiplied.
//
//   CTA = 256 output columns x a k-range, walked in steps of 128 k; 21 warps:
//   warp 2      streams the packed planes + scales (+ q_bias) of a step and the fp16 activation tile through two
//               shared-memory rings (tiled TMA, as in gemm_tc.cuh);
//   warps 3-4   quantise a landed activation tile into the int8 B tile (K-major, 128-byte swizzle, bytes inside every
//               32-k block in the order the expansion's shift leaves the bits) and write the per-row coefficients;
//   warps 5-12  expand one plane of a step into the 0 / 1 byte operand in TENSOR MEMORY (tcgen05.st, thread = output
//               column = lane, 32 columns per plane and step);
//   warps 0-1   issue the MMAs of one column half each (M = 128 columns, N = 48 digit rows, K = 32): per plane and
//               scale unit (min(g, 128) k) a fresh int32 accumulator out of a ring of four, handed over by
//               tcgen05.commit (one issuing warp per ring: a slot's barrier phases are each seen by their producer);
//   warps 13-20 read an accumulator (tcgen05.ld), release it, and fold it into 16 fp32 sums per thread; at the end
//               they store / reduce exactly like the fp16 kernel.
//
// All mbarrier waits are bounded; a wait that runs out sets the status word and the CTA still frees its tensor memory.
#pragma once
#include "gemm_tc.cuh"

namespace lg {

constexpr int kI8Rows = 16;                   // activation rows per launch
constexpr int kI8NB = 3 * kI8Rows;            // rows of the B operand: digits d2, d1, d0 of the 16 rows
constexpr int kI8MmaWarps = 2, kI8TmaWarp = 2, kI8QuantWarp = 3, kI8QuantWarps = 2, kI8FirstExpWarp = 5, kI8ExpWarps = 8,
              kI8FirstEpiWarp = 13, kI8EpiWarps = 8;
constexpr int kI8Threads = (kI8FirstEpiWarp + kI8EpiWarps) * 32;      // 672
constexpr int kI8AStages = 2;                 // operand stages in tensor memory, 64 columns each (32 per column half)
constexpr int kI8DSlots = 4;                  // accumulator slots per column half, 48 columns each
constexpr uint32_t kI8ACol0 = 2u * kI8DSlots * kI8NB;                 // 384; operand stages take the other 128 columns
constexpr int kI8XSlots = 4;                  // both activation rings (fp16 staging, int8 operand)
constexpr int kI8XSlotBytes = kI8Rows * 256;  // fp16 staging: two sub-tiles [16 rows][64 k]
constexpr int kI8BSlotBytes = kI8NB * 128;    // int8 operand: [48 rows][128 k]
constexpr int kI8CoefFloats = kI8Rows * 5;    // per step: c1[16], c2[4 units][16]
constexpr int kI8BOff = 0, kI8XOff = kI8XSlots * kI8BSlotBytes, kI8CoefOff = kI8XOff + kI8XSlots * kI8XSlotBytes,
              kI8ScratchOff = kI8CoefOff + 2048, kI8WOff = kI8ScratchOff + kI8EpiWarps * 16 * 33 * 4;
constexpr int kI8BarBytes = 1024;
constexpr float kI8VMax = 8355711.f;          // 127 * 65536 + 127 * 256 + 127: the largest v three signed digits hold

struct I8Params {
    float* partial;
    unsigned* counters;
    int* status;
    __half* y16;
    float* y32;
    int N, K, g, m;
    int steps_per_cta;
    int units;               // scale units per 128-k step: 128 / min(g, 128)
    int w_packed_bytes, w_alpha_bytes, w_bias_bytes, w_slot_bytes, w_slots;
};

inline bool i8_plan(int q, bool bias, int g, I8Params& p) {
    const int a_rows = g >= kTcStepK ? 1 : kTcStepK / g;
    p.units = a_rows;
    p.w_packed_bytes = kTcStepWords * q * kTcTileN * 4;
    p.w_alpha_bytes = a_rows * q * kTcTileN * 2;
    p.w_bias_bytes = bias ? a_rows * kTcTileN * 2 : 0;
    p.w_slot_bytes = p.w_packed_bytes + p.w_alpha_bytes + p.w_bias_bytes;
    p.w_slots = (kTcSmemTotal - kI8BarBytes - kI8WOff) / p.w_slot_bytes;
    if (p.w_slots > kTcMaxSlots) p.w_slots = kTcMaxSlots;
    return p.w_slots >= 2 && a_rows <= 4;
}

// D[tmem] (+)= A[tmem] * B[smem], int8 inputs, int32 accumulation; issued by one thread.
__device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Instruction descriptor for kind::i8: signed 8-bit x signed 8-bit -> int32, K-major operands, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_s8_s32(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

enum { I8S_wfull = 0, I8S_bfull = 1, I8S_dfull = 2, I8S_aempty = 3, I8S_xfull = 4, I8S_bempty = 5, I8S_wempty = 6, I8S_xempty = 7, I8S_afull = 8, I8S_dempty = 9 };
// Every wait of the kernel: whole warp, bounded (the first argument names the wait site).
#define I8_WAIT(site, bar, par) __all_sync(0xffffffffu, mbar_wait_bounded(bar, par))

//  tmX: 2-D map {K, m} of fp16, box {64, 16}, 128-byte swizzle;  tmW / tmA / tmQ: the maps of gemm_tc_kernel.
template <int Q, bool BIAS>
__global__ void __launch_bounds__(kI8Threads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ, const I8Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int bar_off = kTcSmemTotal - kI8BarBytes;
    const uint32_t bar0 = smem_base + bar_off;
    const uint32_t bar_wfull = bar0;                                   // kTcMaxSlots each
    const uint32_t bar_wempty = bar0 + 8 * kTcMaxSlots;
    const uint32_t bar_xfull = bar0 + 16 * kTcMaxSlots;                // kI8XSlots each: fp16 tile landed
    const uint32_t bar_xempty = bar_xfull + 8 * kI8XSlots;
    const uint32_t bar_bfull = bar_xempty + 8 * kI8XSlots;             // int8 operand + coefficients written
    const uint32_t bar_bempty = bar_bfull + 8 * kI8XSlots;
    const uint32_t bar_afull = bar_bempty + 8 * kI8XSlots;             // kI8AStages each
    const uint32_t bar_aempty = bar_afull + 8 * kI8AStages;
    const uint32_t bar_dfull = bar_aempty + 8 * kI8AStages;            // [2 halves][kI8DSlots]
    const uint32_t bar_dempty = bar_dfull + 8 * 2 * kI8DSlots;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + bar_off + 16 * kTcMaxSlots + 32 * kI8XSlots + 16 * kI8AStages +
                                                   32 * kI8DSlots + 16);
    int* s_flag = reinterpret_cast<int*>(s_tmem + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N;
    const int n0 = blockIdx.x * kTcTileN;
    const int steps_total = (p.K + kTcStepK - 1) / kTcStepK;
    const int step_begin = blockIdx.y * p.steps_per_cta;
    const int nsteps = max(0, min(steps_total, step_begin + p.steps_per_cta) - step_begin);
    const int U = p.units;                                 // 1, 2 or 4
    const int kper = 4 / U;                                // 32-k blocks (MMAs) per unit

    if (tid == 0) {
        for (int s = 0; s < kTcMaxSlots; s++) {
            mbar_init(bar_wfull + 8 * s, 1);
            mbar_init(bar_wempty + 8 * s, kI8ExpWarps + kI8EpiWarps);
        }
        for (int s = 0; s < kI8XSlots; s++) {
            mbar_init(bar_xfull + 8 * s, 1);
            mbar_init(bar_xempty + 8 * s, kI8QuantWarps);
            mbar_init(bar_bfull + 8 * s, kI8QuantWarps);
            mbar_init(bar_bempty + 8 * s, kI8EpiWarps);
        }
        for (int s = 0; s < kI8AStages; s++) {
            mbar_init(bar_afull + 8 * s, kI8ExpWarps);
            mbar_init(bar_aempty + 8 * s, 2);                          // the two column halves
        }
        for (int s = 0; s < 2 * kI8DSlots; s++) {
            mbar_init(bar_dfull + 8 * s, 1);
            mbar_init(bar_dempty + 8 * s, 4);                          // the four lane quarters of that half
        }
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(s_tmem), kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *s_tmem;
    bool timed_out = false;
    pdl_launch_dependents();

    const bool split = gridDim.y > 1;
    float acc[kI8Rows];                                    // epilogue warps: this column's sums
#pragma unroll
    for (int r = 0; r < kI8Rows; r++) acc[r] = 0.f;

    if (warp >= kI8FirstEpiWarp) {
        // ---------------- accumulators -> fp32 sums ----------------
        const int lq = warp & 3, hN = (warp - kI8FirstEpiWarp) >> 2;
        const int col = hN * 128 + lq * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(hN * kI8DSlots * kI8NB);
        int ws = 0, wround = 0, bs = 0, bround = 0, d = 0, dr = 0;
        for (int j = 0; j < nsteps && !timed_out; j++) {
            if (!I8_WAIT(I8S_wfull, bar_wfull + 8 * ws, wround & 1)) { timed_out = true; break; }
            if (!I8_WAIT(I8S_bfull, bar_bfull + 8 * bs, bround & 1)) { timed_out = true; break; }
            const unsigned char* slot = smem + kI8WOff + ws * p.w_slot_bytes;
            const __half* a_sm = reinterpret_cast<const __half*>(slot + p.w_packed_bytes) + col;
            const __half* qsm = reinterpret_cast<const __half*>(slot + p.w_packed_bytes + p.w_alpha_bytes) + col;
            const float* coef = reinterpret_cast<const float*>(smem + kI8CoefOff) + bs * kI8CoefFloats;
            float tg[kI8Rows];
#pragma unroll
            for (int r = 0; r < kI8Rows; r++) tg[r] = 0.f;
#pragma unroll 1
            for (int b = 0; b < Q && !timed_out; b++) {
#pragma unroll 1
                for (int unit = 0; unit < U; unit++) {
                    if (!I8_WAIT(I8S_dfull, bar_dfull + 8 * (hN * kI8DSlots + d), dr & 1)) { timed_out = true; break; }
                    tc_fence_after_sync();
                    const float alpha = __half2float(a_sm[(unit * Q + b) * kTcTileN]);
                    const uint32_t t_src = t_lane + (uint32_t)(d * kI8NB);
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        uint32_t d2[8], d1[8], d0[8];
                        tmem_ld_x8(t_src + 8u * hh, d2);
                        tmem_ld_x8(t_src + 16u + 8u * hh, d1);
                        tmem_ld_x8(t_src + 32u + 8u * hh, d0);
                        tmem_ld_wait();
#pragma unroll
                        for (int r = 0; r < 8; r++)
                            tg[8 * hh + r] = fmaf(alpha, __int2float_rn(((int)d2[r] * 256 + (int)d1[r]) * 256 + (int)d0[r]), tg[8 * hh + r]);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_dempty + 8 * (hN * kI8DSlots + d));
                    if (++d == kI8DSlots) { d = 0; dr++; }
                }
            }
            if (timed_out) break;
            // the step's activation scale, then the terms in S = sum of the step's integers per unit
#pragma unroll
            for (int r = 0; r < kI8Rows; r++) acc[r] = fmaf(coef[r], tg[r], acc[r]);
#pragma unroll 1
            for (int unit = 0; unit < U; unit++) {
                float asum = 0.f;
#pragma unroll
                for (int b = 0; b < Q; b++) asum += __half2float(a_sm[(unit * Q + b) * kTcTileN]);
                if (BIAS) asum -= __half2float(qsm[unit * kTcTileN]);
                const float* c2 = coef + kI8Rows * (1 + unit);
#pragma unroll
                for (int r = 0; r < kI8Rows; r++) acc[r] = fmaf(c2[r], asum, acc[r]);
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_wempty + 8 * ws);
                mbar_arrive(bar_bempty + 8 * bs);
            }
            if (++ws == p.w_slots) { ws = 0; wround++; }
            if (++bs == kI8XSlots) { bs = 0; bround++; }
        }
    } else if (warp >= kI8FirstExpWarp) {
        // ---------------- expansion: packed planes (shared memory) -> 0 / 1 byte operand (tensor memory) ----------------
        const int lq = warp & 3, hN = (warp - kI8FirstExpWarp) >> 2;
        const int col = hN * 128 + lq * 32 + lane;
        const uint32_t t_dst0 = tmem_base + ((uint32_t)(lq * 32) << 16) + kI8ACol0 + (uint32_t)hN * 32u;
        int ws = 0, wround = 0, st = 0, sround = 0;
        for (int j = 0; j < nsteps && !timed_out; j++) {
            if (!I8_WAIT(I8S_wfull, bar_wfull + 8 * ws, wround & 1)) { timed_out = true; break; }
            const uint32_t* wsm = reinterpret_cast<const uint32_t*>(smem + kI8WOff + ws * p.w_slot_bytes) + col;
#pragma unroll 1
            for (int b = 0; b < Q; b++) {
                uint32_t w[4];
#pragma unroll
                for (int wd = 0; wd < 4; wd++) w[wd] = wsm[(wd * Q + b) * kTcTileN];
                if (sround > 0) {
                    if (!I8_WAIT(I8S_aempty, bar_aempty + 8 * st, (sround - 1) & 1)) { timed_out = true; break; }
                    tc_fence_after_sync();
                }
#pragma unroll
                for (int h2 = 0; h2 < 2; h2++) {
                    // register t of word wd: bytes j = 0..3 are bits t + 8 j, i.e. byte 4 t + j of the 32-k block is
                    // weight k = t + 8 j, which is where the quantise warps put the activations
                    uint32_t nat[16];
#pragma unroll
                    for (int wd2 = 0; wd2 < 2; wd2++)
#pragma unroll
                        for (int t = 0; t < 8; t++) nat[wd2 * 8 + t] = (w[2 * h2 + wd2] >> t) & 0x01010101u;
                    tmem_st_x16(t_dst0 + (uint32_t)st * 64u + (uint32_t)h2 * 16u, nat);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull + 8 * st);
                if (++st == kI8AStages) { st = 0; sround++; }
            }
            __syncwarp();
            if (lane == 0 && !timed_out) mbar_arrive(bar_wempty + 8 * ws);
            if (++ws == p.w_slots) { ws = 0; wround++; }
        }
    } else if (warp >= kI8QuantWarp) {
        // ---------------- activations: fp16 tile -> block-scaled int16 as two int8 digit rows + coefficients ----------------
        const int tk = (warp - kI8QuantWarp) * 32 + lane;          // 64 tasks: (row, 32-k word)
        const int r = tk >> 2, wd = tk & 3;
        int xs = 0, xround = 0;
        for (int j = 0; j < nsteps; j++) {
            if (!I8_WAIT(I8S_xfull, bar_xfull + 8 * xs, xround & 1)) { timed_out = true; break; }
            if (xround > 0) {
                if (!I8_WAIT(I8S_bempty, bar_bempty + 8 * xs, (xround - 1) & 1)) { timed_out = true; break; }
            }
            const unsigned char* src = smem + kI8XOff + xs * kI8XSlotBytes + (wd >> 1) * (kI8Rows * 128) + (r >> 3) * 1024 + (r & 7) * 128;
            float xv[32];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 c = *reinterpret_cast<const uint4*>(src + (((4 * (wd & 1) + i) ^ (r & 7)) << 4));
                const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&cw[e]));
                    xv[8 * i + 2 * e] = f.x;
                    xv[8 * i + 2 * e + 1] = f.y;
                    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
            }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            // the largest power of two 2^s with max|x| * 2^s <= kI8VMax; sc = 2^-s (NaN for a non-finite block)
            const uint32_t eb = __float_as_uint(amax) >> 23;
            float inv = __uint_as_float((276u - eb) << 23);
            if (amax * inv > kI8VMax) inv *= 0.5f;
            float sc = 1.f / inv;
            if (amax == 0.f) { inv = 0.f; sc = 0.f; }
            if (eb == 255u) { inv = 0.f; sc = __uint_as_float(0x7fc00000u); }
            int v[32];
            int S = 0;
#pragma unroll
            for (int e = 0; e < 32; e++) {
                v[e] = __float2int_rn(xv[e] * inv);
                S += v[e];
            }
            if (U <= 2) S += __shfl_xor_sync(0xffffffffu, S, 1);
            if (U == 1) S += __shfl_xor_sync(0xffffffffu, S, 2);
            // signed digits: d0 = byte 0 of v, d1 = byte 1 of v + 0x80, d2 = byte 2 of v + 0x8080
            unsigned char* bslot = smem + kI8BOff + xs * kI8BSlotBytes;
#pragma unroll
            for (int dg = 0; dg < 3; dg++) {
                const int add = dg == 0 ? 0 : (dg == 1 ? 0x80 : 0x8080);
                const uint32_t pick = dg == 0 ? 0x0040u : (dg == 1 ? 0x0051u : 0x0062u);
                uint32_t pk[8];
#pragma unroll
                for (int t = 0; t < 8; t++)
                    pk[t] = prmt_b32(prmt_b32((uint32_t)(v[t] + add), (uint32_t)(v[t + 8] + add), pick),
                                     prmt_b32((uint32_t)(v[t + 16] + add), (uint32_t)(v[t + 24] + add), pick), 0x5410u);
                const int rr = r + kI8Rows * (2 - dg);                       // rows 0-15: d2, 16-31: d1, 32-47: d0
                unsigned char* row = bslot + (rr >> 3) * 1024 + (rr & 7) * 128;
#pragma unroll
                for (int i = 0; i < 2; i++)
                    *reinterpret_cast<uint4*>(row + (((2 * wd + i) ^ (rr & 7)) << 4)) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
            float* coef = reinterpret_cast<float*>(smem + kI8CoefOff) + xs * kI8CoefFloats;
            if (wd == 0) coef[r] = 2.f * sc;
            if ((wd & (kper - 1)) == 0) coef[kI8Rows * (1 + wd / kper) + r] = -sc * (float)S;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_bfull + 8 * xs);
                mbar_arrive(bar_xempty + 8 * xs);
            }
            if (++xs == kI8XSlots) { xs = 0; xround++; }
        }
    } else if (warp == kI8TmaWarp) {
        // ---------------- TMA: packed planes + scales (+ q_bias) and fp16 activation tiles ----------------
        if (lane == 0) {
            tma_prefetch_descriptor(&tmX);
            tma_prefetch_descriptor(&tmW);
            tma_prefetch_descriptor(&tmA);
            if (BIAS) tma_prefetch_descriptor(&tmQ);
        }
        int ws = 0, wround = 0, xs = 0, xround = 0;
        for (int j = 0; j < nsteps; j++) {
            const int step = step_begin + j;
            if (wround > 0) {
                if (!I8_WAIT(I8S_wempty, bar_wempty + 8 * ws, (wround - 1) & 1)) { timed_out = true; break; }
            }
            if (lane == 0) {
                const int grp0 = (step * kTcStepK) / p.g;
                const uint32_t wdst = smem_base + kI8WOff + ws * p.w_slot_bytes;
                mbar_arrive_expect_tx(bar_wfull + 8 * ws, (uint32_t)p.w_slot_bytes);
                tma_load_3d(wdst, &tmW, n0, 0, step * kTcStepWords, bar_wfull + 8 * ws);
                tma_load_3d(wdst + p.w_packed_bytes, &tmA, n0, 0, grp0, bar_wfull + 8 * ws);
                if (BIAS) tma_load_2d(wdst + p.w_packed_bytes + p.w_alpha_bytes, &tmQ, n0, grp0, bar_wfull + 8 * ws);
            }
            if (++ws == p.w_slots) { ws = 0; wround++; }

            if (j == 0) pdl_wait_prior_grids();                      // the activations may come from the previous kernel
            if (xround > 0) {
                if (!I8_WAIT(I8S_xempty, bar_xempty + 8 * xs, (xround - 1) & 1)) { timed_out = true; break; }
            }
            if (lane == 0) {
                const uint32_t xdst = smem_base + kI8XOff + xs * kI8XSlotBytes;
                mbar_arrive_expect_tx(bar_xfull + 8 * xs, (uint32_t)kI8XSlotBytes);
                tma_load_2d(xdst, &tmX, step * kTcStepK, 0, bar_xfull + 8 * xs);
                tma_load_2d(xdst + kI8Rows * 128, &tmX, step * kTcStepK + 64, 0, bar_xfull + 8 * xs);
            }
            if (++xs == kI8XSlots) { xs = 0; xround++; }
            __syncwarp();
        }
    } else {
        // ---------------- MMA issue: warp w issues everything of column half w ----------------
        const int hN = warp;
        const uint32_t idesc = umma_idesc_s8_s32(kI8NB);
        const uint64_t db0 = umma_desc_k_sw128(smem_base + kI8BOff);
        const uint32_t d_t0 = tmem_base + (uint32_t)(hN * kI8DSlots * kI8NB);
        const uint32_t a_t0 = tmem_base + kI8ACol0 + (uint32_t)hN * 32u;
        int st = 0, sround = 0, bs = 0, bround = 0, d = 0, dr = 0;
        for (int j = 0; j < nsteps && !timed_out; j++) {
            if (!I8_WAIT(I8S_bfull, bar_bfull + 8 * bs, bround & 1)) { timed_out = true; break; }
#pragma unroll 1
            for (int b = 0; b < Q && !timed_out; b++) {
                if (!I8_WAIT(I8S_afull, bar_afull + 8 * st, sround & 1)) { timed_out = true; break; }
                tc_fence_after_sync();
#pragma unroll 1
                for (int unit = 0; unit < U; unit++) {
                    if (dr > 0) {
                        if (!I8_WAIT(I8S_dempty, bar_dempty + 8 * (hN * kI8DSlots + d), (dr - 1) & 1)) { timed_out = true; break; }
                        tc_fence_after_sync();
                    }
                    if (lane == 0) {
                        for (int kk = 0; kk < kper; kk++) {
                            const int kb = unit * kper + kk;       // 32-k block of the step: 8 operand columns, 32 B of a B row
                            umma_i8_ts(d_t0 + (uint32_t)(d * kI8NB), a_t0 + (uint32_t)st * 64u + (uint32_t)kb * 8u,
                                       db0 + (uint64_t)((bs * kI8BSlotBytes + kb * 32) >> 4), idesc, kk > 0 ? 1u : 0u);
                        }
                        umma_commit(bar_dfull + 8 * (hN * kI8DSlots + d));
                    }
                    __syncwarp();
                    if (++d == kI8DSlots) { d = 0; dr++; }
                }
                if (timed_out) break;
                if (lane == 0) umma_commit(bar_aempty + 8 * st);
                __syncwarp();
                if (++st == kI8AStages) { st = 0; sround++; }
            }
            if (timed_out) break;
            // (no commit on the B slot: the epilogue warps release it after reading the step's last accumulator,
            // which is complete only when every MMA that read the slot is)
            if (++bs == kI8XSlots) { bs = 0; bround++; }
        }
    }
    pdl_wait_prior_grids();                  // before any store to global memory
    if (timed_out) atomicExch(p.status, kStatusTcTimeout);

    if (warp >= kI8FirstEpiWarp && nsteps > 0) {
        const int lq = warp & 3, hN = (warp - kI8FirstEpiWarp) >> 2;
        float* scratch = reinterpret_cast<float*>(smem + kI8ScratchOff) + (warp - kI8FirstEpiWarp) * (16 * 33);
        uint32_t v[16];
#pragma unroll
        for (int r = 0; r < 16; r++) v[r] = __float_as_uint(acc[r]);
        tc_store_block(scratch, v, lane, 0, n0 + hN * 128 + lq * 32, p.m, N, split, p.partial, p.y16, p.y32);
    }
    tc_fence_before_sync();
    __threadfence();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
    if (!split) return;
    tc_splitk_finish(p.partial, p.counters, p.y16, p.y32, p.m, N, n0, s_flag, kI8Threads);
}

}  // namespace lg
