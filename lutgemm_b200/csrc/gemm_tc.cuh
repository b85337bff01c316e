// Batched BCQ matmul (2 <= m <= 128 rows per launch) on the 5th-generation tensor cores, sm_100a.
//
// Replaces the reference's batched path, which writes a dense fp16 copy of the whole weight to a
// global scratch buffer and calls cuBLAS on it (lutGEMM/src/kernels.cu:73-79,
// lutGEMM/src/cuda/kernels/dequant_fp16.hpp:54-107, lutGEMM/src/cuda/kernels/cublas.h:47-55).  Here the
// dense values never leave the SM:
//
//   CTA = 256 output columns x a k-range.  The weights are the MMA's N-side operand (N = 256, the widest
//   instruction: a tcgen05.mma costs about the same time whatever its N, so wide N is what keeps the
//   tensor pipe from being the limit at small batch), the activations the M-side operand (M = 128 rows,
//   rows beyond m zero-filled by TMA).
//   16 expansion warps turn ONE bit plane at a time into a dense fp16 tile B_b[n][k] = +-alpha_b
//   (256 x 64, K-major, 128-byte swizzle) in shared memory, the sign applied by XOR-ing the fp16
//   sign bits of two weights at a time, so every operand value is exact; q_bias is one more "plane"
//   whose tile holds q_bias[g][n] unsigned.  All planes accumulate into the same fp32 accumulator:
//   y = sum_k x (sum_b A_b + q_bias) with exact products and fp32 sums, the accuracy of the matvec path;
//   one lane loads the matching activation tiles x[m][k] with tiled TMA (128-byte swizzle);
//   one lane issues tcgen05.mma (kind::f16, M = 128, N = 256, K = 16 per instruction) accumulating
//   fp32 in tensor memory (128 lanes x 256 columns) over the whole k-range;
//   tcgen05.commit releases each shared-memory stage and finally hands the accumulator to four
//   epilogue warps, which read it with tcgen05.ld and either store fp16/fp32 outputs directly or, with
//   split-k, add their partial sums with fp32 reductions in L2 into a workspace that the last CTA of
//   the column tile converts.
//
// q_bias is honoured for every m (the reference drops it for m > 1).  All mbarrier waits are bounded; a wait that runs out sets the status word, and the CTA
// still frees its tensor memory before leaving.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_async.cuh"

namespace lg {

constexpr int kTcTileN = 256;                 // output columns per CTA (MMA N)
constexpr int kTcTileK = 64;                  // k per sub-tile: one 64-k swizzle atom; a pipeline stage holds two
constexpr int kTcTileM = 128;                 // activation rows per MMA (zero padded)
constexpr int kTcStages = 2;
constexpr int kTcExpWarps = 16;
constexpr int kTcThreads = (kTcExpWarps + 2) * 32;       // + TMA warp + MMA warp = 576
constexpr int kTcASubBytes = kTcTileN * kTcTileK * 2;     // 32768: weight sub-tile [256 rows][128 B]
constexpr int kTcAStageBytes = 2 * kTcASubBytes;          // 65536: two sub-tiles = 128 k per stage
constexpr int kTcBRingBytes = 98304;                     // activation ring: one slot per k tile, [128 rows][128 B]
constexpr int kTcBSlotBytes = kTcTileM * kTcTileK * 2;   // 16384
constexpr int kTcBSlotsMax = kTcBRingBytes / kTcBSlotBytes;   // 6
constexpr int kTcBarOff = kTcStages * kTcAStageBytes + kTcBRingBytes;   // 98304 + 98304
constexpr int kTcSmemBytes = kTcBarOff + 256;

enum { kStatusTcTimeout = 3 };

struct TcParams {
    const uint32_t* bW;      // [K/32][q][N]
    const __half* alpha;     // [G][q][N]
    const __half* q_bias;    // [G][N] or nullptr
    float* partial;          // [m][N] fp32, zero between launches (split-k only)
    unsigned* counters;      // [gridDim.x], zero between launches
    int* status;
    __half* y16;             // [m][N] or nullptr
    float* y32;              // [m][N] or nullptr
    int N, K, q, g;
    int m;                   // rows (<= 128)
    int ktiles_per_cta;      // 64-k tiles per CTA (split-k along gridDim.y)
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulation; issued by one thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 B, 8-row groups
// 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);            // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                                   // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                                   // version
    d |= (uint64_t)2 << 61;                                   // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_f16_f32(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
constexpr uint32_t kTcTmemCols = 256;         // fp32 accumulator: 128 lanes x 256 columns

// Q: number of bit planes; BIAS: container has q_bias.  tmX: 2-D map {K, m} of fp16, box {64, 128}, 128-byte swizzle.
template <int Q, bool BIAS>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t a_base = smem_base;
    const uint32_t b_base = smem_base + kTcStages * kTcAStageBytes;
    const uint32_t bar_afull = smem_base + kTcBarOff;            // kTcStages x 8 B, count = expansion warps
    const uint32_t bar_empty = bar_afull + 8 * kTcStages;        // weight stage free: tcgen05.commit arrives
    const uint32_t bar_acc = bar_empty + 8 * kTcStages;          // accumulator complete
    const uint32_t bar_bfull = bar_acc + 8;                      // activation slot loaded (TMA transaction barriers)
    const uint32_t bar_bempty = bar_bfull + 8 * kTcBSlotsMax;    // activation slot free: tcgen05.commit arrives
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kTcBarOff + 200);
    int* s_flag = reinterpret_cast<int*>(smem + kTcBarOff + 208);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N;
    constexpr int q = Q;
    const int n0 = blockIdx.x * kTcTileN;
    const int kt_begin = blockIdx.y * p.ktiles_per_cta;
    const int kt_total = (p.K + kTcTileK - 1) / kTcTileK;
    const int kt_end = min(kt_total, kt_begin + p.ktiles_per_cta);
    const int nkt = kt_end - kt_begin;
    constexpr int planes = Q + (BIAS ? 1 : 0);            // q_bias rides as one more plane
    const int npairs = (nkt + 1) / 2;                     // a stage = (pair of 64-k sub-tiles, plane)
    const int nst = npairs * planes;
    const size_t rowN = (size_t)N;
    constexpr uint32_t b_slot_bytes = kTcBSlotBytes;
    constexpr int nb_slots = kTcBSlotsMax;

    if (tid == 0) {
        for (int s = 0; s < kTcStages; s++) {
            mbar_init(bar_afull + 8 * s, kTcExpWarps);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kTcBSlotsMax; s++) {
            mbar_init(bar_bfull + 8 * s, 1);
            mbar_init(bar_bempty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_fence_init();
    }
    if (warp == kTcExpWarps + 1) {          // the MMA warp owns the tensor-memory allocation
        tmem_alloc(smem_u32(s_tmem), kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_acc = *s_tmem;
    bool timed_out = false;

    if (warp < kTcExpWarps) {
        // ---------------- expansion: packed planes -> dense fp16 tile in shared memory ----------------
        const int ks = warp >> 3;                         // which of the tile's two packed k-words
        const int row = (warp & 7) * 32 + lane;           // row of the tile = output column n0 + row
        const int n = n0 + row;
        const bool n_ok = n < N;
        // swizzled position of this thread's four 16-byte chunks (4 ks .. 4 ks + 3 of the 128-byte row)
        const uint32_t row_off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
        const int c0 = 4 * ks;
        // One k tile = `planes` pipeline stages.  The packed words and scales of a k tile are fetched two
        // tiles ahead into registers (a tile is far shorter than a trip to HBM); plane indices are
        // compile-time, addresses advance by constant strides.
        constexpr int P = Q + (BIAS ? 1 : 0);
        const int g_words = p.g >> 5;                      // group size in packed words
        int pf_t = 0;                                      // next k tile (local index) to fetch
        int pf_kw = kt_begin * (kTcTileK / 32) + ks;
        int pf_grp = pf_kw / g_words, pf_rem = pf_kw - pf_grp * g_words;
        const uint32_t* wp = p.bW + (size_t)pf_kw * Q * rowN + n;
        const size_t w_tile_stride = (size_t)(kTcTileK / 32) * Q * rowN;
        const unsigned short* alpha_u16 = reinterpret_cast<const unsigned short*>(p.alpha) + n;
        const unsigned short* qbias_u16 = reinterpret_cast<const unsigned short*>(p.q_bias) + n;
        auto load_tile = [&](uint32_t (&w)[P], uint32_t (&a)[P]) {
            const bool ok = (pf_t < nkt) && n_ok && (pf_kw * 32 < p.K);
            const unsigned short* ap = alpha_u16 + (size_t)pf_grp * Q * rowN;
#pragma unroll
            for (int b = 0; b < Q; b++) {
                w[b] = ok ? __ldg(wp + (size_t)b * rowN) : 0u;
                a[b] = (ok ? (uint32_t)__ldg(ap + (size_t)b * rowN) : 0u) * 0x00010001u;
            }
            if (BIAS) {
                w[Q] = 0u;
                a[Q] = (ok ? (uint32_t)__ldg(qbias_u16 + (size_t)pf_grp * rowN) : 0u) * 0x00010001u;
            }
            pf_t++;
            pf_kw += kTcTileK / 32;
            wp += w_tile_stride;
            pf_rem += kTcTileK / 32;
            while (pf_rem >= g_words) { pf_rem -= g_words; pf_grp++; }
        };
        uint32_t chunk_off[4];
#pragma unroll
        for (int c = 0; c < 4; c++) chunk_off[c] = (uint32_t)(((c0 + c) ^ (row & 7)) * 16);
        int cs = 0, cround = 0;                            // shared-memory stage and ring round of the next stage
        // two weights per register: element t (low half) and t + 16 (high half) of the packed word;
        // bit set -> +alpha, bit clear -> -alpha (sign bit flipped where the bit is 0); q_bias plane: no sign
        auto expand_word = [&](uint32_t w, uint32_t a, bool is_bias, unsigned char* dst) {
            uint32_t nat[16];
            if (!is_bias) {
                uint32_t h[16];
#pragma unroll
                for (int t = 0; t < 16; t++) {
                    const uint32_t sh = (t == 15) ? w : (w << (15 - t));
                    h[t] = a ^ (~sh & 0x80008000u);
                }
                // natural k order: (0,1), (2,3), ... then (16,17), ...
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    nat[j] = prmt_b32(h[2 * j], h[2 * j + 1], 0x5410u);
                    nat[j + 8] = prmt_b32(h[2 * j], h[2 * j + 1], 0x7632u);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) nat[j] = a;
            }
#pragma unroll
            for (int c = 0; c < 4; c++)
                *reinterpret_cast<uint4*>(dst + chunk_off[c]) = make_uint4(nat[4 * c], nat[4 * c + 1], nat[4 * c + 2], nat[4 * c + 3]);
        };
        auto expand_pair = [&](const uint32_t (&w0)[P], const uint32_t (&a0)[P], const uint32_t (&w1)[P], const uint32_t (&a1)[P]) {
#pragma unroll
            for (int b = 0; b < P; b++) {
                if (timed_out) break;
                if (cround > 0) {
                    if (!mbar_wait_bounded(bar_empty + 8 * cs, (cround - 1) & 1)) { timed_out = true; break; }
                }
                unsigned char* dst = smem + cs * kTcAStageBytes + row_off;
                expand_word(w0[b], a0[b], b >= Q, dst);
                expand_word(w1[b], a1[b], b >= Q, dst + kTcASubBytes);
                fence_proxy_async_smem();                  // make the generic-proxy stores visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull + 8 * cs);
                if (++cs == kTcStages) { cs = 0; cround++; }
            }
        };
        constexpr int NP = (P <= 5) ? 2 : 1;               // pairs of sub-tiles held in registers ahead of their use
        uint32_t wq[2 * NP][P], aq[2 * NP][P];
#pragma unroll
        for (int u = 0; u < 2 * NP; u++) load_tile(wq[u], aq[u]);
        for (int j = 0; j < npairs && !timed_out; j += NP) {
#pragma unroll
            for (int u = 0; u < NP; u++) {
                if (j + u < npairs && !timed_out) {
                    expand_pair(wq[2 * u], aq[2 * u], wq[2 * u + 1], aq[2 * u + 1]);
                    load_tile(wq[2 * u], aq[2 * u]);
                    load_tile(wq[2 * u + 1], aq[2 * u + 1]);
                }
            }
        }
    } else if (warp == kTcExpWarps) {
        // ---------------- TMA: activation tiles, one slot per k tile, as far ahead as the ring allows ----------------
        if (lane == 0) {
            tma_prefetch_descriptor(&tmX);
            int slot = 0, round = 0;
            for (int j = 0; j < 2 * npairs; j++) {         // sub-tiles, an even number (a trailing one is all padding)
                if (round > 0) {
                    if (!mbar_wait_bounded(bar_bempty + 8 * slot, (round - 1) & 1)) { timed_out = true; break; }
                }
                const int k = (kt_begin + j) * kTcTileK;
                const uint32_t dst = b_base + slot * b_slot_bytes;
                mbar_arrive_expect_tx(bar_bfull + 8 * slot, b_slot_bytes);
                tma_load_2d(dst, &tmX, k, 0, bar_bfull + 8 * slot);
                if (++slot == nb_slots) { slot = 0; round++; }
            }
        }
    } else {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16_f32(kTcTileN);
            int s = 0, sround = 0, bslot = 0, bround = 0;
            const uint64_t dx0 = umma_desc_k_sw128(b_base), dw0 = umma_desc_k_sw128(a_base);
            for (int j = 0; j < npairs && !timed_out; j++) {
                // the pair's two activation slots
                if (!mbar_wait_bounded(bar_bfull + 8 * bslot, bround & 1) ||
                    !mbar_wait_bounded(bar_bfull + 8 * (bslot + 1), bround & 1)) { timed_out = true; break; }
                for (int b = 0; b < planes; b++) {
                    if (!mbar_wait_bounded(bar_afull + 8 * s, sround & 1)) { timed_out = true; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int half = 0; half < 2; half++) {
#pragma unroll
                        for (int k16 = 0; k16 < 4; k16++) {
                            // M-side operand: activations; N-side operand: this plane's +-alpha tile (descriptor start address in 16-byte units)
                            const uint64_t dx = dx0 + (uint64_t)(((bslot + half) * b_slot_bytes + k16 * 32) >> 4);
                            const uint64_t dw = dw0 + (uint64_t)((s * kTcAStageBytes + half * kTcASubBytes + k16 * 32) >> 4);
                            umma_f16_ss(tmem_acc, dx, dw, idesc, (j > 0 || b > 0 || half > 0 || k16 > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(bar_empty + 8 * s);        // weight stage reusable once these MMAs have read it
                    if (++s == kTcStages) { s = 0; sround++; }
                }
                umma_commit(bar_bempty + 8 * bslot);       // activation slots reusable after the last plane of the pair
                umma_commit(bar_bempty + 8 * (bslot + 1));
                bslot += 2;
                if (bslot == nb_slots) { bslot = 0; bround++; }
            }
            umma_commit(bar_acc);                          // accumulator complete
        }
    }
    if (timed_out) atomicExch(p.status, kStatusTcTimeout);

    // ---------------- epilogue: warps 0..3 read the accumulator (TMEM lane = activation row, column = output column) ----
    if (warp < 4) {
        bool ok = (nst > 0) && mbar_wait_bounded(bar_acc, 0);
        if (!ok && nst > 0) atomicExch(p.status, kStatusTcTimeout);
        tc_fence_after_sync();
        const int mrow = warp * 32 + lane;
        const bool split = gridDim.y > 1;
        if (warp * 32 < p.m) {                              // warp-uniform: this quadrant holds real rows
            for (int nc = 0; nc < kTcTileN; nc += 16) {
                uint32_t r[16];
                if (ok) {
                    tmem_ld_x16(tmem_acc + ((uint32_t)(warp * 32) << 16) + (uint32_t)nc, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) r[j] = 0u;
                }
                if (mrow < p.m) {
                    const size_t base = (size_t)mrow * rowN + n0 + nc;
                    if ((N & 7) == 0 && n0 + nc + 16 <= N) {
                        // 16 consecutive columns of one row: vector reductions / vector stores
                        if (split) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.partial + base + j),
                                             "f"(__uint_as_float(r[j])), "f"(__uint_as_float(r[j + 1])),
                                             "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3])) : "memory");
                        } else {
                            if (p.y32) {
#pragma unroll
                                for (int j = 0; j < 16; j += 4)
                                    *reinterpret_cast<float4*>(p.y32 + base + j) =
                                        make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                            }
                            if (p.y16) {
                                uint32_t hh[8];
#pragma unroll
                                for (int j = 0; j < 8; j++) {
                                    __half2 h2 = __floats2half2_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                    hh[j] = *reinterpret_cast<uint32_t*>(&h2);
                                }
                                *reinterpret_cast<uint4*>(p.y16 + base) = make_uint4(hh[0], hh[1], hh[2], hh[3]);
                                *reinterpret_cast<uint4*>(p.y16 + base + 8) = make_uint4(hh[4], hh[5], hh[6], hh[7]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (n0 + nc + j < N) {
                                const float v = __uint_as_float(r[j]);
                                if (split) {
                                    atomicAdd(p.partial + base + j, v);
                                } else {
                                    if (p.y32) p.y32[base + j] = v;
                                    if (p.y16) p.y16[base + j] = __float2half_rn(v);
                                }
                            }
                        }
                    }
                }
            }
        }
        tc_fence_before_sync();
    }
    __threadfence();
    __syncthreads();
    if (warp == kTcExpWarps + 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_acc, kTcTmemCols);
    }
    if (gridDim.y == 1) return;

    // split-k finish: the last CTA of this column tile converts the reduced sums and zeroes the workspace
    if (tid == 0) {
        const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
        *s_flag = (prev == gridDim.y - 1u);
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    for (int idx = tid; idx < p.m * kTcTileN; idx += kTcThreads) {
        const int mrow = idx / kTcTileN, n = n0 + (idx % kTcTileN);
        if (n >= N) continue;
        float* src = p.partial + (size_t)mrow * rowN + n;
        const float v = __ldcg(src);
        __stcg(src, 0.f);
        if (p.y32) p.y32[(size_t)mrow * rowN + n] = v;
        if (p.y16) p.y16[(size_t)mrow * rowN + n] = __float2half_rn(v);
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;
}

}  // namespace lg
