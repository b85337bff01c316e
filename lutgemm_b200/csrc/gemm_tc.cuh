// Batched BCQ matmul (2 <= m <= 128 rows per launch) on the 5th-generation tensor cores, sm_100a.
//
// Replaces the reference's batched path, which writes a dense fp16 copy of the whole weight to a
// global scratch buffer and calls cuBLAS on it (lutGEMM/src/kernels.cu:73-79,
// lutGEMM/src/cuda/kernels/dequant_fp16.hpp:54-107, lutGEMM/src/cuda/kernels/cublas.h:47-55).  Here the
// dense values never leave the SM:
//
//   CTA = 128 output columns (the MMA M dimension: "swap-AB", weights are operand A) x a k-range.
//   16 expansion warps turn ONE bit plane at a time into a dense fp16 tile A_b[n][k] = +-alpha_b
//   (128 x 128, K-major, 128-byte swizzle) in shared memory, the sign applied by XOR-ing the fp16
//   sign bits of two weights at a time, so every operand value is exact; q_bias is one more "plane"
//   whose tile holds q_bias[g][n] unsigned.  All planes accumulate into the same fp32 accumulator:
//   y = sum_k x (sum_b A_b + q_bias) with exact products and fp32 sums, the accuracy of the matvec path;
//   one lane loads the matching activation tiles x[m][k] with tiled TMA (128-byte swizzle, rows
//   beyond m zero-filled); one lane issues tcgen05.mma (kind::f16, M = 128, N = m padded to 16,
//   K = 16 per instruction) accumulating fp32 in tensor memory over the whole k-range;
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

constexpr int kTcTileN = 128;                 // output columns per CTA (MMA M)
constexpr int kTcTileK = 128;                 // k per stage: two 64-k swizzle atoms
constexpr int kTcStages = 3;
constexpr int kTcPrefetch = 8;                // stages of packed words / scales in flight per thread
constexpr int kTcExpWarps = 16;
constexpr int kTcThreads = (kTcExpWarps + 2) * 32;       // + TMA warp + MMA warp = 576
constexpr int kTcAStageBytes = kTcTileN * kTcTileK * 2;   // 32768: [2 halves][128 rows][128 B]
constexpr int kTcBHalfBytesMax = 128 * 128;              // m_pad rows x 128 B, m_pad <= 128
constexpr int kTcBarOff = kTcStages * kTcAStageBytes + kTcStages * 2 * kTcBHalfBytesMax;   // 98304 + 98304
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
    int m, m_pad;            // rows, rows padded to a multiple of 16 (<= 128)
    int ktiles_per_cta;      // 128-k tiles per CTA (split-k along gridDim.y)
    int tmem_cols;           // power of two >= max(32, m_pad)
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

// Q: number of bit planes.  tmX: 2-D map {K, m} of fp16, box {64, m_pad}, 128-byte swizzle.
template <int Q>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t a_base = smem_base;
    const uint32_t b_base = smem_base + kTcStages * kTcAStageBytes;
    const uint32_t bar_afull = smem_base + kTcBarOff;            // kTcStages x 8 B, count = expansion warps
    const uint32_t bar_bfull = bar_afull + 8 * kTcStages;        // TMA transaction barriers
    const uint32_t bar_empty = bar_bfull + 8 * kTcStages;        // tcgen05.commit arrives
    const uint32_t bar_acc = bar_empty + 8 * kTcStages;          // accumulator complete
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kTcBarOff + 128);
    int* s_flag = reinterpret_cast<int*>(smem + kTcBarOff + 136);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N;
    constexpr int q = Q;
    const int n0 = blockIdx.x * kTcTileN;
    const int kt_begin = blockIdx.y * p.ktiles_per_cta;
    const int kt_total = (p.K + kTcTileK - 1) / kTcTileK;
    const int kt_end = min(kt_total, kt_begin + p.ktiles_per_cta);
    const int nkt = kt_end - kt_begin;
    const int planes = Q + (p.q_bias ? 1 : 0);            // q_bias rides as one more plane
    const int nst = nkt * planes;                         // pipeline stages: (k tile, plane) pairs
    const size_t rowN = (size_t)N;
    const uint32_t b_half_bytes = (uint32_t)p.m_pad * 128u;

    if (tid == 0) {
        for (int s = 0; s < kTcStages; s++) {
            mbar_init(bar_afull + 8 * s, kTcExpWarps);
            mbar_init(bar_bfull + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_fence_init();
    }
    if (warp == kTcExpWarps + 1) {          // the MMA warp owns the tensor-memory allocation
        tmem_alloc(smem_u32(s_tmem), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_acc = *s_tmem;
    bool timed_out = false;

    if (warp < kTcExpWarps) {
        // ---------------- expansion: packed planes -> dense fp16 tile in shared memory ----------------
        const int rq = warp & 3, ks = warp >> 2;          // row quarter (32 rows), k-word slot (0..3) of the tile
        const int row = rq * 32 + lane;                   // row of the tile = output column n0 + row
        const int n = n0 + row;
        const bool n_ok = n < N;
        // swizzled position of this thread's four 16-byte chunks: half = ks >> 1, chunks 4 (ks & 1) .. +3
        const uint32_t row_off = (uint32_t)(ks >> 1) * (kTcTileN * 128) + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
        const int c0 = 4 * (ks & 1);
        // Packed words and scales are fetched kTcPrefetch stages ahead (a stage is far shorter than a trip
        // to HBM); the queue lives in registers and is indexed at compile time by unrolling the stage loop.
        uint32_t wq[kTcPrefetch], aq[kTcPrefetch];         // word of the plane; alpha_b (or q_bias) as half2 (a, a)
        auto load_stage = [&](int i, uint32_t& w, uint32_t& v2) {
            w = 0u;
            unsigned short vh = 0;
            if (i < nst) {
                const int kt = kt_begin + i / planes, b = i % planes;
                const int kw = kt * (kTcTileK / 32) + ks;
                if (n_ok && (kw * 32 < p.K)) {
                    const int grp = (kw * 32) / p.g;
                    if (b < Q) {
                        w = __ldg(p.bW + ((size_t)kw * q + b) * rowN + n);
                        vh = __ldg(reinterpret_cast<const unsigned short*>(p.alpha) + ((size_t)grp * q + b) * rowN + n);
                    } else {
                        vh = __ldg(reinterpret_cast<const unsigned short*>(p.q_bias) + (size_t)grp * rowN + n);
                    }
                }
            }
            v2 = (uint32_t)vh * 0x00010001u;
        };
#pragma unroll
        for (int d = 0; d < kTcPrefetch; d++) load_stage(d, wq[d], aq[d]);
        for (int i0 = 0; i0 < nst && !timed_out; i0 += kTcPrefetch) {
#pragma unroll
            for (int d = 0; d < kTcPrefetch; d++) {
                const int i = i0 + d;
                if (i >= nst || timed_out) break;
                const int s = i % kTcStages;
                const bool is_bias = (i % planes) == Q;
                const uint32_t word = wq[d], a2 = aq[d];
                load_stage(i + kTcPrefetch, wq[d], aq[d]);
                if (i >= kTcStages) {
                    if (!mbar_wait_bounded(bar_empty + 8 * s, ((i / kTcStages) - 1) & 1)) { timed_out = true; break; }
                }
                // 16 registers of two weights each: element t (low half) and t + 16 (high half) of the word;
                // bit set -> +alpha, bit clear -> -alpha (sign bits flipped where the bit is 0); q_bias: no sign
                const uint32_t flip_mask = is_bias ? 0u : 0x80008000u;
                uint32_t h[16];
#pragma unroll
                for (int t = 0; t < 16; t++) {
                    const uint32_t sh = (t == 15) ? word : (word << (15 - t));
                    h[t] = a2 ^ (~sh & flip_mask);
                }
                // natural k order: (0,1), (2,3), ... then (16,17), ...
                uint32_t nat[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    nat[j] = prmt_b32(h[2 * j], h[2 * j + 1], 0x5410u);
                    nat[j + 8] = prmt_b32(h[2 * j], h[2 * j + 1], 0x7632u);
                }
                unsigned char* dst = smem + s * kTcAStageBytes + row_off;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int chunk = (c0 + c) ^ (row & 7);
                    *reinterpret_cast<uint4*>(dst + chunk * 16) = make_uint4(nat[4 * c], nat[4 * c + 1], nat[4 * c + 2], nat[4 * c + 3]);
                }
                fence_proxy_async_smem();                  // make the generic-proxy stores visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull + 8 * s);
            }
        }
    } else if (warp == kTcExpWarps) {
        // ---------------- TMA: activation tiles ----------------
        if (lane == 0) {
            tma_prefetch_descriptor(&tmX);
            for (int i = 0; i < nst; i++) {
                const int s = i % kTcStages;
                if (i >= kTcStages) {
                    if (!mbar_wait_bounded(bar_empty + 8 * s, ((i / kTcStages) - 1) & 1)) { timed_out = true; break; }
                }
                const int k = (kt_begin + i / planes) * kTcTileK;     // the same activation tile for every plane of a k tile
                mbar_arrive_expect_tx(bar_bfull + 8 * s, 2 * b_half_bytes);
                tma_load_2d(b_base + s * 2 * kTcBHalfBytesMax, &tmX, k, 0, bar_bfull + 8 * s);
                tma_load_2d(b_base + s * 2 * kTcBHalfBytesMax + kTcBHalfBytesMax, &tmX, k + 64, 0, bar_bfull + 8 * s);
            }
        }
    } else {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16_f32(p.m_pad);
            for (int i = 0; i < nst; i++) {
                const int s = i % kTcStages;
                const uint32_t ph = (i / kTcStages) & 1;
                if (!mbar_wait_bounded(bar_afull + 8 * s, ph) || !mbar_wait_bounded(bar_bfull + 8 * s, ph)) { timed_out = true; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int half = 0; half < 2; half++) {
#pragma unroll
                    for (int k16 = 0; k16 < 4; k16++) {
                        const uint64_t da = umma_desc_k_sw128(a_base + s * kTcAStageBytes + half * (kTcTileN * 128) + k16 * 32);
                        const uint64_t db = umma_desc_k_sw128(b_base + s * 2 * kTcBHalfBytesMax + half * kTcBHalfBytesMax + k16 * 32);
                        umma_f16_ss(tmem_acc, da, db, idesc, (i > 0 || half > 0 || k16 > 0) ? 1u : 0u);
                    }
                }
                umma_commit(bar_empty + 8 * s);            // stage reusable once these MMAs have read it
            }
            umma_commit(bar_acc);                          // accumulator complete
        }
    }
    if (timed_out) atomicExch(p.status, kStatusTcTimeout);

    // ---------------- epilogue: warps 0..3 read the accumulator (TMEM lanes 32 w .. 32 w + 31) ----------------
    if (warp < 4) {
        bool ok = (nst > 0) && mbar_wait_bounded(bar_acc, 0);
        if (!ok && nst > 0) atomicExch(p.status, kStatusTcTimeout);
        tc_fence_after_sync();
        const int n = n0 + warp * 32 + lane;
        const bool split = gridDim.y > 1;
        for (int mc = 0; mc < p.m_pad; mc += 16) {
            uint32_t r[16];
            if (ok) {
                tmem_ld_x16(tmem_acc + ((uint32_t)(warp * 32) << 16) + (uint32_t)mc, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) r[j] = 0u;
            }
            if (n < N) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int mrow = mc + j;
                    if (mrow < p.m) {
                        const float v = __uint_as_float(r[j]);
                        if (split) {
                            atomicAdd(p.partial + (size_t)mrow * rowN + n, v);
                        } else {
                            if (p.y32) p.y32[(size_t)mrow * rowN + n] = v;
                            if (p.y16) p.y16[(size_t)mrow * rowN + n] = __float2half_rn(v);
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
        tmem_dealloc(tmem_acc, (uint32_t)p.tmem_cols);
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
