// Batched BCQ matmul (2 <= m <= 128 rows per launch) on the 5th-generation tensor cores, sm_100a.
//
// Replaces the reference's batched path, which writes a dense fp16 copy of the whole weight to a
// global scratch buffer and calls cuBLAS on it (lutGEMM/src/kernels.cu:73-79,
// lutGEMM/src/cuda/kernels/dequant_fp16.hpp:54-107, lutGEMM/src/cuda/kernels/cublas.h:47-55).  Here the
// dense values exist only inside the SM, in TENSOR MEMORY:
//
//   CTA = 256 output columns x a k-range, walked in steps of 128 k.
//   One lane streams, per step, the packed words of all planes ([4 words][q][256 columns], one tiled TMA
//   load), their scales ([groups][q][256]) and, if present, q_bias into a deep shared-memory ring (the
//   ring is what is in flight from HBM), and the matching activation tiles x[m_pad][128 k] (128-byte
//   swizzle) into a second ring.
//   For up to 64 rows two warps permute every landed activation tile in place (inside each 32-k block, positions
//   (2t, 2t + 1) take activations (t, t + 16): the order in which one shift of a packed word leaves two sign bits in
//   a register); beyond 64 rows the kernel is MMA-bound and the expansion un-permutes its registers instead.
//   16 expansion warps turn ONE bit plane of a step at a time into the dense fp16 operand
//   A_b[n][k] = +-alpha_b (sign applied by XOR-ing the fp16 sign bits of two weights at a time: every
//   operand value is exact; q_bias is one more, unsigned, plane) and write it with tcgen05.st straight
//   into tensor memory: thread = output column = TMEM lane, 64 columns of packed fp16 pairs per 128 k.
//   Nothing of the expanded operand touches shared memory, whose bandwidth was what limited the
//   earlier shared-memory-operand version of this kernel (64 KB written and 96 KB read per plane and step).
//   Six lanes issue tcgen05.mma.kind::f16 with the A operand in tensor memory and the activations as the
//   shared-memory B operand: M = 128 output columns, N = m_pad rows (16..128), K = 16 per instruction,
//   two column halves, all planes accumulating into the same fp32 accumulators (TMEM lane = output column,
//   TMEM column = activation row).  tcgen05.commit releases the operand stage / the activation slot and
//   finally hands the accumulators to the 16 warps, which read them with tcgen05.ld (a warp's lanes are
//   32 consecutive output columns of one row: coalesced) and either store fp16/fp32 or, with split-k, add
//   fp32 reductions in L2 into a workspace that the last CTA of the column tile converts.
//
// Tensor memory (512 columns): accumulators first (half h at columns d_stride * h, d_stride = 64 for up to 64
// rows, else 128), then the operand stages of 128 columns each (half h at + 64 h): three stages for up to 64
// rows, two beyond.
//
// q_bias is honoured for every m (the reference drops it for m > 1).  All mbarrier waits are bounded; a
// wait that runs out sets the status word, and the CTA still frees its tensor memory before leaving.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_async.cuh"

namespace lg {

constexpr int kTcTileN = 256;                 // output columns per CTA: two MMA halves of 128
constexpr int kTcStepK = 128;                 // k per pipeline step
constexpr int kTcStepWords = kTcStepK / 32;   // 4 packed words
constexpr int kTcExpWarps = 16;
constexpr int kTcMaxAStages = 3;             // operand stages in tensor memory (3 for up to 64 rows, else 2)
// Six MMA-issuing warps (lane 0 of warps 0..5 issues): warp w takes column half w & 1 of the operand stages
// t with t mod (number of stages) == w >> 1.  Clock stamps showed a single issuing lane spending most of every stage
// between its own instructions (a handful of mbarrier / tcgen05 instructions taking several hundred cycles while
// the expansion warps' tcgen05.st traffic runs on the same SM sub-partition); several lanes on different
// sub-partitions overlap those waits.  The lanes of a column half accumulate into the same accumulator, which the
// expansion warps zero beforehand; the sums commute.
constexpr int kTcMmaWarps = 2 * kTcMaxAStages, kTcTmaWarp = kTcMmaWarps, kTcPermWarp = kTcMmaWarps + 1, kTcPermWarps = 2,
              kTcFirstExpWarp = kTcPermWarp + kTcPermWarps;
constexpr int kTcThreads = (kTcFirstExpWarp + kTcExpWarps) * 32;       // 6 + 1 + 2 + 16 warps = 800
constexpr uint32_t kTcTmemCols = 512;
constexpr uint32_t kTcDCol = 0;
constexpr int kTcMaxSlots = 8;
constexpr int kTcBarBytes = 512;
constexpr int kTcXBudget = 96 * 1024;         // activation ring
constexpr int kTcSmemTotal = 216 * 1024;      // both rings + barriers; also keeps the kernel at one CTA per SM

enum { kStatusTcTimeout = 3 };

// Shared-memory plan of one launch (computed on the host, passed by value).
struct TcLayout {
    int m_pad;          // activation rows rounded up to 16 (the MMA's N)
    int a_rows;         // scale groups per 128-k step: max(1, 128 / g)
    int w_packed_bytes, w_alpha_bytes, w_bias_bytes, w_slot_bytes, w_slots;
    int x_sub_bytes, x_slot_bytes, x_slots;
    int x_off, w_off, bar_off, smem_bytes;
    int d_stride;       // TMEM columns between the accumulators of the two column halves: 64 (m_pad <= 64) or 128
    int a_stages;       // operand stages in TMEM: 3 when the accumulators leave room for them, else 2
    int permute_x;      // 1: activations are permuted in shared memory and the operand is written in shift order (m_pad <= 64,
                        // where the expansion's instruction count is the limit); 0: the expansion un-permutes its registers
};
inline TcLayout tc_layout(int q, bool bias, int g, int m) {
    TcLayout L;
    L.m_pad = (m + 15) / 16 * 16;
    L.a_rows = g >= kTcStepK ? 1 : kTcStepK / g;
    L.w_packed_bytes = kTcStepWords * q * kTcTileN * 4;
    L.w_alpha_bytes = L.a_rows * q * kTcTileN * 2;
    L.w_bias_bytes = bias ? L.a_rows * kTcTileN * 2 : 0;
    L.w_slot_bytes = L.w_packed_bytes + L.w_alpha_bytes + L.w_bias_bytes;     // every part a multiple of 512 B
    L.x_sub_bytes = L.m_pad * 128;                                            // [m_pad rows][64 k] fp16
    L.x_slot_bytes = 2 * L.x_sub_bytes;
    L.x_slots = kTcXBudget / L.x_slot_bytes;
    if (L.x_slots > kTcMaxSlots) L.x_slots = kTcMaxSlots;
    L.x_off = 0;
    L.w_off = L.x_slots * L.x_slot_bytes;                                     // multiple of 1024
    L.w_slots = (kTcSmemTotal - kTcBarBytes - L.w_off) / L.w_slot_bytes;
    if (L.w_slots > kTcMaxSlots) L.w_slots = kTcMaxSlots;
    L.bar_off = kTcSmemTotal - kTcBarBytes;
    L.smem_bytes = kTcSmemTotal;
    // The epilogue turns accumulator blocks through a per-warp scratch of 16 x 33 floats that starts at x_off and, for
    // m_pad == 16 (activation ring 32 KB), reaches 1 KB into the first weight slot.  That is safe only because both rings
    // are idle by then (the accumulators are complete when every load has been consumed) and the kernel walks one
    // output tile per launch; the plan is refused if the scratch would ever leave the two rings.
    if (kTcExpWarps * 16 * 33 * 4 > L.x_slots * L.x_slot_bytes + L.w_slots * L.w_slot_bytes) L.w_slots = 0;
    L.d_stride = L.m_pad <= 64 ? 64 : 128;
    L.a_stages = L.m_pad <= 64 ? 3 : 2;                    // 2 * d_stride + 128 * a_stages = 512 columns
    L.permute_x = L.m_pad <= 64 ? 1 : 0;
    return L;
}

struct TcParams {
    float* partial;          // [m][N] fp32, zero between launches (split-k only)
    unsigned* counters;      // [gridDim.x], zero between launches
    int* status;
    __half* y16;             // [m][N] or nullptr
    float* y32;              // [m][N] or nullptr
    int N, K, g;
    int m;                   // rows (<= 128)
    int steps_per_cta;       // 128-k steps per CTA (split-k along gridDim.y)
    TcLayout L;
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
// D[tmem] (+)= A[tmem] * B[smem], fp16 inputs, fp32 accumulation; issued by one thread.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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
// 32 lanes x 16 columns: lane i of the warp's TMEM quarter, columns taddr .. taddr + 15.
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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
// Instruction descriptor for kind::f16: fp16 x fp16 -> fp32, K-major operands, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_f16_f32(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// One 16-row x 32-column accumulator block of a warp (lane = output column, v[j] = activation row row0 + j), turned through
// a per-warp scratch of 16 x 33 floats (rows padded: no bank conflicts either way) so that a lane holds 4 consecutive
// columns of one row: vector reductions / 128-bit stores, a quarter of the L2 transactions of scalar ones.
// N % 8 == 0 on this path: whole groups of four columns.
__device__ __forceinline__ void tc_store_block(float* scratch, const uint32_t (&v16)[16], int lane, int row0, int ncol0, int m,
                                               int N, bool split, float* partial, __half* y16, float* y32) {
#pragma unroll
    for (int jj = 0; jj < 16; jj++) scratch[jj * 33 + lane] = __uint_as_float(v16[jj]);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = (lane >> 3) + 4 * i, col4 = (lane & 7) * 4;
        const float* src = scratch + row * 33 + col4;
        const float4 v = make_float4(src[0], src[1], src[2], src[3]);
        const int mrow = row0 + row, n = ncol0 + col4;
        if (mrow < m && n < N) {
            const size_t o = (size_t)mrow * (size_t)N + n;
            if (split) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(partial + o), "f"(v.x), "f"(v.y),
                             "f"(v.z), "f"(v.w) : "memory");
            } else {
                if (y32) *reinterpret_cast<float4*>(y32 + o) = v;
                if (y16) {
                    __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                    uint2 h2;
                    h2.x = *reinterpret_cast<uint32_t*>(&lo);
                    h2.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(y16 + o) = h2;
                }
            }
        }
    }
    __syncwarp();
}

// Split-k finish, called by every thread of the CTA after its reductions (and a __threadfence + __syncthreads): the last
// CTA of this column tile converts the reduced sums and zeroes the workspace.
__device__ __forceinline__ void tc_splitk_finish(float* partial, unsigned* counters, __half* y16, float* y32, int m, int N,
                                                 int n0, int* s_flag, int nthreads) {
    const int tid = threadIdx.x;
    if (tid == 0) {
        const unsigned prev = atomicAdd(counters + blockIdx.x, 1u);
        *s_flag = (prev == gridDim.y - 1u);
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    // whole float4 groups, several loads in flight per thread
    const int nvec = m * (kTcTileN / 4);
    for (int base = tid; base < nvec; base += 4 * nthreads) {
        float4 v[4];
        size_t off[4];
        bool live[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int idx = base + u * nthreads;
            const int mrow = idx / (kTcTileN / 4), n = n0 + 4 * (idx % (kTcTileN / 4));
            live[u] = idx < nvec && n < N;
            off[u] = (size_t)mrow * (size_t)N + n;
            if (live[u]) v[u] = __ldcg(reinterpret_cast<const float4*>(partial + off[u]));
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (!live[u]) continue;
            __stcg(reinterpret_cast<float4*>(partial + off[u]), make_float4(0.f, 0.f, 0.f, 0.f));
            if (y32) *reinterpret_cast<float4*>(y32 + off[u]) = v[u];
            if (y16) {
                __half2 lo = __floats2half2_rn(v[u].x, v[u].y), hi = __floats2half2_rn(v[u].z, v[u].w);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&lo);
                o.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(y16 + off[u]) = o;
            }
        }
    }
    if (tid == 0) counters[blockIdx.x] = 0u;
}

// Q: number of bit planes; BIAS: container has q_bias.
//  tmX: 2-D map {K, m} of fp16, box {64, m_pad}, 128-byte swizzle;
//  tmW: 3-D map {N, q, K/32} of uint32, box {256, q, 4};  tmA: 3-D map {N, q, G} of fp16, box {256, q, a_rows};
//  tmQ: 2-D map {N, G} of fp16, box {256, a_rows} (read only when BIAS).
template <int Q, bool BIAS>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const TcLayout& L = p.L;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar0 = smem_base + L.bar_off;
    const uint32_t bar_wfull = bar0;                              // kTcMaxSlots each
    const uint32_t bar_wempty = bar0 + 8 * kTcMaxSlots;
    const uint32_t bar_xfull = bar0 + 16 * kTcMaxSlots;
    const uint32_t bar_xempty = bar0 + 24 * kTcMaxSlots;
    const uint32_t bar_xready = bar0 + 32 * kTcMaxSlots;          // activation slot permuted, kTcMaxSlots
    const uint32_t bar_afull = bar0 + 40 * kTcMaxSlots;           // kTcMaxAStages
    const uint32_t bar_aempty = bar_afull + 8 * kTcMaxAStages;
    const uint32_t bar_acc = bar_aempty + 8 * kTcMaxAStages;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L.bar_off + 40 * kTcMaxSlots + 16 * kTcMaxAStages + 16);
    const uint32_t a_col0 = 2u * (uint32_t)L.d_stride;             // first operand column in tensor memory
    const int nA = L.a_stages;
    int* s_flag = reinterpret_cast<int*>(s_tmem + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N;
    const int n0 = blockIdx.x * kTcTileN;
    const int steps_total = (p.K + kTcStepK - 1) / kTcStepK;
    const int step_begin = blockIdx.y * p.steps_per_cta;
    const int nsteps = max(0, min(steps_total, step_begin + p.steps_per_cta) - step_begin);
    constexpr int P = Q + (BIAS ? 1 : 0);                  // q_bias rides as one more plane
    const int m_pad = L.m_pad;

    if (tid == 0) {
        for (int s = 0; s < kTcMaxSlots; s++) {
            mbar_init(bar_wfull + 8 * s, 1);
            mbar_init(bar_wempty + 8 * s, kTcExpWarps);
            mbar_init(bar_xfull + 8 * s, 1);
            mbar_init(bar_xempty + 8 * s, kTcMmaWarps);
            mbar_init(bar_xready + 8 * s, kTcPermWarps);
        }
        for (int s = 0; s < kTcMaxAStages; s++) {
            mbar_init(bar_afull + 8 * s, kTcExpWarps);
            mbar_init(bar_aempty + 8 * s, 2);                      // the two column halves of that stage parity
        }
        mbar_init(bar_acc, kTcMmaWarps);
        mbar_fence_init();
    }
    if (warp == 0) {                        // the first MMA warp owns the tensor-memory allocation
        tmem_alloc(smem_u32(s_tmem), kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *s_tmem;
    bool timed_out = false;
    // Launched with programmatic stream serialization: the packed planes and scales are never written by a kernel, so
    // their stream and the expansion into tensor memory start while the previous kernel of the stream drains; the
    // activations, the split-k workspace and the outputs are touched only after griddepcontrol.wait.
    pdl_launch_dependents();

    if (warp >= kTcFirstExpWarp) {
        // ---------------- expansion: packed planes (shared memory) -> dense fp16 operand (tensor memory) ----------------
        const int lq = warp & 3;                          // TMEM lane quarter this warp may access (hardware: warp id mod 4)
        const int gi = (warp - kTcFirstExpWarp) >> 2;     // 0..3, distinct among the four warps of a lane quarter
        const int hN = gi & 1;                            // column half (which accumulator / operand block)
        const int hK = gi >> 1;                           // which two of the step's four packed words
        const int col = hN * 128 + lq * 32 + lane;        // column of the tile; TMEM lane = col & 127
        int arow[2];
#pragma unroll
        for (int u = 0; u < 2; u++) arow[u] = (p.g >= kTcStepK) ? 0 : (32 * (2 * hK + u)) / p.g;
        const uint32_t t_lane = tmem_base + ((uint32_t)(lq * 32) << 16);
        const uint32_t t_col0 = a_col0 + (uint32_t)hN * 64u + (uint32_t)hK * 32u;
        if (hK == 0) {
            // zero this lane quarter of accumulator hN: every MMA accumulates
            uint32_t z[16];
#pragma unroll
            for (int i = 0; i < 16; i++) z[i] = 0u;
            for (int c = 0; c < m_pad; c += 16) tmem_st_x16(t_lane + kTcDCol + (uint32_t)(hN * L.d_stride + c), z);
            tmem_st_wait();
        }
        int ws = 0, wround = 0, st = 0, sround = 0;
        for (int j = 0; j < nsteps && !timed_out; j++) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_wfull + 8 * ws, wround & 1))) { timed_out = true; break; }
            const unsigned char* slot = smem + L.w_off + ws * L.w_slot_bytes;
            const uint32_t* wsm = reinterpret_cast<const uint32_t*>(slot) + col;
            const unsigned short* a_sm = reinterpret_cast<const unsigned short*>(slot + L.w_packed_bytes) + col;
            const unsigned short* qsm = reinterpret_cast<const unsigned short*>(slot + L.w_packed_bytes + L.w_alpha_bytes) + col;
            // not unrolled: the loop body is ~2 KB of straight-line code, and instruction fetch is shared with the
            // MMA-issuing lanes, whose every loop iteration otherwise waits hundreds of cycles for its instructions
#pragma unroll 1
            for (int b = 0; b < P; b++) {
                uint32_t w[2], a[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    if (b < Q) {
                        w[u] = wsm[((2 * hK + u) * Q + b) * kTcTileN];
                        a[u] = (uint32_t)a_sm[(arow[u] * Q + b) * kTcTileN] * 0x00010001u;
                    } else {
                        w[u] = 0u;
                        a[u] = (uint32_t)qsm[arow[u] * kTcTileN] * 0x00010001u;
                    }
                }
                if (sround > 0) {
                    if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_aempty + 8 * st, (sround - 1) & 1))) { timed_out = true; break; }
                    tc_fence_after_sync();
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    // two weights per register: element t (low half) and t + 16 (high half) of the packed word: register t
                    // goes to TMEM column t, i.e. k-positions (2t, 2t + 1) of the block, which is where the permute warp
                    // has put activations t and t + 16.  Bit set -> +alpha, bit clear -> -alpha (sign bit flipped where
                    // the bit is 0); q_bias plane: no sign
                    uint32_t nat[16];
                    if (b < Q) {
#pragma unroll
                        for (int t = 0; t < 16; t++) {
                            const uint32_t sh = (t == 15) ? w[u] : (w[u] << (15 - t));
                            nat[t] = a[u] ^ (~sh & 0x80008000u);
                        }
                        if (!L.permute_x) {
                            // activations in natural order: pairs (0,1), (2,3), ... then (16,17), ...
                            uint32_t h[16];
#pragma unroll
                            for (int t = 0; t < 16; t++) h[t] = nat[t];
#pragma unroll
                            for (int jj = 0; jj < 8; jj++) {
                                nat[jj] = prmt_b32(h[2 * jj], h[2 * jj + 1], 0x5410u);
                                nat[jj + 8] = prmt_b32(h[2 * jj], h[2 * jj + 1], 0x7632u);
                            }
                        }
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 16; jj++) nat[jj] = a[u];
                    }
                    tmem_st_x16(t_lane + t_col0 + (uint32_t)st * 128u + (uint32_t)u * 16u, nat);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull + 8 * st);
                if (++st == nA) { st = 0; sround++; }
            }
            __syncwarp();
            if (lane == 0 && !timed_out) mbar_arrive(bar_wempty + 8 * ws);     // the step's packed words have been read
            if (++ws == L.w_slots) { ws = 0; wround++; }
        }
    } else if (warp == kTcTmaWarp) {
        // ---------------- TMA: packed planes + scales (+ q_bias) and activation tiles, as far ahead as the rings allow --------
        // The whole warp walks the loop and lane 0 issues: a lone lane looping while its 31 siblings already sit at
        // the CTA barrier below is scheduled only now and then (measured: hundreds of cycles for a handful of
        // instructions).
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
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_wempty + 8 * ws, (wround - 1) & 1))) { timed_out = true; break; }
            }
            if (lane == 0) {
                const int grp0 = (step * kTcStepK) / p.g;
                const uint32_t wdst = smem_base + L.w_off + ws * L.w_slot_bytes;
                mbar_arrive_expect_tx(bar_wfull + 8 * ws, (uint32_t)L.w_slot_bytes);    // out-of-range parts are zero-filled and counted
                tma_load_3d(wdst, &tmW, n0, 0, step * kTcStepWords, bar_wfull + 8 * ws);
                tma_load_3d(wdst + L.w_packed_bytes, &tmA, n0, 0, grp0, bar_wfull + 8 * ws);
                if (BIAS) tma_load_2d(wdst + L.w_packed_bytes + L.w_alpha_bytes, &tmQ, n0, grp0, bar_wfull + 8 * ws);
            }
            if (++ws == L.w_slots) { ws = 0; wround++; }

            if (j == 0) pdl_wait_prior_grids();                      // the activations may come from the previous kernel
            if (xround > 0) {
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_xempty + 8 * xs, (xround - 1) & 1))) { timed_out = true; break; }
            }
            if (lane == 0) {
                const uint32_t xdst = smem_base + L.x_off + xs * L.x_slot_bytes;
                mbar_arrive_expect_tx(bar_xfull + 8 * xs, (uint32_t)L.x_slot_bytes);
                tma_load_2d(xdst, &tmX, step * kTcStepK, 0, bar_xfull + 8 * xs);
                tma_load_2d(xdst + L.x_sub_bytes, &tmX, step * kTcStepK + 64, 0, bar_xfull + 8 * xs);
            }
            if (++xs == L.x_slots) { xs = 0; xround++; }
            __syncwarp();
        }
    } else if (warp >= kTcPermWarp) {                      // the permute warps; idle when the layout does not ask for them
        // ---------------- activation permute: inside every 32-k block, positions (2t, 2t + 1) <- activations (t, t + 16) --------
        // (the order in which the expansion's shift leaves two weights in a register; permuting the few activations
        // once per step costs far less than un-permuting every expanded operand register)
        int xs = 0, xround = 0;
        for (int j = 0; j < (L.permute_x ? nsteps : 0); j++) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_xfull + 8 * xs, xround & 1))) { timed_out = true; break; }
            unsigned char* slot = smem + L.x_off + xs * L.x_slot_bytes;
            const int tasks = 4 * p.m;                               // (sub-tile, row < m, 32-k block); rows >= m are zero
            for (int tk = (warp - kTcPermWarp) * 32 + lane; tk < tasks; tk += 32 * kTcPermWarps) {
                const int blk = tk & 1, sub = (tk >> 1) & 1, r = tk >> 2;
                unsigned char* row = slot + sub * L.x_sub_bytes + (r >> 3) * 1024 + (r & 7) * 128;
                uint4 in[4];
#pragma unroll
                for (int i = 0; i < 4; i++) in[i] = *reinterpret_cast<const uint4*>(row + (((4 * blk + i) ^ (r & 7)) << 4));
                const uint32_t v[16] = {in[0].x, in[0].y, in[0].z, in[0].w, in[1].x, in[1].y, in[1].z, in[1].w,
                                        in[2].x, in[2].y, in[2].z, in[2].w, in[3].x, in[3].y, in[3].z, in[3].w};
                uint32_t o[16];
#pragma unroll
                for (int t = 0; t < 16; t++) o[t] = prmt_b32(v[t >> 1], v[(t >> 1) + 8], (t & 1) ? 0x7632u : 0x5410u);
#pragma unroll
                for (int i = 0; i < 4; i++)
                    *reinterpret_cast<uint4*>(row + (((4 * blk + i) ^ (r & 7)) << 4)) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
            fence_proxy_async_smem();                                // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_xready + 8 * xs);
            if (++xs == L.x_slots) { xs = 0; xround++; }
        }
    } else if (warp < kTcMmaWarps) {
        // ---------------- MMA issue: warp w takes column half w & 1 of the stages t with t mod nA == w >> 1 ----------------
        // (whole warp in the loop, lane 0 issues; see the TMA warp)
        const int hN = warp & 1, par = warp >> 1;          // par >= nA: nothing to issue, but the commits below still arrive
        const uint32_t idesc = umma_idesc_f16_f32(m_pad);
        const uint64_t dx0 = umma_desc_k_sw128(smem_base + L.x_off);
        const uint32_t d_t = tmem_base + kTcDCol + (uint32_t)(hN * L.d_stride);
        const uint32_t a_t0 = tmem_base + a_col0 + (uint32_t)par * 128u + (uint32_t)hN * 64u;    // this warp's operand stage
        int t = 0, tmod = 0;                           // running stage index (step * P + plane) and t mod nA
        int sround = 0, xs = 0, xround = 0;
        for (int j = 0; j < nsteps && !timed_out; j++) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded((L.permute_x ? bar_xready : bar_xfull) + 8 * xs, xround & 1))) { timed_out = true; break; }
#pragma unroll 1
            for (int b = 0; b < P; b++, t++, tmod = (tmod + 1 == nA) ? 0 : tmod + 1) {
                if (tmod != par) continue;
                // The expansion warps complete their tcgen05.st with tcgen05.wait::st before they arrive, so the
                // operand is in tensor memory once this wait returns.
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_afull + 8 * par, sround & 1))) { timed_out = true; break; }
                tc_fence_after_sync();
                if (lane == 0) {
#pragma unroll
                    for (int k16 = 0; k16 < 8; k16++) {
                        // B operand: activations [m_pad rows][16 k] of sub-tile k16 / 4 (start address in 16-byte units)
                        const uint64_t dx = dx0 + (uint64_t)((xs * L.x_slot_bytes + (k16 >> 2) * L.x_sub_bytes + (k16 & 3) * 32) >> 4);
                        umma_f16_ts(d_t, a_t0 + (uint32_t)k16 * 8u, dx, idesc, 1u);
                    }
                    umma_commit(bar_aempty + 8 * par);     // operand stage reusable once both halves' MMAs have read it
                }
                __syncwarp();
                sround++;
            }
            if (timed_out) break;
            if (lane == 0) umma_commit(bar_xempty + 8 * xs);   // this warp is done with the step's activation slot
            __syncwarp();
            if (++xs == L.x_slots) { xs = 0; xround++; }
        }
        if (lane == 0) umma_commit(bar_acc);               // this warp's share of the accumulators is complete
        __syncwarp();
    }
    pdl_wait_prior_grids();                  // before any store to global memory (returns at once if already passed)
    if (timed_out) atomicExch(p.status, kStatusTcTimeout);

    // ---------------- epilogue: TMEM lane = output column, TMEM column = activation row ----------------
    const bool split = gridDim.y > 1;
    if (warp >= kTcFirstExpWarp && nsteps > 0) {
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_acc, 0));
        if (!ok) atomicExch(p.status, kStatusTcTimeout);
        tc_fence_after_sync();
        const int lq = warp & 3, gi = (warp - kTcFirstExpWarp) >> 2, hN = gi & 1, hK = gi >> 1;
        const uint32_t t_src = tmem_base + ((uint32_t)(lq * 32) << 16) + kTcDCol + (uint32_t)(hN * L.d_stride);
        // A tcgen05.ld leaves lane = output column, register = activation row.  Each 16 x 32 block is turned through a
        // per-warp scratch in shared memory (the activation ring and, for 16 rows, the first KB of the weight ring: both
        // idle once the accumulators are complete, see tc_layout; rows padded to
        // 33 floats: no bank conflicts either way) so that a lane holds 4 consecutive columns of one row: vector
        // reductions / 128-bit stores, a quarter of the L2 transactions of scalar ones.
        float* scratch = reinterpret_cast<float*>(smem + L.x_off) + (warp - kTcFirstExpWarp) * (16 * 33);
        const int ncol0 = n0 + hN * 128 + lq * 32;
        for (int c = hK; 16 * c < p.m && ok; c += 2) {     // 16 activation rows per tcgen05.ld; warp-uniform
            uint32_t r[16];
            tmem_ld_x16(t_src + 16u * (uint32_t)c, r);
            tmem_ld_wait();
            tc_store_block(scratch, r, lane, 16 * c, ncol0, p.m, N, split, p.partial, p.y16, p.y32);
        }
        tc_fence_before_sync();
    }
    __threadfence();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
    if (!split) return;

    tc_splitk_finish(p.partial, p.counters, p.y16, p.y32, p.m, N, n0, s_flag, kTcThreads);
}

}  // namespace lg
