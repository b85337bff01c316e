// LUT matvec for BCQ weights (m = 1), sm_100a: TMA fed, one CTA per SM.
//
// Replaces _nqmv / _nqmv_bias of the reference (lutGEMM/src/cuda/kernels/mv_fp16.hpp:25-97,
// lutGEMM/src/cuda/kernels/mv_fp16_bias.hpp:24-118).  Same mathematics — a 2^8-entry table of signed
// partial sums per 8 activations, one lookup per packed weight byte — mapped to the machine as follows.
//
//  CTA = (column tile) x (512-k slab).  544 threads: 16 consumer warps + 1 producer warp.
//
//  Table (64 KB).  lut[idx][slot] fp32, TRANSPOSED: the shared-memory bank is chosen by the slot (the
//  8-activation chunk), not by the random weight byte.  The slab's 16 packed k-words are numbered
//  kw = 4 G + jp + 2 u (G = 0..3: a run of four words = 128 k; jp, u = 0..1); chunk (kw, byte beta)
//  lives in slot 32 u + 8 G + 4 jp + beta.  In every lookup instruction the 32 lanes of a warp hold
//  the 8 different (G, jp) and, through a per-lane byte rotation, 4 different beta: 32 different
//  banks, so lookups never conflict, whatever the weights are.  One PRMT turns a packed byte into the
//  shared-memory offset (idx << 8 | slot * 4): a lookup is PRMT + LDS + add.
//
//  Weights and scales.  One producer lane issues, per stage, one tiled TMA load of the box
//  [16 k-words][1 plane][256 columns] of the packed planes (16 KB, dense rows of 1 KB) and one of the
//  box [groups of the slab][1 plane][256 columns] of alpha; completion is counted on an mbarrier, no
//  multicast.  Up to 8 stages (>= 100 KB) are in flight, which is what it takes to keep HBM busy from
//  one CTA per SM; a consumer warp releases a stage as soon as its words are in registers.  Lane
//  (c8 = lane & 7, rr = lane >> 3) of warp (cb = warp & 7, h = warp >> 3) reads columns
//  32 cb + 4 c8 .. +3 of rows 4 rr + ((c8 & 1) ^ h) + 2 u: a quarter warp reads eight consecutive
//  16-byte chunks, which is conflict free on dense rows.
//
//  Scales.  A lane's two words of a stage lie in one 128-k run, so with group size % 128 == 0 they
//  share one alpha: 8 lookups are summed, then one FMA (WPG = 2); otherwise one FMA per word.
//
//  Result.  fp32 throughout; the 4 lanes that share columns are added with shuffles, the two warp
//  halves are added through shared memory.  Across slabs either (default) vector fp32 reductions in
//  L2 into one zeroed workspace row, or (ordered mode) one partial row per slab added in slab order
//  by the last CTA of the column tile, which makes results bit-reproducible run to run.  The last
//  CTA rounds to fp16 once and leaves the workspace zeroed: no memset launch.
//
//  Launch.  The kernel is launched with programmatic stream serialization: its weight stream starts
//  while the previous kernel in the stream drains; everything a predecessor may have produced (the
//  activations) or may still use (workspace, output) is touched only after griddepcontrol.wait.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_async.cuh"

namespace lg {

constexpr int kSlab2 = 512;                                 // k per CTA
constexpr int kSlabWords = kSlab2 / 32;                     // 16 packed k-words per slab
constexpr int kStageCols = 256;                             // columns per stage
constexpr int kConsWarps = 16;
constexpr int kGemv2Threads = (kConsWarps + 1) * 32;        // 544
constexpr int kMaxStages = 8;
constexpr int kRowPitch = kStageCols * 4;                   // 1024: dense TMA box rows
constexpr int kWStageBytes = kSlabWords * kRowPitch;        // 16384
constexpr int kARowPitch = kStageCols * 2;                  // 512: one alpha group row of the box
constexpr int kLut2Bytes = 65536;
constexpr int kSmemLimit = 232448;                          // 227 KB opt-in maximum per CTA
// shared memory: table | half-warp exchange (1 KB) | barriers | stages (weight box + alpha box each)
constexpr int kXchgOff = kLut2Bytes;
constexpr int kBarOff = kXchgOff + 1024;
constexpr int kStage0Off = kBarOff + 256;
__host__ __device__ constexpr int gemv2_stage_bytes(int a_rows) { return kWStageBytes + a_rows * kARowPitch; }
__host__ __device__ constexpr int gemv2_num_stages(int a_rows) {
    return (kSmemLimit - kStage0Off) / gemv2_stage_bytes(a_rows) < kMaxStages
               ? (kSmemLimit - kStage0Off) / gemv2_stage_bytes(a_rows) : kMaxStages;
}
__host__ __device__ constexpr int gemv2_smem_bytes(int a_rows) {
    return kStage0Off + gemv2_num_stages(a_rows) * gemv2_stage_bytes(a_rows);
}

enum { kStatusOk = 0, kStatusProducerTimeout = 1, kStatusConsumerTimeout = 2, kStatusPeerTimeout = 4, kStatusLayout = 8 };

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for a flag that other GPUs increment (about a quarter of a second at most).
__device__ __forceinline__ bool wait_flag_bounded(const unsigned* flag, unsigned target) {
    for (unsigned it = 0; it < (1u << 18); it++) {
        if (ld_acquire_sys(flag) >= target) return true;
        if (it > 16) __nanosleep(200);
    }
    return false;
}

// Tensor-parallel links of one matvec (all zero / null for an ordinary call).
//  Input side:  x_mode 0: p.x is ready when the previous kernel of the stream has finished;
//               x_mode 1: p.x is an fp16 vector in THIS GPU's memory that every rank fills by peer stores
//                         (all-gather); wait until flag_in reaches flag_target;
//               x_mode 2: the activations are the sum, in rank order, of `world` fp32 rows
//                         x_slots[r * x_slot_stride + x_off + k] written by the ranks (all-reduce), rounded to
//                         fp16 once; wait as above.
//  Output side: out_mode 0: p.y16 / p.y32 in local memory;
//               out_mode 1: the fp16 result goes to out16[r] + out_off on every rank r (peer-mapped pointers);
//               out_mode 2: the fp32 result goes to out32[r] (this rank's slot on rank r);
//               then flag_out[r] is incremented once per finished column tile, release at system scope.
//  The last CTA to pass the input wait resets flag_in, so the same words serve the next step (CUDA graphs
//  replay constant parameters).  All waits are bounded.
struct TpLink {
    int x_mode, out_mode, world, out_off;
    const float* x_slots;
    int x_slot_stride, x_off;
    unsigned* flag_in;
    unsigned flag_target;
    unsigned* done_counter;
    __half* out16[8];
    float* out32[8];
    unsigned* flag_out[8];
};

struct Gemv2Params {
    const uint32_t* bW;      // [K/32][q][N]
    const __half* alpha;     // [G][q][N]
    const __half* q_bias;    // [G][N] or nullptr
    const __half* x;         // [K]
    float* partial;          // split-k workspace: [nslabs][N] (ordered) or one zeroed row [N] (reductions)
    unsigned* counters;      // [gridDim.x], zero between launches
    int* status;             // device word; set non-zero if a bounded wait ran out
    __half* y16;             // [N] or nullptr
    float* y32;              // [N] or nullptr
    int N, K, q, g;
    int n_tile;              // columns per CTA, multiple of kStageCols
    int nslabs;              // gridDim.y
    int a_rows;              // alpha groups per slab (rows of the alpha box): max(1, 512 / g)
    int ordered;             // 1: slabs are added in slab order (bit-reproducible); 0: fp32 reductions in L2
    TpLink tp;
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
// Vector fp32 reduction into global memory (performed in L2, no return value).
__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start launching / wait for the
// previous one to finish and flush.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Sum of the four table entries selected by the four bytes of one packed word.  IMM is the
// compile-time part of the slot address (which of the lane's two words).
template <int IMM>
__device__ __forceinline__ float2 lookup_word(const unsigned char* lut, uint32_t word, uint32_t cs,
                                              const uint32_t (&sel)[4]) {
    const float l0 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[0]) + IMM);
    const float l1 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[1]) + IMM);
    const float l2 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[2]) + IMM);
    const float l3 = *reinterpret_cast<const float*>(lut + prmt_b32(word, cs, sel[3]) + IMM);
    return add_f32x2(make_float2(l0, l1), make_float2(l2, l3));
}

// Table for the 64 chunks of one slab.  Consumer thread t owns slot (t & 63) and the 32 entries
// idx in [32 (t >> 6), +32), walked in Gray-code order (one add per entry).  A warp stores 32
// consecutive slots of one idx row: conflict free.
__device__ __forceinline__ int lut_chunk_of(int ctid) {
    const int slot = ctid & 63;
    const int u = slot >> 5, G = (slot >> 3) & 3, jp = (slot >> 2) & 1, beta = slot & 3;
    return 4 * (4 * G + jp + 2 * u) + beta;                   // 8-activation chunk in natural k order
}
// The 8 fp16 activations of this thread's chunk (zero beyond K).
__device__ __forceinline__ uint4 load_x_chunk(const __half* x, int k0, int K, int ctid) {
    const int chunk = lut_chunk_of(ctid);
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (k0 + 8 * chunk < K) raw = __ldcg(reinterpret_cast<const uint4*>(x + k0 + 8 * chunk));
    return raw;
}
__device__ __forceinline__ void build_lut_from(unsigned char* lut, const float (&xv)[8], int ctid) {
    const int slot = ctid & 63, part = ctid >> 6;
    float e = -xv[0] - xv[1] - xv[2] - xv[3] - xv[4];
    e += (part & 1) ? xv[5] : -xv[5];
    e += (part & 2) ? xv[6] : -xv[6];
    e += (part & 4) ? xv[7] : -xv[7];
    unsigned char* base = lut + part * (32 * 256) + slot * 4;
    *reinterpret_cast<float*>(base) = e;
#pragma unroll
    for (int c = 1; c < 32; c++) {
        const int t = (c & 1) ? 0 : (c & 2) ? 1 : (c & 4) ? 2 : (c & 8) ? 3 : 4;   // bit that flips
        const int gcode = c ^ (c >> 1);
        const float two_x = 2.0f * xv[t];
        e = ((gcode >> t) & 1) ? e + two_x : e - two_x;
        *reinterpret_cast<float*>(base + gcode * 256) = e;
    }
}
// The same from the chunk's 8 fp16 values as loaded (16 bytes).
__device__ __forceinline__ void build_lut_from_raw(unsigned char* lut, uint4 raw, int ctid) {
    float xv[8];
    const float2 f0 = half2_bits_to_float2(raw.x), f1 = half2_bits_to_float2(raw.y);
    const float2 f2 = half2_bits_to_float2(raw.z), f3 = half2_bits_to_float2(raw.w);
    xv[0] = f0.x; xv[1] = f0.y; xv[2] = f1.x; xv[3] = f1.y; xv[4] = f2.x; xv[5] = f2.y; xv[6] = f3.x; xv[7] = f3.y;
    build_lut_from(lut, xv, ctid);
}
__device__ __forceinline__ void build_lut2(unsigned char* lut, const __half* x, int k0, int K, int ctid, const TpLink& tp) {
    if (tp.x_mode == 2) {
        // all-reduced input: add the ranks' fp32 rows in rank order, round to fp16 once
        const int chunk = lut_chunk_of(ctid);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (k0 + 8 * chunk < K) {
            for (int r = 0; r < tp.world; r++) {
                const float4* src = reinterpret_cast<const float4*>(tp.x_slots + (size_t)r * tp.x_slot_stride + tp.x_off + k0 + 8 * chunk);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
        }
        float xv[8];
#pragma unroll
        for (int t = 0; t < 8; t++) xv[t] = __half2float(__float2half_rn(acc[t]));
        build_lut_from(lut, xv, ctid);
    } else {
        build_lut_from_raw(lut, load_x_chunk(x, k0, K, ctid), ctid);
    }
}

// Split-k finish shared by the matvec kernels: called by every thread of the CTA after its partial sums are
// out.  The last CTA of the column tile [n_begin, n_end) either adds the slabs in slab order or reads the row
// of L2-reduced sums and zeroes it again for the next launch; one fp16 rounding either way; then the
// tensor-parallel output links, if any.
template <int THREADS>
__device__ __forceinline__ void splitk_finish(const Gemv2Params& p, int tid, int n_begin, int n_end, int* s_flag) {
    const size_t rowN = (size_t)p.N;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(p.counters + blockIdx.x, 1u);
        *s_flag = (prev == (unsigned)p.nslabs - 1u);
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    for (int c = n_begin + 4 * tid; c < n_end; c += 4 * THREADS) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = p.partial + c;
        int sl = 0;
        if (!p.ordered) {
            s = __ldcg(reinterpret_cast<const float4*>(src));
            __stcg(reinterpret_cast<float4*>(p.partial + c), make_float4(0.f, 0.f, 0.f, 0.f));
            sl = p.nslabs;
        }
        for (; sl + 8 <= p.nslabs; sl += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sl + i) * rowN));
#pragma unroll
            for (int i = 0; i < 8; i++) { s.x += v[i].x; s.y += v[i].y; s.z += v[i].z; s.w += v[i].w; }
        }
        for (; sl < p.nslabs; sl++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sl * rowN));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        // Row 0 is also the L2 reduction row of the default mode, which expects to find it zero: leave it so, so
        // that the mode may be switched between calls on one workspace.
        if (p.ordered) __stcg(reinterpret_cast<float4*>(p.partial + c), make_float4(0.f, 0.f, 0.f, 0.f));
        __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        if (p.tp.out_mode == 0) {
            if (p.y32) *reinterpret_cast<float4*>(p.y32 + c) = s;
            if (p.y16) *reinterpret_cast<uint2*>(p.y16 + c) = o;
        } else if (p.tp.out_mode == 1) {
            for (int r = 0; r < p.tp.world; r++) *reinterpret_cast<uint2*>(p.tp.out16[r] + p.tp.out_off + c) = o;   // peer stores
        } else {
            for (int r = 0; r < p.tp.world; r++) *reinterpret_cast<float4*>(p.tp.out32[r] + c) = s;                  // peer stores
        }
    }
    if (p.tp.out_mode != 0) {
        // publish this tile to every rank: data first (system-scope fence by every storing thread), then the flag
        __threadfence_system();
        __syncthreads();
        if (tid < p.tp.world) red_release_sys_add(p.tp.flag_out[tid], 1u);
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;   // ready for the next launch on this stream
}

// WPG: packed words per alpha group among a lane's two words of a stage (2: g % 128 == 0, else 1).
// BIAS: container has q_bias.  tmW: 3-D map {N, q, K/32} of uint32, box {256, 1, 16};
// tmA: 3-D map {N, q, G} of fp16, box {256, 1, a_rows}.
template <int WPG, bool BIAS>
__global__ void __launch_bounds__(kGemv2Threads, 1)
gemv_tma_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                const Gemv2Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* lut = smem;
    const int stage_bytes = gemv2_stage_bytes(p.a_rows);
    const int nstages = gemv2_num_stages(p.a_rows);
    const uint32_t bar_full = smem_u32(smem + kBarOff);          // nstages x 8 B
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    int* s_flag = reinterpret_cast<int*>(smem + kBarOff + 16 * kMaxStages);

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
        // ---------------- producer: one lane, two TMA loads per stage.  Weights and scales are never
        // written by a kernel, so the stream may start before the previous kernel has finished. -------
        if (lane == 0) {
            tma_prefetch_descriptor(&tmW);
            tma_prefetch_descriptor(&tmA);
            const int grp0 = k0 / p.g;
            const uint32_t tx = (uint32_t)stage_bytes;           // out-of-range parts are zero-filled and counted
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
                const uint32_t dst = smem_u32(smem + kStage0Off + slot * stage_bytes);
                mbar_arrive_expect_tx(bar_full + 8 * slot, tx);
                tma_load_3d(dst, &tmW, col0, b, kw0, bar_full + 8 * slot);
                tma_load_3d(dst + kWStageBytes, &tmA, col0, b, grp0, bar_full + 8 * slot);
                if (++slot == nstages) { slot = 0; round++; }
            }
        }
        pdl_wait_prior_grids();
    } else {
        // ---------------- consumers ----------------
        const int c8 = lane & 7;                 // 16-byte column chunk inside the warp's 32 columns
        const int rr = lane >> 3;                // G: which 128-k run of the slab
        const int cb = warp & 7, h = warp >> 3;
        const int jp = (c8 & 1) ^ h;             // this lane's words in the slab: kw = 4 rr + jp + 2 u, u = 0, 1
        // everything that does not depend on the activations comes before the dependency wait
        uint32_t cs = 0, sel[4];
#pragma unroll
        for (int b = 0; b < 4; b++) cs |= (uint32_t)(32 * rr + 16 * jp + 4 * b) << (8 * b);
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const uint32_t beta = (uint32_t)(s + (c8 >> 1)) & 3u;
            sel[s] = 0xCC00u | (beta << 4) | (4u + beta);     // -> {0, 0, word.byte[beta], cs.byte[beta]}
        }

        constexpr int NG = 2 / WPG;                            // alpha groups among the lane's 2 words
        int arow[NG];                                          // row of each group in the alpha box
        int grp[NG];
        bool grp_ok[NG];
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            const int kw_local = 4 * rr + jp + 2 * gi * WPG;   // NG == 2: word u = gi; NG == 1: both words
            grp[gi] = (k0 + 32 * kw_local) / p.g;
            arow[gi] = grp[gi] - k0 / p.g;
            grp_ok[gi] = (k0 + 32 * kw_local) < p.K;
        }
        pdl_wait_prior_grids();                  // the activations may come from the previous kernel
        if (p.tp.x_mode != 0) {
            // ... or from the other GPUs: wait for their pushes (bounded), then let the last CTA re-arm the flag
            if (tid == 0) {
                if (!wait_flag_bounded(p.tp.flag_in, p.tp.flag_target)) atomicExch(p.status, kStatusPeerTimeout);
                const unsigned prev = atomicAdd(p.tp.done_counter, 1u);
                if (prev == gridDim.x * gridDim.y - 1u) {
                    *reinterpret_cast<volatile unsigned*>(p.tp.flag_in) = 0u;
                    *reinterpret_cast<volatile unsigned*>(p.tp.done_counter) = 0u;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
        }
        build_lut2(lut, p.x, k0, p.K, tid, p.tp);
        asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");

        float xsum[NG];
        if (BIAS) {
            // sum of the activations under each group of words: entries idx = 255 (all signs +)
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
        const int col_in_stage = 32 * cb + 4 * c8;
        const uint32_t w_off = (uint32_t)(4 * rr + jp) * kRowPitch + (uint32_t)col_in_stage * 4u;
        bool aborted = false;
        int slot = 0, round = 0;
        for (int cg = 0; cg < ncg; cg++) {
            const int col = n_begin + cg * kStageCols + col_in_stage;
            const bool col_ok = col < n_end;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
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
                const unsigned char* st = smem + kStage0Off + slot * stage_bytes + w_off;
                const unsigned char* sa = smem + kStage0Off + slot * stage_bytes + kWStageBytes + col_in_stage * 2;
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
                    float2 s2[4];
#pragma unroll
                    for (int jj = 0; jj < WPG; jj++) {
                        const int u = gi * WPG + jj;
                        const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const float2 v = (u == 0) ? lookup_word<0>(lut, ww[c], cs, sel)
                                                      : lookup_word<128>(lut, ww[c], cs, sel);
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
            // add the 4 lanes (128-k runs) that share a column quad
#pragma unroll
            for (int off = 8; off < 32; off <<= 1) {
#pragma unroll
                for (int c = 0; c < 4; c++) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
            }
            // add the two warp halves (the other word parity) through shared memory
            if (h == 1 && rr == 0) *xchg = make_float4(acc[0], acc[1], acc[2], acc[3]);
            asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");
            if (h == 0 && rr == 0 && col_ok) {
                const float4 o = *xchg;
                const float4 r4 = make_float4(acc[0] + o.x, acc[1] + o.y, acc[2] + o.z, acc[3] + o.w);
                if (p.ordered) *reinterpret_cast<float4*>(part_out + col) = r4;
                else red_add_v4(p.partial + col, r4);
            }
            asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");   // exchange slot free for the next column group
        }
    }

    splitk_finish<kGemv2Threads>(p, tid, n_begin, n_end, s_flag);
}

// Last consumer of a tensor-parallel chain: waits for the ranks' fp32 rows, adds them in rank order and writes
// the fp16 (and optionally fp32) vector; re-arms the flag.  One CTA.
__global__ void __launch_bounds__(256)
tp_finalize_kernel(__half* y16, float* y32, const float* slots, int slot_stride, int world, int n,
                   unsigned* flag_in, unsigned flag_target, int* status) {
    __shared__ int s_ok;
    pdl_wait_prior_grids();
    if (threadIdx.x == 0) {
        s_ok = wait_flag_bounded(flag_in, flag_target) ? 1 : 0;
        if (!s_ok) atomicExch(status, kStatusPeerTimeout);
        *reinterpret_cast<volatile unsigned*>(flag_in) = 0u;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < world; r++) acc += __ldcg(slots + (size_t)r * slot_stride + i);
        if (y32) y32[i] = acc;
        if (y16) y16[i] = __float2half_rn(acc);
    }
}

}  // namespace lg
