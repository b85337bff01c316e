// A whole sequence of BCQ matvecs (m = 1) in ONE persistent kernel, sm_100a.
//
// The reference launches one kernel (plus a memset) per matvec (lutGEMM/src/kernels.cu:64-71); a decode step of a
// decoder stack is hundreds of such launches, each of which pays a kernel boundary: the tail of the split-k finish,
// the grid drain, the dependency release and a cold start of the weight stream.  Here one CTA per SM stays
// resident for the whole sequence:
//
//  * the producer lane walks ALL matvecs of the sequence and keeps the same ring of TMA stages full across
//    matvec boundaries (weights never depend on anything, so the stream never stops);
//  * the 16 consumer warps do, per (matvec, column tile, 512-k slab): wait for the slab's activations, build
//    the 2^8-entry tables (as gemv_tma_kernel, gemv_tma.cuh), look up and accumulate, reduce across slabs in
//    L2; the last CTA of a column tile rounds once and PUBLISHES the result;
//  * matvecs hand their results over in exchange lines of 16 bytes, {data, seq, data, seq}: the consumer polls
//    the very words it needs until both sequence numbers equal the current step number (no separate flag, no
//    fence between data and flag, no re-arming: one store crosses the bus per hand-over).  A line is written
//    with one 16-byte store and checked per 8-byte half, so only 8-byte store atomicity is assumed.
//    With several GPUs (tensor parallelism, one process each) the publisher stores the same lines into every
//    rank's exchange memory through peer-mapped pointers (plain stores over NVLink; no multicast, no TMA to or
//    from a peer): an fp16 vector for an all-gather, one fp32 row per rank for an all-reduce, which the
//    consumer adds in rank order (deterministic) and rounds to fp16 once.
//
// Every wait is bounded (a time limit on the poll loops, an iteration limit on the mbarrier waits); when one
// runs out the kernel records a status word, stops waiting anywhere else and runs to its end.
#pragma once
#include "gemv_tma.cuh"

namespace lg {

constexpr int kSeqThreads = kGemv2Threads;                   // 16 consumer warps + 1 producer warp
constexpr int kSeqMaxOps = 896;                              // matvecs per sequence (their geometry travels as kernel parameters)
constexpr int kSeqXsOff = kXchgOff + 1024;                   // 512 fp16 activations of the current slab
constexpr int kSeqBarOff = kSeqXsOff + 1024;                 // barriers and the finish flag
constexpr int kSeqStage0Off = kSeqBarOff + 256;
__host__ __device__ constexpr int seq_num_stages(int a_rows) {
    return (kSmemLimit - kSeqStage0Off) / gemv2_stage_bytes(a_rows) < kMaxStages
               ? (kSmemLimit - kSeqStage0Off) / gemv2_stage_bytes(a_rows) : kMaxStages;
}
__host__ __device__ constexpr int seq_smem_bytes(int a_rows) {
    return kSeqStage0Off + seq_num_stages(a_rows) * gemv2_stage_bytes(a_rows);
}

enum { kSeqInExternal = 0, kSeqInVector = 1, kSeqInRows = 2 };
enum { kSeqOutLocal = 0, kSeqOutVector = 1, kSeqOutRow = 2 };

// One matvec of the sequence as the kernel reads it (array in global memory, written by the host before launch).
struct alignas(128) SeqOpDev {
    CUtensorMap tmW;         // {N, q, K/32} uint32, box {256, 1, 16}
    CUtensorMap tmA;         // {N, q, G} fp16, box {256, 1, a_rows}
    const __half* q_bias;    // [G][N] or nullptr
    float* partial;          // zeroed fp32 row [N] of this matvec
    unsigned* counters;      // [tiles], zero
    const void* in_ptr;      // external: fp16 vector; vector / rows: first exchange line of this matvec's input
    void* out_ptr[8];        // local: [0] = fp16 vector; vector / row: first line of the target on every rank
    int N, K, q, g;
    int n_tile, tiles, nslabs, items;
    int in_kind, in_rows, in_row_lines;    // rows: number of rows added and lines per row
    int out_kind, out_world;
    int reduce_only;         // 1: no weights; the input (rows) is added, rounded and written to out_ptr[0] as fp16
    int pad_[2];
};

// What drives the loops of a matvec.  These numbers travel in the kernel's parameter space, not in global
// memory: values read from parameters are known to be the same in every lane, so the loops around the hot path
// stay on the uniform data path and need no divergence bookkeeping.
struct SeqGeo {
    int N, K, n_tile, tiles, nslabs, q, g, reduce_only;
};
struct SeqParams {
    const SeqOpDev* ops;
    int n_ops;
    int a_rows;              // alpha groups per slab, the same for every matvec of the sequence
    unsigned* epoch;         // step number (starts at 1); the kernel adds one when it is done
    unsigned* done;          // CTAs that have finished this step
    int* status;
    unsigned long long wait_ns;   // time limit of a poll loop
    unsigned long long* trace;    // optional: 4 time stamps (ns) per (matvec, CTA), see lutgemm_sequence_set_trace
    SeqGeo geo[kSeqMaxOps];
};

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_line(void* p, uint32_t d0, uint32_t d1, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d0), "r"(seq), "r"(d1), "r"(seq) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Polls up to ROWS exchange lines (row r at base + r * stride lines) until all carry `seq`; bounded by time and
// cut short as soon as any wait anywhere has failed.  Returns false if it gave up (status is set).
template <int ROWS>
__device__ __forceinline__ bool poll_lines(const uint4* base, int rows, int stride, uint32_t seq, uint4 (&v)[ROWS],
                                           const SeqParams& p) {
    unsigned long long t0 = 0;
    for (unsigned it = 0;; it++) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            if (r < rows) v[r] = ld_volatile_v4(base + (size_t)r * stride);
        }
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            if (r < rows) all = all && (v[r].y == seq) && (v[r].w == seq);
        }
        if (all) return true;
        if ((it & 31u) == 31u) {
            if (*reinterpret_cast<volatile int*>(p.status) != 0) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.wait_ns) {
                atomicExch(p.status, kStatusPeerTimeout);
                return false;
            }
        }
    }
}

// The 512 activations of slab [k0, k0 + 512) of matvec `op` as fp16 in shared memory (zero beyond K).
// Called by the 512 consumer threads; ends with their barrier.
__device__ __noinline__ void seq_fetch_input(const SeqOpDev& op, int k0, uint32_t seq, unsigned char* xs, int ctid,
                                                const SeqParams& p) {
    if (op.in_kind == kSeqInExternal) {
        if (ctid < 64) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (k0 + 8 * ctid < op.K) raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(op.in_ptr) + k0 + 8 * ctid));
            *reinterpret_cast<uint4*>(xs + 16 * ctid) = raw;
        }
    } else if (op.in_kind == kSeqInVector) {
        if (ctid < 128) {
            uint2 o = make_uint2(0u, 0u);
            if (k0 + 4 * ctid < op.K) {
                uint4 v[1];
                if (poll_lines<1>(reinterpret_cast<const uint4*>(op.in_ptr) + (k0 >> 2) + ctid, 1, 0, seq, v, p)) o = make_uint2(v[0].x, v[0].z);
            }
            *reinterpret_cast<uint2*>(xs + 8 * ctid) = o;
        }
    } else {
        if (ctid < 256) {
            uint32_t o = 0u;
            if (k0 + 2 * ctid < op.K) {
                uint4 v[8];
                if (poll_lines<8>(reinterpret_cast<const uint4*>(op.in_ptr) + (k0 >> 1) + ctid, op.in_rows, op.in_row_lines, seq, v, p)) {
                    float a = 0.f, b = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        if (r < op.in_rows) { a += __uint_as_float(v[r].x); b += __uint_as_float(v[r].z); }   // rank order
                    }
                    const __half2 h = __floats2half2_rn(a, b);
                    o = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
            *reinterpret_cast<uint32_t*>(xs + 4 * ctid) = o;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
}

// Last CTA of a column tile: the reduced sums -> one fp16 rounding (or the fp32 sums) -> the matvec's target.
__device__ __noinline__ void seq_publish(const SeqOpDev& op, int n_begin, int n_end, uint32_t seq, int ctid) {
    for (int c = n_begin + 4 * ctid; c < n_end; c += 4 * kConsWarps * 32) {
        const float4 s = __ldcg(reinterpret_cast<const float4*>(op.partial + c));
        __stcg(reinterpret_cast<float4*>(op.partial + c), make_float4(0.f, 0.f, 0.f, 0.f));
        if (op.out_kind == kSeqOutRow) {
            for (int r = 0; r < op.out_world; r++) {
                uint4* dst = reinterpret_cast<uint4*>(op.out_ptr[r]) + (c >> 1);
                st_line(dst, __float_as_uint(s.x), __float_as_uint(s.y), seq);
                st_line(dst + 1, __float_as_uint(s.z), __float_as_uint(s.w), seq);
            }
        } else {
            const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
            const uint32_t d0 = *reinterpret_cast<const uint32_t*>(&lo), d1 = *reinterpret_cast<const uint32_t*>(&hi);
            if (op.out_kind == kSeqOutVector) {
                for (int r = 0; r < op.out_world; r++) st_line(reinterpret_cast<uint4*>(op.out_ptr[r]) + (c >> 2), d0, d1, seq);
            } else {
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(op.out_ptr[0]) + c) = make_uint2(d0, d1);
            }
        }
    }
}

// The table sits at the very start of the CTA's dynamic shared memory, whose address in the shared window is a
// fixed number for a kernel without static shared memory (the first kilobyte belongs to the system).  With that
// number folded into the instruction's immediate, a lookup is exactly PRMT + LDS: the byte-permute result IS the
// address register.  The kernel checks the assumption when it starts and refuses to run otherwise.
constexpr uint32_t kSeqSmemBase = 0x400;
template <int IMM>
__device__ __forceinline__ float lds_lut(uint32_t off) {
    float v;
    asm("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(off), "n"(IMM + (int)kSeqSmemBase));
    return v;
}
// Sum of the four table entries selected by the four bytes of one packed word.
template <int IMM>
__device__ __forceinline__ float2 lookup_word_seq(uint32_t word, uint32_t cs, const uint32_t (&sel)[4]) {
    const float l0 = lds_lut<IMM>(prmt_b32(word, cs, sel[0]));
    const float l1 = lds_lut<IMM>(prmt_b32(word, cs, sel[1]));
    const float l2 = lds_lut<IMM>(prmt_b32(word, cs, sel[2]));
    const float l3 = lds_lut<IMM>(prmt_b32(word, cs, sel[3]));
    return add_f32x2(make_float2(l0, l1), make_float2(l2, l3));
}

// One item = one (column tile, 512-k slab) of one matvec: every stage of its column groups is taken from the ring,
// looked up, scaled and added, and the column sums go to the matvec's reduction row in L2.
// slot / round: the consumer side's position in the ring (the same in every thread; kept apart from `aborted`,
// which comes out of a barrier poll and would otherwise make the compiler treat the ring position as divergent).
template <int WPG, bool BIAS>
__device__ __forceinline__ void seq_consume_item(int& slot, int& round, bool& aborted, int n_begin, int n_end, int k0, int q,
                                                 int g, int K, int N, float* partial, const __half* q_bias, int a_rows,
                                                 int* status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* lut = smem;
    const int stage_bytes = gemv2_stage_bytes(a_rows);
    const int nstages = seq_num_stages(a_rows);
    const uint32_t bar_full = smem_u32(smem + kSeqBarOff);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c8 = lane & 7;                 // 16-byte column chunk inside the warp's 32 columns
    const int rr = lane >> 3;                // which 128-k run of the slab
    const int cb = warp & 7, h = warp >> 3;
    const int jp = (c8 & 1) ^ h;             // this lane's words in the slab: kw = 4 rr + jp + 2 u, u = 0, 1
    uint32_t cs = 0, sel[4];
#pragma unroll
    for (int b = 0; b < 4; b++) cs |= (uint32_t)(32 * rr + 16 * jp + 4 * b) << (8 * b);
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const uint32_t beta = (uint32_t)(s + (c8 >> 1)) & 3u;
        sel[s] = 0xCC00u | (beta << 4) | (4u + beta);     // -> {0, 0, word.byte[beta], cs.byte[beta]}
    }
    constexpr int NG = 2 / WPG;                            // alpha groups among the lane's 2 words
    float4* xchg = reinterpret_cast<float4*>(smem + kXchgOff) + cb * 8 + c8;
    const int col_in_stage = 32 * cb + 4 * c8;
    const uint32_t w_off = (uint32_t)(4 * rr + jp) * kRowPitch + (uint32_t)col_in_stage * 4u;
    const size_t rowN = (size_t)N;
    const int ncg = (n_end - n_begin + kStageCols - 1) / kStageCols;

    int arow[NG], grp[NG];
    bool grp_ok[NG];
#pragma unroll
    for (int gi = 0; gi < NG; gi++) {
        const int kw_local = 4 * rr + jp + 2 * gi * WPG;   // NG == 2: word u = gi; NG == 1: both words
        grp[gi] = (k0 + 32 * kw_local) / g;
        arow[gi] = grp[gi] - k0 / g;
        grp_ok[gi] = (k0 + 32 * kw_local) < K;
    }
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

    for (int cg = 0; cg < ncg; cg++) {
        const int col = n_begin + cg * kStageCols + col_in_stage;
        const bool col_ok = col < n_end;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 bv[NG];
        if (BIAS) {
#pragma unroll
            for (int gi = 0; gi < NG; gi++)
                bv[gi] = (col_ok && grp_ok[gi]) ? ldg_nc_v2(q_bias + (size_t)grp[gi] * rowN + col) : make_uint2(0u, 0u);
        }
        for (int b = 0; b < q && !aborted; b++) {
            if (!mbar_wait_bounded(bar_full + 8 * slot, round & 1)) {
                atomicExch(status, kStatusConsumerTimeout);
                aborted = true;     // keep walking the loops (the pair barriers below must stay matched)
                break;
            }
            const unsigned char* st = smem + kSeqStage0Off + slot * stage_bytes + w_off;
            const unsigned char* sa = smem + kSeqStage0Off + slot * stage_bytes + kWStageBytes + col_in_stage * 2;
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
                        const float2 v = (u == 0) ? lookup_word_seq<0>(ww[c], cs, sel) : lookup_word_seq<128>(ww[c], cs, sel);
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
            red_add_v4(partial + col, make_float4(acc[0] + o.x, acc[1] + o.y, acc[2] + o.z, acc[3] + o.w));
        }
        asm volatile("bar.sync %0, 64;" ::"r"(2 + cb) : "memory");   // exchange slot free for the next column group
    }
}

// WPG, BIAS: as gemv_tma_kernel (the same for every matvec of the sequence).  Grid: one CTA per SM, all resident
// (cooperative launch); block: 16 consumer warps + 1 producer warp.
template <int WPG, bool BIAS>
__global__ void __launch_bounds__(kSeqThreads, 1)
gemv_seq_kernel(const __grid_constant__ SeqParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* lut = smem;
    unsigned char* xs = smem + kSeqXsOff;
    const int stage_bytes = gemv2_stage_bytes(p.a_rows);
    const int nstages = seq_num_stages(p.a_rows);
    const uint32_t bar_full = smem_u32(smem + kSeqBarOff);          // nstages x 8 B
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    volatile int* s_flag = reinterpret_cast<volatile int*>(smem + kSeqBarOff + 16 * kMaxStages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;

    if (tid == 0) {
        for (int s = 0; s < nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t seq = *reinterpret_cast<volatile unsigned*>(p.epoch);

    if (smem_u32(smem) != kSeqSmemBase) {                            // see lds_lut: the lookups assume this address
        if (tid == 0) atomicExch(p.status, kStatusLayout);
    } else if (warp == kConsWarps) {
        // ---------------- producer: one lane keeps the ring full across the whole sequence ----------------
        if (lane == 0) {
            const uint32_t tx = (uint32_t)stage_bytes;
            int slot = 0, round = 0;
            bool dead = false;
            for (int j = 0; j < p.n_ops && !dead; j++) {
                const SeqGeo& G = p.geo[j];
                const int N = G.N, q = G.q, g = G.g, n_tile = G.n_tile, tiles = G.tiles, items = G.tiles * G.nslabs;
                if (G.reduce_only || cta >= items) continue;
                const SeqOpDev* op = p.ops + j;
                tma_prefetch_descriptor(&op->tmW);
                tma_prefetch_descriptor(&op->tmA);
                for (int it = cta; it < items && !dead; it += ncta) {
                    const int tile = it % tiles, slab = it / tiles;
                    const int n_begin = tile * n_tile;
                    const int n_end = min(N, n_begin + n_tile);
                    const int ncg = (n_end - n_begin + kStageCols - 1) / kStageCols;
                    const int kw0 = slab * kSlabWords, grp0 = slab * kSlab2 / g;
                    for (int cg = 0; cg < ncg && !dead; cg++) {
                        const int col0 = n_begin + cg * kStageCols;
                        for (int b = 0; b < q; b++) {
                            if (round > 0 && !mbar_wait_bounded(bar_empty + 8 * slot, (round - 1) & 1)) {
                                atomicExch(p.status, kStatusProducerTimeout);
                                dead = true;
                                break;
                            }
                            const uint32_t dst = smem_u32(smem + kSeqStage0Off + slot * stage_bytes);
                            mbar_arrive_expect_tx(bar_full + 8 * slot, tx);
                            tma_load_3d(dst, &op->tmW, col0, b, kw0, bar_full + 8 * slot);
                            tma_load_3d(dst + kWStageBytes, &op->tmA, col0, b, grp0, bar_full + 8 * slot);
                            if (++slot == nstages) { slot = 0; round++; }
                        }
                    }
                }
            }
        }
    } else {
    // ---------------- consumers ----------------
    // The ring position is re-derived per item from the count of stages consumed so far, which depends on the
    // kernel's parameters only: the compiler can then see that it is the same in every lane (carried through the item
    // loops it would inherit the divergence of the barrier polls inside them).
    unsigned stages_done = 0;
    for (int j = 0; j < p.n_ops; j++) {
        const SeqGeo& G = p.geo[j];
        const int items = G.reduce_only ? (G.K + kSlab2 - 1) / kSlab2 : G.tiles * G.nslabs;
        if (cta >= items) continue;
        const SeqOpDev& op = p.ops[j];
        if (tid < 3 && j + 1 < p.n_ops)      // the next matvec's descriptor: on its way to L1 while this one runs
            asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(p.ops + j + 1) + 128 * tid));
        if (G.reduce_only) {
            // the sequence's result: rows added in rank order, one fp16 rounding, plain store
            for (int it = cta; it < items; it += ncta) {
                const int k0 = it * kSlab2;
                seq_fetch_input(op, k0, seq, xs, tid, p);
                if (tid < 64 && k0 + 8 * tid < G.K)
                    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(op.out_ptr[0]) + k0 + 8 * tid) = *reinterpret_cast<const uint4*>(xs + 16 * tid);
                asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
            }
            continue;
        }
        const int N = G.N, tiles = G.tiles, n_tile = G.n_tile, nslabs = G.nslabs;
        for (int it = cta; it < items; it += ncta) {
            const int tile = it % tiles, slab = it / tiles;
            const int k0 = slab * kSlab2;
            const int n_begin = tile * n_tile;
            const int n_end = min(N, n_begin + n_tile);
            // the slab's activations (waits for whoever produces them), then the tables
            unsigned long long* tr = (p.trace && tid == 0 && it == cta) ? p.trace + ((size_t)j * ncta + cta) * 4 : nullptr;
            seq_fetch_input(op, k0, seq, xs, tid, p);
            if (tr) tr[0] = global_ns();
            build_lut_from_raw(lut, *reinterpret_cast<const uint4*>(xs + 16 * lut_chunk_of(tid)), tid);
            asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
            if (tr) tr[1] = global_ns();

            int slot = (int)(stages_done % (unsigned)nstages), round = (int)(stages_done / (unsigned)nstages);
            bool aborted = false;
            seq_consume_item<WPG, BIAS>(slot, round, aborted, n_begin, n_end, k0, G.q, G.g, G.K, N, op.partial, op.q_bias, p.a_rows, p.status);
            stages_done += (unsigned)(((n_end - n_begin + kStageCols - 1) / kStageCols) * G.q);

            // split-k finish: the last CTA of the column tile publishes it
            asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
            if (tr) tr[2] = global_ns();
            if (tid == 0) {
                __threadfence();
                const unsigned prev = atomicAdd(op.counters + tile, 1u);
                *s_flag = (prev == (unsigned)nslabs - 1u);
                if (prev == (unsigned)nslabs - 1u) op.counters[tile] = 0u;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
            if (*s_flag) {
                __threadfence();
                seq_publish(op, n_begin, n_end, seq, tid);
            }
            if (tr) tr[3] = global_ns() | (*s_flag ? 1ull : 0ull);      // bit 0: this CTA published the tile
            // (the barrier of the next seq_fetch_input keeps s_flag and the tables apart from the next item)
        }
    }

    // step done: the last CTA advances the step number
    asm volatile("bar.sync 1, %0;" ::"n"(kConsWarps * 32) : "memory");
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(p.done, 1u);
        if (prev == (unsigned)ncta - 1u) {
            *reinterpret_cast<volatile unsigned*>(p.done) = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(p.epoch) = seq + 1u;
        }
    }
    }
}

}  // namespace lg
