// C ABI of the library (declared in include/lutgemm_b200.h): container handle, argument checks,
// kernel selection and launch.  There is no CPU fallback anywhere in this file: without a usable
// CUDA device every compute entry point returns LUTGEMM_ERR_NO_DEVICE / LUTGEMM_ERR_CUDA.
#include "../../include/lutgemm_b200.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "aux_kernels.cuh"
#include "gemv_tma.cuh"
#include "gemv_reg.cuh"
#include "gemv_tma2.cuh"
#include "gemv_seq.cuh"
#include "gemm_tc.cuh"
#include "gemm_i8.cuh"
#include "bcq_quantize.cuh"
#include "gptq3.cuh"

// Split-k scratch of the matmul kernels: everything a call writes besides its output.  One per container by
// default; lutgemm_workspace_create makes more, so that several streams can use one container at a time.
struct lutgemm_workspace {
    float* partial = nullptr;    // partial sums [slabs][n_cap] fp32 (ordered mode) / row 0 = zeroed L2 reduction row
    float* partial2 = nullptr;   // second zeroed reduction row [n_cap] of the two-row matvec
    unsigned* counters = nullptr;   // per-tile arrival counters, zero between launches
    int* status = nullptr;       // device word set by a kernel whose bounded wait ran out
    float* tc_partial = nullptr; // fp32 split-k rows of the batched (tensor-core) path, [tc_rows][n_cap], kept zeroed
    int tc_rows = 0;
    int n_cap = 0, slabs = 0;    // widest N and most 512-k slabs this workspace serves
    // transposed copies for the (output, nqW, input, n) overload: input [n][K] and output [n][N] fp16
    void* t_in = nullptr;
    void* t_out = nullptr;
    size_t t_in_bytes = 0, t_out_bytes = 0;
    std::atomic<int> ordered{-1};   // split-k mode of calls on this workspace: -1 = the process-wide setting, 0 / 1 = fixed
};

struct lutgemm_weight {
    uint32_t* bW = nullptr;
    __half* alpha = nullptr;
    __half* q_bias = nullptr;
    int N = 0, K = 0, q = 0, G = 0, g = 0;
    bool row_wise = false;
    bool owns = true;
    int device = 0;
    // the container's own split-k workspace (calls that name no other workspace use it)
    lutgemm_workspace own;
    // TMA descriptors of the packed planes and of alpha (valid when tma_ok)
    CUtensorMap tmW, tmA;
    bool tma_ok = false;
    int a_rows = 1;            // alpha groups per 512-k slab
    // TMA descriptors of the batched (tensor-core) path: planes box {256, q, 4}, alpha box {256, q, groups per 128 k},
    // q_bias box {256, groups per 128 k} (valid when tc_ok)
    CUtensorMap tmWtc, tmAtc, tmQtc;
    bool tc_ok = false;
    // staging for lutgemm_matmul_host
    void* h_stage_in = nullptr;
    void* d_stage_in = nullptr;
    void* d_stage_out = nullptr;
    size_t stage_rows = 0;
    // lutgemm_matmul_host: its own non-blocking stream, and the last call's copy-run-copy sequence as an
    // instantiated graph (relaunched while the caller keeps passing the same buffers and batch)
    cudaStream_t host_stream = nullptr;
    cudaGraphExec_t host_graph = nullptr;
    const void* hg_in = nullptr;
    void* hg_out = nullptr;
    int hg_m = 0;
    int hg_launches = 0;
    // page-locked buffers: the copy engine and the stream synchronisation are replaced by a fetch kernel, result
    // stores straight into the host buffer and a completion word in page-locked memory that the host polls
    bool hg_pinned = false;
    volatile unsigned* h_done = nullptr;   // page-locked, 64 B
    unsigned* d_done = nullptr;            // its device alias
};

struct lutgemm_sequence {
    int rank = 0, world = 1, device = 0;
    std::vector<lutgemm_seq_op> ops;
    std::vector<lutgemm_seq_buffer> bufs;
    std::vector<size_t> buf_off;           // byte offset of every buffer inside the exchange memory
    size_t xchg_bytes = 0;
    unsigned char* xchg[8] = {};           // [rank] = this GPU's exchange memory, others: peer mappings
    bool mapped[8] = {};
    std::vector<lg::SeqOpDev> h_ops;
    lg::SeqOpDev* d_ops = nullptr;
    lg::SeqParams* params = nullptr;       // the kernel's parameter block (host copy; holds every matvec's geometry)
    float* partial = nullptr;              // one zeroed fp32 row per matvec, back to back
    unsigned* counters = nullptr;          // arrival counters per column tile, back to back
    unsigned* words = nullptr;             // [0] step number, [1] finished CTAs, [2] status
    int a_rows = 1, wpg = 2, grid = 0;
    bool bias = false, committed = false;
    unsigned long long wait_ns = 2000000000ull;
    unsigned long long* trace = nullptr;   // caller's device buffer, or null
};

namespace {

thread_local int g_last_cuda = 0;
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_ntile_override{0};
std::atomic<int> g_pdl{1};
std::atomic<int> g_ordered{0};
std::atomic<int> g_pairs{1};     // 1: rows that go through the LUT matvec are taken two at a time where possible
std::atomic<int> g_batched{1};   // 0: one matvec per row; 1: tensor-core kernel from kBatchedFromRows rows; 2: from 2 rows
std::atomic<int> g_int8{0};      // 1: batches of up to 16 rows take the integer tensor-core kernel (measured slower: off)
std::atomic<int> g_variant{0};   // 0: bulk-copy fed kernel (default); 1: register-streaming kernel
// Split-k mode of a call on this workspace (read once per call).
inline int ordered_for(const lutgemm_workspace* ws);
constexpr int kMaxCounters = 4096;
constexpr int kMaxBatch = 65536;
constexpr int kBatchedFromRows = 4;      // m >= 4 goes to the tensor-core kernel

#define LG_CUDA(call)                                  \
    do {                                               \
        cudaError_t e__ = (call);                      \
        if (e__ != cudaSuccess) {                      \
            g_last_cuda = (int)e__;                    \
            return (e__ == cudaErrorNoDevice || e__ == cudaErrorInsufficientDriver) \
                       ? LUTGEMM_ERR_NO_DEVICE : LUTGEMM_ERR_CUDA; \
        }                                              \
    } while (0)

int check_shape(int row, int col, int q, int is_row_wise, int groups, int* N, int* K) {
    if (row < 1 || col < 1 || groups < 1) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    *N = is_row_wise ? row : col;
    *K = is_row_wise ? col : row;
    if (*K % 32 != 0 || *K % groups != 0) return LUTGEMM_ERR_SHAPE;
    if ((*K / groups) % 32 != 0) return LUTGEMM_ERR_SHAPE;
    if ((long long)(*K / 32) * q * (long long)*N > (1ll << 40)) return LUTGEMM_ERR_TOO_LARGE;
    return LUTGEMM_OK;
}

// cuTensorMapEncodeTiled, fetched through the runtime so that the library does not link libcuda
// (and therefore still loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// Descriptors for the TMA-fed matvec: planes as {N, q, K/32} uint32 with box {256, 1, 16}; alpha as
// {N, q, G} fp16 with box {256, 1, groups per 512-k slab}.  Leaves tma_ok false when the shape does
// not qualify (N % 8, group size neither dividing nor a multiple of 512) or the driver refuses.
void make_tc_tensor_maps(lutgemm_weight* w, EncodeTiledFn enc) {
    w->tc_ok = false;
    const int g = w->g;
    if (w->N % 8 != 0 || !((lg::kTcStepK % g == 0) || (g % lg::kTcStepK == 0))) return;
    const int a_rows = g >= lg::kTcStepK ? 1 : lg::kTcStepK / g;
    const cuuint64_t N = (cuuint64_t)w->N, q = (cuuint64_t)w->q;
    cuuint32_t es[3] = {1, 1, 1};
    {
        cuuint64_t dims[3] = {N, q, (cuuint64_t)(w->K / 32)};
        cuuint64_t strides[2] = {N * 4, q * N * 4};
        cuuint32_t box[3] = {(cuuint32_t)lg::kTcTileN, (cuuint32_t)w->q, (cuuint32_t)lg::kTcStepWords};
        if (enc(&w->tmWtc, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w->bW, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return;
    }
    {
        cuuint64_t dims[3] = {N, q, (cuuint64_t)w->G};
        cuuint64_t strides[2] = {N * 2, q * N * 2};
        cuuint32_t box[3] = {(cuuint32_t)lg::kTcTileN, (cuuint32_t)w->q, (cuuint32_t)a_rows};
        if (enc(&w->tmAtc, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, w->alpha, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return;
    }
    w->tmQtc = w->tmAtc;                                   // placeholder when there is no q_bias (never read)
    if (w->q_bias) {
        cuuint64_t dims[2] = {N, (cuuint64_t)w->G};
        cuuint64_t strides[1] = {N * 2};
        cuuint32_t box[2] = {(cuuint32_t)lg::kTcTileN, (cuuint32_t)a_rows};
        if (enc(&w->tmQtc, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->q_bias, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return;
    }
    w->tc_ok = true;
}

void make_tensor_maps(lutgemm_weight* w, bool with_batched = true) {
    w->tma_ok = false;
    w->tc_ok = false;
    if (with_batched)
        if (EncodeTiledFn e = encode_tiled_fn()) make_tc_tensor_maps(w, e);
    const int g = w->g;
    if (w->N % 8 != 0 || !((lg::kSlab2 % g == 0) || (g % lg::kSlab2 == 0))) return;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return;
    w->a_rows = (g >= lg::kSlab2) ? 1 : lg::kSlab2 / g;
    const cuuint64_t N = (cuuint64_t)w->N, q = (cuuint64_t)w->q;
    {
        cuuint64_t dims[3] = {N, q, (cuuint64_t)(w->K / 32)};
        cuuint64_t strides[2] = {N * 4, q * N * 4};
        cuuint32_t box[3] = {(cuuint32_t)lg::kStageCols, 1, (cuuint32_t)lg::kSlabWords};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&w->tmW, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w->bW, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return;
    }
    {
        cuuint64_t dims[3] = {N, q, (cuuint64_t)w->G};
        cuuint64_t strides[2] = {N * 2, q * N * 2};
        cuuint32_t box[3] = {(cuuint32_t)lg::kStageCols, 1, (cuuint32_t)w->a_rows};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&w->tmA, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, w->alpha, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return;
    }
    w->tma_ok = true;
}

void free_workspace_buffers(lutgemm_workspace* ws) {
    if (ws->partial) cudaFree(ws->partial);
    if (ws->partial2) cudaFree(ws->partial2);
    if (ws->counters) cudaFree(ws->counters);
    if (ws->status) cudaFree(ws->status);
    if (ws->tc_partial) cudaFree(ws->tc_partial);
    if (ws->t_in) cudaFree(ws->t_in);
    if (ws->t_out) cudaFree(ws->t_out);
    ws->partial = ws->partial2 = ws->tc_partial = nullptr;
    ws->counters = nullptr;
    ws->status = nullptr;
    ws->t_in = ws->t_out = nullptr;
    ws->tc_rows = ws->n_cap = ws->slabs = 0;
    ws->t_in_bytes = ws->t_out_bytes = 0;
    ws->ordered.store(-1);
}

// Rows of the batched path's fp32 workspace for a batch of m (a multiple of 16, at most 128 per launch).
inline int ordered_for(const lutgemm_workspace* ws) {
    const int o = ws ? ws->ordered.load() : -1;
    return o >= 0 ? o : g_ordered.load();
}

int tc_rows_for(int m) {
    const int rows = m > 128 ? 128 : m;
    return (rows + 15) / 16 * 16;
}

int fill_workspace(lutgemm_workspace* ws, int N, int K, int batch_rows) {
    const size_t nslabs = (size_t)(K + lg::kSlab2 - 1) / lg::kSlab2;
    ws->n_cap = N; ws->slabs = (int)nslabs;
    LG_CUDA(cudaMalloc(&ws->partial, nslabs * (size_t)N * sizeof(float)));
    LG_CUDA(cudaMemset(ws->partial, 0, nslabs * (size_t)N * sizeof(float)));   // row 0 doubles as the reduction row
    LG_CUDA(cudaMalloc(&ws->partial2, (size_t)N * sizeof(float)));
    LG_CUDA(cudaMemset(ws->partial2, 0, (size_t)N * sizeof(float)));
    LG_CUDA(cudaMalloc(&ws->counters, kMaxCounters * sizeof(unsigned)));
    LG_CUDA(cudaMemset(ws->counters, 0, kMaxCounters * sizeof(unsigned)));
    LG_CUDA(cudaMalloc(&ws->status, sizeof(int)));
    LG_CUDA(cudaMemset(ws->status, 0, sizeof(int)));
    if (batch_rows > 0) {
        const int rows = tc_rows_for(batch_rows);
        LG_CUDA(cudaMalloc(&ws->tc_partial, (size_t)rows * N * sizeof(float)));
        LG_CUDA(cudaMemset(ws->tc_partial, 0, (size_t)rows * N * sizeof(float)));
        ws->tc_rows = rows;
    }
    return LUTGEMM_OK;
}

int alloc_workspace(lutgemm_weight* w) {
    make_tensor_maps(w);
    return fill_workspace(&w->own, w->N, w->K, 0);
}

int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev].load() > 0) return cached[dev].load();
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
    if (dev >= 0 && dev < 64) cached[dev].store(sms);
    return sms;
}

// Columns per CTA (a multiple of `quantum`).  Every CTA rebuilds its table, so wide tiles are cheaper, but the
// grid should fill whole waves of `per_sm` CTAs per SM: among the candidate widths the widest one whose wave
// efficiency is within 5 % of the best is taken.
int choose_ntile(int N, int nslabs, int per_sm, int quantum) {
    int forced = g_ntile_override.load();
    int ntile;
    if (forced > 0) {
        ntile = (forced + quantum - 1) / quantum * quantum;
    } else {
        const int slots = per_sm * sm_count();
        const int n_max = (N + quantum - 1) / quantum * quantum;
        int lo = quantum;
        if (lo > n_max) lo = n_max;
        double best = 0.0;
        for (int t = lo; t <= n_max; t += quantum) {
            const long long ctas = (long long)((N + t - 1) / t) * nslabs;
            const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
            if (eff > best) best = eff;
        }
        ntile = lo;
        for (int t = lo; t <= n_max; t += quantum) {
            const long long ctas = (long long)((N + t - 1) / t) * nslabs;
            const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
            if (eff >= 0.95 * best) ntile = t;      // keeps the widest qualifying tile
        }
        // same number of tiles, equal widths
        const int tiles = (N + ntile - 1) / ntile;
        ntile = ((N + tiles - 1) / tiles + quantum - 1) / quantum * quantum;
    }
    while ((N + ntile - 1) / ntile > kMaxCounters) ntile *= 2;
    return ntile;
}

template <int WPG>
int launch_gemv_tma(const lutgemm_weight* w, const lg::Gemv2Params& p, dim3 grid, bool bias, cudaStream_t st) {
    static bool configured[64][2] = {};   // the attribute is per device
    auto kern = bias ? lg::gemv_tma_kernel<WPG, true> : lg::gemv_tma_kernel<WPG, false>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev][bias]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kSmemLimit));
        if (dev < 64) configured[dev][bias] = true;
    }
    // Programmatic stream serialization: the kernel may begin (and start its weight stream) while the
    // previous kernel in the stream drains; it orders itself with griddepcontrol.wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lg::kGemv2Threads);
    cfg.dynamicSmemBytes = (size_t)lg::gemv2_smem_bytes(p.a_rows);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    LG_CUDA(cudaLaunchKernelEx(&cfg, kern, w->tmW, w->tmA, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

template <int WPG>
int launch_gemv_reg(const lg::Gemv2Params& p, dim3 grid, bool bias, cudaStream_t st) {
    static bool configured[64][2] = {};   // the attribute is per device
    auto kern = bias ? lg::gemv_reg_kernel<WPG, true> : lg::gemv_reg_kernel<WPG, false>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev][bias]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kRegSmemBytes));
        if (dev < 64) configured[dev][bias] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lg::kRegThreads);
    cfg.dynamicSmemBytes = (size_t)lg::kRegSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    LG_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

// Grid of the TMA-fed matvec for a container: columns per CTA and the number of column tiles.
void gemv_tma_geometry(const lutgemm_weight* w, int* nslabs, int* n_tile, int* tiles) {
    *nslabs = (w->K + lg::kSlab2 - 1) / lg::kSlab2;
    *n_tile = choose_ntile(w->N, *nslabs, 1, lg::kStageCols);
    *tiles = (w->N + *n_tile - 1) / *n_tile;
}

int launch_gemv_tma_any(const lutgemm_weight* w, const lutgemm_workspace* ws, const __half* x, __half* y16, float* y32,
                        const lg::TpLink* link, cudaStream_t st) {
    lg::Gemv2Params p2 = {};
    p2.bW = w->bW; p2.alpha = w->alpha; p2.q_bias = w->q_bias; p2.x = x;
    p2.partial = ws->partial; p2.counters = ws->counters; p2.status = ws->status; p2.y16 = y16; p2.y32 = y32;
    p2.N = w->N; p2.K = w->K; p2.q = w->q; p2.g = w->g;
    int tiles = 0;
    gemv_tma_geometry(w, &p2.nslabs, &p2.n_tile, &tiles);
    p2.a_rows = w->a_rows;
    p2.ordered = ordered_for(ws);
    if (link) p2.tp = *link;
    dim3 grid2(tiles, p2.nslabs);
    const bool bias2 = w->q_bias != nullptr;
    if (w->g % 128 == 0) return launch_gemv_tma<2>(w, p2, grid2, bias2, st);
    return launch_gemv_tma<1>(w, p2, grid2, bias2, st);
}

template <int WPG>
int launch_gemv_tma2(const lutgemm_weight* w, const lg::Gemv22Params& p, dim3 grid, bool bias, cudaStream_t st) {
    static bool configured[64][2] = {};   // the attribute is per device
    auto kern = bias ? lg::gemv_tma2_kernel<WPG, true> : lg::gemv_tma2_kernel<WPG, false>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev][bias]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kSmemLimit));
        if (dev < 64) configured[dev][bias] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lg::kGemv2Threads);
    cfg.dynamicSmemBytes = (size_t)lg::gemv22_smem_bytes(p.b.a_rows);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    LG_CUDA(cudaLaunchKernelEx(&cfg, kern, w->tmW, w->tmA, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

// Two matvec rows in one pass over the weights (rows r and r + 1 of x / y); the caller has checked gemv_pair_ok().
int gemv_pair(const lutgemm_weight* w, const lutgemm_workspace* ws, const __half* x, __half* y16, float* y32, cudaStream_t st) {
    lg::Gemv22Params p = {};
    lg::Gemv2Params& b = p.b;
    b.bW = w->bW; b.alpha = w->alpha; b.q_bias = w->q_bias; b.x = x;
    b.partial = ws->partial; b.counters = ws->counters; b.status = ws->status; b.y16 = y16; b.y32 = y32;
    b.N = w->N; b.K = w->K; b.q = w->q; b.g = w->g;
    int tiles = 0;
    gemv_tma_geometry(w, &b.nslabs, &b.n_tile, &tiles);
    b.a_rows = w->a_rows;
    p.x1 = x + w->K;
    p.y16_1 = y16 ? y16 + w->N : nullptr;
    p.y32_1 = y32 ? y32 + w->N : nullptr;
    p.partial1 = ws->partial2;
    dim3 grid(tiles, b.nslabs);
    const bool bias = w->q_bias != nullptr;
    if (w->g % 128 == 0) return launch_gemv_tma2<2>(w, p, grid, bias, st);
    return launch_gemv_tma2<1>(w, p, grid, bias, st);
}
bool gemv_pair_ok(const lutgemm_weight* w, const lutgemm_workspace* ws) {
    return g_variant.load() == 0 && w->tma_ok && ws->partial2 && !ordered_for(ws) && g_pairs.load() &&
           lg::gemv22_num_stages(w->a_rows) >= 2;
}

// One matvec row: y (fp16 and/or fp32) = x . W
int gemv_row(const lutgemm_weight* w, const lutgemm_workspace* ws, const __half* x, __half* y16, float* y32, cudaStream_t st) {
    const bool use_tma = (g_variant.load() == 0) && w->tma_ok;
    if (use_tma) return launch_gemv_tma_any(w, ws, x, y16, y32, nullptr, st);
    if (w->N % 4 == 0) {
        // register-fed kernel: any group size that is a multiple of 32
        lg::Gemv2Params p = {};
        p.bW = w->bW; p.alpha = w->alpha; p.q_bias = w->q_bias; p.x = x;
        p.partial = ws->partial; p.counters = ws->counters; p.status = ws->status; p.y16 = y16; p.y32 = y32;
        p.N = w->N; p.K = w->K; p.q = w->q; p.g = w->g;
        p.nslabs = (w->K + lg::kSlab2 - 1) / lg::kSlab2;
        p.n_tile = choose_ntile(w->N, p.nslabs, 1, lg::kStageCols);
        p.ordered = ordered_for(ws);
        dim3 grid((w->N + p.n_tile - 1) / p.n_tile, p.nslabs);
        const bool bias = w->q_bias != nullptr;
        if (w->g % 128 == 0) return launch_gemv_reg<2>(p, grid, bias, st);
        return launch_gemv_reg<1>(p, grid, bias, st);
    }
    dim3 grid((w->N + 127) / 128);
    lg::gemv_generic_kernel<<<grid, 128, 0, st>>>(w->bW, w->alpha, w->q_bias, x, y16, y32, w->N, w->K, w->q, w->g);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

template <int Q>
int launch_gemm_tc_q(const lutgemm_weight* w, const CUtensorMap& tmX, const lg::TcParams& p, dim3 grid, cudaStream_t st) {
    static bool configured[64][2] = {};   // the attribute is per device
    const bool bias = w->q_bias != nullptr;
    auto kern = bias ? lg::gemm_tc_kernel<Q, true> : lg::gemm_tc_kernel<Q, false>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev][bias]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kTcSmemTotal));
        if (dev < 64) configured[dev][bias] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lg::kTcThreads);
    cfg.dynamicSmemBytes = (size_t)p.L.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    LG_CUDA(cudaLaunchKernelEx(&cfg, kern, tmX, w->tmWtc, w->tmAtc, w->tmQtc, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

// Split-k plan of a batched launch (256-column tiles x k-ranges of whole 128-k steps) and, when it splits, the fp32
// reduction rows of the workspace.
int tc_split(lutgemm_weight* w, lutgemm_workspace* ws, int m, cudaStream_t st, int* splitk_out, int* steps_per_cta_out) {
    const int tiles = (w->N + lg::kTcTileN - 1) / lg::kTcTileN;
    const int steps_total = (w->K + lg::kTcStepK - 1) / lg::kTcStepK;
    // split-k factor: fill whole waves of one CTA per SM; among equally full choices take the smallest
    const int sms = sm_count();
    int splitk = 1, steps_per_cta = 0;
    double best = 0.0;
    for (int c = 1; c <= 8 && c <= steps_total; c++) {
        const int ctas = tiles * c;
        const double eff = (double)ctas / ((double)((ctas + sms - 1) / sms) * sms);
        if (eff > best + 0.02) { best = eff; splitk = c; }
    }
    if (ordered_for(ws)) splitk = 1;             // bit-reproducible mode: no unordered reductions across k-ranges
    steps_per_cta = (steps_total + splitk - 1) / splitk;
    splitk = (steps_total + steps_per_cta - 1) / steps_per_cta;
    if (tiles > kMaxCounters) return LUTGEMM_ERR_TOO_LARGE;
    if (splitk > 1 && ws->tc_rows < m) {
        // Not reserved (lutgemm_weight_reserve_batch / lutgemm_workspace_create): only the container's own workspace
        // grows by itself, which synchronises the device and cannot happen inside a stream capture.
        if (ws != &w->own) return LUTGEMM_ERR_TOO_LARGE;
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return LUTGEMM_ERR_BATCH;
        if (ws->tc_partial) LG_CUDA(cudaFree(ws->tc_partial));
        ws->tc_partial = nullptr;
        ws->tc_rows = 0;
        const int rows = tc_rows_for(m);
        LG_CUDA(cudaMalloc(&ws->tc_partial, (size_t)rows * w->N * sizeof(float)));
        LG_CUDA(cudaMemset(ws->tc_partial, 0, (size_t)rows * w->N * sizeof(float)));
        ws->tc_rows = rows;
    }
    *splitk_out = splitk;
    *steps_per_cta_out = steps_per_cta;
    return LUTGEMM_OK;
}

// Batched rows [0, m), m in 2..128, through the tensor-core kernel (container must have tc_ok).
int gemm_tc_rows(lutgemm_weight* w, lutgemm_workspace* ws, const __half* x, __half* y16, float* y32, int m, cudaStream_t st) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc || !w->tc_ok) return LUTGEMM_ERR_CUDA;
    lg::TcParams p = {};
    p.m = m;
    p.L = lg::tc_layout(w->q, w->q_bias != nullptr, w->g, m);
    if (p.L.w_slots < 1 || p.L.x_slots < 1) return LUTGEMM_ERR_TOO_LARGE;
    CUtensorMap tmX;
    {
        cuuint64_t dims[2] = {(cuuint64_t)w->K, (cuuint64_t)m};
        cuuint64_t strides[1] = {(cuuint64_t)w->K * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)p.L.m_pad};
        cuuint32_t es[2] = {1, 1};
        if (enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return LUTGEMM_ERR_CUDA;
    }
    int splitk = 1;
    {
        int rc = tc_split(w, ws, m, st, &splitk, &p.steps_per_cta);
        if (rc != LUTGEMM_OK) return rc;
    }
    const int tiles = (w->N + lg::kTcTileN - 1) / lg::kTcTileN;
    p.partial = ws->tc_partial; p.counters = ws->counters; p.status = ws->status;
    p.y16 = y16; p.y32 = y32;
    p.N = w->N; p.K = w->K; p.g = w->g;
    dim3 grid(tiles, splitk);
    switch (w->q) {
        case 1: return launch_gemm_tc_q<1>(w, tmX, p, grid, st);
        case 2: return launch_gemm_tc_q<2>(w, tmX, p, grid, st);
        case 3: return launch_gemm_tc_q<3>(w, tmX, p, grid, st);
        case 4: return launch_gemm_tc_q<4>(w, tmX, p, grid, st);
        case 5: return launch_gemm_tc_q<5>(w, tmX, p, grid, st);
        case 6: return launch_gemm_tc_q<6>(w, tmX, p, grid, st);
        case 7: return launch_gemm_tc_q<7>(w, tmX, p, grid, st);
        case 8: return launch_gemm_tc_q<8>(w, tmX, p, grid, st);
    }
    return LUTGEMM_ERR_BITS;
}

template <int Q>
int launch_gemm_i8_q(const lutgemm_weight* w, const CUtensorMap& tmX, const lg::I8Params& p, dim3 grid, cudaStream_t st) {
    static bool configured[64][2] = {};   // the attribute is per device
    const bool bias = w->q_bias != nullptr;
    auto kern = bias ? lg::gemm_i8_kernel<Q, true> : lg::gemm_i8_kernel<Q, false>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev][bias]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kTcSmemTotal));
        if (dev < 64) configured[dev][bias] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(lg::kI8Threads);
    cfg.dynamicSmemBytes = (size_t)lg::kTcSmemTotal;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    LG_CUDA(cudaLaunchKernelEx(&cfg, kern, tmX, w->tmWtc, w->tmAtc, w->tmQtc, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

// True when a batch of m rows on this container can take the integer tensor-core kernel.
bool gemm_i8_ok(const lutgemm_weight* w, int m) {
    if (!w->tc_ok || m < 2 || m > lg::kI8Rows || w->q > 4 || !g_int8.load()) return false;
    lg::I8Params p = {};
    return lg::i8_plan(w->q, w->q_bias != nullptr, w->g, p);
}

// Batched rows [0, m), m in 2..16, through the integer tensor-core kernel (gemm_i8_ok holds).
int gemm_i8_rows(lutgemm_weight* w, lutgemm_workspace* ws, const __half* x, __half* y16, float* y32, int m, cudaStream_t st) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc || !w->tc_ok) return LUTGEMM_ERR_CUDA;
    lg::I8Params p = {};
    if (!lg::i8_plan(w->q, w->q_bias != nullptr, w->g, p)) return LUTGEMM_ERR_TOO_LARGE;
    p.m = m;
    CUtensorMap tmX;
    {
        cuuint64_t dims[2] = {(cuuint64_t)w->K, (cuuint64_t)m};
        cuuint64_t strides[1] = {(cuuint64_t)w->K * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)lg::kI8Rows};
        cuuint32_t es[2] = {1, 1};
        if (enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return LUTGEMM_ERR_CUDA;
    }
    int splitk = 1;
    int rc = tc_split(w, ws, m, st, &splitk, &p.steps_per_cta);
    if (rc != LUTGEMM_OK) return rc;
    p.partial = ws->tc_partial; p.counters = ws->counters; p.status = ws->status;
    p.y16 = y16; p.y32 = y32;
    p.N = w->N; p.K = w->K; p.g = w->g;
    dim3 grid((w->N + lg::kTcTileN - 1) / lg::kTcTileN, splitk);
    switch (w->q) {
        case 1: return launch_gemm_i8_q<1>(w, tmX, p, grid, st);
        case 2: return launch_gemm_i8_q<2>(w, tmX, p, grid, st);
        case 3: return launch_gemm_i8_q<3>(w, tmX, p, grid, st);
        case 4: return launch_gemm_i8_q<4>(w, tmX, p, grid, st);
    }
    return LUTGEMM_ERR_BITS;
}

// ---- scratch for lutgemm_matvec_static_scratch: lives in the library image, never allocated ----
constexpr int kStaticMaxN = 65536;                       // widest output the static entry point takes
constexpr size_t kStaticRowBytes = (size_t)kStaticMaxN * sizeof(float);
constexpr size_t kStaticCounterBytes = (size_t)kMaxCounters * sizeof(unsigned);
constexpr size_t kStaticScratchBytes = kStaticRowBytes + kStaticCounterBytes + 256;
// [0, 256 KB): the split-k reduction row; then the per-tile arrival counters; then the status word.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use, so the address is asked for once per
// device (with that device current) and cached.
int static_scratch_address(unsigned char** out) {
    static unsigned char* cached[64] = {};
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return LUTGEMM_ERR_TOO_LARGE;
    if (!cached[dev]) {
        unsigned char* ptr = nullptr;
        LG_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        if (!ptr) return LUTGEMM_ERR_CUDA;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return LUTGEMM_OK;
}

int matmul_impl(__half* y16, float* y32, const void* in, lutgemm_weight_t w, int m, lutgemm_workspace* ws, void* stream) {
    if (!w || !in || (!y16 && !y32)) return LUTGEMM_ERR_NULL;
    if (m < 1 || m > kMaxBatch) return LUTGEMM_ERR_BATCH;
    if (((uintptr_t)in & 15) || ((uintptr_t)y16 & 15) || ((uintptr_t)y32 & 15)) return LUTGEMM_ERR_ALIGN;
    if (!ws) ws = &w->own;
    if (ws->n_cap < w->N || ws->slabs < (w->K + lg::kSlab2 - 1) / lg::kSlab2) return LUTGEMM_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    const __half* x = (const __half*)in;
    // Up to three rows one LUT matvec per row is cheaper than the tensor-core kernel, whose cost is nearly
    // independent of m up to 64 rows (measured: 8192^2, q = 2: m x 10.2 us against 29 us; 12288^2, q = 3:
    // m x 17.6 us against 64 us).
    const int batched_mode = g_batched.load();
    if (m == 1 || batched_mode == 0 || (batched_mode == 1 && m < kBatchedFromRows) || !w->tc_ok) {
        const bool pairs = gemv_pair_ok(w, ws);
        for (int r = 0; r < m;) {
            const int take = (pairs && r + 2 <= m) ? 2 : 1;
            const __half* xr = x + (size_t)r * w->K;
            __half* y16r = y16 ? y16 + (size_t)r * w->N : nullptr;
            float* y32r = y32 ? y32 + (size_t)r * w->N : nullptr;
            int rc = take == 2 ? gemv_pair(w, ws, xr, y16r, y32r, st) : gemv_row(w, ws, xr, y16r, y32r, st);
            if (rc != LUTGEMM_OK) return rc;
            r += take;
        }
        return LUTGEMM_OK;
    }
    // batched: 128 rows per tensor-core launch
    for (int r0 = 0; r0 < m; r0 += 128) {
        const int rows = (m - r0 < 128) ? (m - r0) : 128;
        const __half* xr = x + (size_t)r0 * w->K;
        __half* y16r = y16 ? y16 + (size_t)r0 * w->N : nullptr;
        float* y32r = y32 ? y32 + (size_t)r0 * w->N : nullptr;
        int rc = gemm_i8_ok(w, rows) ? gemm_i8_rows(w, ws, xr, y16r, y32r, rows, st) : gemm_tc_rows(w, ws, xr, y16r, y32r, rows, st);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

// fp16 [rows][cols] -> [cols][rows] through a 32 x 32 shared-memory tile (both sides coalesced)
__global__ void __launch_bounds__(256)
transpose_fp16_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int rows, int cols) {
    __shared__ __half tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[i][threadIdx.x] = src[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][i];
    }
}

// Host-buffer call, page-locked buffers: the activations come over the bus through this kernel instead of the copy
// engine (whose 24 KB copy costs ~8 us of fixed latency), ...
__global__ void __launch_bounds__(1024)
host_fetch_kernel(const uint4* __restrict__ src_host, uint4* __restrict__ dst, int n16) {
    lg::pdl_launch_dependents();                       // the matvec behind it may start streaming its weights
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) dst[i] = src_host[i];
}
// ... and completion is a word in page-locked memory written behind the last kernel, which the host polls: that
// takes a bus write instead of the driver's synchronisation path (~15 us).
__global__ void host_done_kernel(unsigned* done_host, unsigned value) {
    lg::pdl_wait_prior_grids();                        // every kernel before it has finished and flushed
    __threadfence_system();
    *reinterpret_cast<volatile unsigned*>(done_host) = value;
}

int grow(void** buf, size_t* have, size_t need, cudaStream_t st) {
    if (*have >= need) return LUTGEMM_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return LUTGEMM_ERR_BATCH;
    if (*buf) LG_CUDA(cudaFree(*buf));
    *buf = nullptr; *have = 0;
    LG_CUDA(cudaMalloc(buf, need));
    *have = need;
    return LUTGEMM_OK;
}

int finish_create(lutgemm_weight* w, lutgemm_weight_t* out) {
    int rc = alloc_workspace(w);
    if (rc != LUTGEMM_OK) {
        lutgemm_weight_destroy(w);
        return rc;
    }
    *out = w;
    return LUTGEMM_OK;
}

size_t seq_buffer_bytes(const lutgemm_seq_buffer& b, int world) {
    // one 16-byte line per 4 fp16 values / per 2 fp32 values
    const size_t raw = b.kind == 1 ? (size_t)b.n * 4 : (size_t)world * b.n * 8;
    return (raw + 255) / 256 * 256;
}

template <int WPG, bool BIAS>
int launch_sequence(lutgemm_sequence* s, cudaStream_t st) {
    static bool configured[64] = {};
    auto kern = lg::gemv_seq_kernel<WPG, BIAS>;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[dev]) {
        LG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lg::kSmemLimit));
        if (dev < 64) configured[dev] = true;
    }
    lg::SeqParams& p = *s->params;
    p.wait_ns = s->wait_ns;
    p.trace = s->trace;
    // cooperative launch: the runtime guarantees that all CTAs are resident together (they wait on one another),
    // or refuses the launch
    void* args[] = {&p};
    LG_CUDA(cudaLaunchCooperativeKernel((void*)kern, dim3(s->grid), dim3(lg::kSeqThreads), args,
                                        (size_t)lg::seq_smem_bytes(s->a_rows), st));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return LUTGEMM_OK;
}

}  // namespace

extern "C" {

int lutgemm_weight_create(lutgemm_weight_t* out, const uint32_t* bW, const float* A, int row, int col,
                          int num_bits, int is_row_wise, int num_alpha_groups, const float* q_bias) {
    if (!out || !bW || !A) return LUTGEMM_ERR_NULL;
    int N, K;
    int rc = check_shape(row, col, num_bits, is_row_wise, num_alpha_groups, &N, &K);
    if (rc != LUTGEMM_OK) return rc;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    lutgemm_weight* w = new (std::nothrow) lutgemm_weight();
    if (!w) return LUTGEMM_ERR_TOO_LARGE;
    w->N = N; w->K = K; w->q = num_bits; w->G = num_alpha_groups; w->g = K / num_alpha_groups;
    w->row_wise = is_row_wise != 0; w->device = dev; w->owns = true;
    const size_t n_words = (size_t)(K / 32) * num_bits * N;
    const size_t n_alpha = (size_t)w->G * num_bits * N;
    const size_t n_bias = (size_t)w->G * N;
#define LG_TRY(call) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) { g_last_cuda = (int)e__; lutgemm_weight_destroy(w); \
        return (e__ == cudaErrorNoDevice) ? LUTGEMM_ERR_NO_DEVICE : LUTGEMM_ERR_CUDA; } } while (0)
    LG_TRY(cudaMalloc(&w->bW, n_words * sizeof(uint32_t)));
    LG_TRY(cudaMalloc(&w->alpha, n_alpha * sizeof(__half)));
    LG_TRY(cudaMemcpy(w->bW, bW, n_words * sizeof(uint32_t), cudaMemcpyHostToDevice));
    {
        std::vector<__half> tmp(n_alpha);
        for (size_t i = 0; i < n_alpha; i++) tmp[i] = __float2half_rn(A[i]);
        LG_TRY(cudaMemcpy(w->alpha, tmp.data(), n_alpha * sizeof(__half), cudaMemcpyHostToDevice));
    }
    if (q_bias) {
        LG_TRY(cudaMalloc(&w->q_bias, n_bias * sizeof(__half)));
        std::vector<__half> tmp(n_bias);
        for (size_t i = 0; i < n_bias; i++) tmp[i] = __float2half_rn(q_bias[i]);
        LG_TRY(cudaMemcpy(w->q_bias, tmp.data(), n_bias * sizeof(__half), cudaMemcpyHostToDevice));
    }
    return finish_create(w, out);
}

int lutgemm_weight_create_device(lutgemm_weight_t* out, const uint32_t* d_bW, const void* d_alpha,
                                 const void* d_q_bias, int row, int col, int num_bits, int is_row_wise,
                                 int num_alpha_groups, int copy) {
    if (!out || !d_bW || !d_alpha) return LUTGEMM_ERR_NULL;
    int N, K;
    int rc = check_shape(row, col, num_bits, is_row_wise, num_alpha_groups, &N, &K);
    if (rc != LUTGEMM_OK) return rc;
    if (((uintptr_t)d_bW & 15) || ((uintptr_t)d_alpha & 15) || ((uintptr_t)d_q_bias & 15)) return LUTGEMM_ERR_ALIGN;
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    lutgemm_weight* w = new (std::nothrow) lutgemm_weight();
    if (!w) return LUTGEMM_ERR_TOO_LARGE;
    w->N = N; w->K = K; w->q = num_bits; w->G = num_alpha_groups; w->g = K / num_alpha_groups;
    w->row_wise = is_row_wise != 0; w->device = dev;
    const size_t n_words = (size_t)(K / 32) * num_bits * N;
    const size_t n_alpha = (size_t)w->G * num_bits * N;
    const size_t n_bias = (size_t)w->G * N;
    if (!copy) {
        w->owns = false;
        w->bW = const_cast<uint32_t*>(d_bW);
        w->alpha = (__half*)const_cast<void*>(d_alpha);
        w->q_bias = (__half*)const_cast<void*>(d_q_bias);
    } else {
        w->owns = true;
        LG_TRY(cudaMalloc(&w->bW, n_words * sizeof(uint32_t)));
        LG_TRY(cudaMalloc(&w->alpha, n_alpha * sizeof(__half)));
        LG_TRY(cudaMemcpy(w->bW, d_bW, n_words * sizeof(uint32_t), cudaMemcpyDeviceToDevice));
        LG_TRY(cudaMemcpy(w->alpha, d_alpha, n_alpha * sizeof(__half), cudaMemcpyDeviceToDevice));
        if (d_q_bias) {
            LG_TRY(cudaMalloc(&w->q_bias, n_bias * sizeof(__half)));
            LG_TRY(cudaMemcpy(w->q_bias, d_q_bias, n_bias * sizeof(__half), cudaMemcpyDeviceToDevice));
        }
    }
    return finish_create(w, out);
}

int lutgemm_weight_destroy(lutgemm_weight_t w) {
    if (!w) return LUTGEMM_OK;
    if (w->owns) {
        if (w->bW) cudaFree(w->bW);
        if (w->alpha) cudaFree(w->alpha);
        if (w->q_bias) cudaFree(w->q_bias);
    }
    free_workspace_buffers(&w->own);
    if (w->h_done) cudaFreeHost((void*)w->h_done);
    if (w->host_graph) cudaGraphExecDestroy(w->host_graph);
    if (w->host_stream) cudaStreamDestroy(w->host_stream);
    if (w->h_stage_in) cudaFreeHost(w->h_stage_in);
    if (w->d_stage_in) cudaFree(w->d_stage_in);
    if (w->d_stage_out) cudaFree(w->d_stage_out);
    delete w;
    return LUTGEMM_OK;
}

int lutgemm_weight_describe(lutgemm_weight_t w, lutgemm_weight_desc* d) {
    if (!w || !d) return LUTGEMM_ERR_NULL;
    d->bWeight = w->bW; d->alpha = w->alpha; d->q_bias = w->q_bias;
    d->num_groups = w->G; d->group_size = w->g; d->mSize = w->N; d->kSize = w->K; d->nb = w->q;
    d->is_row_wise_quantize = w->row_wise ? 1 : 0; d->device = w->device;
    return LUTGEMM_OK;
}

int lutgemm_matmul(void* out, const void* in, lutgemm_weight_t w, int m, void* stream) {
    if (!out) return LUTGEMM_ERR_NULL;
    return matmul_impl((__half*)out, nullptr, in, w, m, nullptr, stream);
}

int lutgemm_matmul_f32(float* out, const void* in, lutgemm_weight_t w, int m, void* stream) {
    if (!out) return LUTGEMM_ERR_NULL;
    return matmul_impl(nullptr, out, in, w, m, nullptr, stream);
}

int lutgemm_matmul_ws(void* out, const void* in, lutgemm_weight_t w, int m, lutgemm_workspace_t ws, void* stream) {
    if (!out) return LUTGEMM_ERR_NULL;
    return matmul_impl((__half*)out, nullptr, in, w, m, ws, stream);
}

int lutgemm_matmul_f32_ws(float* out, const void* in, lutgemm_weight_t w, int m, lutgemm_workspace_t ws, void* stream) {
    if (!out) return LUTGEMM_ERR_NULL;
    return matmul_impl(nullptr, out, in, w, m, ws, stream);
}

int lutgemm_workspace_create(lutgemm_workspace_t* out, int max_n, int max_k, int max_m) {
    if (!out) return LUTGEMM_ERR_NULL;
    if (max_n < 1 || max_k < 32 || max_m < 1 || max_m > kMaxBatch) return LUTGEMM_ERR_SHAPE;
    lutgemm_workspace* ws = new (std::nothrow) lutgemm_workspace();
    if (!ws) return LUTGEMM_ERR_TOO_LARGE;
    int rc = fill_workspace(ws, max_n, max_k, max_m >= 2 ? max_m : 0);
    if (rc != LUTGEMM_OK) {
        free_workspace_buffers(ws);
        delete ws;
        return rc;
    }
    *out = ws;
    return LUTGEMM_OK;
}

int lutgemm_workspace_destroy(lutgemm_workspace_t ws) {
    if (!ws) return LUTGEMM_OK;
    free_workspace_buffers(ws);
    delete ws;
    return LUTGEMM_OK;
}

int lutgemm_workspace_status(lutgemm_workspace_t ws, int* status) {
    if (!ws || !status) return LUTGEMM_ERR_NULL;
    LG_CUDA(cudaMemcpy(status, ws->status, sizeof(int), cudaMemcpyDeviceToHost));
    return LUTGEMM_OK;
}

int lutgemm_workspace_set_ordered(lutgemm_workspace_t ws, int mode) {
    if (!ws) return LUTGEMM_ERR_NULL;
    if (mode < -1 || mode > 1) return LUTGEMM_ERR_SHAPE;
    ws->ordered.store(mode);
    return LUTGEMM_OK;
}

int lutgemm_weight_set_ordered(lutgemm_weight_t w, int mode) {
    if (!w) return LUTGEMM_ERR_NULL;
    return lutgemm_workspace_set_ordered(&w->own, mode);
}

int lutgemm_weight_reserve_batch(lutgemm_weight_t w, int m) {
    if (!w) return LUTGEMM_ERR_NULL;
    if (m < 1 || m > kMaxBatch) return LUTGEMM_ERR_BATCH;
    lutgemm_workspace* ws = &w->own;
    const int rows = tc_rows_for(m);
    if (m >= 2 && ws->tc_rows < rows) {
        if (ws->tc_partial) LG_CUDA(cudaFree(ws->tc_partial));
        ws->tc_partial = nullptr; ws->tc_rows = 0;
        LG_CUDA(cudaMalloc(&ws->tc_partial, (size_t)rows * w->N * sizeof(float)));
        LG_CUDA(cudaMemset(ws->tc_partial, 0, (size_t)rows * w->N * sizeof(float)));
        ws->tc_rows = rows;
    }
    // transposed copies of the (output, nqW, input, n) overload
    int rc = grow(&ws->t_in, &ws->t_in_bytes, (size_t)m * w->K * sizeof(__half), nullptr);
    if (rc == LUTGEMM_OK) rc = grow(&ws->t_out, &ws->t_out_bytes, (size_t)m * w->N * sizeof(__half), nullptr);
    return rc;
}

int lutgemm_matmul_wx(void* out, lutgemm_weight_t w, const void* in, int n, void* stream) {
    if (!out || !w || !in) return LUTGEMM_ERR_NULL;
    if (n < 1 || n > kMaxBatch) return LUTGEMM_ERR_BATCH;
    if (n == 1) return matmul_impl((__half*)out, nullptr, in, w, 1, nullptr, stream);   // [K][1] and [N][1] are plain vectors
    if (((uintptr_t)in & 15) || ((uintptr_t)out & 15)) return LUTGEMM_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    lutgemm_workspace* ws = &w->own;
    int rc = grow(&ws->t_in, &ws->t_in_bytes, (size_t)n * w->K * sizeof(__half), st);
    if (rc == LUTGEMM_OK) rc = grow(&ws->t_out, &ws->t_out_bytes, (size_t)n * w->N * sizeof(__half), st);
    if (rc != LUTGEMM_OK) return rc;
    // input [K][n] -> [n][K]; X.W; output [n][N] -> [N][n]
    dim3 tb(32, 8);
    transpose_fp16_kernel<<<dim3((n + 31) / 32, (w->K + 31) / 32), tb, 0, st>>>((const __half*)in, (__half*)ws->t_in, w->K, n);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    rc = matmul_impl((__half*)ws->t_out, nullptr, ws->t_in, w, n, ws, stream);
    if (rc != LUTGEMM_OK) return rc;
    transpose_fp16_kernel<<<dim3((w->N + 31) / 32, (n + 31) / 32), tb, 0, st>>>((const __half*)ws->t_out, (__half*)out, n, w->N);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

// The copy-in / run / copy-out sequence of lutgemm_matmul_host on `st`.  d_in / d_out: device aliases of the buffers
// when both are page-locked (then no copy engine: a fetch kernel, the result stored straight to the host buffer by the
// kernels' last CTAs, and the completion word), else null.
static int host_sequence(lutgemm_weight_t w, void* out_host, const void* in_host, int m, cudaStream_t st, void* d_in, void* d_out) {
    if (d_in && d_out) {
        const int n16 = (int)((size_t)m * w->K * sizeof(__half) / 16);
        host_fetch_kernel<<<(n16 + 1023) / 1024 > 8 ? 8 : (n16 + 1023) / 1024, 1024, 0, st>>>((const uint4*)d_in, (uint4*)w->d_stage_in, n16);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        int rc = matmul_impl((__half*)d_out, nullptr, w->d_stage_in, w, m, nullptr, st);
        if (rc != LUTGEMM_OK) return rc;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1); cfg.blockDim = dim3(1); cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        LG_CUDA(cudaLaunchKernelEx(&cfg, host_done_kernel, w->d_done, 1u));
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return LUTGEMM_OK;
    }
    LG_CUDA(cudaMemcpyAsync(w->d_stage_in, in_host, (size_t)m * w->K * sizeof(__half), cudaMemcpyHostToDevice, st));
    int rc = matmul_impl((__half*)w->d_stage_out, nullptr, w->d_stage_in, w, m, nullptr, st);
    if (rc != LUTGEMM_OK) return rc;
    LG_CUDA(cudaMemcpyAsync(out_host, w->d_stage_out, (size_t)m * w->N * sizeof(__half), cudaMemcpyDeviceToHost, st));
    return LUTGEMM_OK;
}

// Waits for the completion word (bounded: a few seconds of polling, then the ordinary synchronisation, which also
// reports a failed kernel).
static int host_wait(lutgemm_weight_t w, cudaStream_t st, bool pinned) {
    if (pinned) {
        for (long it = 0; it < 400000000L; it++) {
            if (*w->h_done == 1u) return LUTGEMM_OK;
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        }
    }
    LG_CUDA(cudaStreamSynchronize(st));
    return LUTGEMM_OK;
}

static int host_prepare(lutgemm_weight_t w, int m) {
    if (!w->host_stream) LG_CUDA(cudaStreamCreateWithFlags(&w->host_stream, cudaStreamNonBlocking));
    if (w->stage_rows < (size_t)m) {
        if (w->host_graph) { cudaGraphExecDestroy(w->host_graph); w->host_graph = nullptr; }
        if (w->d_stage_in) cudaFree(w->d_stage_in);
        if (w->d_stage_out) cudaFree(w->d_stage_out);
        w->d_stage_in = w->d_stage_out = nullptr;
        w->stage_rows = 0;
        LG_CUDA(cudaMalloc(&w->d_stage_in, (size_t)m * w->K * sizeof(__half)));
        LG_CUDA(cudaMalloc(&w->d_stage_out, (size_t)m * w->N * sizeof(__half)));
        w->stage_rows = (size_t)m;
        int rc = lutgemm_weight_reserve_batch(w, m);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

// Device alias of a page-locked host pointer, or null when the memory is pageable / not 16-byte aligned.
static void* pinned_alias(const void* p) {
    if ((uintptr_t)p & 15) return nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

int lutgemm_matmul_host(void* out_host, const void* in_host, lutgemm_weight_t w, int m) {
    if (!w || !out_host || !in_host) return LUTGEMM_ERR_NULL;
    if (m < 1 || m > kMaxBatch) return LUTGEMM_ERR_BATCH;
    int rc = host_prepare(w, m);
    if (rc != LUTGEMM_OK) return rc;
    cudaStream_t st = w->host_stream;
    if (w->host_graph && w->hg_in == in_host && w->hg_out == out_host && w->hg_m == m) {
        // the same buffers and batch as last time: one graph launch replays the whole call
        if (w->hg_pinned) *w->h_done = 0u;
        LG_CUDA(cudaGraphLaunch(w->host_graph, st));
        g_launches.fetch_add((unsigned long long)w->hg_launches, std::memory_order_relaxed);
        return host_wait(w, st, w->hg_pinned);
    }
    void* d_in = pinned_alias(in_host);
    void* d_out = pinned_alias(out_host);
    if (!w->h_done) {
        void* hp = nullptr;
        if (cudaHostAlloc(&hp, 64, cudaHostAllocMapped) == cudaSuccess) {
            w->h_done = (volatile unsigned*)hp;
            void* dp = nullptr;
            if (cudaHostGetDevicePointer(&dp, hp, 0) == cudaSuccess) w->d_done = (unsigned*)dp;
        } else {
            (void)cudaGetLastError();
        }
    }
    const bool pinned = d_in && d_out && w->h_done && w->d_done && ((size_t)m * w->K * sizeof(__half)) % 16 == 0;
    if (!pinned) d_in = d_out = nullptr;
    if (pinned) *w->h_done = 0u;
    rc = host_sequence(w, out_host, in_host, m, st, d_in, d_out);
    if (rc != LUTGEMM_OK) return rc;
    rc = host_wait(w, st, pinned);
    if (rc != LUTGEMM_OK) return rc;
    // record the sequence for the next call with these buffers (capture runs nothing)
    if (w->host_graph) { cudaGraphExecDestroy(w->host_graph); w->host_graph = nullptr; }
    const unsigned long long before = g_launches.load();
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int rc2 = host_sequence(w, out_host, in_host, m, st, d_in, d_out);
        const cudaError_t e = cudaStreamEndCapture(st, &graph);
        if (rc2 == LUTGEMM_OK && e == cudaSuccess && graph &&
            cudaGraphInstantiate(&w->host_graph, graph, 0) == cudaSuccess) {
            w->hg_in = in_host; w->hg_out = out_host; w->hg_m = m; w->hg_pinned = pinned;
            w->hg_launches = (int)(g_launches.load() - before);
        } else {
            w->host_graph = nullptr;
            (void)cudaGetLastError();
        }
        if (graph) cudaGraphDestroy(graph);
        g_launches.store(before);                 // captured launches did not run
    } else {
        (void)cudaGetLastError();
    }
    return LUTGEMM_OK;
}

int lutgemm_matmul_host_profile(void* out_host, const void* in_host, lutgemm_weight_t w, int m, float* us4) {
    if (!w || !out_host || !in_host || !us4) return LUTGEMM_ERR_NULL;
    if (m < 1 || m > kMaxBatch) return LUTGEMM_ERR_BATCH;
    int rc = host_prepare(w, m);
    if (rc != LUTGEMM_OK) return rc;
    cudaStream_t st = w->host_stream;
    cudaEvent_t ev[4];
    for (int i = 0; i < 4; i++) LG_CUDA(cudaEventCreate(&ev[i]));
    LG_CUDA(cudaEventRecord(ev[0], st));
    LG_CUDA(cudaMemcpyAsync(w->d_stage_in, in_host, (size_t)m * w->K * sizeof(__half), cudaMemcpyHostToDevice, st));
    LG_CUDA(cudaEventRecord(ev[1], st));
    rc = matmul_impl((__half*)w->d_stage_out, nullptr, w->d_stage_in, w, m, nullptr, st);
    if (rc == LUTGEMM_OK) {
        LG_CUDA(cudaEventRecord(ev[2], st));
        LG_CUDA(cudaMemcpyAsync(out_host, w->d_stage_out, (size_t)m * w->N * sizeof(__half), cudaMemcpyDeviceToHost, st));
        LG_CUDA(cudaEventRecord(ev[3], st));
        LG_CUDA(cudaStreamSynchronize(st));
        float ms = 0.f;
        for (int i = 0; i < 3; i++) { LG_CUDA(cudaEventElapsedTime(&ms, ev[i], ev[i + 1])); us4[i] = ms * 1e3f; }
        LG_CUDA(cudaEventElapsedTime(&ms, ev[0], ev[3]));
        us4[3] = ms * 1e3f;
    }
    for (int i = 0; i < 4; i++) cudaEventDestroy(ev[i]);
    return rc;
}

int lutgemm_matvec_static_scratch(void* out_fp16, const void* in_fp16, const uint32_t* d_bW, const void* d_alpha_fp16,
                                  const void* d_q_bias_fp16, int K, int N, int num_bits, int num_alpha_groups,
                                  void* stream) {
    if (!out_fp16 || !in_fp16 || !d_bW || !d_alpha_fp16) return LUTGEMM_ERR_NULL;
    int n_chk = 0, k_chk = 0;
    int rc = check_shape(K, N, num_bits, 0, num_alpha_groups, &n_chk, &k_chk);
    if (rc != LUTGEMM_OK) return rc;
    if (N > kStaticMaxN) return LUTGEMM_ERR_TOO_LARGE;          // the reduction row holds kStaticMaxN floats
    if (((uintptr_t)out_fp16 & 15) || ((uintptr_t)in_fp16 & 15) || ((uintptr_t)d_bW & 15) ||
        ((uintptr_t)d_alpha_fp16 & 15) || ((uintptr_t)d_q_bias_fp16 & 15))
        return LUTGEMM_ERR_ALIGN;
    // A container that lives on this stack frame only: it borrows the caller's arrays and the static scratch.
    lutgemm_weight w;
    w.bW = const_cast<uint32_t*>(d_bW);
    w.alpha = (__half*)const_cast<void*>(d_alpha_fp16);
    w.q_bias = (__half*)const_cast<void*>(d_q_bias_fp16);
    w.N = N; w.K = K; w.q = num_bits; w.G = num_alpha_groups; w.g = K / num_alpha_groups;
    w.owns = false;
    make_tensor_maps(&w, false);                                // the two matvec descriptors only
    if (!w.tma_ok) return LUTGEMM_ERR_SHAPE;                    // needs N % 8 == 0 and a group size the TMA kernel takes
    unsigned char* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != LUTGEMM_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // The array keeps whatever the last call left in it: start from zero sums, counters and status.
    const int nslabs = (K + lg::kSlab2 - 1) / lg::kSlab2;
    const int n_tile = choose_ntile(N, nslabs, 1, lg::kStageCols);
    const int tiles = (N + n_tile - 1) / n_tile;
    LG_CUDA(cudaMemsetAsync(scratch, 0, (size_t)N * sizeof(float), st));
    LG_CUDA(cudaMemsetAsync(scratch + kStaticRowBytes, 0, (size_t)tiles * sizeof(unsigned), st));
    LG_CUDA(cudaMemsetAsync(scratch + kStaticRowBytes + kStaticCounterBytes, 0, sizeof(int), st));
    lg::Gemv2Params p = {};
    p.bW = w.bW; p.alpha = w.alpha; p.q_bias = w.q_bias; p.x = (const __half*)in_fp16;
    p.partial = (float*)scratch;
    p.counters = (unsigned*)(scratch + kStaticRowBytes);
    p.status = (int*)(scratch + kStaticRowBytes + kStaticCounterBytes);
    p.y16 = (__half*)out_fp16; p.y32 = nullptr;
    p.N = N; p.K = K; p.q = num_bits; p.g = w.g;
    p.n_tile = n_tile; p.nslabs = nslabs; p.a_rows = w.a_rows;
    p.ordered = 0;                                              // one reduction row is all the scratch holds
    dim3 grid(tiles, nslabs);
    const bool bias = d_q_bias_fp16 != nullptr;
    if (w.g % 128 == 0) return launch_gemv_tma<2>(&w, p, grid, bias, st);
    return launch_gemv_tma<1>(&w, p, grid, bias, st);
}

int lutgemm_static_scratch_status(int* status) {
    if (!status) return LUTGEMM_ERR_NULL;
    unsigned char* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != LUTGEMM_OK) return rc;
    LG_CUDA(cudaMemcpy(status, scratch + kStaticRowBytes + kStaticCounterBytes, sizeof(int), cudaMemcpyDeviceToHost));
    return LUTGEMM_OK;
}

int lutgemm_matvec_tiles(lutgemm_weight_t w, int* tiles) {
    if (!w || !tiles) return LUTGEMM_ERR_NULL;
    if (!w->tma_ok) return LUTGEMM_ERR_SHAPE;
    int nslabs = 0, n_tile = 0;
    gemv_tma_geometry(w, &nslabs, &n_tile, tiles);
    return LUTGEMM_OK;
}

int lutgemm_matvec_tp(const void* in_fp16, lutgemm_weight_t w, const lutgemm_tp_link* link, void* out_fp16,
                      float* out_f32, void* stream) {
    if (!w || !link) return LUTGEMM_ERR_NULL;
    if (!w->tma_ok) return LUTGEMM_ERR_SHAPE;
    if (link->world < 1 || link->world > 8 || link->x_mode < 0 || link->x_mode > 2 || link->out_mode < 0 || link->out_mode > 2)
        return LUTGEMM_ERR_SHAPE;
    if (link->x_mode != 2 && !in_fp16) return LUTGEMM_ERR_NULL;
    if (link->x_mode == 2 && (!link->x_slots || (link->x_off % 8) || (link->x_slot_stride % 4))) return LUTGEMM_ERR_ALIGN;
    if (link->x_mode != 0 && (!link->flag_in || !link->done_counter)) return LUTGEMM_ERR_NULL;
    if (link->out_mode == 0 && !out_fp16 && !out_f32) return LUTGEMM_ERR_NULL;
    if (((uintptr_t)in_fp16 & 15) || ((uintptr_t)out_fp16 & 15) || ((uintptr_t)out_f32 & 15)) return LUTGEMM_ERR_ALIGN;
    lg::TpLink t = {};
    t.x_mode = link->x_mode; t.out_mode = link->out_mode; t.world = link->world; t.out_off = link->out_off;
    t.x_slots = link->x_slots; t.x_slot_stride = link->x_slot_stride; t.x_off = link->x_off;
    t.flag_in = link->flag_in; t.flag_target = link->flag_target; t.done_counter = link->done_counter;
    for (int r = 0; r < link->world; r++) {
        if (link->out_mode == 1 && (!link->out16[r] || ((uintptr_t)link->out16[r] & 15) || (link->out_off % 8))) return LUTGEMM_ERR_ALIGN;
        if (link->out_mode == 2 && (!link->out32[r] || ((uintptr_t)link->out32[r] & 15))) return LUTGEMM_ERR_ALIGN;
        if (link->out_mode != 0 && !link->flag_out[r]) return LUTGEMM_ERR_NULL;
        t.out16[r] = (__half*)link->out16[r]; t.out32[r] = link->out32[r]; t.flag_out[r] = link->flag_out[r];
    }
    return launch_gemv_tma_any(w, &w->own, (const __half*)in_fp16, (__half*)out_fp16, out_f32, &t, (cudaStream_t)stream);
}

int lutgemm_tp_finalize(void* out_fp16, float* out_f32, const float* slots, int slot_stride, int world, int n,
                        unsigned* flag_in, unsigned flag_target, lutgemm_weight_t status_owner, void* stream) {
    if ((!out_fp16 && !out_f32) || !slots || !flag_in || !status_owner) return LUTGEMM_ERR_NULL;
    if (world < 1 || world > 8 || n < 1) return LUTGEMM_ERR_SHAPE;
    lg::tp_finalize_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((__half*)out_fp16, out_f32, slots, slot_stride, world, n,
                                                                 flag_in, flag_target, status_owner->own.status);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_ipc_alloc(size_t bytes, void** dptr, void* handle64) {
    if (!dptr || !handle64 || bytes == 0) return LUTGEMM_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    LG_CUDA(cudaMalloc(&p, bytes));
    LG_CUDA(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { g_last_cuda = (int)e; cudaFree(p); return LUTGEMM_ERR_CUDA; }
    std::memcpy(handle64, &h, 64);
    *dptr = p;
    return LUTGEMM_OK;
}

int lutgemm_ipc_open(const void* handle64, void** dptr) {
    if (!handle64 || !dptr) return LUTGEMM_ERR_NULL;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    LG_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return LUTGEMM_OK;
}

int lutgemm_ipc_close(void* dptr) {
    if (!dptr) return LUTGEMM_OK;
    LG_CUDA(cudaIpcCloseMemHandle(dptr));
    return LUTGEMM_OK;
}

int lutgemm_ipc_free(void* dptr) {
    if (!dptr) return LUTGEMM_OK;
    LG_CUDA(cudaFree(dptr));
    return LUTGEMM_OK;
}

// ---------------------------------------------------------------------------------------------------------
// sequences of matvecs in one persistent kernel (gemv_seq.cuh)
int lutgemm_sequence_create(lutgemm_sequence_t* out, const lutgemm_seq_op* ops, int n_ops,
                            const lutgemm_seq_buffer* buffers, int n_buffers, int rank, int world) {
    if (!out || !ops || (n_buffers > 0 && !buffers)) return LUTGEMM_ERR_NULL;
    if (n_ops < 1 || n_buffers < 0 || world < 1 || world > 8 || rank < 0 || rank >= world) return LUTGEMM_ERR_SHAPE;
    if (n_ops > lg::kSeqMaxOps) return LUTGEMM_ERR_TOO_LARGE;
    for (int b = 0; b < n_buffers; b++)
        if ((buffers[b].kind != 1 && buffers[b].kind != 2) || buffers[b].n < 4 || buffers[b].n % 4 != 0) return LUTGEMM_ERR_SHAPE;
    const lutgemm_weight* first = nullptr;
    for (int i = 0; i < n_ops; i++) {
        const lutgemm_seq_op& o = ops[i];
        if (o.in_kind < 0 || o.in_kind > 2 || o.out_kind < 0 || o.out_kind > 2) return LUTGEMM_ERR_SHAPE;
        const int K = o.w ? o.w->K : o.n, N = o.w ? o.w->N : o.n;
        if (!o.w && (o.in_kind != 2 || o.out_kind != 0 || o.n < 4 || o.n % 4 != 0)) return LUTGEMM_ERR_SHAPE;
        if (o.in_kind == 0) {
            if (!o.x_ext) return LUTGEMM_ERR_NULL;
            if ((uintptr_t)o.x_ext & 15) return LUTGEMM_ERR_ALIGN;
        } else {
            if (o.in_buf < 0 || o.in_buf >= n_buffers || buffers[o.in_buf].kind != o.in_kind) return LUTGEMM_ERR_SHAPE;
            if (o.in_off < 0 || o.in_off % 4 != 0 || o.in_off + K > buffers[o.in_buf].n) return LUTGEMM_ERR_SHAPE;
        }
        if (o.out_kind == 0) {
            if (!o.y_ext) return LUTGEMM_ERR_NULL;
            if ((uintptr_t)o.y_ext & 15) return LUTGEMM_ERR_ALIGN;
        } else {
            if (o.out_buf < 0 || o.out_buf >= n_buffers || buffers[o.out_buf].kind != o.out_kind) return LUTGEMM_ERR_SHAPE;
            if (o.out_off < 0 || o.out_off % 4 != 0 || o.out_off + N > buffers[o.out_buf].n) return LUTGEMM_ERR_SHAPE;
        }
        if (o.w) {
            if (!o.w->tma_ok) return LUTGEMM_ERR_SHAPE;
            if (!first) first = o.w;
            if (o.w->a_rows != first->a_rows || (o.w->g % 128 == 0) != (first->g % 128 == 0) ||
                (o.w->q_bias != nullptr) != (first->q_bias != nullptr))
                return LUTGEMM_ERR_SHAPE;
        }
    }
    int dev = 0;
    LG_CUDA(cudaGetDevice(&dev));
    lutgemm_sequence* s = new (std::nothrow) lutgemm_sequence();
    if (!s) return LUTGEMM_ERR_TOO_LARGE;
    s->rank = rank; s->world = world; s->device = dev;
    s->ops.assign(ops, ops + n_ops);
    if (n_buffers) s->bufs.assign(buffers, buffers + n_buffers);
    if (first) { s->a_rows = first->a_rows; s->wpg = first->g % 128 == 0 ? 2 : 1; s->bias = first->q_bias != nullptr; }
    size_t off = 0;
    for (int b = 0; b < n_buffers; b++) { s->buf_off.push_back(off); off += seq_buffer_bytes(buffers[b], world); }
    s->xchg_bytes = off ? off : 256;
#define LG_SEQ_TRY(call) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) { g_last_cuda = (int)e__; lutgemm_sequence_destroy(s); \
        return (e__ == cudaErrorNoDevice || e__ == cudaErrorInsufficientDriver) ? LUTGEMM_ERR_NO_DEVICE : LUTGEMM_ERR_CUDA; } } while (0)
    LG_SEQ_TRY(cudaMalloc(&s->xchg[rank], s->xchg_bytes));
    LG_SEQ_TRY(cudaMemset(s->xchg[rank], 0, s->xchg_bytes));           // step numbers start at 1: nothing is valid yet
    s->mapped[rank] = true;
    // geometry and workspace of every matvec
    s->h_ops.resize(n_ops);
    size_t n_partial = 0, n_counters = 0;
    s->grid = sm_count();
    for (int i = 0; i < n_ops; i++) {
        lg::SeqOpDev& d = s->h_ops[i];
        std::memset(&d, 0, sizeof(d));
        const lutgemm_seq_op& o = ops[i];
        if (!o.w) {
            d.reduce_only = 1; d.N = d.K = o.n; d.items = (o.n + lg::kSlab2 - 1) / lg::kSlab2;
        } else {
            d.tmW = o.w->tmW; d.tmA = o.w->tmA; d.q_bias = o.w->q_bias;
            d.N = o.w->N; d.K = o.w->K; d.q = o.w->q; d.g = o.w->g;
            gemv_tma_geometry(o.w, &d.nslabs, &d.n_tile, &d.tiles);
            d.items = d.tiles * d.nslabs;
            n_partial += ((size_t)d.N + 63) / 64 * 64;
            n_counters += (size_t)d.tiles;
        }
        d.in_kind = o.in_kind; d.out_kind = o.out_kind; d.out_world = world;
        d.in_rows = world;
        if (o.in_kind == 2) d.in_row_lines = s->bufs[o.in_buf].n / 2;
    }
    LG_SEQ_TRY(cudaMalloc(&s->partial, (n_partial + 64) * sizeof(float)));
    LG_SEQ_TRY(cudaMemset(s->partial, 0, (n_partial + 64) * sizeof(float)));
    LG_SEQ_TRY(cudaMalloc(&s->counters, (n_counters + 64) * sizeof(unsigned)));
    LG_SEQ_TRY(cudaMemset(s->counters, 0, (n_counters + 64) * sizeof(unsigned)));
    LG_SEQ_TRY(cudaMalloc(&s->words, 64));
    {
        const unsigned init[4] = {1u, 0u, 0u, 0u};
        LG_SEQ_TRY(cudaMemcpy(s->words, init, sizeof(init), cudaMemcpyHostToDevice));
    }
    LG_SEQ_TRY(cudaMalloc(&s->d_ops, (size_t)n_ops * sizeof(lg::SeqOpDev)));
    size_t po = 0, co = 0;
    for (int i = 0; i < n_ops; i++) {
        lg::SeqOpDev& d = s->h_ops[i];
        if (d.reduce_only) continue;
        d.partial = s->partial + po; po += ((size_t)d.N + 63) / 64 * 64;
        d.counters = s->counters + co; co += (size_t)d.tiles;
    }
#undef LG_SEQ_TRY
    *out = s;
    if (world == 1) return lutgemm_sequence_commit(s);
    return LUTGEMM_OK;
}

int lutgemm_sequence_export(lutgemm_sequence_t s, void* handle64) {
    if (!s || !handle64) return LUTGEMM_ERR_NULL;
    cudaIpcMemHandle_t h;
    LG_CUDA(cudaIpcGetMemHandle(&h, s->xchg[s->rank]));
    std::memcpy(handle64, &h, 64);
    return LUTGEMM_OK;
}

int lutgemm_sequence_connect(lutgemm_sequence_t s, int peer_rank, const void* handle64) {
    if (!s || !handle64) return LUTGEMM_ERR_NULL;
    if (peer_rank < 0 || peer_rank >= s->world || peer_rank == s->rank || s->mapped[peer_rank]) return LUTGEMM_ERR_SHAPE;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* ptr = nullptr;
    LG_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    s->xchg[peer_rank] = (unsigned char*)ptr;
    s->mapped[peer_rank] = true;
    s->committed = false;
    return LUTGEMM_OK;
}

int lutgemm_sequence_commit(lutgemm_sequence_t s) {
    if (!s) return LUTGEMM_ERR_NULL;
    for (int r = 0; r < s->world; r++)
        if (!s->mapped[r]) return LUTGEMM_ERR_NULL;
    for (size_t i = 0; i < s->ops.size(); i++) {
        const lutgemm_seq_op& o = s->ops[i];
        lg::SeqOpDev& d = s->h_ops[i];
        if (o.in_kind == 0) d.in_ptr = o.x_ext;
        else d.in_ptr = s->xchg[s->rank] + s->buf_off[o.in_buf] + (size_t)(o.in_off / (o.in_kind == 1 ? 4 : 2)) * 16;
        for (int r = 0; r < 8; r++) d.out_ptr[r] = nullptr;
        if (o.out_kind == 0) d.out_ptr[0] = o.y_ext;
        else if (o.out_kind == 1)
            for (int r = 0; r < s->world; r++) d.out_ptr[r] = s->xchg[r] + s->buf_off[o.out_buf] + (size_t)(o.out_off / 4) * 16;
        else
            for (int r = 0; r < s->world; r++)
                d.out_ptr[r] = s->xchg[r] + s->buf_off[o.out_buf] + ((size_t)s->rank * (s->bufs[o.out_buf].n / 2) + o.out_off / 2) * 16;
    }
    LG_CUDA(cudaMemcpy(s->d_ops, s->h_ops.data(), s->h_ops.size() * sizeof(lg::SeqOpDev), cudaMemcpyHostToDevice));
    if (!s->params) s->params = new (std::nothrow) lg::SeqParams();
    if (!s->params) return LUTGEMM_ERR_TOO_LARGE;
    lg::SeqParams& p = *s->params;
    std::memset(&p, 0, sizeof(p));
    p.ops = s->d_ops; p.n_ops = (int)s->h_ops.size(); p.a_rows = s->a_rows;
    p.epoch = s->words; p.done = s->words + 1; p.status = (int*)(s->words + 2); p.wait_ns = s->wait_ns;
    for (size_t i = 0; i < s->h_ops.size(); i++) {
        const lg::SeqOpDev& d = s->h_ops[i];
        p.geo[i] = lg::SeqGeo{d.N, d.K, d.n_tile, d.tiles, d.nslabs, d.q, d.g, d.reduce_only};
    }
    s->committed = true;
    return LUTGEMM_OK;
}

int lutgemm_sequence_run(lutgemm_sequence_t s, void* stream) {
    if (!s) return LUTGEMM_ERR_NULL;
    if (!s->committed) return LUTGEMM_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (s->wpg == 2) return s->bias ? launch_sequence<2, true>(s, st) : launch_sequence<2, false>(s, st);
    return s->bias ? launch_sequence<1, true>(s, st) : launch_sequence<1, false>(s, st);
}

int lutgemm_sequence_status(lutgemm_sequence_t s, int* status) {
    if (!s || !status) return LUTGEMM_ERR_NULL;
    LG_CUDA(cudaMemcpy(status, s->words + 2, sizeof(int), cudaMemcpyDeviceToHost));
    return LUTGEMM_OK;
}

int lutgemm_sequence_clear_status(lutgemm_sequence_t s) {
    if (!s) return LUTGEMM_ERR_NULL;
    LG_CUDA(cudaDeviceSynchronize());
    LG_CUDA(cudaMemset(s->words + 2, 0, sizeof(int)));
    return LUTGEMM_OK;
}

int lutgemm_sequence_set_wait_limit(lutgemm_sequence_t s, int milliseconds) {
    if (!s) return LUTGEMM_ERR_NULL;
    if (milliseconds < 1 || milliseconds > 60000) return LUTGEMM_ERR_SHAPE;
    s->wait_ns = (unsigned long long)milliseconds * 1000000ull;
    return LUTGEMM_OK;
}

int lutgemm_sequence_set_trace(lutgemm_sequence_t s, unsigned long long* d_stamps, size_t entries) {
    if (!s) return LUTGEMM_ERR_NULL;
    if (d_stamps && entries < s->h_ops.size() * (size_t)s->grid * 4) return LUTGEMM_ERR_SHAPE;
    s->trace = d_stamps;
    return LUTGEMM_OK;
}

int lutgemm_sequence_describe(lutgemm_sequence_t s, int* launches_per_run, int* ctas, size_t* exchange_bytes) {
    if (!s) return LUTGEMM_ERR_NULL;
    if (launches_per_run) *launches_per_run = 1;
    if (ctas) *ctas = s->grid;
    if (exchange_bytes) *exchange_bytes = s->xchg_bytes;
    return LUTGEMM_OK;
}

int lutgemm_sequence_destroy(lutgemm_sequence_t s) {
    if (!s) return LUTGEMM_OK;
    for (int r = 0; r < 8; r++) {
        if (!s->xchg[r]) continue;
        if (r == s->rank) cudaFree(s->xchg[r]);
        else cudaIpcCloseMemHandle(s->xchg[r]);
    }
    if (s->partial) cudaFree(s->partial);
    if (s->counters) cudaFree(s->counters);
    if (s->words) cudaFree(s->words);
    if (s->d_ops) cudaFree(s->d_ops);
    delete s->params;
    delete s;
    return LUTGEMM_OK;
}

int lutgemm_dequantize(lutgemm_weight_t w, void* d_fW, void* stream) {
    if (!w || !d_fW) return LUTGEMM_ERR_NULL;
    if ((uintptr_t)d_fW & 15) return LUTGEMM_ERR_ALIGN;
    dim3 grid((w->N + 255) / 256, w->K / 32);
    if (grid.y > 65535) return LUTGEMM_ERR_TOO_LARGE;
    lg::dequantize_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w->bW, w->alpha, (__half*)d_fW, w->N, w->K, w->q,
                                                                  w->g, w->row_wise ? 1 : 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_pack_planes(const int8_t* planes, int K, int q, int N, uint32_t* bW) {
    if (!planes || !bW) return LUTGEMM_ERR_NULL;
    if (K < 32 || K % 32 != 0 || N < 1) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    const size_t qn = (size_t)q * N;
    for (int kw = 0; kw < K / 32; kw++) {
        uint32_t* dst = bW + (size_t)kw * qn;
        std::memset(dst, 0, qn * sizeof(uint32_t));
        for (int t = 0; t < 32; t++) {
            const int8_t* src = planes + (size_t)(kw * 32 + t) * qn;
            const uint32_t bit = 1u << t;
            for (size_t c = 0; c < qn; c++)
                if (src[c] > 0) dst[c] |= bit;
        }
    }
    return LUTGEMM_OK;
}

int lutgemm_pack_planes_device(const int8_t* d_planes, int K, int q, int N, uint32_t* d_bW, void* stream) {
    if (!d_planes || !d_bW) return LUTGEMM_ERR_NULL;
    if (K < 32 || K % 32 != 0 || N < 1) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    dim3 grid((unsigned)(((size_t)q * N + 255) / 256), K / 32);
    if (grid.y > 65535) return LUTGEMM_ERR_TOO_LARGE;
    lg::pack_planes_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d_planes, d_bW, K, q, N);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_uniform_to_bcq(const float* scale, const float* zero, const int32_t* code, int N, int G, int g, int q,
                           uint32_t* bW, float* alpha, float* q_bias) {
    if (!scale || !zero || !code || !bW || !alpha || !q_bias) return LUTGEMM_ERR_NULL;
    if (N < 1 || G < 1 || g < 32 || g % 32 != 0) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    const int K = G * g;
    std::memset(bW, 0, (size_t)(K / 32) * q * N * sizeof(uint32_t));
    for (int n = 0; n < N; n++) {
        for (int grp = 0; grp < G; grp++) {
            const size_t ng = (size_t)n * G + grp;
            const float z = scale[ng] * zero[ng];
            const float half_s = scale[ng] / 2.0f;
            float sum = 0.f;
            for (int b = 0; b < q; b++) {
                const float a = half_s * (float)(1u << b);
                alpha[((size_t)grp * q + b) * N + n] = a;
                sum += a;
            }
            q_bias[(size_t)grp * N + n] = sum - z;
            const int32_t* c = code + ng * g;
            for (int j = 0; j < g; j++) {
                const int k = grp * g + j;
                const int v = c[j];
                for (int b = 0; b < q; b++)
                    if ((v >> b) & 1) bW[((size_t)(k / 32) * q + b) * N + n] |= 1u << (k % 32);
            }
        }
    }
    return LUTGEMM_OK;
}

int lutgemm_uniform_to_bcq_device(const float* d_scale, const float* d_zero, const int32_t* d_code, int N, int G,
                                  int g, int q, uint32_t* d_bW, void* d_alpha, void* d_q_bias, void* stream) {
    if (!d_scale || !d_zero || !d_code || !d_bW || !d_alpha || !d_q_bias) return LUTGEMM_ERR_NULL;
    if (N < 1 || G < 1 || g < 32 || g % 32 != 0) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    dim3 grid((N + 255) / 256, (unsigned)((size_t)G * g / 32));
    if (grid.y > 65535) return LUTGEMM_ERR_TOO_LARGE;
    lg::uniform_to_bcq_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d_scale, d_zero, d_code, N, G, g, q, d_bW,
                                                                      (__half*)d_alpha, (__half*)d_q_bias);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_from_python_layout(const float* alpha_py, const int8_t* binary_py, const float* offset_py, int N, int K,
                               int g, int q, uint32_t* bW, float* alpha, float* q_bias) {
    if (!alpha_py || !binary_py || !bW || !alpha) return LUTGEMM_ERR_NULL;
    if (offset_py && !q_bias) return LUTGEMM_ERR_NULL;
    if (N < 1 || K < 32 || K % 32 != 0 || g < 1 || K % g != 0) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    const int G = K / g;
    std::memset(bW, 0, (size_t)(K / 32) * q * N * sizeof(uint32_t));
    for (int n = 0; n < N; n++)
        for (int grp = 0; grp < G; grp++) {
            const size_t ng = (size_t)n * G + grp;
            if (offset_py) q_bias[(size_t)grp * N + n] = offset_py[ng];
            for (int b = 0; b < q; b++) alpha[((size_t)grp * q + b) * N + n] = alpha_py[ng * q + b];
            const int8_t* bin = binary_py + ng * g * q;
            for (int j = 0; j < g; j++) {
                const int k = grp * g + j;
                for (int b = 0; b < q; b++)
                    if (bin[(size_t)j * q + b] > 0) bW[((size_t)(k / 32) * q + b) * N + n] |= 1u << (k % 32);
            }
        }
    return LUTGEMM_OK;
}

int lutgemm_packer_pack(const int8_t* flat, size_t L, uint8_t* packed) {
    if (!flat || !packed) return LUTGEMM_ERR_NULL;
    if (L % 8 != 0) return LUTGEMM_ERR_SHAPE;
    const size_t cols = L / 8;
    std::memset(packed, 0, cols);
    for (int i = 0; i < 8; i++) {
        const int8_t* src = flat + (size_t)i * cols;
        const uint8_t bit = (uint8_t)(1u << i);
        for (size_t j = 0; j < cols; j++)
            if (src[j] > 0) packed[j] |= bit;
    }
    return LUTGEMM_OK;
}

int lutgemm_packer_unpack(const uint8_t* packed, size_t L, int8_t* flat) {
    if (!flat || !packed) return LUTGEMM_ERR_NULL;
    if (L % 8 != 0) return LUTGEMM_ERR_SHAPE;
    const size_t cols = L / 8;
    for (int i = 0; i < 8; i++) {
        int8_t* dst = flat + (size_t)i * cols;
        for (size_t j = 0; j < cols; j++) dst[j] = ((packed[j] >> i) & 1) ? 1 : -1;
    }
    return LUTGEMM_OK;
}

int lutgemm_packer_pack_device(const int8_t* d_flat, size_t L, uint8_t* d_packed, void* stream) {
    if (!d_flat || !d_packed) return LUTGEMM_ERR_NULL;
    if (L == 0 || L % 8 != 0) return LUTGEMM_ERR_SHAPE;
    const size_t cols = L / 8;
    if ((cols + 255) / 256 > 0x7fffffffull) return LUTGEMM_ERR_TOO_LARGE;
    lg::packer_pack_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_flat, cols, d_packed);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_packer_unpack_device(const uint8_t* d_packed, size_t L, int8_t* d_flat, void* stream) {
    if (!d_flat || !d_packed) return LUTGEMM_ERR_NULL;
    if (L == 0 || L % 8 != 0) return LUTGEMM_ERR_SHAPE;
    const size_t cols = L / 8;
    if ((cols + 255) / 256 > 0x7fffffffull) return LUTGEMM_ERR_TOO_LARGE;
    lg::packer_unpack_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_packed, cols, d_flat);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_from_python_layout_device(const float* d_alpha_py, const int8_t* d_binary_py, const uint8_t* d_binary_packed,
                                      const float* d_offset_py, int N, int K, int g, int q, uint32_t* d_bW,
                                      void* d_alpha_fp16, void* d_q_bias_fp16, void* stream) {
    if (!d_alpha_py || (!d_binary_py && !d_binary_packed) || (d_binary_py && d_binary_packed) || !d_bW || !d_alpha_fp16)
        return LUTGEMM_ERR_NULL;
    if (d_offset_py && !d_q_bias_fp16) return LUTGEMM_ERR_NULL;
    if (N < 1 || K < 32 || K % 32 != 0 || g < 32 || g % 32 != 0 || K % g != 0) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > 8) return LUTGEMM_ERR_BITS;
    if (d_binary_packed && ((size_t)N * K * q) % 8 != 0) return LUTGEMM_ERR_SHAPE;
    dim3 grid((N + 127) / 128, K / 32);
    if (grid.y > 65535) return LUTGEMM_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (d_binary_packed)
        lg::python_layout_kernel<true><<<grid, 128, 0, st>>>(d_alpha_py, d_binary_packed, d_offset_py, N, K, g, q, d_bW,
                                                              (__half*)d_alpha_fp16, (__half*)d_q_bias_fp16);
    else
        lg::python_layout_kernel<false><<<grid, 128, 0, st>>>(d_alpha_py, d_binary_py, d_offset_py, N, K, g, q, d_bW,
                                                               (__half*)d_alpha_fp16, (__half*)d_q_bias_fp16);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_matmul_gptq(int m, int n, int k_packed, const void* scale_fp16, const void* zero_fp16,
                        const void* in_fp16, const uint32_t* mat, void* out_fp16, void* stream) {
    if (!scale_fp16 || !zero_fp16 || !in_fp16 || !mat || !out_fp16) return LUTGEMM_ERR_NULL;
    if (m < 1 || m > kMaxBatch) return LUTGEMM_ERR_BATCH;
    if (n < 1 || k_packed < 3 || k_packed % 3 != 0) return LUTGEMM_ERR_SHAPE;
    const int K = k_packed / 3 * 32;
    const long long ctas = ((long long)n + lg::kG3Cols - 1) / lg::kG3Cols;
    if (ctas > 0x7fffffffLL) return LUTGEMM_ERR_TOO_LARGE;
    lg::G3Params p;
    p.mat = mat; p.scale = (const __half*)scale_fp16; p.zero = (const __half*)zero_fp16; p.N = n; p.K = K;
    for (int r = 0; r < m; r++) {
        p.x = (const __half*)in_fp16 + (size_t)r * K;
        p.y = (__half*)out_fp16 + (size_t)r * n;
        lg::gptq3_gemv_kernel<<<(unsigned)ctas, lg::kG3Threads, 0, (cudaStream_t)stream>>>(p);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_bcq_quantize_device(const float* d_w, int N, int K, int q, int group_size, int rounds,
                                float* d_alpha_py, signed char* d_binary_py, uint32_t* d_bW, void* d_alpha_fp16,
                                void* stream) {
    if (!d_w || (!d_alpha_py && !d_binary_py && !d_bW && !d_alpha_fp16)) return LUTGEMM_ERR_NULL;
    if (q < 1 || q > lg::kBqMaxQ) return LUTGEMM_ERR_BITS;
    const int g = group_size > 0 ? group_size : K;
    if (N < 1 || K < 1 || rounds < 0 || K % g != 0 || g > 65536) return LUTGEMM_ERR_SHAPE;
    if ((d_bW || d_alpha_fp16) && (g % 32 != 0)) return LUTGEMM_ERR_SHAPE;
    lg::BqParams p;
    p.w = d_w; p.N = N; p.K = K; p.g = g; p.q = q; p.rounds = rounds;
    p.alpha_py = d_alpha_py; p.binary_py = d_binary_py; p.bW = d_bW; p.alpha_k = (__half*)d_alpha_fp16;
    const long long groups = (long long)N * (K / g);
    const long long ctas = (groups + lg::kBqWarps - 1) / lg::kBqWarps;
    if (ctas > 0x7fffffffLL) return LUTGEMM_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (g <= 128) lg::bcq_quantize_kernel<4><<<(unsigned)ctas, lg::kBqWarps * 32, 0, st>>>(p);
    else if (g <= 256) lg::bcq_quantize_kernel<8><<<(unsigned)ctas, lg::kBqWarps * 32, 0, st>>>(p);
    else if (g <= 1024) lg::bcq_quantize_kernel<32><<<(unsigned)ctas, lg::kBqWarps * 32, 0, st>>>(p);
    else {
        // one CTA per group, its codes (2 bytes per weight) in dynamic shared memory
        if (groups > 0x7fffffffLL) return LUTGEMM_ERR_TOO_LARGE;
        const size_t smem = (size_t)g * sizeof(unsigned short);
        static bool configured[64] = {};
        int dev = 0;
        LG_CUDA(cudaGetDevice(&dev));
        if (dev >= 64 || !configured[dev]) {
            LG_CUDA(cudaFuncSetAttribute(lg::bcq_quantize_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
            if (dev < 64) configured[dev] = true;
        }
        lg::bcq_quantize_block_kernel<<<(unsigned)groups, lg::kBqBlockThreads, smem, st>>>(p);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    LG_CUDA(cudaGetLastError());
    return LUTGEMM_OK;
}

int lutgemm_bcq_quantize(const float* w, int N, int K, int q, int group_size, int rounds,
                         float* alpha_py, signed char* binary_py) {
    if (!w || !alpha_py || !binary_py) return LUTGEMM_ERR_NULL;
    if (N < 1 || K < 1) return LUTGEMM_ERR_SHAPE;
    if (q < 1 || q > lg::kBqMaxQ) return LUTGEMM_ERR_BITS;
    const int g = group_size > 0 ? group_size : K;
    if (K % g != 0) return LUTGEMM_ERR_SHAPE;
    const size_t nw = (size_t)N * K, na = (size_t)N * (K / g) * q;
    float *d_w = nullptr, *d_a = nullptr;
    signed char* d_b = nullptr;
    int rc = LUTGEMM_OK;
    auto fail = [&](cudaError_t e) {
        g_last_cuda = (int)e;
        rc = (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? LUTGEMM_ERR_NO_DEVICE : LUTGEMM_ERR_CUDA;
    };
    cudaError_t e;
    if ((e = cudaMalloc(&d_w, nw * sizeof(float))) != cudaSuccess) fail(e);
    if (rc == LUTGEMM_OK && (e = cudaMalloc(&d_a, na * sizeof(float))) != cudaSuccess) fail(e);
    if (rc == LUTGEMM_OK && (e = cudaMalloc(&d_b, nw * q)) != cudaSuccess) fail(e);
    if (rc == LUTGEMM_OK && (e = cudaMemcpy(d_w, w, nw * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) fail(e);
    if (rc == LUTGEMM_OK) rc = lutgemm_bcq_quantize_device(d_w, N, K, q, group_size, rounds, d_a, d_b, nullptr, nullptr, nullptr);
    if (rc == LUTGEMM_OK && (e = cudaMemcpy(alpha_py, d_a, na * sizeof(float), cudaMemcpyDeviceToHost)) != cudaSuccess) fail(e);
    if (rc == LUTGEMM_OK && (e = cudaMemcpy(binary_py, d_b, nw * q, cudaMemcpyDeviceToHost)) != cudaSuccess) fail(e);
    if (d_w) cudaFree(d_w);
    if (d_a) cudaFree(d_a);
    if (d_b) cudaFree(d_b);
    return rc;
}

const char* lutgemm_status_string(int s) {
    switch (s) {
        case LUTGEMM_OK: return "ok";
        case LUTGEMM_ERR_NULL: return "a required pointer is NULL";
        case LUTGEMM_ERR_SHAPE: return "unsupported shape (K % 32, K % num_groups, group size % 32, sizes >= 1)";
        case LUTGEMM_ERR_BITS: return "num_bits must be in 1..8";
        case LUTGEMM_ERR_BATCH: return "batch size out of range";
        case LUTGEMM_ERR_CUDA: return "a CUDA call failed (see lutgemm_last_cuda_error)";
        case LUTGEMM_ERR_NO_DEVICE: return "no usable CUDA device; this library has no CPU fallback";
        case LUTGEMM_ERR_TOO_LARGE: return "size beyond the supported maximum";
        case LUTGEMM_ERR_ALIGN: return "pointer or row pitch not 16-byte aligned";
    }
    return "unknown status";
}

int lutgemm_weight_device_status(lutgemm_weight_t w, int* status) {
    if (!w || !status) return LUTGEMM_ERR_NULL;
    LG_CUDA(cudaMemcpy(status, w->own.status, sizeof(int), cudaMemcpyDeviceToHost));
    return LUTGEMM_OK;
}

int lutgemm_set_gemv_variant(int variant) {
    if (variant < 0 || variant > 1) return LUTGEMM_ERR_SHAPE;
    g_variant.store(variant);
    return LUTGEMM_OK;
}

int lutgemm_set_ordered_reduction(int enabled) {
    g_ordered.store(enabled ? 1 : 0);
    return LUTGEMM_OK;
}
int lutgemm_set_row_pairs(int enabled) {
    g_pairs.store(enabled ? 1 : 0);
    return LUTGEMM_OK;
}

int lutgemm_set_batched_path(int mode) {
    if (mode < 0 || mode > 2) return LUTGEMM_ERR_SHAPE;
    g_batched.store(mode);
    return LUTGEMM_OK;
}

int lutgemm_set_batched_int8(int enabled) {
    g_int8.store(enabled ? 1 : 0);
    return LUTGEMM_OK;
}

int lutgemm_set_dependent_launch(int enabled) {
    g_pdl.store(enabled ? 1 : 0);
    return LUTGEMM_OK;
}

int lutgemm_last_cuda_error(void) { return g_last_cuda; }
unsigned long long lutgemm_kernel_launch_count(void) { return g_launches.load(); }
int lutgemm_set_gemv_ntile(int columns) {
    if (columns < 0) return LUTGEMM_ERR_SHAPE;
    g_ntile_override.store(columns);
    return LUTGEMM_OK;
}

}  // extern "C"
