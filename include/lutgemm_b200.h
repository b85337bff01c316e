/*
 * lutgemm_b200 — C ABI of the B200 (sm_100a) LUT-GEMM library.
 *
 * Drop-in boundary for the BCQ matmul path of naver-aics/lut-gemm.  Every entry
 * point is `extern "C"`, takes plain pointers and sizes, and returns an int
 * status (LUTGEMM_OK == 0).  Beside each declaration is the reference interface
 * it replaces, as <file>:<line> inside the reference project.
 *
 * Container layout (identical to the reference, column-wise mode):
 *   bW      uint32 [K/32][q][N]   bit (k % 32) of bW[k/32][b][n] set <=> plane b of weight (k, n) is +1
 *   alpha   fp16   [G][q][N]      G = num_groups, group size g = K / G along k
 *   q_bias  fp16   [G][N]         optional per-group offset (uniform quantisation folded into BCQ)
 *   y[m][n] = sum_g ( q_bias[g][n] * sum_{k in g} x[m][k]
 *                     + sum_b alpha[g][b][n] * sum_{k in g} (+-1)(k,b,n) * x[m][k] )
 * with N = mSize (output features), K = kSize (input features), q = nb.
 */
#ifndef LUTGEMM_B200_H
#define LUTGEMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    LUTGEMM_OK = 0,
    LUTGEMM_ERR_NULL = 1,          /* a required pointer is NULL */
    LUTGEMM_ERR_SHAPE = 2,         /* K % 32 != 0, K % num_groups != 0, group size % 32 != 0, N < 1, ... */
    LUTGEMM_ERR_BITS = 3,          /* num_bits outside 1..8 */
    LUTGEMM_ERR_BATCH = 4,         /* m < 1 or above the supported maximum */
    LUTGEMM_ERR_CUDA = 5,          /* a CUDA runtime call failed; see lutgemm_last_cuda_error() */
    LUTGEMM_ERR_NO_DEVICE = 6,     /* no usable CUDA device: there is no CPU fallback */
    LUTGEMM_ERR_TOO_LARGE = 7,     /* size beyond what the entry point supports */
    LUTGEMM_ERR_ALIGN = 8          /* pointer not aligned as the entry point requires */
};

/* Opaque weight container.  Replaces class lutGEMM::nQWeight_fp16
 * (lutGEMM/include/nQWeight_fp16.h:27-52). */
typedef struct lutgemm_weight* lutgemm_weight_t;

/* The public fields of the reference container (lutGEMM/include/nQWeight_fp16.h:29-37),
 * as device pointers. */
typedef struct lutgemm_weight_desc {
    uint32_t* bWeight;   /* device, [K/32][q][N] */
    void* alpha;         /* device fp16, [G][q][N] */
    void* q_bias;        /* device fp16, [G][N], or NULL */
    int num_groups;
    int group_size;
    int mSize;           /* N */
    int kSize;           /* K */
    int nb;              /* q */
    int is_row_wise_quantize;
    int device;
} lutgemm_weight_desc;

/* Uploads a container from host arrays to the current CUDA device.
 * Replaces nQWeight_fp16::parsing (lutGEMM/src/nQWeight_fp16.cu:60-91) with the same
 * argument meaning: bW [K/32][q][N] uint32; A float [G][q][N] and q_bias float [G][N]
 * (or NULL) are rounded to fp16 (round-to-nearest-even); column-wise (is_row_wise == 0)
 * means K = row, N = col; row-wise means N = row, K = col.
 * The copy lives in plain device memory owned by the handle. */
int lutgemm_weight_create(lutgemm_weight_t* out, const uint32_t* bW, const float* A,
                          int row, int col, int num_bits, int is_row_wise,
                          int num_alpha_groups, const float* q_bias);

/* Same, from arrays that are already on the current device in their final types
 * (uint32 planes, fp16 alpha, fp16 q_bias or NULL).  With copy == 0 the handle
 * borrows the caller's buffers, which must outlive it.  No reference counterpart: the
 * reference exposes its fields publicly (lutGEMM/include/nQWeight_fp16.h:29-37) and a caller
 * would assign them by hand. */
int lutgemm_weight_create_device(lutgemm_weight_t* out, const uint32_t* d_bW, const void* d_alpha_fp16,
                                 const void* d_q_bias_fp16, int row, int col, int num_bits,
                                 int is_row_wise, int num_alpha_groups, int copy);

/* Replaces nQWeight_fp16::~nQWeight_fp16 (lutGEMM/src/nQWeight_fp16.cu:101-105); frees each
 * owned buffer exactly once.  NULL is accepted. */
int lutgemm_weight_destroy(lutgemm_weight_t w);

/* Reads the container's fields (lutGEMM/include/nQWeight_fp16.h:29-37). */
int lutgemm_weight_describe(lutgemm_weight_t w, lutgemm_weight_desc* desc);

/* out[m][N] (fp16, device) = in[m][K] (fp16, device) x W.
 * Replaces lutGEMM::matmul(output, input, nqW, m) (lutGEMM/include/kernels.h:27, lutGEMM/src/kernels.cu:64-71);
 * q_bias is applied whenever the container has one, for every m.
 * Asynchronous on `stream` (a cudaStream_t, NULL = default stream); no host synchronisation.
 * The call uses the container's own split-k workspace, so calls that share a container must be ordered on one
 * stream; to run one container from several streams at a time give every stream a workspace of its own
 * (lutgemm_matmul_ws below).  A first batched call (m >= 4) on a container that was not told its batch size
 * (lutgemm_weight_reserve_batch) allocates the batched path's fp32 rows, which synchronises the device; inside a
 * stream capture that call fails with LUTGEMM_ERR_BATCH instead. */
int lutgemm_matmul(void* out_fp16, const void* in_fp16, lutgemm_weight_t w, int m, void* stream);

/* Same computation with the result left in fp32 (no final fp16 rounding). */
int lutgemm_matmul_f32(float* out_f32, const void* in_fp16, lutgemm_weight_t w, int m, void* stream);

/* The (output, nqW, input, n) overload of the reference (lutGEMM/include/kernels.h:26, lutGEMM/src/kernels.cu:56-63,
 * 73-75; operand order of lutGEMM/src/cuda/kernels/cublas.h:47-55): W . X with the activations as COLUMNS,
 * in[K][n] and out[N][n], both fp16 row-major.  For n == 1 these are the plain vectors of lutgemm_matmul.  For n > 1
 * the library transposes in and out around the X . W kernels (two small extra launches) in scratch that belongs to
 * the container (sized by lutgemm_weight_reserve_batch(w, n), else grown on first use as described above).
 * The reference runs this overload on a dense weight laid out [N][K], i.e. on row-wise containers; here it is the same
 * mathematical product for either container kind. */
int lutgemm_matmul_wx(void* out_fp16, lutgemm_weight_t w, const void* in_fp16, int n, void* stream);

/* Sizes everything lutgemm_matmul / lutgemm_matmul_wx / lutgemm_matmul_host may need for batches of up to m rows
 * (fp32 split-k rows of the batched path, transposed copies of the W . X form), so that no later call allocates:
 * call it once after creation, before capturing a CUDA graph that holds a batched call.  No reference counterpart
 * (its scratch is a process-wide singleton grown inside the call, lutGEMM/src/cuda/tmpWeight.hpp:28-35). */
int lutgemm_weight_reserve_batch(lutgemm_weight_t w, int m);

/* An explicit split-k workspace: partial rows, arrival counters, a status word and the batched path's fp32 rows for
 * containers up to max_n output features, max_k input features and batches up to max_m.  One workspace serves one
 * stream at a time; two streams may run the SAME container concurrently when each passes its own workspace.
 * lutgemm_matmul_ws / _f32_ws are lutgemm_matmul / _f32 on that workspace (NULL = the container's own) and never
 * allocate: a container or batch beyond the workspace's sizes is refused with LUTGEMM_ERR_TOO_LARGE.
 * lutgemm_workspace_status synchronises and reads the workspace's status word (see lutgemm_weight_device_status).
 * No reference counterpart: the reference runs on the legacy default stream only. */
typedef struct lutgemm_workspace* lutgemm_workspace_t;
int lutgemm_workspace_create(lutgemm_workspace_t* out, int max_n, int max_k, int max_m);
int lutgemm_workspace_destroy(lutgemm_workspace_t ws);
int lutgemm_workspace_status(lutgemm_workspace_t ws, int* status);
/* Split-k mode of the calls made on this workspace / on the container's own workspace: 0 = unordered fp32 reductions,
 * 1 = bit-reproducible (see lutgemm_set_ordered_reduction), -1 (initial) = whatever the process-wide setting is when the
 * call is made.  Each call reads the mode once; a workspace may change mode between calls. */
int lutgemm_workspace_set_ordered(lutgemm_workspace_t ws, int mode);
int lutgemm_weight_set_ordered(lutgemm_weight_t w, int mode);
int lutgemm_matmul_ws(void* out_fp16, const void* in_fp16, lutgemm_weight_t w, int m, lutgemm_workspace_t ws, void* stream);
int lutgemm_matmul_f32_ws(float* out_f32, const void* in_fp16, lutgemm_weight_t w, int m, lutgemm_workspace_t ws, void* stream);

/* Same computation from and to HOST buffers: copies in (m*K fp16) to the device, runs,
 * copies out (m*N fp16) back and synchronises.  This is the call a host program holding
 * CPU activations makes (the reference test keeps them in managed memory,
 * tests/opt/fp16/int3_col_wise_matmul_fp16.cu:246-256).  It runs on a non-blocking stream of the container's own.
 * m = 1 with both buffers page-locked (cudaHostAlloc / cudaHostRegister, 16-byte aligned): no copy engine is involved;
 * one kernel reads the activations from the host buffer (each CTA the 1 KB its k-slab needs, while its weight stream
 * starts) and stores the result into the host buffer.  Otherwise: copy-in, kernels, copy-out, replayed as one
 * instantiated graph while the caller keeps passing the same two buffers and batch.
 * lutgemm_matmul_host_profile runs the same call once with events between its parts and returns, in microseconds,
 * us4 = {copy in, kernels, copy out, all three on the device}. */
int lutgemm_matmul_host(void* out_fp16_host, const void* in_fp16_host, lutgemm_weight_t w, int m);
int lutgemm_matmul_host_profile(void* out_fp16_host, const void* in_fp16_host, lutgemm_weight_t w, int m, float* us4);

/* Matvec (m = 1) that allocates nothing: out[N] (fp16) = in[K] (fp16) x W, with every array passed
 * by the caller as a device pointer in the container's layout (d_bW uint32 [K/32][q][N], d_alpha fp16
 * [G][q][N], d_q_bias fp16 [G][N] or NULL).  It has no counterpart in the reference, whose matvec needs
 * a parsed container and a memset before each call.
 *
 * It is meant for programs that must not call cudaMalloc once they are running: a serving process that
 * has handed all free device memory to its own pool at start-up (a later cudaMalloc would fail, or
 * would stall every stream while the driver maps new memory), or a host whose rules freeze the memory
 * map after initialisation.  The other matvec entry points keep a split-k workspace that
 * lutgemm_weight_create allocates; here that workspace is a fixed array inside the library image
 * (about 272 KB, resident on every GPU that loads the library until the process exits).  The call
 * makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *   - N <= 65536 (LUTGEMM_ERR_TOO_LARGE beyond: the array holds one fp32 row of that width); N % 8 == 0
 *     and a group size that divides 512 or is a multiple of 512 (LUTGEMM_ERR_SHAPE otherwise);
 *     16-byte aligned pointers (LUTGEMM_ERR_ALIGN).
 *   - The first call on each device looks up the array's device address (that device must be current);
 *     make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  Each call clears the part it uses on `stream` before
 *     the kernel, so a call never sees the previous call's sums, but two calls that can run at the same
 *     time on the GPU (different streams, no ordering between them) corrupt each other: order them.
 *   - k-slabs are added by fp32 reductions in L2 (unordered), as in the default mode of lutgemm_matmul. */
int lutgemm_matvec_static_scratch(void* out_fp16, const void* in_fp16, const uint32_t* d_bW,
                                  const void* d_alpha_fp16, const void* d_q_bias_fp16,
                                  int K, int N, int num_bits, int num_alpha_groups, void* stream);
/* The status word of lutgemm_matvec_static_scratch lives in the same fixed array (that entry point has no
 * container whose status could be asked): this call synchronises with the current device and reads it.
 * 0 = the last call's bounded waits were all met; 1 / 2 = its weight stream stalled and the output is invalid.
 * Each call of the entry point clears the word before its kernel.  No counterpart in the reference. */
int lutgemm_static_scratch_status(int* status);

/* ---- Tensor-parallel matvec: the exchange steps fused into the kernel (no counterpart in the reference,
 * which is single-GPU; lutGEMM/CMakeLists.txt:13 links no communication library). ----
 *
 * A decoder linear sharded over `world` GPUs (one process each) needs an all-gather after a column-parallel
 * matvec and an all-reduce after a row-parallel one.  Instead of separate collectives, the producing kernel
 * stores its result straight into every rank's buffer (peer-mapped pointers, see lutgemm_ipc_*) and bumps a
 * flag there; the consuming kernel starts streaming its weights at once and waits for the flag (bounded)
 * only before it reads the activations.
 *   x_mode   0: `in_fp16` is ready in stream order.  1: `in_fp16` (local memory) is filled by all ranks' pushes;
 *            wait until *flag_in >= flag_target.  2: the input is sum_r x_slots[r*x_slot_stride + x_off + k]
 *            (fp32 rows pushed by the ranks, added in rank order, rounded to fp16 once); same wait.
 *   out_mode 0: out_fp16 / out_f32 in local memory.  1: fp16 result to out16[r] + out_off for every rank r.
 *            2: fp32 result to out32[r] (this rank's row on rank r).  Then *flag_out[r] += 1 per finished column
 *            tile (lutgemm_matvec_tiles gives the count; the consumer's flag_target is the sum over producers).
 * The kernel re-arms flag_in (and done_counter, a zeroed word of the caller's) itself, so a CUDA graph with
 * constant arguments can be replayed.  Needs a container the TMA-fed kernel takes; world <= 8. */
typedef struct lutgemm_tp_link {
    int x_mode, out_mode, world, out_off;
    const float* x_slots;
    int x_slot_stride, x_off;
    unsigned* flag_in;
    unsigned flag_target;
    unsigned* done_counter;
    void* out16[8];
    float* out32[8];
    unsigned* flag_out[8];
} lutgemm_tp_link;
int lutgemm_matvec_tp(const void* in_fp16, lutgemm_weight_t w, const lutgemm_tp_link* link, void* out_fp16,
                      float* out_f32, void* stream);
/* Column tiles (= flag increments per launch) of the TMA-fed matvec on this container. */
int lutgemm_matvec_tiles(lutgemm_weight_t w, int* tiles);
/* Last consumer of a chain: waits for the flag, adds `world` fp32 rows of n values in rank order, writes fp16
 * and/or fp32, re-arms the flag.  `status_owner` receives a time-out in its status word. */
int lutgemm_tp_finalize(void* out_fp16, float* out_f32, const float* slots, int slot_stride, int world, int n,
                        unsigned* flag_in, unsigned flag_target, lutgemm_weight_t status_owner, void* stream);
/* Peer-visible device memory: allocate (zero-filled) and export a 64-byte handle / map another process's
 * handle into this process / unmap / free. */
int lutgemm_ipc_alloc(size_t bytes, void** dptr, void* handle64);
int lutgemm_ipc_open(const void* handle64, void** dptr);
int lutgemm_ipc_close(void* dptr);
int lutgemm_ipc_free(void* dptr);

/* ---- A sequence of matvecs in one persistent kernel (no counterpart in the reference, which launches a memset
 * and a kernel per matvec, lutGEMM/src/kernels.cu:64-71, and has no multi-GPU code). ----
 *
 * A decode step of a decoder stack is a fixed list of m = 1 matvecs, most of which consume what an earlier one
 * produced.  lutgemm_sequence_run executes the whole list in ONE kernel launch: one CTA per SM stays resident,
 * the weight stream runs across matvec boundaries, and results travel between matvecs (and between the GPUs of a
 * tensor-parallel group, one process per GPU) in exchange memory whose every 16-byte line carries the step number,
 * so that a consumer waits on exactly the words it needs and no flag, fence or collective kernel is involved.
 *
 * Exchange buffers (lutgemm_seq_buffer; owned by the sequence, identical on every rank):
 *   kind 1  an fp16 vector of n values, filled by matvecs with out_kind 1 (each rank writes its columns into
 *           EVERY rank's copy: an all-gather);
 *   kind 2  `world` fp32 rows of n values, row r filled by rank r's matvec with out_kind 2 on every rank's
 *           copy; a consumer adds the rows in rank order and rounds to fp16 once (an all-reduce).
 * Matvec i (lutgemm_seq_op):
 *   w         the container (a shape the TMA-fed matvec kernel takes; all containers of one sequence have the same
 *             group size and agree on having q_bias); NULL = no matvec: the `n` values at in_off of a kind-2
 *             buffer are added, rounded and written to y_ext (the usual last step after a row-parallel matvec)
 *   in_kind   0: x_ext, an fp16 device vector that is complete when the sequence is launched;
 *             1 / 2: K values starting at element in_off of buffer in_buf (kind 1 / kind 2)
 *   out_kind  0: y_ext, an fp16 device vector of N values; 1: N values at element out_off of buffer out_buf;
 *             2: N values at element out_off of this rank's row of buffer out_buf
 *   in_off and out_off are multiples of 4.
 * Pointers are fixed at creation, so a captured launch can be replayed.  Within a step every buffer region is
 * written once and must be consumed by a later matvec of the same step; all ranks of a group run the same
 * list the same number of times (the step number is the handshake), and the last matvecs of the list must depend,
 * directly or not, on every rank (as a row-parallel matvec followed by the NULL step does), so that no rank can
 * run a step ahead of a reader.
 *
 * Set-up with world > 1: every rank creates its sequence, exports the 64-byte handle of its exchange memory,
 * passes it to the other ranks by any host channel, connects theirs, then commits.  world == 1 needs only create.
 * lutgemm_sequence_run is asynchronous on `stream`, allocates nothing and synchronises nothing.  Every in-kernel
 * wait is bounded (lutgemm_sequence_set_wait_limit, 2 s by default): when a producer never shows up the kernel
 * records a status (lutgemm_sequence_status: 4 = a peer's data did not arrive, 1 / 2 = weight stream), stops waiting
 * and ends; results of that step are then invalid. */
typedef struct lutgemm_sequence* lutgemm_sequence_t;
typedef struct lutgemm_seq_buffer {
    int kind;            /* 1: fp16 vector; 2: `world` fp32 rows */
    int n;               /* values (per row); a multiple of 4 */
} lutgemm_seq_buffer;
typedef struct lutgemm_seq_op {
    lutgemm_weight_t w;
    int in_kind, in_buf, in_off;
    int out_kind, out_buf, out_off;
    int n;               /* w == NULL only: how many values to add and write */
    const void* x_ext;   /* in_kind 0 */
    void* y_ext;         /* out_kind 0 */
} lutgemm_seq_op;
int lutgemm_sequence_create(lutgemm_sequence_t* out, const lutgemm_seq_op* ops, int n_ops,
                            const lutgemm_seq_buffer* buffers, int n_buffers, int rank, int world);
int lutgemm_sequence_export(lutgemm_sequence_t s, void* handle64);
int lutgemm_sequence_connect(lutgemm_sequence_t s, int peer_rank, const void* handle64);
int lutgemm_sequence_commit(lutgemm_sequence_t s);
int lutgemm_sequence_run(lutgemm_sequence_t s, void* stream);
/* Synchronises with the device and reads the sequence's status word (0 = every wait was met). */
int lutgemm_sequence_status(lutgemm_sequence_t s, int* status);
/* Synchronises and sets the status word back to 0.  A failed step leaves the sequence consistent (every CTA still walks
 * the whole list, counters and reduction rows are left as a good step leaves them), but while the word is set every wait
 * gives up at once; clear it once the cause (a peer that was late or gone) is dealt with. */
int lutgemm_sequence_clear_status(lutgemm_sequence_t s);
/* Time limit of one in-kernel wait for another matvec's or rank's data, in milliseconds (default 2000). */
int lutgemm_sequence_set_wait_limit(lutgemm_sequence_t s, int milliseconds);
/* Tracing: with a device buffer of n_ops * ctas * 4 uint64 (ctas from lutgemm_sequence_describe) every later run
 * records, per (matvec i, CTA c) at [(i * ctas + c) * 4 ..], the device clock in ns when (0) the CTA's activations had
 * arrived, (1) its tables were built, (2) its last stage was consumed, (3) it left the matvec (bit 0 set if it was
 * the one that published the column tile).  NULL switches tracing off.  Costs one predicated store per stamp. */
int lutgemm_sequence_set_trace(lutgemm_sequence_t s, unsigned long long* d_stamps, size_t entries);
/* Kernel launches one lutgemm_sequence_run makes (1) and the CTAs it uses; for reports. */
int lutgemm_sequence_describe(lutgemm_sequence_t s, int* launches_per_run, int* ctas, size_t* exchange_bytes);
int lutgemm_sequence_destroy(lutgemm_sequence_t s);

/* Dense fp16 weight on the device: W[k][N] (column-wise) or W[n][K] (row-wise),
 * W = sum_b +-alpha, fp32 sum over planes b = 0..q-1 and one fp16 rounding, no q_bias.
 * Replaces lutGEMM::dequantize_gpu (lutGEMM/src/nQWeight_fp16.cu:29-35) and is bit-identical to
 * lutGEMM::dequantize_cpu (lutGEMM/src/nQWeight_fp16.cu:38-59). */
int lutgemm_dequantize(lutgemm_weight_t w, void* d_fW_fp16, void* stream);

/* Host packer: +-1 planes int8 [K][q][N] -> bW uint32 [K/32][q][N].
 * Replaces makeRandomWeight's packing (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:200-215). */
int lutgemm_pack_planes(const int8_t* planes, int K, int q, int N, uint32_t* bW);

/* Device packer: the same mapping with both arrays on the current device. */
int lutgemm_pack_planes_device(const int8_t* d_planes, int K, int q, int N, uint32_t* d_bW, void* stream);

/* Host converter, uniform quantisation -> BCQ with offset, written straight into the
 * kernel layout.  Inputs in the Python examples' shapes: scale, zero float [N][G],
 * code int32 [N][G][g] with values in [0, 2^q).  Outputs: bW [K/32][q][N] (plane b = bit b
 * of the code), alpha float [G][q][N] = scale/2 * 2^b, q_bias float [G][N] =
 * sum_b alpha_b - scale*zero.  Replaces RTNParameter.convert_bcq_format
 * (examples/rtn_parameter.py:77-96) followed by the layout transposition the reference
 * leaves to the caller. */
int lutgemm_uniform_to_bcq(const float* scale, const float* zero, const int32_t* code,
                           int N, int G, int g, int q, uint32_t* bW, float* alpha, float* q_bias);

/* Device converter: same mapping, all arrays on the current device; alpha and q_bias are
 * written as fp16 (the container's types), ready for lutgemm_weight_create_device. */
int lutgemm_uniform_to_bcq_device(const float* d_scale, const float* d_zero, const int32_t* d_code,
                                  int N, int G, int g, int q, uint32_t* d_bW, void* d_alpha_fp16,
                                  void* d_q_bias_fp16, void* stream);

/* The Python examples' tensors (alpha float [N][G][q], binary int8 [N][G][g][q] of +-1,
 * offset float [N][G] or NULL; examples/bcq_parameter.py:41-48) -> kernel layout on the host. */
int lutgemm_from_python_layout(const float* alpha_py, const int8_t* binary_py, const float* offset_py,
                               int N, int K, int g, int q, uint32_t* bW, float* alpha, float* q_bias);

/* The 3-bit uniform (GPTQ-format) comparison rows of the reference's header: replaces lutGEMM::matmul_gptq and
 * lutGEMM::matmul_gptq_faster (lutGEMM/include/kernels.h:28-33, lutGEMM/src/kernels.cu:40-54; kernels
 * lutGEMM/src/cuda/kernels/gptq_fp16_bias.hpp, gptq_faster_fp16_bias.hpp), same argument order and meaning:
 * k_packed = K * 3 / 32 rows of `mat` [k_packed][n] (32 codes of 3 bits in three words along k),
 * out[r][c] = sum_k (scale[c] * code[k][c] - zero[c]) * in[r][k].  fp32 accumulation, one fp16 rounding, no
 * memset and no atomics; every one of the m rows is computed (the reference kernels compute row 0 only). */
int lutgemm_matmul_gptq(int m, int n, int k_packed, const void* scale_fp16, const void* zero_fp16,
                        const void* in_fp16, const uint32_t* mat, void* out_fp16, void* stream);

/* BCQ quantiser: replaces quantize() of examples/bcq.py:23-98 (greedy_mean_torch :100-128, refine_mean_torch
 * :130-157, find_B_torch :165-188, batch_cg_torch :190-206) for its default unweighted case (exponent 0,
 * clipping 1, pruning 0).  w float [N][K] (output rows, groups of `group_size` consecutive input features;
 * group_size <= 0: one group per row); `rounds` refinements after the greedy start (the reference's default is
 * 15; ignored for q == 1).  One warp quantises a group of up to 1024 weights, one CTA a wider one (up to 65536).
 * Outputs, each optional
 * (NULL to skip) in the device form: the quantiser's own layout alpha [N][G][q] / binary int8 [N][G][g][q]
 * in {-1, 0, +1} (0 only where the greedy start met an exactly zero residual), and the container layout of this
 * library, bW [K/32][q][N] and alpha fp16 [G][q][N] (needs group_size % 32 == 0; a zero code packs as -1),
 * ready for lutgemm_weight_create_device.  The host form copies w in and the quantiser's layout out. */
int lutgemm_bcq_quantize_device(const float* d_w, int N, int K, int q, int group_size, int rounds,
                                float* d_alpha_py, signed char* d_binary_py, uint32_t* d_bW, void* d_alpha_fp16,
                                void* stream);
int lutgemm_bcq_quantize(const float* w, int N, int K, int q, int group_size, int rounds,
                         float* alpha_py, signed char* binary_py);

/* The Python examples' uint8 interchange format (Packer.pack / Packer.unpack,
 * examples/utils.py:162-181): L values of +-1 <-> L/8 bytes, byte j = sum_i 2^i * [flat[i*L/8 + j] > 0]. */
int lutgemm_packer_pack(const int8_t* flat_pm1, size_t L, uint8_t* packed);
int lutgemm_packer_unpack(const uint8_t* packed, size_t L, int8_t* flat_pm1);
/* The same two mappings with both arrays on the current device (the reference's Packer runs its torch ops wherever
 * the tensor lives, examples/utils.py:162-181). */
int lutgemm_packer_pack_device(const int8_t* d_flat_pm1, size_t L, uint8_t* d_packed, void* stream);
int lutgemm_packer_unpack_device(const uint8_t* d_packed, size_t L, int8_t* d_flat_pm1, void* stream);
/* Device form of lutgemm_from_python_layout: the quantisers' tensors, already on the device, straight into the
 * container layout in its final types (alpha and q_bias fp16), ready for lutgemm_weight_create_device.  The binary
 * tensor [N][G][g][q] comes either as int8 +-1 (d_binary_py) or as the Packer's uint8 stream of the flattened tensor
 * (d_binary_packed, N*K*q/8 bytes; examples/utils.py:162-172) - exactly one of the two - and in the packed case is
 * read bit by bit without ever being expanded.  Group sizes are multiples of 32. */
int lutgemm_from_python_layout_device(const float* d_alpha_py, const int8_t* d_binary_py, const uint8_t* d_binary_packed,
                                      const float* d_offset_py, int N, int K, int g, int q, uint32_t* d_bW,
                                      void* d_alpha_fp16, void* d_q_bias_fp16, void* stream);

/* Text for a status code; never NULL. */
const char* lutgemm_status_string(int status);
/* The cudaError_t of the last failing CUDA call on this thread (0 if none). */
int lutgemm_last_cuda_error(void);
/* How many kernels this library has launched in this process (all threads). */
unsigned long long lutgemm_kernel_launch_count(void);
/* Tuning knob: columns per CTA of the LUT matvec (0 = automatic).  Process-wide. */
int lutgemm_set_gemv_ntile(int columns);
/* Tuning knob: 0 = bulk-copy (TMA) fed matvec kernel (default), 1 = register-streaming kernel.
 * Process-wide; both compute the same function. */
int lutgemm_set_gemv_variant(int variant);
/* 0 (default): the TMA-fed matvec adds its k-slabs with fp32 reductions in L2, whose order is not
 * fixed (results agree to fp32 rounding of a 24-term sum, then one fp16 rounding).  1: one partial
 * row per slab, added in slab order: bit-reproducible run to run, about 10 % slower; the batched
 * (tensor-core) path then gives every column tile its whole k-range instead of reducing across k-ranges.
 * Switch only while no matmul is in flight; a workspace may be used in either mode from call to call.  (The reference's half2 atomicAdd accumulation,
 * lutGEMM/src/cuda/kernels/mv_fp16.hpp:95, has no ordered mode.) */
int lutgemm_set_ordered_reduction(int enabled);
/* 1 (default): rows that go through the LUT matvec (m = 2, 3; any m with lutgemm_set_batched_path(0)) are taken
 * two at a time by a two-table kernel that reads the weights once for both; 0: one row per launch.  The pair
 * kernel is used only with the default reductions (not in ordered mode) and the default matvec variant. */
int lutgemm_set_row_pairs(int enabled);
/* 1 (default): m >= 4 runs the tensor-core (tcgen05) kernel, 128 rows per launch, smaller batches one LUT
 * matvec per row; 0: always one LUT matvec per row; 2: tensor-core kernel from m = 2.  All compute the same
 * function. */
int lutgemm_set_batched_path(int mode);
/* 0 (default): every batch on the tensor-core path takes the fp16 kernel (operand = +-alpha in fp16, exact products).
 * 1: a batch of up to 16 rows on a container of up to 4 planes runs the integer kernel (tcgen05.mma.kind::i8): the packed
 * bits are the operand as they are, the activations are taken as block-scaled 24-bit integers per 128 k and row (every
 * fp16 input within 2^13 of its block's maximum exactly, the rest to 2^-24 of that maximum; a block with a non-finite
 * input yields NaN for its row), the scales are applied in fp32 to exact int32 sums.  Same results to fp32 rounding;
 * measured slower than the fp16 kernel on B200 (one accumulator hand-over per scale group and plane), kept as an
 * alternative. */
int lutgemm_set_batched_int8(int enabled);
/* Tuning knob: 1 (default) launches the TMA-fed matvec with programmatic stream serialization, so
 * that its weight stream starts while the previous kernel of the stream drains; 0 = plain launches. */
int lutgemm_set_dependent_launch(int enabled);
/* Synchronises with the device and reads the container's kernel status word: 0 = every kernel
 * that used this container ran to completion; non-zero = a bounded in-kernel wait ran out
 * (1 producer, 2 consumer) and the affected output is invalid.  The reference has no error
 * reporting of any kind (all its entry points return void). */
int lutgemm_weight_device_status(lutgemm_weight_t w, int* status);

#ifdef __cplusplus
}
#endif
#endif /* LUTGEMM_B200_H */
