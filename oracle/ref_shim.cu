/*
 * Thin C entry points around the UNMODIFIED reference sources, which are
 * compiled where they lie (never copied) by oracle/Makefile into oracle/_ref/.
 *
 * TEST INFRASTRUCTURE ONLY: used to pin the C restatement in
 * lutgemm_oracle.c against the reference's own code and, in the benchmark,
 * as the timed reference baseline.  The shipped library never loads it.
 *
 * ref_dequantize_cpu   -> lutGEMM::dequantize_cpu   (lutGEMM/src/nQWeight_fp16.cu:38-59), host only
 * ref_gpu_matmul_gptq -> lutGEMM::matmul_gptq / matmul_gptq_faster (lutGEMM/src/kernels.cu:40-54)
 * ref_gpu_*            -> nQWeight_fp16::parsing + lutGEMM::matmul on the GPU
 *                         (lutGEMM/src/nQWeight_fp16.cu:60-91, lutGEMM/src/kernels.cu:56-71);
 *                         built only into libref_gpu.so (REF_WITH_GPU).
 */
#include <cstdint>
#include <cstdlib>
#include <new>
#include "nQWeight_fp16.h"
#ifdef REF_WITH_GPU
#include "kernels.h"
#include <cuda_runtime.h>
#endif

extern "C" {

/* Fills the container's public fields by hand instead of calling parsing():
 * parsing() needs managed device memory, and it computes group_size from an
 * unset kSize (lutGEMM/src/nQWeight_fp16.cu:62-63), so the field is set here.
 * The object is placement-constructed in a raw buffer and never destroyed: the
 * reference destructor would cudaFree host pointers. */
void ref_dequantize_cpu(const uint32_t* bW, const uint16_t* alpha_h, int K, int N, int q,
                        int group_size, int row_wise, uint16_t* fW) {
    alignas(16) static thread_local unsigned char raw[sizeof(lutGEMM::nQWeight_fp16)];
    lutGEMM::nQWeight_fp16* w = new (raw) lutGEMM::nQWeight_fp16();
    w->bWeight = const_cast<uint32_t*>(bW);
    w->alpha = (void*)alpha_h;
    w->q_bias = nullptr;
    w->num_groups = K / group_size;
    w->group_size = group_size;
    w->mSize = N;
    w->kSize = K;
    w->nb = q;
    w->is_row_wise_quantize = row_wise != 0;
    lutGEMM::dequantize_cpu(*w, (void*)fW);
}

#ifdef REF_WITH_GPU
/* Creates a reference container through the reference's own parsing() (managed
 * memory) and returns it as an opaque pointer.  Leaked on purpose at exit: the
 * reference destructor double-frees alpha (lutGEMM/src/nQWeight_fp16.cu:101-105). */
void* ref_gpu_create(uint32_t* bW, float* alpha, float* q_bias, int K, int N, int q, int num_groups) {
    auto* w = new lutGEMM::nQWeight_fp16();
    w->parsing(bW, alpha, K, N, q, false, num_groups, q_bias);
    /* parsing() computes group_size from kSize before kSize is set (lutGEMM/src/nQWeight_fp16.cu:62-63), leaving it
     * indeterminate; the m = 1 kernels never read it, but the batched path's _dequantize_t divides by it
     * (lutGEMM/src/cuda/kernels/dequant_fp16.hpp:66), so the public field is given the value it was meant to have. */
    w->group_size = K / num_groups;
    cudaDeviceSynchronize();
    return (void*)w;
}
/* out, in: device (or managed) fp16 pointers.  m == 1 runs the reference LUT matvec kernels, m > 1 its
 * dequantise-to-scratch + cuBLAS path (q <= 4 only: beyond that its dequantiser launches nothing,
 * lutGEMM/src/cuda/kernels/dequant_fp16.hpp:102-105); legacy default stream, as the reference does. */
void ref_gpu_matmul(void* out, void* in, void* w, int m) {
    lutGEMM::matmul(out, in, *(lutGEMM::nQWeight_fp16*)w, m);
}
/* The reference's 3-bit uniform kernels (lutGEMM/src/kernels.cu:40-54): k = packed rows, all pointers device or
 * managed; they read whole 24-row x 256-column blocks without bounds checks, so call them only with
 * K % 256 == 0 and n % 256 == 0. */
void ref_gpu_matmul_gptq(int m, int n, int k, void* scale, void* bias, void* A, void* B, void* C, int faster) {
    if (faster) lutGEMM::matmul_gptq_faster(m, n, k, scale, bias, A, B, C);
    else lutGEMM::matmul_gptq(m, n, k, scale, bias, A, B, C);
}
int ref_gpu_last_error() { return (int)cudaGetLastError(); }
#endif
}
