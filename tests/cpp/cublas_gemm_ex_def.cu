// The reference's benchmark translation unit (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:25-27) declares
//     template <typename T, typename S> cublasStatus_t cublas_gemm_ex(T* A, T* B, S* C, int m, int n, int k);
// and leaves the definition to the library it links (lutGEMM/src/cuda/kernels/cublas.h:24-56).  This file gives that
// symbol for fp16 so that the unmodified translation unit links against liblutgemm_b200.so:
// row-major C[m][n] = A[m][k] * B[k][n], fp16 in and out, through cublasGemmEx with the operands swapped.
#include <cublas_v2.h>
#include <cuda_fp16.h>

template <typename T, typename S>
cublasStatus_t cublas_gemm_ex(T* A, T* B, S* C, int m, int n, int k) {
    static cublasHandle_t handle = nullptr;
    if (!handle && cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return CUBLAS_STATUS_NOT_INITIALIZED;
    const __half one = __float2half(1.0f), zero = __float2half(0.0f);
    return cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, &one, B, CUDA_R_16F, n, A, CUDA_R_16F, k, &zero,
                        C, CUDA_R_16F, n, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT);
}
template cublasStatus_t cublas_gemm_ex<__half, __half>(__half*, __half*, __half*, int, int, int);
