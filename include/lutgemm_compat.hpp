// Source-compatible C++ surface of naver-aics/lut-gemm's BCQ path, implemented on the C ABI of
// liblutgemm_b200 (include/lutgemm_b200.h).  A translation unit written against the reference's
//   #include "lutGEMM"
//   lutGEMM::nQWeight_fp16 w(bW, A, row, col, nb, false, groups, q_bias);
//   lutGEMM::matmul(out, in, w, m);
// compiles against this header unchanged and links with -llutgemm_b200.
//
// Replaces: class nQWeight_fp16 (lutGEMM/include/nQWeight_fp16.h:27-52), matmul x2
// (lutGEMM/include/kernels.h:26-27), dequantize_gpu / dequantize_cpu (lutGEMM/include/nQWeight_fp16.h:24-25).
// Differences that a caller can observe: the container's arrays live in plain device memory
// (cudaMalloc) instead of managed memory, so bWeight / alpha / q_bias must not be dereferenced on the
// host; q_bias is applied for every batch size, not only for batch 1; every call records a status
// readable through lutGEMM::last_status() instead of failing silently; the destructor frees each
// buffer exactly once; matmul_gptq* compute all m rows in fp32 (the reference kernels compute row 0 in fp16).
#ifndef LUTGEMM_COMPAT_HPP
#define LUTGEMM_COMPAT_HPP

#include <cuda_runtime_api.h>

#include "lutgemm_b200.h"

namespace lutGEMM {

inline int& last_status_ref() {
    static thread_local int s = LUTGEMM_OK;
    return s;
}
// Status of the last lutGEMM:: call on this thread (LUTGEMM_OK == 0); text via lutgemm_status_string().
inline int last_status() { return last_status_ref(); }

class nQWeight_fp16 {
public:
    // Same public fields as the reference container; pointers are device pointers.
    unsigned int* bWeight = nullptr;   // [kSize/32][nb][mSize]
    void* alpha = nullptr;             // fp16 [num_groups][nb][mSize]
    void* q_bias = nullptr;            // fp16 [num_groups][mSize] or nullptr
    int num_groups = 0;
    int group_size = 0;
    int mSize = 0;
    int kSize = 0;
    int nb = 0;
    bool is_row_wise_quantize = false;

    nQWeight_fp16() {}
    nQWeight_fp16(unsigned int* bW, float* A, int row, int col, int num_bits, bool is_row_wise,
                  int num_alpha_groups = 1, float* q_bias_host = nullptr) {
        parsing(bW, A, row, col, num_bits, is_row_wise, num_alpha_groups, q_bias_host);
    }
    nQWeight_fp16(const nQWeight_fp16&) = delete;
    nQWeight_fp16& operator=(const nQWeight_fp16&) = delete;

    void parsing(unsigned int* bW, float* A, int row, int col, int num_bits, bool is_row_wise,
                 int num_alpha_groups = 1, float* q_bias_host = nullptr) {
        release();
        last_status_ref() = lutgemm_weight_create(&handle_, bW, A, row, col, num_bits, is_row_wise ? 1 : 0,
                                                  num_alpha_groups, q_bias_host);
        if (last_status_ref() != LUTGEMM_OK) return;
        lutgemm_weight_desc d;
        lutgemm_weight_describe(handle_, &d);
        bWeight = d.bWeight; alpha = d.alpha; q_bias = d.q_bias;
        num_groups = d.num_groups; group_size = d.group_size; mSize = d.mSize; kSize = d.kSize; nb = d.nb;
        is_row_wise_quantize = d.is_row_wise_quantize != 0;
    }

    // Dense fp16 weight in a device buffer owned by this container (the reference returns a
    // process-wide scratch buffer, lutGEMM/src/nQWeight_fp16.cu:93-99).  Only the GPU path exists.
    void* getDequantiedWeight(bool onGPU = true) {
        (void)onGPU;
        if (!handle_) { last_status_ref() = LUTGEMM_ERR_NULL; return nullptr; }
        if (!dense_) {
            if (cudaMalloc(&dense_, sizeof(unsigned short) * (size_t)mSize * (size_t)kSize) != cudaSuccess) {
                dense_ = nullptr;
                last_status_ref() = LUTGEMM_ERR_CUDA;
                return nullptr;
            }
        }
        last_status_ref() = lutgemm_dequantize(handle_, dense_, nullptr);
        return dense_;
    }

    ~nQWeight_fp16() { release(); }

    lutgemm_weight_t handle() const { return handle_; }

private:
    void release() {
        if (handle_) lutgemm_weight_destroy(handle_);
        handle_ = nullptr;
        if (dense_) cudaFree(dense_);
        dense_ = nullptr;
        bWeight = nullptr; alpha = nullptr; q_bias = nullptr;
    }
    lutgemm_weight_t handle_ = nullptr;
    void* dense_ = nullptr;
};

// The W . X form (lutGEMM/include/kernels.h:26, lutGEMM/src/kernels.cu:56-63,73-75): input[kSize][n] and
// output[mSize][n], fp16 row-major on the device, as the reference's cuBLAS call lays them out
// (lutGEMM/src/cuda/kernels/cublas.h:47-55); for n == 1 plain vectors.  `algo` is accepted and ignored, as in the reference.
inline void matmul(void* output, nQWeight_fp16& nqW, void* input, int n, int algo = 0) {
    (void)algo;
    last_status_ref() = lutgemm_matmul_wx(output, nqW.handle(), input, n, nullptr);
}
// output[m][mSize] (fp16, device) = input[m][kSize] (fp16, device) x W.
inline void matmul(void* output, void* input, nQWeight_fp16& nqW, int m, int algo = 0) {
    (void)algo;
    last_status_ref() = lutgemm_matmul(output, input, nqW.handle(), m, nullptr);
}
// The 3-bit uniform comparison rows (lutGEMM/include/kernels.h:28-33): k = packed rows K * 3 / 32, scale / bias
// (the zero term) fp16 [n], A fp16 [m][K], B uint32 [k][n], C fp16 [m][n]; out = sum_k (scale * code - bias) * in.
inline void matmul_gptq(int m, int n, int k, void* scale, void* bias, void* A, void* B, void* C) {
    last_status_ref() = lutgemm_matmul_gptq(m, n, k, scale, bias, A, (const uint32_t*)B, C, nullptr);
}
inline void matmul_gptq_faster(int m, int n, int k, void* scale, void* bias, void* A, void* B, void* C) {
    last_status_ref() = lutgemm_matmul_gptq(m, n, k, scale, bias, A, (const uint32_t*)B, C, nullptr);
}
// Dense fp16 weight into a device buffer, then waits for it (the reference synchronises too,
// lutGEMM/src/nQWeight_fp16.cu:34).
inline void dequantize_gpu(nQWeight_fp16& nqw, void* d_fW, int algo = 0) {
    (void)algo;
    last_status_ref() = lutgemm_dequantize(nqw.handle(), d_fW, nullptr);
    if (last_status_ref() == LUTGEMM_OK && cudaDeviceSynchronize() != cudaSuccess) last_status_ref() = LUTGEMM_ERR_CUDA;
}
// Dense fp16 weight into a HOST buffer.  Computed by the same GPU kernel (bit-identical to the
// reference's host loop, lutGEMM/src/nQWeight_fp16.cu:38-59) and copied back: this library has no CPU path.
inline void dequantize_cpu(nQWeight_fp16& nqw, void* fW) {
    void* d = nqw.getDequantiedWeight(true);
    if (!d || last_status_ref() != LUTGEMM_OK) return;
    if (cudaMemcpy(fW, d, sizeof(unsigned short) * (size_t)nqw.mSize * (size_t)nqw.kSize, cudaMemcpyDeviceToHost) != cudaSuccess)
        last_status_ref() = LUTGEMM_ERR_CUDA;
}

}  // namespace lutGEMM
#endif  // LUTGEMM_COMPAT_HPP
