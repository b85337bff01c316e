// Written the way the reference's benchmark uses the library (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:
// parsing at :70, matmul at :123, managed buffers at :246-256), compiled against include/lutGEMM.
// Prints "shim ok <max abs diff>" and returns 0 when the GPU result matches a host fp32 evaluation.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "lutGEMM"

int main() {
    const int M = 1, N = 512, K = 1024, NB = 3, GS = 128, G = K / GS;
    std::vector<uint32_t> bW((size_t)K / 32 * NB * N);
    std::vector<float> alpha((size_t)G * NB * N), q_bias((size_t)G * N), x(K);
    uint32_t s = 12345u;
    auto rnd = [&]() { s = s * 1664525u + 1013904223u; return s; };
    for (auto& w : bW) w = rnd();
    for (auto& a : alpha) a = __half2float(__float2half((rnd() >> 8) * (0.04f / 16777216.0f)));
    for (auto& b : q_bias) b = __half2float(__float2half(((int)(rnd() >> 8) - 8388608) * (0.02f / 8388608.0f)));
    for (auto& v : x) v = __half2float(__float2half(((int)(rnd() >> 8) - 8388608) * (1.0f / 8388608.0f)));

    __half *d_in, *d_out;
    if (cudaMallocManaged(&d_in, sizeof(__half) * M * K) != cudaSuccess) { printf("no device\n"); return 2; }
    cudaMallocManaged(&d_out, sizeof(__half) * M * N);
    for (int k = 0; k < K; k++) d_in[k] = __float2half(x[k]);

    lutGEMM::nQWeight_fp16 nqW;
    nqW.parsing(bW.data(), alpha.data(), K, N, NB, false, G, q_bias.data());
    if (lutGEMM::last_status() != 0) { printf("parsing failed: %s\n", lutgemm_status_string(lutGEMM::last_status())); return 1; }
    lutGEMM::matmul((void*)d_out, (void*)d_in, nqW, M);
    cudaDeviceSynchronize();
    if (lutGEMM::last_status() != 0) { printf("matmul failed: %s\n", lutgemm_status_string(lutGEMM::last_status())); return 1; }

    // the X.W call against a host fp32 evaluation: max relative error (floor 1e-2 rms) <= 1e-2, mean absolute error <= 1e-3
    std::vector<float> ref(N);
    double rms = 0;
    for (int n = 0; n < N; n++) {
        float acc = 0;
        for (int k = 0; k < K; k++) {
            float w = q_bias[(size_t)(k / GS) * N + n];
            for (int b = 0; b < NB; b++) {
                float sgn = ((bW[((size_t)(k / 32) * NB + b) * N + n] >> (k % 32)) & 1) ? 1.f : -1.f;
                w += alpha[((size_t)(k / GS) * NB + b) * N + n] * sgn;
            }
            acc += x[k] * w;
        }
        ref[n] = acc;
        rms += (double)acc * acc;
    }
    rms = std::sqrt(rms / N);
    double max_rel = 0, mae = 0;
    for (int n = 0; n < N; n++) {
        const double d = std::fabs(ref[n] - __half2float(d_out[n]));
        max_rel = std::fmax(max_rel, d / std::fmax(std::fabs((double)ref[n]), 1e-2 * rms));
        mae += d / N;
    }
    // the W.X overload with n = 4 columns: input [K][4], output [N][4]; column c carries 2^(c-2) * x (exact in fp16)
    const int NC = 4;
    __half *d_in2, *d_out2;
    cudaMallocManaged(&d_in2, sizeof(__half) * K * NC);
    cudaMallocManaged(&d_out2, sizeof(__half) * N * NC);
    for (int k = 0; k < K; k++)
        for (int c = 0; c < NC; c++) d_in2[k * NC + c] = __float2half(x[k] * 0.25f * (float)(1 << c));
    lutGEMM::matmul((void*)d_out2, nqW, (void*)d_in2, NC);
    cudaDeviceSynchronize();
    double max_rel2 = 0;
    for (int n = 0; n < N; n++)
        for (int c = 0; c < NC; c++) {
            const double want = ref[n] * 0.25 * (double)(1 << c);
            const double d = std::fabs(want - __half2float(d_out2[n * NC + c]));
            max_rel2 = std::fmax(max_rel2, d / std::fmax(std::fabs(want), 1e-2 * rms));
        }
    std::vector<__half> dense((size_t)K * N);
    lutGEMM::dequantize_cpu(nqW, dense.data());
    printf("shim ok %.3e %.3e wx %.3e fields %d %d %d %d %d\n", max_rel, mae, max_rel2, nqW.mSize, nqW.kSize, nqW.nb, nqW.num_groups,
           nqW.group_size);
    cudaFree(d_in); cudaFree(d_out); cudaFree(d_in2); cudaFree(d_out2);
    return (max_rel <= 1e-2 && mae <= 1e-3 && max_rel2 <= 1e-2 && lutGEMM::last_status() == 0) ? 0 : 1;
}
