/*
 * CPU oracle for the BCQ (binary-coding-quantised) matmul path of naver-aics/lut-gemm.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the host-side
 * semantics of the reference so that the CUDA library can be checked against
 * it.  Nothing in the shipped library links, loads or calls it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity pinning: the reference ships no golden vectors or asserting tests for
 * this path.  The restatement is therefore pinned in two ways: (1) against the
 * reference's own `lutGEMM::dequantize_cpu`, compiled unmodified from the
 * reference sources into oracle/_ref/ (see oracle/Makefile) and compared on
 * seeded inputs; (2) against outputs of the reference's Python converter
 * (examples/rtn_parameter.py, examples/utils.py) stored as fixtures under
 * tests/golden/.  The test-side functions of the reference (packing, fp32
 * dequantisation with q_bias, the serial fp32 matmul) live inside a GoogleTest
 * translation unit that cannot be linked; they are restated here line by line
 * with the file:line each follows.
 *
 * Layouts (column-wise container, the only mode the reference kernels index):
 *   bW     uint32 [K/32][q][N]   bit (k % 32) of bW[k/32][b][n] set  <=>  plane value +1
 *   alpha  fp16   [G][q][N]      G = K / group_size
 *   q_bias fp16   [G][N]
 *   x      [M][K],  y [M][N]
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) { f16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { f16 v = (f16)f; uint16_t h; memcpy(&h, &v, 2); return h; } /* round-to-nearest-even, as __float2half */

/* float -> fp16 bits, the conversion `parsing` applies to alpha and q_bias
 * (lutGEMM/src/nQWeight_fp16.cu:81,85). */
void lgo_float_to_half(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f2h(src[i]);
}
void lgo_half_to_float(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = h2f(src[i]);
}

/* Pack +-1 planes into the kernel layout.
 * Follows makeRandomWeight (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:200-215):
 * bW[k/32][b][n] has bit t set iff plane[k+t][b][n] == +1.
 * planes: int8 [K][q][N] holding +1 / -1. */
void lgo_pack_planes(const int8_t* planes, int K, int q, int N, uint32_t* bW) {
    for (int n = 0; n < N; n++)
        for (int b = 0; b < q; b++)
            for (int k = 0; k < K; k += 32) {
                uint32_t s = 0;
                for (int t = 0; t < 32; t++)
                    if (planes[((size_t)(k + t) * q + b) * N + n] > 0) s |= 1u << t;
                bW[((size_t)(k / 32) * q + b) * N + n] = s;
            }
}

/* Inverse of lgo_pack_planes; the bit test is the one dequantize_cpu uses
 * (lutGEMM/src/nQWeight_fp16.cu:50). */
void lgo_unpack_planes(const uint32_t* bW, int K, int q, int N, int8_t* planes) {
    for (int k = 0; k < K; k++)
        for (int b = 0; b < q; b++)
            for (int n = 0; n < N; n++)
                planes[((size_t)k * q + b) * N + n] =
                    ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) ? 1 : -1;
}

/* Dense fp16 weight from the container, without q_bias.
 * Follows lutGEMM::dequantize_cpu (lutGEMM/src/nQWeight_fp16.cu:38-59):
 * fp32 running sum over planes in order b = 0..q-1, one fp16 rounding at the
 * store; output W[k][n] (column-wise) or W[n][k] (row-wise). */
void lgo_dequantize_cpu(const uint32_t* bW, const uint16_t* alpha, int K, int N, int q,
                        int group_size, int row_wise, uint16_t* fW) {
#pragma omp parallel for schedule(static)
    for (int k = 0; k < K; k++) {
        for (int n = 0; n < N; n++) {
            float tmp = 0.0f;
            for (int b = 0; b < q; b++) {
                float a = h2f(alpha[((size_t)(k / group_size) * q + b) * N + n]);
                if ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) tmp += a;
                else tmp -= a;
            }
            if (row_wise) fW[(size_t)n * K + k] = f2h(tmp);
            else          fW[(size_t)k * N + n] = f2h(tmp);
        }
    }
}

/* Dense fp32 weight including the per-group offset.
 * Follows dequantizeFrom_qW (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:235-244):
 * W[k][n] = q_bias[k/g][n] + sum_b alpha[k/g][b][n] * plane[k][b][n], fp32,
 * planes in order b = 0..q-1.  alpha / q_bias are host floats here, as in the test. */
void lgo_dequantize_from_qw(const uint32_t* bW, const float* alpha, const float* q_bias,
                            int K, int N, int q, int group_size, float* W) {
#pragma omp parallel for schedule(static)
    for (int k = 0; k < K; k++) {
        int g = k / group_size;
        for (int n = 0; n < N; n++) {
            float w = q_bias ? q_bias[(size_t)g * N + n] : 0.0f;
            for (int b = 0; b < q; b++) {
                float s = ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) ? 1.0f : -1.0f;
                w += alpha[((size_t)g * q + b) * N + n] * s;
            }
            W[(size_t)k * N + n] = w;
        }
    }
}

/* out[m][n] = sum_k in[m][k] * W[k][n], fp32, k ascending.
 * Follows matmul_cpu (tests/opt/fp16/int3_col_wise_matmul_fp16.cu:174-183). */
void lgo_matmul_cpu(const float* in, const float* W, float* out, int M, int N, int K) {
    for (int m = 0; m < M; m++) {
#pragma omp parallel for schedule(static)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) acc += in[(size_t)m * K + k] * W[(size_t)k * N + n];
            out[(size_t)m * N + n] = acc;
        }
    }
}

/* The reference's host "dequant-and-matmul" result for fp16 inputs:
 *   W_h   = dequantize_cpu(container)                   (fp16, no offset)
 *   y     = matmul_cpu(float(x_h), float(W_h))          (fp32, k ascending)
 *   y    += sum_g float(q_bias_h[g][n]) * sum_{k in g} float(x_h[k])   (offset term of
 *           dequantizeFrom_qW, tests/...fp16.cu:238, which dequantize_cpu omits)
 * x: fp16 bits [M][K]; alpha/q_bias: fp16 bits; y: fp32 [M][N].
 * Never materialises more than one k-row of W, but rounds each W[k][n] to fp16
 * exactly as the dense path does, and adds in the same k order. */
void lgo_bcq_matmul_ref(const uint16_t* x, const uint32_t* bW, const uint16_t* alpha,
                        const uint16_t* q_bias, int M, int N, int K, int q, int group_size,
                        float* y) {
    int G = K / group_size;
    for (int m = 0; m < M; m++) {
        float* gsum = (float*)calloc((size_t)G, sizeof(float));
        if (q_bias)
            for (int k = 0; k < K; k++) gsum[k / group_size] += h2f(x[(size_t)m * K + k]);
#pragma omp parallel for schedule(static)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                float tmp = 0.0f;
                for (int b = 0; b < q; b++) {
                    float a = h2f(alpha[((size_t)(k / group_size) * q + b) * N + n]);
                    if ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) tmp += a;
                    else tmp -= a;
                }
                acc += h2f(x[(size_t)m * K + k]) * h2f(f2h(tmp));
            }
            if (q_bias) {
                float off = 0.0f;
                for (int g = 0; g < G; g++) off += h2f(q_bias[(size_t)g * N + n]) * gsum[g];
                acc += off;
            }
            y[(size_t)m * N + n] = acc;
        }
        free(gsum);
    }
}

/* The reference's fp32 host result, test-side semantics, never materialising W:
 *   W[k][n] = q_bias[k/g][n] + sum_b alpha[k/g][b][n] * plane[k][b][n]     (dequantizeFrom_qW,
 *             tests/opt/fp16/int3_col_wise_matmul_fp16.cu:235-244; fp32, b ascending)
 *   y[m][n] = sum_k x[m][k] * W[k][n]                                      (matmul_cpu, :174-183; fp32, k ascending)
 * alpha and q_bias are the container's fp16 values (what parsing stores, lutGEMM/src/nQWeight_fp16.cu:81,85)
 * widened to float; x is the fp16 activation widened to float.  This is the "fp32 reference" the
 * matvec tolerance is stated against. */
void lgo_bcq_matmul_fp32(const uint16_t* x, const uint32_t* bW, const uint16_t* alpha,
                         const uint16_t* q_bias, int M, int N, int K, int q, int group_size,
                         float* y) {
    for (int m = 0; m < M; m++) {
#pragma omp parallel for schedule(static)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                int g = k / group_size;
                float w = q_bias ? h2f(q_bias[(size_t)g * N + n]) : 0.0f;
                for (int b = 0; b < q; b++) {
                    float s = ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) ? 1.0f : -1.0f;
                    w += h2f(alpha[((size_t)g * q + b) * N + n]) * s;
                }
                acc += h2f(x[(size_t)m * K + k]) * w;
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

/* Independent restatement in double precision with no intermediate fp16
 * rounding of W; bounds the oracle's own rounding error. */
void lgo_bcq_matmul_f64(const uint16_t* x, const uint32_t* bW, const uint16_t* alpha,
                        const uint16_t* q_bias, int M, int N, int K, int q, int group_size,
                        double* y) {
    for (int m = 0; m < M; m++) {
#pragma omp parallel for schedule(static)
        for (int n = 0; n < N; n++) {
            double acc = 0.0;
            for (int k = 0; k < K; k++) {
                int g = k / group_size;
                double w = q_bias ? (double)h2f(q_bias[(size_t)g * N + n]) : 0.0;
                for (int b = 0; b < q; b++) {
                    double a = (double)h2f(alpha[((size_t)g * q + b) * N + n]);
                    w += ((bW[((size_t)(k / 32) * q + b) * N + n] >> (k % 32)) & 1) ? a : -a;
                }
                acc += (double)h2f(x[(size_t)m * K + k]) * w;
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

/* Uniform (scale, zero, code) -> BCQ with offset.
 * Follows RTNParameter.convert_bcq_format (examples/rtn_parameter.py:77-96), fp32:
 *   alpha[n][g][i]     = (scale[n][g] / 2) * 2^i
 *   binary[n][g][j][i] = ((code[n][g][j] >> i) & 1) * 2 - 1
 *   offset[n][g]       = sum_i alpha[n][g][i] - scale[n][g] * zero[n][g]
 * The alpha row is the fp32 matmul of a 1-element row by [2^0 .. 2^(q-1)], i.e.
 * one fp32 product each; the sum over i is taken in ascending i as torch.sum
 * does for a short contiguous row. */
void lgo_uniform_to_bcq(const float* scale, const float* zero, const int32_t* code,
                        int N, int G, int g, int q,
                        float* alpha, int8_t* binary, float* offset) {
    for (size_t ng = 0; ng < (size_t)N * G; ng++) {
        float z = scale[ng] * zero[ng];
        float half = scale[ng] / 2.0f;
        float s = 0.0f;
        for (int i = 0; i < q; i++) {
            float a = half * (float)(1u << i);
            alpha[ng * q + i] = a;
            s += a;
        }
        offset[ng] = s - z;
        for (int j = 0; j < g; j++)
            for (int i = 0; i < q; i++)
                binary[(ng * g + j) * q + i] = (int8_t)(((code[ng * g + j] >> i) & 1) * 2 - 1);
    }
}

/* Python-side tensors (in_ch_wise = False; W is [N][K]) -> kernel layout.
 *   alpha_k[g][b][n]  = alpha_py[n][g][b]
 *   q_bias_k[g][n]    = offset_py[n][g]
 *   bit (k%32) of bW[k/32][b][n] = binary_py[n][k/gs][k%gs][b] > 0
 * Shapes follow examples/bcq_parameter.py:41-48; the bit convention is the
 * kernel's (lutGEMM/src/nQWeight_fp16.cu:50). */
void lgo_python_to_kernel_layout(const float* alpha_py, const int8_t* binary_py, const float* offset_py,
                                 int N, int K, int gs, int q,
                                 float* alpha_k, uint32_t* bW, float* q_bias_k) {
    int G = K / gs;
    memset(bW, 0, (size_t)(K / 32) * q * N * sizeof(uint32_t));
    for (int n = 0; n < N; n++)
        for (int g = 0; g < G; g++) {
            if (offset_py) q_bias_k[(size_t)g * N + n] = offset_py[(size_t)n * G + g];
            for (int b = 0; b < q; b++)
                alpha_k[((size_t)g * q + b) * N + n] = alpha_py[((size_t)n * G + g) * q + b];
            for (int j = 0; j < gs; j++) {
                int k = g * gs + j;
                for (int b = 0; b < q; b++)
                    if (binary_py[(((size_t)n * G + g) * gs + j) * q + b] > 0)
                        bW[((size_t)(k / 32) * q + b) * N + n] |= 1u << (k % 32);
            }
        }
}

/* The Python examples' uint8 interchange format.
 * Follows Packer.pack (examples/utils.py:162-172): the +-1 tensor is flattened,
 * mapped to {0,1}, viewed as [8][L/8]; byte j = sum_i 2^i * flat[i*L/8 + j]. */
void lgo_packer_pack(const int8_t* flat_pm1, size_t L, uint8_t* out) {
    size_t cols = L / 8;
    for (size_t j = 0; j < cols; j++) {
        unsigned v = 0;
        for (int i = 0; i < 8; i++)
            if (flat_pm1[(size_t)i * cols + j] > 0) v |= 1u << i;
        out[j] = (uint8_t)v;
    }
}
/* Follows Packer.unpack (examples/utils.py:174-181). */
void lgo_packer_unpack(const uint8_t* packed, size_t L, int8_t* flat_pm1) {
    size_t cols = L / 8;
    for (int i = 0; i < 8; i++)
        for (size_t j = 0; j < cols; j++)
            flat_pm1[(size_t)i * cols + j] = ((packed[j] >> i) & 1) ? 1 : -1;
}

int lgo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void lgo_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
