/*
 * ORACLE -- TEST INFRASTRUCTURE ONLY. Nothing in the product (the package under
 * flash-train_b200/) may include, link or call this file; only tests/, the
 * smoke check and the benchmark's CPU-baseline leg use it, as the checker.
 *
 * Plain C restatement of the reference's FP32 GEMM arithmetic
 *   d[i,j] = alpha * sum_k a[i,k] * b[k,j] + beta * c[i,j]
 * following, line by line:
 *   - the device kernel, src/primitive/hygon/gemm/fp32_gemm.hip:24-30
 *     (float accumulator starting at 0, k ascending, then
 *     alpha * acc + (c ? beta * c : 0));
 *   - the host reference of the reference's own numerics test,
 *     tests/api/gemm_numerics_test.cpp:34-51 (same loop order);
 *   - that test's deterministic fill, tests/api/gemm_numerics_test.cpp:30-32.
 * Pinned against the reference's golden vectors (tests/golden/) and against
 * the reference's own sources compiled for the CPU (oracle/_ref).
 *
 * Two FP32 variants exist because a compiler may or may not contract
 * `acc += a * b` into a fused multiply-add: ftoracle_gemm_f32 rounds the
 * product and the sum separately (this file is built with -ffp-contract=off),
 * ftoracle_gemm_f32_fma uses fmaf as GPU compilers do. ftoracle_gemm_f64
 * accumulates in double and is the accuracy yardstick.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/* Element strides allow any layout; dense row-major is (cols, 1). */
typedef struct {
    int64_t row;
    int64_t col;
} ftoracle_strides;

float ftoracle_element_value(uint64_t linear) {
    return (float)((linear * 2654435761ULL) % 199ULL) / 199.0F - 0.5F;
}

void ftoracle_fill(float* out, uint64_t count, uint64_t offset) {
    for (uint64_t i = 0; i < count; ++i) { out[i] = ftoracle_element_value(i + offset); }
}

void ftoracle_gemm_f32(const float* a, ftoracle_strides sa, const float* b, ftoracle_strides sb, const float* c,
                       ftoracle_strides sc, float* d, ftoracle_strides sd, int64_t m, int64_t n, int64_t k, float alpha,
                       float beta) {
    for (int64_t row = 0; row < m; ++row) {
        for (int64_t column = 0; column < n; ++column) {
            float accumulator = 0.0F;
            for (int64_t depth = 0; depth < k; ++depth) {
                const float product = a[row * sa.row + depth * sa.col] * b[depth * sb.row + column * sb.col];
                accumulator         = accumulator + product;
            }
            const float scaled = alpha * accumulator;
            const float addend = c != NULL ? beta * c[row * sc.row + column * sc.col] : 0.0F;
            d[row * sd.row + column * sd.col] = scaled + addend;
        }
    }
}

void ftoracle_gemm_f32_fma(const float* a, ftoracle_strides sa, const float* b, ftoracle_strides sb, const float* c,
                           ftoracle_strides sc, float* d, ftoracle_strides sd, int64_t m, int64_t n, int64_t k,
                           float alpha, float beta) {
    for (int64_t row = 0; row < m; ++row) {
        for (int64_t column = 0; column < n; ++column) {
            float accumulator = 0.0F;
            for (int64_t depth = 0; depth < k; ++depth) {
                accumulator = fmaf(a[row * sa.row + depth * sa.col], b[depth * sb.row + column * sb.col], accumulator);
            }
            float value = alpha * accumulator;
            if (c != NULL) { value = fmaf(beta, c[row * sc.row + column * sc.col], value); }
            d[row * sd.row + column * sd.col] = value;
        }
    }
}

void ftoracle_gemm_f64(const float* a, ftoracle_strides sa, const float* b, ftoracle_strides sb, const float* c,
                       ftoracle_strides sc, double* d, int64_t m, int64_t n, int64_t k, float alpha, float beta) {
    for (int64_t row = 0; row < m; ++row) {
        for (int64_t column = 0; column < n; ++column) {
            double accumulator = 0.0;
            for (int64_t depth = 0; depth < k; ++depth) {
                accumulator += (double)a[row * sa.row + depth * sa.col] * (double)b[depth * sb.row + column * sb.col];
            }
            double value = (double)alpha * accumulator;
            if (c != NULL) { value += (double)beta * (double)c[row * sc.row + column * sc.col]; }
            d[row * n + column] = value;
        }
    }
}
