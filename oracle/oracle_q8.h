/*
 * oracle_q8.h - CPU restatement of Laplace's int8-activation quantized matmul.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped CUDA library includes,
 * links or calls this code; it exists so the parity tests, the smoke check and
 * the CPU-baseline leg of the benchmark have something to compare against.
 *
 * What it restates (paths inside the Laplace project):
 *   src/matmul_simd.cpp:26-32    ActQ8 activation block
 *   src/matmul_simd.cpp:348-410  quantize_act_q8_neon
 *   src/matmul_simd.cpp:143-160  dot_row_q8_0_int_neon
 *   src/matmul_simd.cpp:162-182  dot_row_q4_0_int_neon
 *   src/matmul_simd.cpp:184-224  dot_row_q5_0_int_neon
 *   src/matmul_simd.cpp:226-283  dot_row_q4_k_int_neon
 *   src/matmul_simd.cpp:285-342  dot_row_q6_k_int_neon
 *   src/matmul_simd.cpp:432-455  gemm_int row loop
 *   src/matmul_simd.cpp:506-544  moe_gemv_int / moe_gemv_multi_int
 *   src/kernels.h:21-54,82-90    block layouts, 6-bit scale/min unpack
 *   src/fp16.h:9-69              software binary16 conversions
 *   src/matmul.cpp:84-198        scalar fp32-activation dots (cross-check)
 *   src/matmul.cpp:504-603       dequantize()
 *
 * PARITY PIN. The reference's NEON path cannot be executed on an x86 host and
 * the reference's tests hold no literal output vectors for it, so at the
 * 1e-5 / bit-exact level this restatement is itself the pin. It is anchored
 * three ways (see tests/): it passes the reference test's Q8-round-trip check
 * (tests/test_matmul.cpp:57-97) on that test's own seeded inputs, its fp16
 * conversions reproduce the known answers of tests/test_matmul.cpp:252-268,
 * and its dequantizers/scalar dots agree with the reference's own scalar code
 * compiled unmodified into oracle/_ref.
 */
#ifndef LAPLACE_ORACLE_Q8_H
#define LAPLACE_ORACLE_Q8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids used on this path (src/tensor.h:11-34). */
enum { LPO_Q4_0 = 2, LPO_Q5_0 = 6, LPO_Q8_0 = 8, LPO_Q4_K = 12, LPO_Q6_K = 14 };

/* Same 44-byte layout as the reference's private ActQ8. */
typedef struct {
    float   d;
    float   sum;
    int16_t sum_lo;
    int16_t sum_hi;
    int8_t  qs[32];
} lpo_actq8;

/* Result modes of the dot products. */
enum {
    LPO_MODE_F32_LANES = 0, /* fp32, same accumulator lanes and fma order as the NEON code */
    LPO_MODE_F64       = 1, /* every product and sum in double; for error measurement */
    LPO_MODE_MASS      = 2  /* sum of |term| in double: the magnitude that fp32 accumulation
                               error scales with when the terms cancel */
};

float    lpo_fp16_to_fp32(uint16_t h);
uint16_t lpo_fp32_to_fp16(float f);

size_t lpo_row_bytes(uint32_t type, int K);          /* 0 when the type is not handled */
int    lpo_block_elems(uint32_t type);               /* 32 or 256, 0 when unhandled */

/* Activation quantizer: K/32 blocks for one row / for M rows. */
void lpo_quantize_row(const float* x, int K, lpo_actq8* out);
void lpo_quantize_rows(const float* x, int M, int K, lpo_actq8* out);

/* One weight row against one quantized activation row. */
double lpo_dot(uint32_t type, const lpo_actq8* xa, const uint8_t* row, int K, int mode);

/* Integer block sums of one row. Q8_0/Q4_0/Q5_0/Q4_K: K/32 values; Q6_K: K/16 values.
 * Returns how many were written. */
int lpo_row_blocksums(uint32_t type, const lpo_actq8* xa, const uint8_t* row, int K, int32_t* out);

/* y[m*N+j] for all m<M, j<N. threads<=1 runs serially. Returns 0, or 1 when
 * the type is not one of the five. */
int lpo_gemm(const float* x, const uint8_t* w, uint32_t type, float* y,
             int M, int K, int N, int mode, int threads);
int lpo_moe_gemv(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                 int n_experts, float* y, int K, int N, int mode, int threads);
int lpo_moe_gemv_multi(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                       int n_experts, float* y, int K, int N, int mode, int threads);

/* Block sums for a whole matrix: out[(m*N+j)*per_row + b]. */
int lpo_gemm_blocksums(const float* x, const uint8_t* w, uint32_t type, int32_t* out,
                       int M, int K, int N);

/* fp32-activation scalar path and dequantizer (secondary cross-check). */
float lpo_dot_scalar(uint32_t type, const float* x, const uint8_t* row, int K);
int   lpo_gemm_scalar(const float* x, const uint8_t* w, uint32_t type, float* y,
                      int M, int K, int N, int threads);
int   lpo_dequantize(uint32_t type, const uint8_t* w, float* dst, size_t n);

/* The seeded inputs of the reference's own tests/test_matmul.cpp (XorShift32,
 * tests/test_util.h:47-61): x of check_against_ref (:60-61) and the weight
 * blocks of test_q4_0/q8_0/q4_k/q6_k (:142-212). */
void lpo_testgen_x(uint32_t type, int K, float* x);
int  lpo_testgen_weights(uint32_t type, int K, int N, uint8_t* out);

#ifdef __cplusplus
}
#endif
#endif
