/* CPU oracle for picograd's dense matrix-multiply path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (picograd_b200/, include/)
 * may call, link or load this; only tests/, the smoke check and the benchmark's
 * CPU-baseline leg do, and there only as the checker.
 *
 * Each function restates, in plain C, what one function of picograd computes
 * (the file:line it follows is given at its definition in pg_oracle.c).
 * Parity of this restatement is pinned two ways: against the golden vectors
 * that picograd's own tests hold for the path, and against outputs of the
 * unmodified picograd CPU library compiled from its sources (oracle/_ref).
 */
#ifndef PG_ORACLE_H
#define PG_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes: core/dtype.h:11-16 */
enum { PGO_F32 = 0, PGO_F16 = 1, PGO_BF16 = 2 };

uint16_t pgo_f32_to_bf16(float f);
float    pgo_bf16_to_f32(uint16_t h);
uint16_t pgo_f32_to_f16(float f);
float    pgo_f16_to_f32(uint16_t h);
void pgo_f32_to_bf16_n(uint16_t *dst, const float *src, size_t n);
void pgo_f32_to_f16_n(uint16_t *dst, const float *src, size_t n);
void pgo_bf16_to_f32_n(float *dst, const uint16_t *src, size_t n);
void pgo_f16_to_f32_n(float *dst, const uint16_t *src, size_t n);

/* C[m,n] (f32, overwritten) = A[m,k] * B[k,n]; row-major, ld* in elements. */
void pgo_gemm_ex(int dtype, size_t m, size_t n, size_t k,
                 const void *a, size_t lda, const void *b, size_t ldb,
                 float *c, size_t ldc);

/* Only rows [r0,r1) x columns [c0,c1) of C are computed (same arithmetic);
 * lets a test check panels of a full-size product in seconds. */
/* pg_cpu_gemm_fused_ex: C = act(bias[j] + A*B), the chain of column j starting at bias[j]
 * (bias may be NULL).  act: PGO_ACT_* = PG_ACT_* of backend/cpu/gemm.h:37-39. */
#define PGO_ACT_NONE 0
#define PGO_ACT_RELU 1
#define PGO_ACT_GELU 2
void pgo_gemm_fused_ex(int dtype, size_t m, size_t n, size_t k,
                       const void *a, size_t lda, const void *b, size_t ldb,
                       float *c, size_t ldc, const float *bias, int act);
void pgo_gemm_ex_panel(int dtype, size_t m, size_t n, size_t k,
                       const void *a, size_t lda, const void *b, size_t ldb,
                       float *c, size_t ldc,
                       size_t r0, size_t r1, size_t c0, size_t c1);

/* Batched strict 3-D case: [batch,m,k] x [batch,k,n] -> f32 [batch,m,n]. */
void pgo_bmm(int dtype, size_t batch, size_t m, size_t n, size_t k,
             const void *a, const void *b, float *c);

/* Matmul backward for one 2-D pair: ga[m,k] += g[m,n] * B^T ; gb[k,n] += A^T * g.
 * A, B in `dtype` (upcast exactly to f32 first), g and the gradients f32.
 * ga or gb may be NULL. */
void pgo_matmul_backward(int dtype, size_t m, size_t n, size_t k,
                         const void *a, const void *b, const float *g,
                         float *ga, float *gb);

/* Row softmax over the last axis and erf-GELU, the two harness steps between
 * the GEMMs of the attention-shaped and MLP workloads. */
/* pg_addmm (ops/matmul.c:371-405): c = beta * input + alpha * (a * b), input read through element strides
 * (0 = broadcast along that dimension), every step a separate rounded f32 operation as in picograd. */
void pgo_addmm(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
               float *c, size_t ldc, const float *input, size_t in_rs, size_t in_cs, float alpha, float beta);
/* pg_conv2d (ops/conv.c:10-146): x [n,cin,h,w], wt [cout,cin,kh,kw], bias [cout] or NULL ->
 * out [n,cout,oh,ow], oh = (h + 2 pad - kh) / stride + 1.  Returns -1 for shapes pg_conv2d rejects. */
int pgo_conv2d(size_t n, size_t cin, size_t h, size_t w, size_t cout, size_t kh, size_t kw,
               int stride, int pad, const float *x, const float *wt, const float *bias, float *out);
void pgo_softmax_rows(float *out, const float *src, size_t rows, size_t len);
void pgo_gelu(float *out, const float *src, size_t n);
void pgo_gelu_grad(float *out, const float *x, const float *gy, size_t n);

/* Number of threads the loops above use (OpenMP). */
int pgo_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
