/* Drop-in check of the CALLERS: picograd's own, unmodified pg_matmul / pg_bmm / pg_tensordot
 * (src/ops/matmul.c) and pg_gemm_ex, linked against picograd's objects plus OUR CUDA seat
 * (oracle/Makefile target `dropin`).  Each product is computed twice through picograd's public
 * API — once with pg_set_device(PG_DEV_CPU), once with pg_set_device(PG_DEV_CUDA) — and compared.
 * f32 goes through picograd's try_matmul_gpu (pg_dev_malloc / pg_copy_h2d / pg_gemm / pg_copy_d2h,
 * matmul.c:56-184); f16/bf16 go through pg_gemm_ex with host pointers (matmul.c:264-271), which our
 * seat stages.  Exit code 0 = all within tolerance, 77 = no CUDA device (skipped).
 *
 * Built only where picograd's sources are present; includes picograd's headers, copies none.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "backend/backend.h"
#include "core/convert.h"
#include "core/tensor.h"
#include "ops/matmul.h"

static int fails;

static double relerr(const pg_tensor *x, const pg_tensor *y)
{
    double num = 0, den = 0;
    if (!x || !y || x->numel != y->numel) return 1e9;
    for (size_t i = 0; i < x->numel; i++) {
        double d = (double)x->data[i] - (double)y->data[i];
        num += d * d;
        den += (double)y->data[i] * (double)y->data[i];
    }
    return den > 0 ? sqrt(num / den) : sqrt(num);
}

static pg_tensor *rounded(const pg_tensor *f32, pg_dtype dt)
{
    pg_tensor *t = pg_tensor_empty_dtype(dt, f32->ndim, f32->shape);
    for (size_t i = 0; i < f32->numel; i++)
        t->data_u16[i] = dt == PG_DTYPE_BF16 ? pg_f32_to_bf16_scalar(f32->data[i]) : pg_f32_to_f16_scalar(f32->data[i]);
    return t;
}

typedef pg_tensor *(*binop)(const pg_tensor *, const pg_tensor *);

static void check(const char *what, binop op, const pg_tensor *a, const pg_tensor *b, double tol)
{
    pg_set_device(PG_DEV_CPU);
    pg_tensor *want = op(a, b);
    pg_set_device(PG_DEV_CUDA);
    pg_tensor *got = op(a, b);
    pg_dev_sync();
    pg_set_device(PG_DEV_CPU);
    double e = relerr(got, want);
    printf("%-44s rel.err %.3e (tol %.1e) %s\n", what, e, tol, e <= tol ? "ok" : "FAIL");
    if (!(e <= tol)) fails++;
    pg_tensor_free(want);
    pg_tensor_free(got);
}

static pg_tensor *tdot(const pg_tensor *a, const pg_tensor *b)
{
    size_t aa[1] = {2}, ab[1] = {0};
    return pg_tensordot(a, b, 1, aa, ab);
}

int main(void)
{
    if (pg_set_device(PG_DEV_CUDA) != PG_OK) {
        printf("dropin_callers: cuda not available, skipping\n");
        return 77;
    }
    pg_set_device(PG_DEV_CPU);
    pg_seed(7);
    size_t s2a[2] = {192, 256}, s2b[2] = {256, 136};
    size_t s3a[3] = {4, 72, 64}, s3b[3] = {4, 64, 40};
    size_t t3a[3] = {6, 5, 16}, t3b[3] = {16, 24, 3};
    pg_tensor *a = pg_tensor_uniform(2, s2a, -1, 1), *b = pg_tensor_uniform(2, s2b, -1, 1);
    pg_tensor *a3 = pg_tensor_uniform(3, s3a, -1, 1), *b3 = pg_tensor_uniform(3, s3b, -1, 1);
    pg_tensor *ta = pg_tensor_uniform(3, t3a, -1, 1), *tb = pg_tensor_uniform(3, t3b, -1, 1);
    size_t s2c[2] = {64, 40};
    pg_tensor *b2 = pg_tensor_uniform(2, s2c, -1, 1);

    check("pg_matmul f32 [192,256]x[256,136]", pg_matmul, a, b, 1e-6);
    check("pg_bmm    f32 [4,72,64]x[4,64,40]", pg_bmm, a3, b3, 1e-6);
    check("pg_matmul f32 batched [4,72,64] x unbatched [64,40]", pg_matmul, a3, b2, 1e-6);
    check("pg_tensordot f32 axes ([2],[0])", tdot, ta, tb, 1e-6);

    pg_tensor *ab = rounded(a, PG_DTYPE_BF16), *bb = rounded(b, PG_DTYPE_BF16);
    pg_tensor *ah = rounded(a, PG_DTYPE_F16), *bh = rounded(b, PG_DTYPE_F16);
    pg_tensor *a3b = rounded(a3, PG_DTYPE_BF16), *b3b = rounded(b3, PG_DTYPE_BF16);
    check("pg_matmul bf16 (pg_gemm_ex, host pointers)", pg_matmul, ab, bb, 1e-5 * sqrt(256.0));
    check("pg_matmul f16  (pg_gemm_ex, host pointers)", pg_matmul, ah, bh, 1e-5 * sqrt(256.0));
    check("pg_bmm    bf16 [4,72,64]x[4,64,40]", pg_bmm, a3b, b3b, 1e-5 * sqrt(64.0));

    printf(fails ? "dropin_callers: %d FAILED\n" : "dropin_callers: all passed\n", fails);
    return fails ? 1 : 0;
}
