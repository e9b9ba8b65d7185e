/* Types of picograd's backend seat, restated so that the host side builds without
 * picograd's tree.  Layout and values must equal picograd's:
 *   pg_status        backend/backend.h:25-32
 *   pg_dtype         core/dtype.h:11-16
 *   pg_backend_ops   backend/backend_i.h:8-34
 * When built inside picograd (-DPG_B200_USE_REFERENCE_HEADERS) picograd's own headers are
 * used instead, so a drift would be a compile error there.
 */
#ifndef PG_SEAT_H
#define PG_SEAT_H

#include <stddef.h>
#include <stdint.h>

#if defined(PG_B200_USE_REFERENCE_HEADERS)
#include "backend/backend_i.h"
#else

typedef enum {
    PG_OK = 0,
    PG_ERR_UNSUPPORTED = -1,
    PG_ERR_ALLOC = -2,
    PG_ERR_COPY = -3,
    PG_ERR_SYNC = -4,
    PG_ERR_GEMM = -5,
} pg_status;

typedef enum { PG_DTYPE_F32 = 0, PG_DTYPE_F16 = 1, PG_DTYPE_BF16 = 2, PG_DTYPE_COUNT = 3 } pg_dtype;

typedef struct pg_backend_ops {
    const char *name;
    pg_status (*init)(void);
    void *(*malloc)(size_t nbytes);
    void (*free)(void *p);
    pg_status (*copy_h2d)(void *dst, const void *src, size_t nbytes);
    pg_status (*copy_d2h)(void *dst, const void *src, size_t nbytes);
    pg_status (*sync)(void);
    void (*gemm)(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b, size_t ldb,
                 float *c, size_t ldc);
    void (*hgemm)(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb,
                  float *c, size_t ldc);
    void (*bgemm)(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb,
                  float *c, size_t ldc);
    pg_status (*gemm_ex)(pg_dtype dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                         const void *b, size_t ldb, float *c, size_t ldc);
} pg_backend_ops;

extern const pg_backend_ops pg_backend_cuda;
#endif

/* Last error text of the device library ("" before it is loaded). */
const char *pg_cuda_last_error(void);

#endif
