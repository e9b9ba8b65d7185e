/* The CUDA seat of picograd's backend dispatcher, for B200.
 *
 * Replaces picograd's src/backend/cuda/cuda.c + driver.c: exports the one symbol the
 * dispatcher binds, `const pg_backend_ops pg_backend_cuda` (backend/backend_i.h:38-40,
 * selected in backend/backend.c:54-74 under -DPICOGRAD_BACKEND_CUDA), with every entry
 * filled in — picograd's own seat registers only .gemm (cuda.c:282-291).
 *
 * Like picograd's seat it has no link-time CUDA dependency (docs/gpu-plan.md:17-23): the
 * device library libpg_b200.so (include/pg_b200.h) is dlopen'd on first use, and when it
 * or a B200 is absent init returns PG_ERR_UNSUPPORTED, which makes pg_set_device leave the
 * device unchanged (backend.c:82-86) — the same graceful skip as driver.c:85-92.
 *
 * Host C11; no locks, single caller thread, as the backend it replaces (cuda.c:32-33).
 */
#define _GNU_SOURCE
#include "pg_seat.h"

#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    void *handle;
    int (*init)(void);
    void *(*dmalloc)(size_t);
    void (*dfree)(void *);
    int (*h2d)(void *, const void *, size_t);
    int (*d2h)(void *, const void *, size_t);
    int (*sync)(void);
    void (*gemm)(size_t, size_t, size_t, const float *, size_t, const float *, size_t, float *, size_t);
    void (*hgemm)(size_t, size_t, size_t, const uint16_t *, size_t, const uint16_t *, size_t, float *, size_t);
    void (*bgemm)(size_t, size_t, size_t, const uint16_t *, size_t, const uint16_t *, size_t, float *, size_t);
    int (*gemm_ex)(int, size_t, size_t, size_t, const void *, size_t, const void *, size_t, float *, size_t);
    const char *(*last_error)(void);
} pg_b200_api;

static pg_b200_api g_api;
static int g_tried;
static pg_status g_status = PG_ERR_UNSUPPORTED;
static char g_err[256];

static int debug(void) { return getenv("PG_CUDA_DEBUG") != NULL; }

/* $PG_B200_LIB, else lib/libpg_b200.so beside this object's own shared library, else the
 * loader's search path. */
static void *open_device_library(void)
{
    const char *env = getenv("PG_B200_LIB");
    if (env && *env) {
        void *h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
        if (h || debug()) { if (!h) fprintf(stderr, "picograd/cuda: dlopen(%s): %s\n", env, dlerror()); }
        if (h) return h;
    }
    Dl_info info;
    if (dladdr((void *)&open_device_library, &info) && info.dli_fname) {
        char path[4096];
        const char *slash = strrchr(info.dli_fname, '/');
        size_t dirlen = slash ? (size_t)(slash - info.dli_fname) : 0;
        const char *rel[] = {"/libpg_b200.so", "/../lib/libpg_b200.so", "/../../picograd_b200/lib/libpg_b200.so"};
        for (size_t i = 0; i < sizeof rel / sizeof rel[0]; i++) {
            if (dirlen + strlen(rel[i]) + 2 > sizeof path) continue;
            memcpy(path, info.dli_fname, dirlen);
            strcpy(path + dirlen, rel[i]);
            void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
            if (h) return h;
        }
    }
    return dlopen("libpg_b200.so", RTLD_NOW | RTLD_LOCAL);
}

#define BIND(field, symbol)                                                        \
    do {                                                                           \
        *(void **)(&g_api.field) = dlsym(g_api.handle, symbol);                    \
        if (!g_api.field) {                                                        \
            snprintf(g_err, sizeof g_err, "libpg_b200.so lacks %s", symbol);       \
            return PG_ERR_UNSUPPORTED;                                             \
        }                                                                          \
    } while (0)

static pg_status load_api(void)
{
    g_api.handle = open_device_library();
    if (!g_api.handle) {
        snprintf(g_err, sizeof g_err, "libpg_b200.so not found (set PG_B200_LIB): %s", dlerror());
        return PG_ERR_UNSUPPORTED;
    }
    BIND(init, "pg_b200_init");
    BIND(dmalloc, "pg_b200_malloc");
    BIND(dfree, "pg_b200_free");
    BIND(h2d, "pg_b200_copy_h2d");
    BIND(d2h, "pg_b200_copy_d2h");
    BIND(sync, "pg_b200_sync");
    BIND(gemm, "pg_b200_gemm");
    BIND(hgemm, "pg_b200_hgemm");
    BIND(bgemm, "pg_b200_bgemm");
    BIND(gemm_ex, "pg_b200_gemm_ex");
    BIND(last_error, "pg_b200_last_error");
    return PG_OK;
}

/* cuda.c:30-105: cached; a failure is remembered and returned again. */
static pg_status cuda_init(void)
{
    if (g_tried) return g_status;
    g_tried = 1;
    g_status = load_api();
    if (g_status == PG_OK) {
        int st = g_api.init();
        g_status = (pg_status)st;
        if (st != PG_OK) snprintf(g_err, sizeof g_err, "%s", g_api.last_error());
    }
    if (debug())
        fprintf(stderr, "picograd/cuda: init %s%s%s\n", g_status == PG_OK ? "ok (B200 tensor-core GEMM)" : "failed: ",
                g_status == PG_OK ? "" : g_err, "");
    return g_status;
}

const char *pg_cuda_last_error(void)
{
    if (g_status == PG_OK && g_api.last_error) return g_api.last_error();
    return g_err;
}

static void *cuda_malloc(size_t nbytes) { return cuda_init() == PG_OK ? g_api.dmalloc(nbytes) : NULL; }

static void cuda_free(void *p)
{
    if (p && cuda_init() == PG_OK) g_api.dfree(p);
}

static pg_status cuda_h2d(void *dst, const void *src, size_t nbytes)
{
    return cuda_init() == PG_OK ? (pg_status)g_api.h2d(dst, src, nbytes) : PG_ERR_COPY;
}

static pg_status cuda_d2h(void *dst, const void *src, size_t nbytes)
{
    return cuda_init() == PG_OK ? (pg_status)g_api.d2h(dst, src, nbytes) : PG_ERR_COPY;
}

static pg_status cuda_sync(void) { return cuda_init() == PG_OK ? (pg_status)g_api.sync() : PG_ERR_SYNC; }

/* The three void entries cannot report; like cuda.c:150-174 they return silently when the
 * device is unavailable.  Failures inside the device library are kept in its last-error text
 * and asynchronous ones surface at .sync. */
static void cuda_gemm(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b, size_t ldb,
                      float *c, size_t ldc)
{
    if (cuda_init() == PG_OK) g_api.gemm(m, n, k, a, lda, b, ldb, c, ldc);
}

static void cuda_hgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b,
                       size_t ldb, float *c, size_t ldc)
{
    if (cuda_init() == PG_OK) g_api.hgemm(m, n, k, a, lda, b, ldb, c, ldc);
}

static void cuda_bgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b,
                       size_t ldb, float *c, size_t ldc)
{
    if (cuda_init() == PG_OK) g_api.bgemm(m, n, k, a, lda, b, ldb, c, ldc);
}

/* backend.c:164-166: a non-OK return makes the dispatcher try hgemm/bgemm, then the CPU. */
static pg_status cuda_gemm_ex(pg_dtype dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                              const void *b, size_t ldb, float *c, size_t ldc)
{
    if (cuda_init() != PG_OK) return PG_ERR_UNSUPPORTED;
    return (pg_status)g_api.gemm_ex((int)dtype, m, n, k, a, lda, b, ldb, c, ldc);
}

const pg_backend_ops pg_backend_cuda = {
    .name = "cuda",
    .init = cuda_init,
    .malloc = cuda_malloc,
    .free = cuda_free,
    .copy_h2d = cuda_h2d,
    .copy_d2h = cuda_d2h,
    .sync = cuda_sync,
    .gemm = cuda_gemm,
    .hgemm = cuda_hgemm,
    .bgemm = cuda_bgemm,
    .gemm_ex = cuda_gemm_ex,
};
