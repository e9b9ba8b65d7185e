/* CPU oracle for picograd's dense matrix-multiply path — TEST INFRASTRUCTURE
 * ONLY (see pg_oracle.h).  A restatement of the algorithm, not a copy of the
 * source: every product is formed from exactly-upcast f32 operands and added
 * into an f32 accumulator with one rounding per k-step, k ascending, which is
 * what picograd's CPU micro-kernels do:
 *
 *   - f32: the 8x16 / 8x8 assembly kernels keep C in registers and issue one
 *     vfmadd231ps per k (backend/cpu/asm/sgemm_avx512.S:126-154); the driver
 *     splits k in blocks of 256 and re-loads C from memory between blocks
 *     (backend/cpu/gemm.c:503-507, gemm_par_fn) — storing and re-loading an
 *     f32 is exact, so the result is one fused-multiply-add chain over all k.
 *   - f16: upcast with vcvtph2ps, then _mm512_fmadd_ps per k
 *     (backend/cpu/hgemm_avx512fp16.c:22-67), driver gemm.c:575-599.
 *   - bf16: scalar upcast and `acc += a*b` (backend/cpu/bgemm_avx512bf16.c:
 *     10-19), compiled with -ffast-math, so the compiler chooses contraction
 *     and association; this restatement uses the fused chain.  bf16 results
 *     therefore agree with the compiled reference to rounding noise
 *     (measured in tests/test_oracle.py), f32 and f16 bit for bit.
 *
 * Parity pins: the golden vectors of picograd's tests (tests/test_backend.c:
 * 62-96 exact 2x1x2 case and 13x9x7 grid; benchmarks/bench_gemm_cuda.c:16-65
 * dyadic 512^3 data that is exact in f32; tests/test_gemm.c:126-189 shape
 * grid) and the outputs of the unmodified library built into oracle/_ref:
 * products, fused epilogues, conv, addmm, and — for pgo_matmul_backward — the
 * gradients of picograd's own pg_ag_matmul -> pg_backward on f32, bf16 and f16
 * leaves (tests/golden/make_golden.py), reproduced bit for bit where
 * bwd_matmul takes its GEMM route (autograd/autograd.c:635).
 */
#include "pg_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

/* ---- a plain pthread parallel-for (no OpenMP runtime in the image) ------- */

int pgo_num_threads(void)
{
    static int cached = 0;
    if (cached) return cached;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    const char *e = getenv("PGO_THREADS");
    if (e && atoi(e) > 0) n = atoi(e);
    if (n < 1) n = 1;
    if (n > 256) n = 256;
    cached = (int)n;
    return cached;
}

typedef void (*pgo_range_fn)(void *ctx, size_t begin, size_t end);
typedef struct { pgo_range_fn fn; void *ctx; size_t begin, end; } pgo_job;

static void *pgo_job_main(void *p)
{
    pgo_job *j = (pgo_job *)p;
    j->fn(j->ctx, j->begin, j->end);
    return NULL;
}

static void pgo_parallel_for(size_t n, pgo_range_fn fn, void *ctx)
{
    int t = pgo_num_threads();
    if ((size_t)t > n) t = (int)n;
    if (t <= 1) { if (n) fn(ctx, 0, n); return; }
    pthread_t th[256];
    pgo_job jobs[256];
    size_t chunk = (n + (size_t)t - 1) / (size_t)t;
    int started = 0;
    for (int i = 0; i < t; i++) {
        size_t b = (size_t)i * chunk, e = b + chunk < n ? b + chunk : n;
        if (b >= e) break;
        jobs[i] = (pgo_job){fn, ctx, b, e};
        if (pthread_create(&th[i], NULL, pgo_job_main, &jobs[i]) != 0) {
            fn(ctx, b, e);              /* run inline if a thread cannot start */
            th[i] = 0;
        }
        started = i + 1;
    }
    for (int i = 0; i < started; i++)
        if (th[i]) pthread_join(th[i], NULL);
}

/* ---- converters: core/convert.h:15-104 (round-to-nearest-even) ---------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* core/convert.h:85-97: NaN -> 0x7FC0 | bit16; else add 0x7FFF + lsb, keep top half */
uint16_t pgo_f32_to_bf16(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu))
        return (uint16_t)(0x7FC0u | ((u >> 16) & 1u));
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* core/convert.h:99-104 */
float pgo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* core/convert.h:15-52: Inf/NaN kept (NaN quieted), overflow -> Inf,
 * subnormal halves produced with RNE, anything below 2^-25 flushed to zero. */
uint16_t pgo_f32_to_f16(float f)
{
    uint32_t u = f2u(f);
    uint32_t s = (u >> 16) & 0x8000u;
    uint32_t ex = (u >> 23) & 0xFFu;
    uint32_t man = u & 0x7FFFFFu;
    if (ex == 255) {
        if (!man) return (uint16_t)(s | 0x7C00u);
        uint16_t q = (uint16_t)(s | 0x7C00u | (man >> 13));
        if (!(q & 0x3FFu)) q |= 1;
        return q | 0x0200u;
    }
    int e = (int)ex - 112;                     /* re-bias 127 -> 15 */
    if (e >= 31) return (uint16_t)(s | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        /* The reference rounds the 24-bit significand at bit (1-e) and
         * returns sign|mantissa WITHOUT dropping the 13 low bits a half has
         * no room for (core/convert.h:33-44), so its subnormal results are
         * not IEEE halves.  Restated as it is; harness inputs are rounded
         * with an IEEE converter instead and both sides read the same bytes. */
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(1 - e);
        uint32_t rb = 1u << (shift - 1);
        uint32_t extra = man & ((1u << shift) - 1u);
        uint32_t m2 = man >> shift;
        if (extra > rb || (extra == rb && (m2 & 1u))) m2++;
        return (uint16_t)(s | m2);
    }
    man += 0x0FFFu + ((man >> 13) & 1u);
    if (man & 0x800000u) { man = 0; e++; }
    if (e >= 31) return (uint16_t)(s | 0x7C00u);
    return (uint16_t)(s | ((uint32_t)e << 10) | (man >> 13));
}

/* core/convert.h:54-83 */
float pgo_f16_to_f32(uint16_t h)
{
    uint32_t s = ((uint32_t)h & 0x8000u) << 16;
    uint32_t ex = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (ex == 0) {
        if (!man) return u2f(s);
        int e = 1;
        while (!(man & 0x400u)) { man <<= 1; e--; }
        man &= 0x3FFu;
        return u2f(s | ((uint32_t)(e + 112) << 23) | (man << 13));
    }
    if (ex == 31) return u2f(s | 0x7F800000u | (man << 13));
    return u2f(s | ((ex + 112) << 23) | (man << 13));
}

void pgo_f32_to_bf16_n(uint16_t *d, const float *s, size_t n)
{
    for (size_t i = 0; i < n; i++) d[i] = pgo_f32_to_bf16(s[i]);
}
void pgo_f32_to_f16_n(uint16_t *d, const float *s, size_t n)
{
    for (size_t i = 0; i < n; i++) d[i] = pgo_f32_to_f16(s[i]);
}
void pgo_bf16_to_f32_n(float *d, const uint16_t *s, size_t n)
{
    for (size_t i = 0; i < n; i++) d[i] = pgo_bf16_to_f32(s[i]);
}
void pgo_f16_to_f32_n(float *d, const uint16_t *s, size_t n)
{
    for (size_t i = 0; i < n; i++) d[i] = pgo_f16_to_f32(s[i]);
}

/* ---- GEMM --------------------------------------------------------------- */

/* Upcast one row segment of B (or A) to f32. */
static void upcast_row(int dtype, float *dst, const void *src, size_t off, size_t n)
{
    if (dtype == PGO_F32) {
        memcpy(dst, (const float *)src + off, n * sizeof(float));
    } else if (dtype == PGO_BF16) {
        const uint16_t *p = (const uint16_t *)src + off;
        for (size_t j = 0; j < n; j++) dst[j] = pgo_bf16_to_f32(p[j]);
    } else {
        const uint16_t *p = (const uint16_t *)src + off;
        for (size_t j = 0; j < n; j++) dst[j] = pgo_f16_to_f32(p[j]);
    }
}

static inline float load1(int dtype, const void *p, size_t i)
{
    if (dtype == PGO_F32) return ((const float *)p)[i];
    if (dtype == PGO_BF16) return pgo_bf16_to_f32(((const uint16_t *)p)[i]);
    return pgo_f16_to_f32(((const uint16_t *)p)[i]);
}

#define PGO_JB 256   /* columns of C per strip */
#define PGO_IB 8     /* rows of C per strip: B rows are upcast once per 8 rows */

typedef struct {
    int dtype; size_t k; const void *a; size_t lda; const void *b; size_t ldb;
    float *c; size_t ldc; size_t r0, r1, c0, c1, nstrip;
    const float *bias; int act;
} panel_ctx;

/* backend/cpu/gemm.c:632-636 (act_apply) */
static inline float act_apply(float x, int act)
{
    if (act == PGO_ACT_RELU) return x > 0 ? x : 0;
    if (act == PGO_ACT_GELU) return 0.5f * x * (1.0f + erff(x * 0.70710678118f));
    return x;
}

static void panel_range(void *vctx, size_t begin, size_t end)
{
    const panel_ctx *x = (const panel_ctx *)vctx;
    float brow[PGO_JB], acc[PGO_IB][PGO_JB], av[PGO_IB];
    for (size_t t = begin; t < end; t++) {
        size_t i0 = x->r0 + (t / x->nstrip) * PGO_IB;
        size_t h = x->r1 - i0 < PGO_IB ? x->r1 - i0 : PGO_IB;
        size_t j0 = x->c0 + (t % x->nstrip) * PGO_JB;
        size_t w = x->c1 - j0 < PGO_JB ? x->c1 - j0 : PGO_JB;
        memset(acc, 0, sizeof acc);
        if (x->bias)                 /* gemm.c:729-735: the C rows start as the bias row */
            for (size_t r = 0; r < h; r++)
                memcpy(acc[r], x->bias + j0, w * sizeof(float));
        for (size_t p = 0; p < x->k; p++) {
            const float *bp;
            if (x->dtype == PGO_F32) {
                bp = (const float *)x->b + p * x->ldb + j0;
            } else {
                upcast_row(x->dtype, brow, x->b, p * x->ldb + j0, w);
                bp = brow;
            }
            for (size_t r = 0; r < h; r++) av[r] = load1(x->dtype, x->a, (i0 + r) * x->lda + p);
            /* each C element owns one accumulator: one fused multiply-add per k,
             * k ascending — rows and columns are independent chains */
            for (size_t r = 0; r < h; r++)
                for (size_t j = 0; j < w; j++)
                    acc[r][j] = __builtin_fmaf(av[r], bp[j], acc[r][j]);
        }
        if (x->act != PGO_ACT_NONE)  /* gemm.c:770-779: over the finished rows */
            for (size_t r = 0; r < h; r++)
                for (size_t j = 0; j < w; j++) acc[r][j] = act_apply(acc[r][j], x->act);
        for (size_t r = 0; r < h; r++)
            memcpy(x->c + (i0 + r) * x->ldc + j0, acc[r], w * sizeof(float));
    }
}

/* backend/backend.c:150-177 -> backend/cpu/gemm.c:456-508 (f32),
 * :575-599 (f16), :600-624 (bf16): C rows are zeroed, then C += A*B. */
void pgo_gemm_ex_panel(int dtype, size_t m, size_t n, size_t k,
                       const void *a, size_t lda, const void *b, size_t ldb,
                       float *c, size_t ldc,
                       size_t r0, size_t r1, size_t c0, size_t c1)
{
    if (r1 > m) r1 = m;
    if (c1 > n) c1 = n;
    if (r0 >= r1 || c0 >= c1) return;
    panel_ctx x = {dtype, k, a, lda, b, ldb, c, ldc, r0, r1, c0, c1,
                   (c1 - c0 + PGO_JB - 1) / PGO_JB, NULL, PGO_ACT_NONE};
    pgo_parallel_for(((r1 - r0 + PGO_IB - 1) / PGO_IB) * x.nstrip, panel_range, &x);
}

/* backend/cpu/gemm.c:685-716 (pg_cpu_gemm_fused) and :718-817 (pg_cpu_gemm_fused_ex): every
 * row of C is set to the bias row (zeros without a bias), the same micro-kernels as pg_gemm_ex
 * accumulate A*B onto it K block by K block -- so each element is ONE chain of fused
 * multiply-adds that starts at bias[j], k ascending -- and the activation runs over the
 * finished rows.  With k == 0 the result is act(bias). */
void pgo_gemm_fused_ex(int dtype, size_t m, size_t n, size_t k,
                       const void *a, size_t lda, const void *b, size_t ldb,
                       float *c, size_t ldc, const float *bias, int act)
{
    if (m == 0 || n == 0) return;
    panel_ctx x = {dtype, k, a, lda, b, ldb, c, ldc, 0, m, 0, n,
                   (n + PGO_JB - 1) / PGO_JB, bias, act};
    pgo_parallel_for(((m + PGO_IB - 1) / PGO_IB) * x.nstrip, panel_range, &x);
}

void pgo_gemm_ex(int dtype, size_t m, size_t n, size_t k,
                 const void *a, size_t lda, const void *b, size_t ldb,
                 float *c, size_t ldc)
{
    if (k == 0) {                               /* gemm.c:539: rows zeroed first */
        for (size_t i = 0; i < m; i++) memset(c + i * ldc, 0, n * sizeof(float));
        return;
    }
    pgo_gemm_ex_panel(dtype, m, n, k, a, lda, b, ldb, c, ldc, 0, m, 0, n);
}

/* ops/matmul.c:340-369: one pg_gemm[_ex] per batch element, contiguous operands. */
void pgo_bmm(int dtype, size_t batch, size_t m, size_t n, size_t k,
             const void *a, const void *b, float *c)
{
    size_t es = dtype == PGO_F32 ? 4 : 2;
    for (size_t s = 0; s < batch; s++)
        pgo_gemm_ex(dtype, m, n, k, (const char *)a + s * m * k * es, k,
                    (const char *)b + s * k * n * es, n, c + s * m * n, n);
}

/* autograd/autograd.c:561-706 (bwd_matmul): operands upcast to f32 (:566-590),
 * B^T / A^T materialised on the host (:659-665, :684-687), an f32 GEMM into a
 * zeroed temporary (:666-668, :688-689) and `grad += temporary` (:669-670,
 * :690-691).  The f32 GEMM is the same fused chain as above. */
void pgo_matmul_backward(int dtype, size_t m, size_t n, size_t k,
                         const void *a, const void *b, const float *g,
                         float *ga, float *gb)
{
    if (ga) {
        /* tmp[m,k] = g[m,n] * B^T[n,k] */
        float *bt = (float *)malloc(n * k * sizeof(float));
        float *tmp = (float *)malloc(m * k * sizeof(float));
        for (size_t i = 0; i < k; i++)
            for (size_t j = 0; j < n; j++) bt[j * k + i] = load1(dtype, b, i * n + j);
        pgo_gemm_ex(PGO_F32, m, k, n, g, n, bt, k, tmp, k);
        for (size_t i = 0; i < m * k; i++) ga[i] += tmp[i];
        free(bt); free(tmp);
    }
    if (gb) {
        /* tmp[k,n] = A^T[k,m] * g[m,n] */
        float *at = (float *)malloc(k * m * sizeof(float));
        float *tmp = (float *)malloc(k * n * sizeof(float));
        for (size_t i = 0; i < m; i++)
            for (size_t j = 0; j < k; j++) at[j * m + i] = load1(dtype, a, i * k + j);
        pgo_gemm_ex(PGO_F32, k, n, m, at, m, g, n, tmp, n);
        for (size_t i = 0; i < k * n; i++) gb[i] += tmp[i];
        free(at); free(tmp);
    }
}

/* ops/matmul.c:371-405 (pg_addmm): tmp = pg_matmul(m1, m2); tmp *= alpha (if alpha != 1); with beta == 0 that is
 * the result; else base = 0 + broadcast(input) ; base *= beta (if beta != 1); result = base + tmp -- separate
 * f32 operations, each rounded.  input is read through (row, column) element strides, 0 for a broadcast one. */
void pgo_addmm(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
               float *c, size_t ldc, const float *input, size_t in_rs, size_t in_cs, float alpha, float beta)
{
    pgo_gemm_ex(dtype, m, n, k, a, lda, b, ldb, c, ldc);
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            volatile float t = c[i * ldc + j];
            if (alpha != 1.0f) t = t * alpha;
            if (beta != 0.0f) {
                volatile float base = 0.0f + input[i * in_rs + j * in_cs];
                if (beta != 1.0f) base = base * beta;
                t = base + t;
            }
            c[i * ldc + j] = t;
        }
}

/* ops/conv.c:10-146 (pg_conv2d): NCHW, per batch element an im2col matrix (K = cin*kh*kw rows in
 * (ci, ki, kj) order, one column per output pixel, zeros where the window leaves the image), then
 * pg_cpu_gemm(cout, columns, K, w, K, col, ...) and `+= bias[co]` over the finished rows (:127-133).
 * The chunking into 1024 columns (:43-58) does not change any element's arithmetic: each output is one
 * fused multiply-add chain over the K rows, zeros included, followed by one addition of the bias. */
typedef struct {
    size_t cin, h, w, cout, kh, kw, oh, ow; int stride, pad;
    const float *x, *wt, *bias; float *out;
} conv_ctx;

static void conv_range(void *vctx, size_t begin, size_t end)
{
    const conv_ctx *c = (const conv_ctx *)vctx;
    for (size_t o = begin; o < end; o++) {               /* o = (n * cout + co) */
        size_t n = o / c->cout, co = o % c->cout;
        const float *xb = c->x + n * c->cin * c->h * c->w;
        const float *wr = c->wt + co * c->cin * c->kh * c->kw;
        float *orow = c->out + o * c->oh * c->ow;
        for (size_t oh = 0; oh < c->oh; oh++)
            for (size_t ow = 0; ow < c->ow; ow++) {
                float acc = 0.0f;
                size_t k = 0;
                for (size_t ci = 0; ci < c->cin; ci++)
                    for (size_t ki = 0; ki < c->kh; ki++)
                        for (size_t kj = 0; kj < c->kw; kj++, k++) {
                            long ih = (long)oh * c->stride - c->pad + (long)ki;
                            long iw = (long)ow * c->stride - c->pad + (long)kj;
                            float v = 0.0f;
                            if (ih >= 0 && ih < (long)c->h && iw >= 0 && iw < (long)c->w)
                                v = xb[(ci * c->h + (size_t)ih) * c->w + (size_t)iw];
                            acc = __builtin_fmaf(wr[k], v, acc);
                        }
                if (c->bias) acc += c->bias[co];
                orow[oh * c->ow + ow] = acc;
            }
    }
}

int pgo_conv2d(size_t n, size_t cin, size_t h, size_t w, size_t cout, size_t kh, size_t kw,
               int stride, int pad, const float *x, const float *wt, const float *bias, float *out)
{
    if (stride <= 0) return -1;
    long vh = (long)h + 2L * pad - (long)kh, vw = (long)w + 2L * pad - (long)kw;   /* conv.h:19-25 */
    if (vh < 0 || vw < 0) return -1;
    conv_ctx c = {cin, h, w, cout, kh, kw, (size_t)(vh / stride) + 1, (size_t)(vw / stride) + 1,
                  stride, pad, x, wt, bias, out};
    pgo_parallel_for(n * cout, conv_range, &c);
    return 0;
}

/* ---- harness steps between the GEMMs ------------------------------------ */

typedef struct { float *out; const float *a; const float *b; size_t len; } ew_ctx;

static void softmax_range(void *vctx, size_t begin, size_t end)
{
    const ew_ctx *x = (const ew_ctx *)vctx;
    for (size_t o = begin; o < end; o++) {
        const float *s = x->a + o * x->len;
        float *d = x->out + o * x->len;
        float mx = s[0];
        for (size_t j = 1; j < x->len; j++) if (s[j] > mx) mx = s[j];
        float sum = 0.0f;
        for (size_t j = 0; j < x->len; j++) sum += expf(s[j] - mx);
        float inv = 1.0f / sum;
        for (size_t j = 0; j < x->len; j++) d[j] = expf(s[j] - mx) * inv;
    }
}

/* ops/activations.c:22-45 (sm1_par_fn, non-log branch) */
void pgo_softmax_rows(float *out, const float *src, size_t rows, size_t len)
{
    ew_ctx x = {out, src, NULL, len};
    pgo_parallel_for(rows, softmax_range, &x);
}

static void gelu_range(void *vctx, size_t begin, size_t end)
{
    const ew_ctx *x = (const ew_ctx *)vctx;
    for (size_t i = begin; i < end; i++)
        x->out[i] = 0.5f * x->a[i] * (1.0f + erff(x->a[i] * 0.70710678118f));
}

/* ops/activations.c:114 (fgelu) */
void pgo_gelu(float *out, const float *src, size_t n)
{
    ew_ctx x = {out, src, NULL, 0};
    pgo_parallel_for(n, gelu_range, &x);
}

static void gelu_grad_range(void *vctx, size_t begin, size_t end)
{
    const ew_ctx *x = (const ew_ctx *)vctx;
    for (size_t i = begin; i < end; i++) {
        float v = x->a[i];
        float e = erff(v * 0.70710678118f);
        float phi = expf(-0.5f * v * v) / 2.50662827463f;
        x->out[i] = x->b[i] * (0.5f * (1.0f + e) + v * phi);
    }
}

/* autograd/autograd.c:794-801 (grad_gelu) applied as :531-532 does: gy * local(x) */
void pgo_gelu_grad(float *out, const float *xin, const float *gy, size_t n)
{
    ew_ctx x = {out, xin, gy, 0};
    pgo_parallel_for(n, gelu_grad_range, &x);
}
