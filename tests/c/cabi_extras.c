/* The C-ABI entries beyond picograd's vtable, called from plain C (no Python, no torch): the fused
 * bias/activation GEMM (pg_cpu_gemm_fused_ex), pg_conv2d and the attention-shaped chain.  Each result is
 * compared with loops written here from the definitions in picograd's sources:
 *   gemm.c:718-817  C = act(bias[j] + A*B), one fused multiply-add chain per element starting at bias[j]
 *   conv.c:10-146   im2col rows in (ci,ki,kj) order, zeros outside the image, GEMM, then + bias
 *   matmul.c:340-369 + activations.c:22-45  O = bf16(softmax_rows(Q*Kt)) * V
 *   matmul.c:186-490  pg_matmul / pg_bmm / pg_tensordot shape rules, autograd.c:561-706 the matmul node's backward
 * usage: cabi_extras /path/to/libpg_b200.so      exit code 0 and "all passed" on success. */
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef int (*init_fn)(void);
typedef void *(*malloc_fn)(size_t);
typedef void (*free_fn)(void *);
typedef int (*copy_fn)(void *, const void *, size_t);
typedef int (*sync_fn)(void);
typedef const char *(*str_fn)(void);
typedef int (*fused_fn)(int, size_t, size_t, size_t, const void *, size_t, const void *, size_t, float *, size_t, const float *, int);
typedef int (*conv_fn)(size_t, size_t, size_t, size_t, size_t, size_t, size_t, int, int, const float *, const float *, const float *, float *);
typedef int (*attn_fn)(int, size_t, size_t, size_t, size_t, const void *, const void *, const void *, float *);
/* pg_b200_tensor of include/pg_b200.h, restated here so that this file needs no header of the library */
typedef struct { int dtype; size_t ndim; size_t shape[8]; size_t stride[8]; void *data; } tensor_t;
typedef int (*mm_fn)(const tensor_t *, const tensor_t *, tensor_t *);
typedef int (*td_fn)(const tensor_t *, const tensor_t *, size_t, const size_t *, const size_t *, tensor_t *);
typedef int (*bwd_fn)(const tensor_t *, const tensor_t *, const float *, float *, float *, int);

static tensor_t make_tensor(int dtype, size_t ndim, const size_t *shape, void *data) {
    tensor_t t; memset(&t, 0, sizeof t);
    t.dtype = dtype; t.ndim = ndim; t.data = data;
    size_t run = 1;
    for (size_t d = ndim; d-- > 0;) { t.shape[d] = shape[d]; t.stride[d] = run; run *= shape[d]; }
    return t;
}

static int fails = 0;
#define CHECK(c) do { if (!(c)) { printf("FAIL:%d %s\n", __LINE__, #c); fails++; } } while (0)

static uint32_t rng_state = 12345u;
static float urand(void) {                       /* uniform in [-1, 1) */
    rng_state = rng_state * 1664525u + 1013904223u;
    return (float)(rng_state >> 8) / 8388608.0f - 1.0f;
}
static uint16_t to_bf16(float f) {               /* round to nearest even */
    uint32_t u; memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }

int main(int argc, char **argv) {
    const char *path = argc > 1 ? argv[1] : getenv("PG_B200_LIB");
    if (!path) { printf("usage: cabi_extras libpg_b200.so\n"); return 2; }
    void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { printf("dlopen: %s\n", dlerror()); return 2; }
    init_fn init = (init_fn)dlsym(h, "pg_b200_init");
    malloc_fn dmalloc = (malloc_fn)dlsym(h, "pg_b200_malloc");
    free_fn dfree = (free_fn)dlsym(h, "pg_b200_free");
    copy_fn h2d = (copy_fn)dlsym(h, "pg_b200_copy_h2d"), d2h = (copy_fn)dlsym(h, "pg_b200_copy_d2h");
    sync_fn dsync = (sync_fn)dlsym(h, "pg_b200_sync");
    str_fn last_path = (str_fn)dlsym(h, "pg_b200_last_path"), last_error = (str_fn)dlsym(h, "pg_b200_last_error");
    fused_fn fused = (fused_fn)dlsym(h, "pg_b200_gemm_fused_ex");
    conv_fn conv = (conv_fn)dlsym(h, "pg_b200_conv2d");
    attn_fn attn = (attn_fn)dlsym(h, "pg_b200_attention_bmm");
    mm_fn matmul = (mm_fn)dlsym(h, "pg_b200_matmul"), bmm = (mm_fn)dlsym(h, "pg_b200_bmm");
    td_fn tensordot = (td_fn)dlsym(h, "pg_b200_tensordot");
    bwd_fn backward = (bwd_fn)dlsym(h, "pg_b200_matmul_backward_nd");
    if (!matmul || !bmm || !tensordot || !backward) { printf("missing symbol (tensor-level callers)\n"); return 2; }
    if (!init || !dmalloc || !dfree || !h2d || !d2h || !dsync || !fused || !conv || !attn || !last_path || !last_error) {
        printf("missing symbol\n"); return 2;
    }
    if (init() != 0) { printf("pg_b200_init failed: %s\n", last_error()); return 3; }

    /* ---- fused GEMM, f32, bias + ReLU: bit for bit ---- */
    {
        enum { M = 33, N = 47, K = 65 };
        static float a[M * K], b[K * N], bias[N], c[M * N], want[M * N];
        for (int i = 0; i < M * K; i++) a[i] = urand();
        for (int i = 0; i < K * N; i++) b[i] = urand();
        for (int j = 0; j < N; j++) bias[j] = urand();
        for (int i = 0; i < M; i++)
            for (int j = 0; j < N; j++) {
                float acc = bias[j];
                for (int k = 0; k < K; k++) acc = fmaf(a[i * K + k], b[k * N + j], acc);
                want[i * N + j] = acc > 0 ? acc : 0;
            }
        void *da = dmalloc(sizeof a), *db = dmalloc(sizeof b), *dbias = dmalloc(sizeof bias), *dc = dmalloc(sizeof c);
        CHECK(da && db && dbias && dc);
        CHECK(h2d(da, a, sizeof a) == 0 && h2d(db, b, sizeof b) == 0 && h2d(dbias, bias, sizeof bias) == 0);
        CHECK(fused(0, M, N, K, da, K, db, N, (float *)dc, N, (const float *)dbias, 1) == 0);
        CHECK(dsync() == 0 && d2h(c, dc, sizeof c) == 0);
        CHECK(memcmp(c, want, sizeof c) == 0);
        /* the same call with HOST pointers, as nn/nn.c:60 passes them */
        memset(c, 0xFF, sizeof c);
        CHECK(fused(0, M, N, K, a, K, b, N, c, N, bias, 1) == 0);
        CHECK(memcmp(c, want, sizeof c) == 0);
        printf("fused gemm f32 33x47x65 bias+relu: exact (%s)\n", last_path());
        dfree(da); dfree(db); dfree(dbias); dfree(dc);
    }

    /* ---- conv2d: bit for bit ---- */
    {
        enum { NB = 2, CI = 3, H = 9, W = 11, CO = 4, KH = 3, KW = 2, S = 2, P = 1 };
        enum { OH = (H + 2 * P - KH) / S + 1, OW = (W + 2 * P - KW) / S + 1 };
        static float x[NB * CI * H * W], wt[CO * CI * KH * KW], bias[CO], y[NB * CO * OH * OW], want[NB * CO * OH * OW];
        for (size_t i = 0; i < sizeof x / 4; i++) x[i] = urand();
        for (size_t i = 0; i < sizeof wt / 4; i++) wt[i] = urand();
        for (int i = 0; i < CO; i++) bias[i] = urand();
        for (int n = 0; n < NB; n++)
            for (int co = 0; co < CO; co++)
                for (int oh = 0; oh < OH; oh++)
                    for (int ow = 0; ow < OW; ow++) {
                        float acc = 0.0f;
                        for (int ci = 0; ci < CI; ci++)
                            for (int ki = 0; ki < KH; ki++)
                                for (int kj = 0; kj < KW; kj++) {
                                    int ih = oh * S - P + ki, iw = ow * S - P + kj;
                                    float v = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? x[((n * CI + ci) * H + ih) * W + iw] : 0.0f;
                                    acc = fmaf(wt[((co * CI + ci) * KH + ki) * KW + kj], v, acc);
                                }
                        want[((n * CO + co) * OH + oh) * OW + ow] = acc + bias[co];
                    }
        void *dx = dmalloc(sizeof x), *dw = dmalloc(sizeof wt), *dbias = dmalloc(sizeof bias), *dy = dmalloc(sizeof y);
        CHECK(dx && dw && dbias && dy);
        CHECK(h2d(dx, x, sizeof x) == 0 && h2d(dw, wt, sizeof wt) == 0 && h2d(dbias, bias, sizeof bias) == 0);
        CHECK(conv(NB, CI, H, W, CO, KH, KW, S, P, (const float *)dx, (const float *)dw, (const float *)dbias, (float *)dy) == 0);
        CHECK(dsync() == 0 && d2h(y, dy, sizeof y) == 0);
        CHECK(memcmp(y, want, sizeof y) == 0);
        printf("conv2d 2x3x9x11 k3x2 s2 p1: exact (%s)\n", last_path());
        dfree(dx); dfree(dw); dfree(dbias); dfree(dy);
    }

    /* ---- attention-shaped chain, bf16, one kernel ---- */
    {
        enum { B = 2, SQ = 160, SK = 264, D = 128 };
        uint16_t *q = malloc(2 * B * SQ * D), *kt = malloc(2 * B * D * SK), *v = malloc(2 * B * SK * D);
        float *o = malloc(4 * B * SQ * D);
        double *want = malloc(8 * B * SQ * D), *srow = malloc(8 * SK);
        for (int i = 0; i < B * SQ * D; i++) q[i] = to_bf16(urand() * 0.5f);
        for (int i = 0; i < B * D * SK; i++) kt[i] = to_bf16(urand() * 0.5f);
        for (int i = 0; i < B * SK * D; i++) v[i] = to_bf16(urand());
        for (int b = 0; b < B; b++)
            for (int i = 0; i < SQ; i++) {
                double mx = -1e300, sum = 0;
                for (int j = 0; j < SK; j++) {
                    double s = 0;
                    for (int d = 0; d < D; d++) s += (double)from_bf16(q[(b * SQ + i) * D + d]) * from_bf16(kt[(b * D + d) * SK + j]);
                    srow[j] = (double)(float)s;
                    if (srow[j] > mx) mx = srow[j];
                }
                for (int j = 0; j < SK; j++) sum += exp(srow[j] - mx);
                for (int d = 0; d < D; d++) want[(b * SQ + i) * D + d] = 0;
                for (int j = 0; j < SK; j++) {
                    double p = from_bf16(to_bf16((float)(exp(srow[j] - mx) / sum)));
                    for (int d = 0; d < D; d++) want[(b * SQ + i) * D + d] += p * from_bf16(v[(b * SK + j) * D + d]);
                }
            }
        void *dq = dmalloc(2 * B * SQ * D), *dk = dmalloc(2 * B * D * SK), *dv = dmalloc(2 * B * SK * D), *dout = dmalloc(4 * B * SQ * D);
        CHECK(dq && dk && dv && dout);
        CHECK(h2d(dq, q, 2 * B * SQ * D) == 0 && h2d(dk, kt, 2 * B * D * SK) == 0 && h2d(dv, v, 2 * B * SK * D) == 0);
        CHECK(attn(2, B, SQ, SK, D, dq, dk, dv, (float *)dout) == 0);
        CHECK(dsync() == 0 && d2h(o, dout, 4 * B * SQ * D) == 0);
        double num = 0, den = 0;
        for (int i = 0; i < B * SQ * D; i++) { num += (o[i] - want[i]) * (o[i] - want[i]); den += want[i] * want[i]; }
        double rel = sqrt(num / den);
        CHECK(strcmp(last_path(), "attn:fused_128x128") == 0);
        CHECK(rel < 1e-3);
        printf("attention bf16 2x160x264x128: rel err %.2e (%s)\n", rel, last_path());
        dfree(dq); dfree(dk); dfree(dv); dfree(dout);
        free(q); free(kt); free(v); free(o); free(want); free(srow);
    }


    /* ---- picograd's tensor-level callers with its shape rules (the shapes of picograd's tests/test_ops.c:368-492):
     *      2-D x 2-D, vector x vector, vector x matrix, matrix x vector, batched, batch-shared b, pg_bmm,
     *      pg_tensordot over two axes, the refusals, and the matmul node's backward with a batch-shared b ---- */
    {
        enum { BT = 2, BM = 3, BK = 4, BN = 5 };
        float a[BT * BM * BK], b[BT * BK * BN], w[BK * BN], v[BK], c[BT * BM * BN];
        for (int i = 0; i < BT * BM * BK; i++) a[i] = urand();
        for (int i = 0; i < BT * BK * BN; i++) b[i] = urand();
        for (int i = 0; i < BK * BN; i++) w[i] = urand();
        for (int i = 0; i < BK; i++) v[i] = urand();
        void *da = dmalloc(sizeof a), *db = dmalloc(sizeof b), *dw = dmalloc(sizeof w), *dv = dmalloc(sizeof v);
        CHECK(da && db && dw && dv);
        CHECK(h2d(da, a, sizeof a) == 0 && h2d(db, b, sizeof b) == 0 && h2d(dw, w, sizeof w) == 0 && h2d(dv, v, sizeof v) == 0);
        tensor_t ta3 = make_tensor(0, 3, (size_t[]){BT, BM, BK}, da), tb3 = make_tensor(0, 3, (size_t[]){BT, BK, BN}, db);
        tensor_t ta2 = make_tensor(0, 2, (size_t[]){BM, BK}, da), tw = make_tensor(0, 2, (size_t[]){BK, BN}, dw);
        tensor_t tv = make_tensor(0, 1, (size_t[]){BK}, dv);
        tensor_t out; memset(&out, 0, sizeof out);            /* out.data == NULL: the library allocates */
        /* batched x batched */
        CHECK(matmul(&ta3, &tb3, &out) == 0 && out.ndim == 3 && out.shape[0] == BT && out.shape[1] == BM && out.shape[2] == BN && out.data);
        CHECK(dsync() == 0 && d2h(c, out.data, sizeof c) == 0);
        for (int s2 = 0; s2 < BT; s2++) for (int i = 0; i < BM; i++) for (int j = 0; j < BN; j++) {
            float acc = 0; for (int k = 0; k < BK; k++) acc = fmaf(a[(s2 * BM + i) * BK + k], b[(s2 * BK + k) * BN + j], acc);
            CHECK(c[(s2 * BM + i) * BN + j] == acc);
        }
        /* pg_bmm gives the same bits */
        tensor_t out2; memset(&out2, 0, sizeof out2);
        float c2[BT * BM * BN];
        CHECK(bmm(&ta3, &tb3, &out2) == 0 && out2.ndim == 3 && dsync() == 0 && d2h(c2, out2.data, sizeof c2) == 0);
        CHECK(memcmp(c, c2, sizeof c) == 0);
        dfree(out.data); dfree(out2.data);
        /* batched a x shared 2-D b */
        memset(&out, 0, sizeof out);
        CHECK(matmul(&ta3, &tw, &out) == 0 && out.ndim == 3 && out.shape[2] == BN && dsync() == 0 && d2h(c, out.data, sizeof c) == 0);
        for (int s2 = 0; s2 < BT; s2++) for (int i = 0; i < BM; i++) for (int j = 0; j < BN; j++) {
            float acc = 0; for (int k = 0; k < BK; k++) acc = fmaf(a[(s2 * BM + i) * BK + k], w[k * BN + j], acc);
            CHECK(c[(s2 * BM + i) * BN + j] == acc);
        }
        dfree(out.data);
        /* vector x vector -> [1]; vector x matrix -> [n]; matrix x vector -> [m] */
        memset(&out, 0, sizeof out);
        CHECK(matmul(&tv, &tv, &out) == 0 && out.ndim == 1 && out.shape[0] == 1 && dsync() == 0 && d2h(c, out.data, 4) == 0);
        { float acc = 0; for (int k = 0; k < BK; k++) acc = fmaf(v[k], v[k], acc); CHECK(c[0] == acc); }
        dfree(out.data); memset(&out, 0, sizeof out);
        CHECK(matmul(&tv, &tw, &out) == 0 && out.ndim == 1 && out.shape[0] == BN && dsync() == 0 && d2h(c, out.data, 4 * BN) == 0);
        for (int j = 0; j < BN; j++) { float acc = 0; for (int k = 0; k < BK; k++) acc = fmaf(v[k], w[k * BN + j], acc); CHECK(c[j] == acc); }
        dfree(out.data); memset(&out, 0, sizeof out);
        CHECK(matmul(&ta2, &tv, &out) == 0 && out.ndim == 1 && out.shape[0] == BM && dsync() == 0 && d2h(c, out.data, 4 * BM) == 0);
        for (int i = 0; i < BM; i++) { float acc = 0; for (int k = 0; k < BK; k++) acc = fmaf(a[i * BK + k], v[k], acc); CHECK(c[i] == acc); }
        dfree(out.data);
        /* refusals: inner dimensions, batch dimensions, dtypes */
        memset(&out, 0, sizeof out);
        CHECK(matmul(&tw, &ta2, &out) == -1 && out.data == NULL);
        tensor_t tb_other = make_tensor(0, 3, (size_t[]){BT + 1, BK, BN}, db);
        CHECK(matmul(&ta3, &tb_other, &out) == -1);
        tensor_t tw16 = tw; tw16.dtype = 2;
        CHECK(matmul(&ta2, &tw16, &out) == -1 && strlen(last_error()) > 0);
        CHECK(bmm(&ta2, &tw, &out) == -1);
        /* pg_tensordot: a [2,3,4] (viewed from `a`), b [4,3,5]: contract a's axes (1,2) with b's axes (1,0) -> [2,5] */
        float tb[BK * BM * BN], td[BT * BN];
        for (int i = 0; i < BK * BM * BN; i++) tb[i] = urand();
        void *dtb = dmalloc(sizeof tb);
        CHECK(dtb && h2d(dtb, tb, sizeof tb) == 0);
        tensor_t tdb = make_tensor(0, 3, (size_t[]){BK, BM, BN}, dtb);
        memset(&out, 0, sizeof out);
        CHECK(tensordot(&ta3, &tdb, 2, (size_t[]){1, 2}, (size_t[]){1, 0}, &out) == 0 && out.ndim == 2 && out.shape[0] == BT && out.shape[1] == BN);
        CHECK(dsync() == 0 && d2h(td, out.data, sizeof td) == 0);
        for (int s2 = 0; s2 < BT; s2++) for (int j = 0; j < BN; j++) {
            double acc = 0;
            for (int i = 0; i < BM; i++) for (int k = 0; k < BK; k++) acc += (double)a[(s2 * BM + i) * BK + k] * tb[(k * BM + i) * BN + j];
            CHECK(fabs(td[s2 * BN + j] - acc) < 1e-5);
        }
        dfree(out.data);
        CHECK(tensordot(&ta3, &tdb, 2, (size_t[]){1, 2}, (size_t[]){0, 1}, &out) == -1);     /* lengths 3,4 against 4,3 */
        /* backward of batched a x shared b, loss = sum: ga[s] = 1 * w^T, gw = sum_s a[s]^T * 1 */
        float g[BT * BM * BN], ga[BT * BM * BK], gw[BK * BN];
        for (int i = 0; i < BT * BM * BN; i++) g[i] = 1.0f;
        void *dg = dmalloc(sizeof g), *dga = dmalloc(sizeof ga), *dgw = dmalloc(sizeof gw);
        CHECK(dg && dga && dgw && h2d(dg, g, sizeof g) == 0);
        CHECK(backward(&ta3, &tw, (const float *)dg, (float *)dga, (float *)dgw, 0) == 0);
        CHECK(dsync() == 0 && d2h(ga, dga, sizeof ga) == 0 && d2h(gw, dgw, sizeof gw) == 0);
        for (int s2 = 0; s2 < BT; s2++) for (int i = 0; i < BM; i++) for (int k = 0; k < BK; k++) {
            double acc = 0; for (int j = 0; j < BN; j++) acc += w[k * BN + j];
            CHECK(fabs(ga[(s2 * BM + i) * BK + k] - acc) < 1e-5);
        }
        for (int k = 0; k < BK; k++) for (int j = 0; j < BN; j++) {
            double acc = 0; for (int s2 = 0; s2 < BT; s2++) for (int i = 0; i < BM; i++) acc += a[(s2 * BM + i) * BK + k];
            CHECK(fabs(gw[k * BN + j] - acc) < 1e-5);
        }
        printf("tensor-level callers: matmul shape modes, bmm, tensordot, refusals, backward: done\n");
        dfree(da); dfree(db); dfree(dw); dfree(dv); dfree(dtb); dfree(dg); dfree(dga); dfree(dgw);
    }

    /* ---- a column shard stored into two full matrices by the GEMM kernel (pg_b200_gemm_ex_scatter) ---- */
    {
        typedef int (*scatter_fn)(int, size_t, size_t, size_t, const void *, size_t, const void *, size_t, float *const *, size_t,
                                  size_t, size_t);
        typedef int (*gemm_ex_fn)(int, size_t, size_t, size_t, const void *, size_t, const void *, size_t, float *, size_t);
        scatter_fn scatter = (scatter_fn)dlsym(h, "pg_b200_gemm_ex_scatter");
        gemm_ex_fn gemm_ex = (gemm_ex_fn)dlsym(h, "pg_b200_gemm_ex");
        if (!scatter || !gemm_ex) { printf("missing symbol (scatter)\n"); return 2; }
        enum { SM = 256, SN = 128, SK = 128, LD = 384, COL0 = 128 };
        static uint16_t a[SM * SK], b[SK * SN];
        static float full[2][SM * LD], own[SM * SN];
        for (int i = 0; i < SM * SK; i++) a[i] = to_bf16(urand());
        for (int i = 0; i < SK * SN; i++) b[i] = to_bf16(urand());
        void *da = dmalloc(sizeof a), *db = dmalloc(sizeof b), *d0 = dmalloc(sizeof full[0]), *d1 = dmalloc(sizeof full[0]),
             *down = dmalloc(sizeof own);
        CHECK(da && db && d0 && d1 && down);
        for (int i = 0; i < SM * LD; i++) full[0][i] = -3.0f;
        CHECK(h2d(da, a, sizeof a) == 0 && h2d(db, b, sizeof b) == 0 && h2d(d0, full[0], sizeof full[0]) == 0 &&
              h2d(d1, full[0], sizeof full[0]) == 0);
        float *dst[2] = {(float *)d0, (float *)d1};
        CHECK(scatter(2, SM, SN, SK, da, SK, db, SN, dst, 2, LD, COL0) == 0);
        CHECK(gemm_ex(2, SM, SN, SK, da, SK, db, SN, (float *)down, SN) == 0);
        CHECK(dsync() == 0 && d2h(full[0], d0, sizeof full[0]) == 0 && d2h(full[1], d1, sizeof full[1]) == 0 &&
              d2h(own, down, sizeof own) == 0);
        CHECK(memcmp(full[0], full[1], sizeof full[0]) == 0);
        for (int i = 0; i < SM; i++)
            for (int j = 0; j < LD; j++) {
                float want = (j >= COL0 && j < COL0 + SN) ? own[i * SN + j - COL0] : -3.0f;
                if (full[0][i * LD + j] != want) { CHECK(!"scatter: element differs"); i = SM; break; }
            }
        CHECK(scatter(2, SM, SN - 2, SK, da, SK, db, SN, dst, 2, LD, COL0) == -1);     /* width not a multiple of 4 */
        printf("gemm_ex_scatter bf16 256x128x128 into two 256x384 matrices: same bits as gemm_ex, rest untouched\n");
        dfree(da); dfree(db); dfree(d0); dfree(d1); dfree(down);
    }

    if (fails) { printf("%d check(s) failed: %s\n", fails, last_error()); return 1; }
    printf("all passed\n");
    return 0;
}
