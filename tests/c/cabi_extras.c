/* The C-ABI entries beyond picograd's vtable, called from plain C (no Python, no torch): the fused
 * bias/activation GEMM (pg_cpu_gemm_fused_ex), pg_conv2d and the attention-shaped chain.  Each result is
 * compared with loops written here from the definitions in picograd's sources:
 *   gemm.c:718-817  C = act(bias[j] + A*B), one fused multiply-add chain per element starting at bias[j]
 *   conv.c:10-146   im2col rows in (ci,ki,kj) order, zeros outside the image, GEMM, then + bias
 *   matmul.c:340-369 + activations.c:22-45  O = bf16(softmax_rows(Q*Kt)) * V
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

    if (fails) { printf("%d check(s) failed: %s\n", fails, last_error()); return 1; }
    printf("all passed\n");
    return 0;
}
