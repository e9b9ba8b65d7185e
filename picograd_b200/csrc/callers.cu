// Tensor-level callers of the GEMM with picograd's shape rules, device-resident: pg_matmul, pg_bmm,
// pg_tensordot (ops/matmul.c:186-284, :340-369, :407-490) and the matmul node of the autograd (bwd_matmul,
// autograd/autograd.c:561-706) over operands described the way pg_tensor describes them (core/tensor.h:21-36:
// dtype, ndim, shape, element strides, data pointer — here a device pointer).  Where picograd returns NULL these
// return PG_ERR_UNSUPPORTED with the reason in pg_b200_last_error().  Everything below is host-side shape logic;
// the arithmetic is pg_b200_gemm_batched / pg_b200_matmul_backward_ex / the permute kernel.

#include "../../include/pg_b200.h"
#include "pg_internal.h"

#include <string.h>

using namespace pgb;

namespace {

bool valid_dtype(int dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }
size_t esize_of(int dt) { return dt == DT_F32 ? 4 : 2; }

bool valid_tensor(const pg_b200_tensor *t, const char *who, const char *name) {
    if (!t || !t->data) { set_error("%s: operand %s is NULL or has no data", who, name); return false; }
    if (t->ndim < 1 || t->ndim > PG_B200_MAX_NDIM) { set_error("%s: operand %s has %zu dimensions", who, name, t->ndim); return false; }
    if (!valid_dtype(t->dtype)) { set_error("%s: operand %s has dtype %d", who, name, t->dtype); return false; }
    return true;
}

// Result tensor: contiguous f32 of `shape`; allocated with pg_b200_malloc when out->data is NULL on entry.
int prepare_out(pg_b200_tensor *out, size_t ndim, const size_t *shape, const char *who, bool shape_only = false) {
    if (!out) { set_error("%s: no result tensor", who); return ST_UNSUPPORTED; }
    size_t numel = 1;
    for (size_t d = 0; d < ndim; ++d) numel *= shape[d];
    out->dtype = DT_F32;
    out->ndim = ndim;
    size_t run = 1;
    for (size_t d = ndim; d-- > 0;) { out->shape[d] = shape[d]; out->stride[d] = run; run *= shape[d]; }
    for (size_t d = ndim; d < PG_B200_MAX_NDIM; ++d) { out->shape[d] = 0; out->stride[d] = 0; }
    if (shape_only) return ST_OK;
    if (!out->data) {
        out->data = pg_b200_malloc(numel * sizeof(float));
        if (!out->data) return ST_ALLOC;
    }
    return ST_OK;
}

// Do the leading `nd` dimensions of t collapse into one batch index with a single stride?
bool single_batch_stride(const pg_b200_tensor *t, size_t nd, size_t *stride) {
    if (nd == 0) { *stride = 0; return true; }
    for (size_t d = 0; d + 1 < nd; ++d)
        if (t->stride[d] != t->stride[d + 1] * t->shape[d + 1]) return false;
    *stride = t->stride[nd - 1];
    return true;
}

bool contiguous(const pg_b200_tensor *t) {
    size_t run = 1;
    for (size_t d = t->ndim; d-- > 0;) {
        if (t->shape[d] != 1 && t->stride[d] != run) return false;
        run *= t->shape[d];
    }
    return true;
}

struct MatmulShape {
    bool av, bv;
    size_t am, ak, bn, abn, bbn, bnd, nbatch;
    const size_t *bshape;
};

// picograd's operand rules (ops/matmul.c:195-231).  One rule is stricter here: a vector b must have ak elements
// (picograd does not check and would read past the end of b).
int matmul_shape(const pg_b200_tensor *a, const pg_b200_tensor *b, MatmulShape &s, const char *who) {
    if (a->dtype != b->dtype) { set_error("%s: operand dtypes differ (%d, %d)", who, a->dtype, b->dtype); return ST_UNSUPPORTED; }
    const size_t ra = a->ndim, rb = b->ndim;
    s.av = ra == 1; s.bv = rb == 1;
    const size_t bk = s.bv ? b->shape[0] : b->shape[rb - 2];
    if (a->shape[ra - 1] != bk) { set_error("%s: inner dimensions differ (%zu, %zu)", who, a->shape[ra - 1], bk); return ST_UNSUPPORTED; }
    if (a->stride[ra - 1] != 1 || (!s.bv && b->stride[rb - 1] != 1)) { set_error("%s: the last dimension must have stride 1", who); return ST_UNSUPPORTED; }
    s.am = s.av ? 1 : a->shape[ra - 2];
    s.ak = a->shape[ra - 1];
    s.bn = s.bv ? 1 : b->shape[rb - 1];
    s.abn = s.av ? 0 : ra - 2;
    s.bbn = s.bv ? 0 : rb - 2;
    if (s.abn == 0 && s.bbn == 0) { s.bnd = 0; s.bshape = nullptr; }
    else if (s.abn == 0) { s.bnd = s.bbn; s.bshape = b->shape; }
    else if (s.bbn == 0) { s.bnd = s.abn; s.bshape = a->shape; }
    else {
        if (s.abn != s.bbn || memcmp(a->shape, b->shape, s.abn * sizeof(size_t)) != 0) {
            set_error("%s: batch dimensions differ", who);
            return ST_UNSUPPORTED;
        }
        s.bnd = s.abn; s.bshape = a->shape;
    }
    s.nbatch = 1;
    for (size_t d = 0; d < s.bnd; ++d) {
        if (s.bshape[d] == 0 || s.nbatch > SIZE_MAX / s.bshape[d]) { set_error("%s: empty or overflowing batch", who); return ST_UNSUPPORTED; }
        s.nbatch *= s.bshape[d];
    }
    return ST_OK;
}

// Walks picograd's batch odometer (ops/matmul.c:262-282): calls fn(batch index, offset into a, offset into b).
template <typename F>
int for_each_batch(const pg_b200_tensor *a, const pg_b200_tensor *b, const MatmulShape &s, F fn) {
    size_t midx[PG_B200_MAX_NDIM] = {0}, oa = 0, ob = 0;
    for (size_t i = 0; i < s.nbatch; ++i) {
        const int st = fn(i, oa, ob);
        if (st != ST_OK) return st;
        for (size_t d = s.bnd; d-- > 0;) {
            const size_t sa = s.abn ? a->stride[d] : 0, sb = s.bbn ? b->stride[d] : 0;
            midx[d]++; oa += sa; ob += sb;
            if (midx[d] < s.bshape[d]) break;
            midx[d] = 0; oa -= sa * s.bshape[d]; ob -= sb * s.bshape[d];
        }
    }
    return ST_OK;
}

}  // namespace

extern "C" {

static int matmul_impl(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out, bool shape_only) {
    const char *who = "pg_b200_matmul";
    if (!valid_tensor(a, who, "a") || !valid_tensor(b, who, "b")) return ST_UNSUPPORTED;
    MatmulShape s;
    int st = matmul_shape(a, b, s, who);
    if (st != ST_OK) return st;
    size_t rshape[PG_B200_MAX_NDIM], rndim = 0;
    for (size_t d = 0; d < s.bnd; ++d) rshape[rndim++] = s.bshape[d];
    if (!s.av) rshape[rndim++] = s.am;
    if (!s.bv) rshape[rndim++] = s.bn;
    if (rndim == 0) rshape[rndim++] = 1;
    if ((st = prepare_out(out, rndim, rshape, who, shape_only)) != ST_OK || shape_only) return st;
    const size_t lda = s.av ? (s.ak ? s.ak : 1) : a->stride[a->ndim - 2];
    const size_t ldb = s.bv ? b->stride[0] : b->stride[b->ndim - 2];
    float *c = (float *)out->data;
    size_t sa = 0, sb = 0;
    if (single_batch_stride(a, s.abn, &sa) && single_batch_stride(b, s.bbn, &sb))
        return pg_b200_gemm_batched(a->dtype, b->dtype, 0, 0, s.nbatch, s.am, s.bn, s.ak, a->data, lda, sa, b->data, ldb, sb,
                                    c, s.bn, s.am * s.bn, 0);
    const size_t es = esize_of(a->dtype);
    return for_each_batch(a, b, s, [&](size_t i, size_t oa, size_t ob) {
        return pg_b200_gemm_batched(a->dtype, b->dtype, 0, 0, 1, s.am, s.bn, s.ak, (const char *)a->data + oa * es, lda, 0,
                                    (const char *)b->data + ob * es, ldb, 0, c + i * s.am * s.bn, s.bn, 0, 0);
    });
}

int pg_b200_matmul(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out) {
    return matmul_impl(a, b, out, false);
}
int pg_b200_matmul_result_shape(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out) {
    return matmul_impl(a, b, out, true);
}

int pg_b200_bmm(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out) {
    const char *who = "pg_b200_bmm";
    if (!valid_tensor(a, who, "a") || !valid_tensor(b, who, "b")) return ST_UNSUPPORTED;
    if (a->ndim != 3 || b->ndim != 3 || a->shape[0] != b->shape[0] || a->shape[2] != b->shape[1] || a->dtype != b->dtype) {
        set_error("%s: needs [B,M,K] x [B,K,N] of one dtype", who);
        return ST_UNSUPPORTED;
    }
    // picograd indexes both operands as contiguous blocks (ops/matmul.c:360-362); say so instead of reading wrongly
    if (!contiguous(a) || !contiguous(b)) { set_error("%s: operands must be contiguous", who); return ST_UNSUPPORTED; }
    const size_t batch = a->shape[0], m = a->shape[1], k = a->shape[2], n = b->shape[2];
    const size_t shape[3] = {batch, m, n};
    const int st = prepare_out(out, 3, shape, who);
    if (st != ST_OK) return st;
    return pg_b200_gemm_batched(a->dtype, b->dtype, 0, 0, batch, m, n, k, a->data, k, m * k, b->data, n, k * n,
                                (float *)out->data, n, m * n, 0);
}

static int tensordot_impl(const pg_b200_tensor *a, const pg_b200_tensor *b, size_t ndims, const size_t *axes_a,
                          const size_t *axes_b, pg_b200_tensor *out, bool shape_only) {
    const char *who = "pg_b200_tensordot";
    if (!valid_tensor(a, who, "a") || !valid_tensor(b, who, "b") || !axes_a || !axes_b) return ST_UNSUPPORTED;
    if (ndims < 1 || ndims > a->ndim || ndims > b->ndim || a->dtype != b->dtype) {
        set_error("%s: bad number of contracted axes or operand dtypes differ", who);
        return ST_UNSUPPORTED;
    }
    const size_t free_a = a->ndim - ndims, rest_b = b->ndim - ndims;
    if (free_a + rest_b > PG_B200_MAX_NDIM) { set_error("%s: result would have more than %d dimensions", who, PG_B200_MAX_NDIM); return ST_UNSUPPORTED; }
    for (size_t i = 0; i < ndims; ++i)
        if (axes_a[i] >= a->ndim || axes_b[i] >= b->ndim || a->shape[axes_a[i]] != b->shape[axes_b[i]]) {
            set_error("%s: contracted axis %zu out of range or of different length", who, i);
            return ST_UNSUPPORTED;
        }
    // a -> (free..., contracted...), b -> (contracted..., rest...)
    uint32_t pa[PG_B200_MAX_NDIM], pb[PG_B200_MAX_NDIM];
    size_t w = 0;
    auto contracted = [&](const size_t *axes, size_t d) { for (size_t i = 0; i < ndims; ++i) if (axes[i] == d) return true; return false; };
    for (size_t d = 0; d < a->ndim; ++d) if (!contracted(axes_a, d)) pa[w++] = (uint32_t)d;
    if (w != free_a) { set_error("%s: an axis of a is contracted twice", who); return ST_UNSUPPORTED; }
    for (size_t i = 0; i < ndims; ++i) pa[w++] = (uint32_t)axes_a[i];
    w = 0;
    for (size_t i = 0; i < ndims; ++i) pb[w++] = (uint32_t)axes_b[i];
    for (size_t d = 0; d < b->ndim; ++d) if (!contracted(axes_b, d)) pb[w++] = (uint32_t)d;
    if (w != b->ndim) { set_error("%s: an axis of b is contracted twice", who); return ST_UNSUPPORTED; }
    size_t mdim = 1, kdim = 1, ndim_n = 1;
    for (size_t d = 0; d < free_a; ++d) mdim *= a->shape[pa[d]];
    for (size_t d = 0; d < ndims; ++d) kdim *= a->shape[axes_a[d]];
    for (size_t d = ndims; d < b->ndim; ++d) ndim_n *= b->shape[pb[d]];
    size_t fshape[PG_B200_MAX_NDIM], j = 0;
    for (size_t d = 0; d < free_a; ++d) fshape[j++] = a->shape[pa[d]];
    for (size_t d = ndims; d < b->ndim; ++d) fshape[j++] = b->shape[pb[d]];
    if (j == 0) fshape[j++] = 1;
    int st = prepare_out(out, j, fshape, who, shape_only);
    if (st != ST_OK || shape_only) return st;
    if (mdim == 0 || ndim_n == 0) return ST_OK;
    // permuted copies (ops/matmul.c:21-42), skipped for an operand that already lies in the wanted order
    const size_t es = esize_of(a->dtype);
    const void *ra = a->data, *rb = b->data;
    const pg_b200_tensor *ops[2] = {a, b};
    const uint32_t *perms[2] = {pa, pb};
    for (int which = 0; which < 2; ++which) {
        const pg_b200_tensor *t = ops[which];
        bool identity = contiguous(t);
        for (size_t d = 0; d < t->ndim; ++d) identity = identity && perms[which][d] == d;
        if (identity) continue;
        size_t numel = 1;
        uint64_t sh[PG_B200_MAX_NDIM], sstr[PG_B200_MAX_NDIM];
        for (size_t d = 0; d < t->ndim; ++d) { numel *= t->shape[d]; sh[d] = t->shape[d]; sstr[d] = t->stride[d]; }
        void *dst = caller_scratch(which, numel * es);
        if (!dst) return ST_ALLOC;
        st = permute_copy_launch(t->data, dst, es, (uint32_t)t->ndim, sh, perms[which], current_stream(), sstr);
        if (st != ST_OK) return st;
        (which == 0 ? ra : rb) = dst;
    }
    return pg_b200_gemm_batched(a->dtype, b->dtype, 0, 0, 1, mdim, ndim_n, kdim, ra, kdim ? kdim : 1, 0, rb, ndim_n, 0,
                                (float *)out->data, ndim_n, 0, 0);
}

int pg_b200_tensordot(const pg_b200_tensor *a, const pg_b200_tensor *b, size_t ndims, const size_t *axes_a,
                      const size_t *axes_b, pg_b200_tensor *out) {
    return tensordot_impl(a, b, ndims, axes_a, axes_b, out, false);
}
int pg_b200_tensordot_result_shape(const pg_b200_tensor *a, const pg_b200_tensor *b, size_t ndims, const size_t *axes_a,
                                   const size_t *axes_b, pg_b200_tensor *out) {
    return tensordot_impl(a, b, ndims, axes_a, axes_b, out, true);
}

int pg_b200_matmul_backward_nd(const pg_b200_tensor *a, const pg_b200_tensor *b, const float *grad_out, float *grad_a,
                               float *grad_b, int accumulate) {
    const char *who = "pg_b200_matmul_backward_nd";
    if (!valid_tensor(a, who, "a") || !valid_tensor(b, who, "b")) return ST_UNSUPPORTED;
    if (!grad_out) { set_error("%s: no incoming gradient", who); return ST_UNSUPPORTED; }
    if (!grad_a && !grad_b) return ST_OK;
    MatmulShape s;
    int st = matmul_shape(a, b, s, who);
    if (st != ST_OK) return st;
    // bwd_matmul reads both operands as contiguous blocks (autograd.c:603-612: step_a = am * ak, step_b = ak * bn)
    if (!contiguous(a) || !contiguous(b)) { set_error("%s: operands must be contiguous", who); return ST_UNSUPPORTED; }
    const bool abat = s.abn > 0, bbat = s.bbn > 0;
    if (abat || !bbat)    // a carries the batch (b batched alike, or shared), or there is no batch at all
        return pg_b200_matmul_backward_ex(a->dtype, s.nbatch, s.am, s.bn, s.ak, a->data, b->data, bbat ? 1 : 0, grad_out,
                                          grad_a, grad_b, accumulate);
    // a shared by a batched b: grad_a sums over the batch (autograd.c:645: gap = ga->data + 0), grad_b is per element
    const size_t es = esize_of(a->dtype);
    for (size_t i = 0; i < s.nbatch; ++i) {
        const void *bi = (const char *)b->data + i * s.ak * s.bn * es;
        const float *gi = grad_out + i * s.am * s.bn;
        if (grad_a) {
            st = pg_b200_matmul_backward_ex(a->dtype, 1, s.am, s.bn, s.ak, a->data, bi, 0, gi, grad_a, nullptr,
                                            (accumulate || i > 0) ? 1 : 0);
            if (st != ST_OK) return st;
        }
        if (grad_b) {
            st = pg_b200_matmul_backward_ex(a->dtype, 1, s.am, s.bn, s.ak, a->data, bi, 0, gi, nullptr,
                                            grad_b + i * s.ak * s.bn, accumulate);
            if (st != ST_OK) return st;
        }
    }
    return ST_OK;
}

}  // extern "C"
