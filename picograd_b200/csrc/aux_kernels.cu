// Small HBM-bound helper kernels around the GEMMs: exact f32 -> bf16-pieces
// split (feeds the tensor cores with f32 data without rounding it), split-K
// reduction, gradient accumulation, and the element-wise harness steps of the
// attention-shaped and MLP workloads (softmax rows, GELU and its gradient,
// f32 -> 16-bit casts).  All are grid-stride / one-warp-per-row kernels with
// 16-byte accesses where alignment allows.

#include "pg_internal.h"
#include "fast_math.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace pgb {

static inline unsigned grid_for(uint64_t work_items, unsigned block) {
    uint64_t blocks = (work_items + block - 1) / block;
    uint64_t cap = (uint64_t)device_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

__device__ __forceinline__ unsigned short bf16_rne(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bf16_up(unsigned short h) { return __uint_as_float((unsigned)h << 16); }

// x = p0 + p1 (+ p2) with every piece a bf16 and every subtraction exact:
// p0 = bf16(x), p1 = bf16(x - p0), p2 = bf16(x - p0 - p1).
// Layout of dst: [batch][part][rows][ld_dst].
__device__ __forceinline__ void split3(float x, unsigned short &h0, unsigned short &h1, unsigned short &h2) {
    h0 = bf16_rne(x);
    const float r1 = x - bf16_up(h0);
    h1 = bf16_rne(r1);
    h2 = bf16_rne(r1 - bf16_up(h1));
}

// Which pieces hold something: bit i for a non-zero element (either sign of zero counts as zero) in piece i.
__device__ __forceinline__ uint32_t piece_bits(unsigned short h0, unsigned short h1, unsigned short h2) {
    return ((h0 & 0x7FFFu) ? 1u : 0u) | ((h1 & 0x7FFFu) ? 2u : 0u) | ((h2 & 0x7FFFu) ? 4u : 0u);
}
__device__ __forceinline__ void publish_piece_mask(uint32_t *mask, uint32_t seen) {
    if (!mask) return;
    seen = __reduce_or_sync(0xffffffffu, seen);
    if ((threadIdx.x & 31) == 0 && seen) atomicOr(mask, seen);
}

// General form: any leading dimensions, one element per thread step.
__global__ void split_f32_kernel(const float *__restrict__ src, uint64_t ld_src, uint64_t src_bs,
                                 unsigned short *__restrict__ dst, uint64_t ld_dst, uint32_t rows, uint32_t cols,
                                 uint32_t batch, uint32_t nparts, uint32_t *mask) {
    const uint64_t per_batch = (uint64_t)rows * cols;
    const uint64_t total = per_batch * batch;
    const uint64_t part_stride = (uint64_t)rows * ld_dst;
    uint32_t seen = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i / per_batch;
        const uint64_t r = (i - b * per_batch) / cols;
        const uint64_t c = i - b * per_batch - r * cols;
        unsigned short h0, h1, h2;
        split3(src[b * src_bs + r * ld_src + c], h0, h1, h2);
        unsigned short *d = dst + b * nparts * part_stride + r * ld_dst + c;
        d[0] = h0;
        d[part_stride] = h1;
        if (nparts > 2) d[2 * part_stride] = h2;
        seen |= piece_bits(h0, h1, nparts > 2 ? h2 : 0);
    }
    publish_piece_mask(mask, seen);
}

// Fast form for the common case (cols and both leading dimensions multiples of 4, 16-byte aligned
// bases): four elements per thread step, one 16-byte load and one 8-byte store per piece.
__global__ void split_f32_vec4_kernel(const float *__restrict__ src, uint64_t ld_src, uint64_t src_bs,
                                      unsigned short *__restrict__ dst, uint64_t ld_dst, uint32_t rows, uint32_t cols4,
                                      uint32_t batch, uint32_t nparts, uint32_t *mask) {
    uint32_t seen = 0;
    const uint64_t per_batch = (uint64_t)rows * cols4;
    const uint64_t total = per_batch * batch;
    const uint64_t part_stride = (uint64_t)rows * ld_dst;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i / per_batch;
        const uint64_t r = (i - b * per_batch) / cols4;
        const uint64_t c = (i - b * per_batch - r * cols4) * 4;
        const float4 x = *reinterpret_cast<const float4 *>(src + b * src_bs + r * ld_src + c);
        unsigned short h[3][4];
        split3(x.x, h[0][0], h[1][0], h[2][0]);
        split3(x.y, h[0][1], h[1][1], h[2][1]);
        split3(x.z, h[0][2], h[1][2], h[2][2]);
        split3(x.w, h[0][3], h[1][3], h[2][3]);
        unsigned short *d = dst + b * nparts * part_stride + r * ld_dst + c;
        for (uint32_t p = 0; p < nparts; ++p) {
            uint2 v;
            v.x = (uint32_t)h[p][0] | ((uint32_t)h[p][1] << 16);
            v.y = (uint32_t)h[p][2] | ((uint32_t)h[p][3] << 16);
            *reinterpret_cast<uint2 *>(d + p * part_stride) = v;
            if ((v.x | v.y) & 0x7FFF7FFFu) seen |= 1u << p;
        }
    }
    publish_piece_mask(mask, seen);
}

int split_f32_to_bf16_launch(const float *src, uint64_t ld_src, uint64_t src_bs, uint16_t *dst, uint64_t ld_dst,
                             uint32_t rows, uint32_t cols, uint32_t batch, uint32_t nparts, cudaStream_t s, uint32_t *mask) {
    const uint64_t total = (uint64_t)rows * cols * batch;
    if (!total) return ST_OK;
    if (mask && cudaMemsetAsync(mask, 0, sizeof(uint32_t), s) != cudaSuccess) { cudaGetLastError(); return ST_GEMM; }
    const bool vec = cols % 4 == 0 && ld_src % 4 == 0 && ld_dst % 4 == 0 && src_bs % 4 == 0 &&
                     ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 7) == 0;
    if (vec)
        split_f32_vec4_kernel<<<grid_for(total / 4, 256), 256, 0, s>>>(src, ld_src, src_bs, dst, ld_dst, rows, cols / 4,
                                                                       batch, nparts, mask);
    else
        split_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, ld_src, src_bs, dst, ld_dst, rows, cols, batch, nparts, mask);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// An f16 value is the exact sum of two bf16 pieces (11 significant bits <= 8 + 8, and bf16 has
// the wider exponent range).  Layout of dst as above with two parts.
__global__ void split_f16_kernel(const unsigned short *__restrict__ src, uint64_t ld_src, uint64_t src_bs,
                                 unsigned short *__restrict__ dst, uint64_t ld_dst, uint32_t rows, uint32_t cols,
                                 uint32_t batch) {
    const uint64_t per_batch = (uint64_t)rows * cols;
    const uint64_t total = per_batch * batch;
    const uint64_t part_stride = (uint64_t)rows * ld_dst;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i / per_batch;
        const uint64_t r = (i - b * per_batch) / cols;
        const uint64_t c = i - b * per_batch - r * cols;
        const float x = __half2float(__ushort_as_half(src[b * src_bs + r * ld_src + c]));
        unsigned short *d = dst + b * 2 * part_stride + r * ld_dst + c;
        const unsigned short h0 = bf16_rne(x);
        d[0] = h0;
        d[part_stride] = bf16_rne(x - bf16_up(h0));
    }
}

int split_f16_to_bf16_launch(const uint16_t *src, uint64_t ld_src, uint64_t src_bs, uint16_t *dst, uint64_t ld_dst,
                             uint32_t rows, uint32_t cols, uint32_t batch, cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * cols * batch;
    if (!total) return ST_OK;
    split_f16_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, ld_src, src_bs, dst, ld_dst, rows, cols, batch);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// C[m][n] (=|+=) sum_s ws[s][m][n], slices summed in ascending order.
__global__ void reduce_splits_kernel(const float *__restrict__ ws, uint64_t slice_stride, uint32_t splits,
                                     float *__restrict__ c, uint64_t ldc, uint32_t M, uint32_t N, uint64_t ws_ld,
                                     int accumulate) {
    const uint64_t total = (uint64_t)M * N;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / N, col = i - r * N;
        const float *w = ws + r * ws_ld + col;
        float acc = w[0];
        for (uint32_t s = 1; s < splits; ++s) acc += w[(uint64_t)s * slice_stride];
        float *d = c + r * ldc + col;
        *d = accumulate ? (*d + acc) : acc;
    }
}

int reduce_splits_launch(const float *ws, uint64_t slice_stride, uint32_t splits, float *c, uint64_t ldc, uint32_t M,
                         uint32_t N, uint64_t ws_ld, int accumulate, cudaStream_t s) {
    const uint64_t total = (uint64_t)M * N;
    if (!total) return ST_OK;
    reduce_splits_kernel<<<grid_for(total, 256), 256, 0, s>>>(ws, slice_stride, splits, c, ldc, M, N, ws_ld, accumulate);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

__global__ void add_inplace_kernel(float *__restrict__ dst, const float *__restrict__ src, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] += src[i];
}
int add_inplace_launch(float *dst, const float *src, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    add_inplace_kernel<<<grid_for(n, 256), 256, 0, s>>>(dst, src, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

__device__ __forceinline__ unsigned short to16(float v, int dtype) {
    return dtype == DT_BF16 ? bf16_rne(v) : __half_as_ushort(__float2half_rn(v));
}

__global__ void cast_f32_kernel(const float *__restrict__ src, unsigned short *__restrict__ dst, uint64_t n, int dtype) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = to16(src[i], dtype);
}
int cast_f32_launch(const float *src, uint16_t *dst, uint64_t n, int dtype, cudaStream_t s) {
    if (!n) return ST_OK;
    cast_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst, n, dtype);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118f)); }
__device__ __forceinline__ float gelu_grad_f(float v, float gy) {
    const float e = erff(v * 0.70710678118f);
    const float phi = expf(-0.5f * v * v) / 2.50662827463f;
    return gy * (0.5f * (1.0f + e) + v * phi);
}

// 0.5 x (1 + erf(x / sqrt 2))   (picograd ops/activations.c:114); four elements per thread step when
// the buffers are 16-byte aligned, the tail (and unaligned buffers) one by one.
__global__ void gelu_kernel(const float *__restrict__ src, float *__restrict__ d32, unsigned short *__restrict__ d16,
                            int dtype16, uint64_t n, int vec) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t n4 = vec ? n / 4 : 0;
    for (uint64_t i = tid; i < n4; i += stride) {
        const float4 x = reinterpret_cast<const float4 *>(src)[i];
        const float4 y = make_float4(gelu_f(x.x), gelu_f(x.y), gelu_f(x.z), gelu_f(x.w));
        if (d32) reinterpret_cast<float4 *>(d32)[i] = y;
        if (d16) {
            uint2 v;
            v.x = (uint32_t)to16(y.x, dtype16) | ((uint32_t)to16(y.y, dtype16) << 16);
            v.y = (uint32_t)to16(y.z, dtype16) | ((uint32_t)to16(y.w, dtype16) << 16);
            reinterpret_cast<uint2 *>(d16)[i] = v;
        }
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) {
        const float y = gelu_f(src[i]);
        if (d32) d32[i] = y;
        if (d16) d16[i] = to16(y, dtype16);
    }
}
int gelu_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    const int vec = (((uintptr_t)src | (uintptr_t)dst_f32) & 15) == 0 && ((uintptr_t)dst_16 & 7) == 0;
    gelu_kernel<<<grid_for(vec ? n / 4 + 1 : n, 256), 256, 0, s>>>(src, dst_f32, dst_16, dtype16, n, vec);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// permute_copy of picograd's pg_tensordot (ops/matmul.c:21-42): dst, contiguous with shape out_shape, takes
// element (c0, .., c_{nd-1}) from src offset sum(c_d * src_stride[d]) (the strides of the source dimension that
// lands in position d).  One thread per destination element: writes coalesced, reads strided; when the last
// dimension keeps its place the reads run along it too.
struct PermuteParams {
    uint32_t ndim;
    uint64_t out_shape[8];
    uint64_t src_stride[8];
    uint64_t total;
};
template <typename T>
__global__ void permute_copy_kernel(const T *__restrict__ src, T *__restrict__ dst, const PermuteParams p) {
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += step) {
        uint64_t rest = i, off = 0;
#pragma unroll
        for (int d = 7; d >= 0; --d) {
            if (d < (int)p.ndim) {
                const uint64_t c = rest % p.out_shape[d];
                rest /= p.out_shape[d];
                off += c * p.src_stride[d];
            }
        }
        dst[i] = src[off];
    }
}
int permute_copy_launch(const void *src, void *dst, size_t elem_size, uint32_t ndim, const uint64_t *shape, const uint32_t *perm,
                        cudaStream_t s, const uint64_t *src_stride) {
    if (ndim == 0 || ndim > 8 || (elem_size != 2 && elem_size != 4)) return ST_UNSUPPORTED;
    PermuteParams p = {};
    p.ndim = ndim;
    uint64_t stride[8], run = 1;
    for (int d = (int)ndim - 1; d >= 0; --d) { stride[d] = src_stride ? src_stride[d] : run; run *= shape[d]; }
    uint32_t seen = 0;
    p.total = 1;
    for (uint32_t d = 0; d < ndim; ++d) {
        if (perm[d] >= ndim || (seen >> perm[d]) & 1u) return ST_UNSUPPORTED;
        seen |= 1u << perm[d];
        p.out_shape[d] = shape[perm[d]];
        p.src_stride[d] = stride[perm[d]];
        p.total *= shape[perm[d]];
    }
    if (!p.total) return ST_OK;
    if (elem_size == 4) permute_copy_kernel<uint32_t><<<grid_for(p.total, 256), 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, p);
    else permute_copy_kernel<uint16_t><<<grid_for(p.total, 256), 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// Re-layout after an all-gather of N-column shards: `staging` holds the G shards one after the other, shard g as a
// row-major [rows][width] block (the layout an all-gather of contiguous shards produces); dst is the row-major
// [rows][n] matrix whose columns [g*width, g*width + width) (clipped at n) are shard g.  HBM-bound: every element is
// read once and written once, 16 bytes per thread per step when width, n, ld and the bases allow it.
template <typename V>
__global__ void gather_relayout_kernel(const V *__restrict__ staging, V *__restrict__ dst, uint32_t shards, uint64_t rows,
                                       uint64_t width_v, uint64_t n_v, uint64_t ld_v) {
    // one "v" = one V (4 floats or 1 float); n_v columns of dst in units of V
    const uint64_t total = rows * n_v;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const uint64_t r = i / n_v, c = i - r * n_v;
        const uint64_t g = c / width_v, j = c - g * width_v;
        dst[r * ld_v + c] = __ldcs(staging + (g * rows + r) * width_v + j);
    }
}
int gather_relayout_launch(const float *staging, float *dst, uint32_t shards, uint64_t rows, uint64_t width, uint64_t n,
                           uint64_t ld, cudaStream_t s) {
    if (!rows || !n) return ST_OK;
    if (!shards || !width || (uint64_t)shards * width < n || ld < n) return ST_UNSUPPORTED;
    const bool vec = width % 4 == 0 && n % 4 == 0 && ld % 4 == 0 && ((uintptr_t)staging & 15u) == 0 && ((uintptr_t)dst & 15u) == 0;
    const int sms = device_sm_count();
    if (vec) {
        const uint64_t total = rows * (n / 4);
        uint64_t blocks = (total + 255) / 256;
        if (blocks > (uint64_t)sms * 16) blocks = (uint64_t)sms * 16;
        gather_relayout_kernel<float4><<<(unsigned)blocks, 256, 0, s>>>((const float4 *)staging, (float4 *)dst, shards, rows,
                                                                       width / 4, n / 4, ld / 4);
    } else {
        const uint64_t total = rows * n;
        uint64_t blocks = (total + 255) / 256;
        if (blocks > (uint64_t)sms * 16) blocks = (uint64_t)sms * 16;
        gather_relayout_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(staging, dst, shards, rows, width, n, ld);
    }
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// The element-wise tail of pg_addmm (ops/matmul.c:383-404): c = (0 + input) * beta + c * alpha with every step a
// separate rounded f32 operation (no contraction into an FMA), input read through (row, column) element strides.
__global__ void addmm_finish_kernel(float *__restrict__ c, uint64_t ldc, const float *__restrict__ input, uint64_t in_rs,
                                    uint64_t in_cs, float alpha, float beta, uint64_t rows, uint64_t n) {
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * n; i += step) {
        const uint64_t r = i / n, j = i - r * n;
        float t = c[r * ldc + j];
        if (alpha != 1.0f) t = __fmul_rn(t, alpha);
        if (beta != 0.0f) {
            float base = __fadd_rn(0.0f, input[r * in_rs + j * in_cs]);
            if (beta != 1.0f) base = __fmul_rn(base, beta);
            t = __fadd_rn(base, t);
        }
        c[r * ldc + j] = t;
    }
}
int addmm_finish_launch(float *c, uint64_t ldc, const float *input, uint64_t in_rs, uint64_t in_cs, float alpha, float beta,
                        uint64_t rows, uint64_t n, cudaStream_t s) {
    if (!rows || !n || (alpha == 1.0f && beta == 0.0f)) return ST_OK;
    addmm_finish_kernel<<<grid_for(rows * n, 256), 256, 0, s>>>(c, ldc, input, in_rs, in_cs, alpha, beta, rows, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// im2col of picograd's pg_conv2d (ops/conv.c:92-113): col[b][row][j], row = (ci*kh + ki)*kw + kj, j = oh*OW + ow,
// zero where the window leaves the image.  One thread per element of col, j fastest (coalesced writes; reads
// run along a row of the image).
__global__ void im2col_kernel(const float *__restrict__ x, float *__restrict__ col, uint32_t cin, uint32_t h, uint32_t w,
                              uint32_t kh, uint32_t kw, uint32_t oh, uint32_t ow, int stride, int pad, uint64_t total) {
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t ncols = (uint64_t)oh * ow, krows = (uint64_t)cin * kh * kw;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const uint64_t j = i % ncols, t = i / ncols, row = t % krows, b = t / krows;
        const uint32_t o_h = (uint32_t)(j / ow), o_w = (uint32_t)(j % ow);
        const uint32_t kj = (uint32_t)(row % kw), ki = (uint32_t)((row / kw) % kh), ci = (uint32_t)(row / ((uint64_t)kw * kh));
        const long ih = (long)o_h * stride - pad + (long)ki, iw = (long)o_w * stride - pad + (long)kj;
        float v = 0.0f;
        if (ih >= 0 && ih < (long)h && iw >= 0 && iw < (long)w) v = x[((b * cin + ci) * h + (uint64_t)ih) * w + (uint64_t)iw];
        col[i] = v;
    }
}
int im2col_launch(const float *x, float *col, uint32_t batch, uint32_t cin, uint32_t h, uint32_t w, uint32_t kh, uint32_t kw,
                  uint32_t oh, uint32_t ow, int stride, int pad, cudaStream_t s) {
    const uint64_t total = (uint64_t)batch * cin * kh * kw * oh * ow;
    if (!total) return ST_OK;
    im2col_kernel<<<grid_for(total, 256), 256, 0, s>>>(x, col, cin, h, w, kh, kw, oh, ow, stride, pad, total);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}
// out[r][j] += bias[r % cout] over rows of `n` elements: the bias step of pg_conv2d (ops/conv.c:127-133)
__global__ void bias_rows_kernel(float *__restrict__ out, const float *__restrict__ bias, uint32_t cout, uint64_t n, uint64_t total) {
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
        out[i] += bias[(i / n) % cout];
}
int bias_rows_launch(float *out, const float *bias, uint32_t cout, uint64_t rows, uint64_t n, cudaStream_t s) {
    if (!rows || !n) return ST_OK;
    bias_rows_kernel<<<grid_for(rows * n, 256), 256, 0, s>>>(out, bias, cout, n, rows * n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// Bias and activation over a finished C (rows x n, leading dimension ldc), for the products whose
// tensor-core route cannot apply them in its own epilogue (K-slices, swapped operands): picograd's
// act_apply (backend/cpu/gemm.c:632-636) after the bias row of gemm.c:729-735.
__global__ void bias_act_kernel(float *__restrict__ c, uint64_t ldc, const float *__restrict__ bias, int act, int copy_only,
                                uint16_t *__restrict__ c16, uint64_t ld16, int dtype16, uint64_t rows, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * n; i += stride) {
        const uint64_t r = i / n, j = i - r * n;
        float x = c[r * ldc + j];
        if (bias) x += bias[j];
        float y = x;
        if (act == 1) y = x > 0.0f ? x : 0.0f;
        else if (act == 2) y = 0.5f * x * (1.0f + erff(x * 0.70710678118f));
        c[r * ldc + j] = copy_only ? x : y;
        if (c16) c16[r * ld16 + j] = to16(y, dtype16);
    }
}
int bias_act_launch(float *c, uint64_t ldc, const float *bias, int act, int act_copy_only, uint16_t *c16, uint64_t ld16,
                    int dtype16, uint64_t rows, uint64_t n, cudaStream_t s) {
    if (!rows || !n) return ST_OK;
    bias_act_kernel<<<grid_for(rows * n, 256), 256, 0, s>>>(c, ldc, bias, act, act_copy_only, c16, ld16, dtype16, rows, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// gy * (0.5 (1 + erf(x/sqrt 2)) + x phi(x))   (picograd autograd/autograd.c:794-801, :531-532)
__global__ void gelu_grad_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ out,
                                 uint64_t n, int vec) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t n4 = vec ? n / 4 : 0;
    for (uint64_t i = tid; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4 *>(x)[i];
        const float4 g = reinterpret_cast<const float4 *>(gy)[i];
        reinterpret_cast<float4 *>(out)[i] =
            make_float4(gelu_grad_f(v.x, g.x), gelu_grad_f(v.y, g.y), gelu_grad_f(v.z, g.z), gelu_grad_f(v.w, g.w));
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) out[i] = gelu_grad_f(x[i], gy[i]);
}
int gelu_grad_launch(const float *x, const float *gy, float *out, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    const int vec = (((uintptr_t)x | (uintptr_t)gy | (uintptr_t)out) & 15) == 0;
    gelu_grad_kernel<<<grid_for(vec ? n / 4 + 1 : n, 256), 256, 0, s>>>(x, gy, out, n, vec);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// The backward of an activation node folded into the split that feeds the next matmul node's backward:
// g' = gy * act'(x) (autograd/autograd.c:794-801 for GELU, :557 for ReLU) is cut into bf16 pieces as it is made and
// never stored as f32 (unless out32 is given).  Same arithmetic as gelu_grad_kernel followed by the split kernel.
// Layout of dst: [part][rows*cols padded to ld]: one "batch" of rows x cols with leading dimension ld_dst.
__global__ void act_grad_split_kernel(const float *__restrict__ x, const float *__restrict__ gy, int act,
                                      float *__restrict__ out32, unsigned short *__restrict__ dst, uint64_t ld_dst,
                                      uint32_t rows, uint32_t cols4, uint32_t nparts, uint32_t *mask) {
    const uint64_t total = (uint64_t)rows * cols4;
    const uint64_t part_stride = (uint64_t)rows * ld_dst;
    const uint64_t cols = (uint64_t)cols4 * 4;
    uint32_t seen = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / cols4, c = (i - r * cols4) * 4;
        const float4 v = *reinterpret_cast<const float4 *>(x + r * cols + c);
        const float4 g = *reinterpret_cast<const float4 *>(gy + r * cols + c);
        float4 y;
        if (act == 2) y = make_float4(gelu_grad_fast(v.x, g.x), gelu_grad_fast(v.y, g.y), gelu_grad_fast(v.z, g.z), gelu_grad_fast(v.w, g.w));
        else y = make_float4(v.x > 0.0f ? g.x : 0.0f, v.y > 0.0f ? g.y : 0.0f, v.z > 0.0f ? g.z : 0.0f, v.w > 0.0f ? g.w : 0.0f);
        if (out32) *reinterpret_cast<float4 *>(out32 + r * cols + c) = y;
        unsigned short h[3][4];
        split3(y.x, h[0][0], h[1][0], h[2][0]);
        split3(y.y, h[0][1], h[1][1], h[2][1]);
        split3(y.z, h[0][2], h[1][2], h[2][2]);
        split3(y.w, h[0][3], h[1][3], h[2][3]);
        unsigned short *d = dst + r * ld_dst + c;
        for (uint32_t p = 0; p < nparts; ++p) {
            uint2 w;
            w.x = (uint32_t)h[p][0] | ((uint32_t)h[p][1] << 16);
            w.y = (uint32_t)h[p][2] | ((uint32_t)h[p][3] << 16);
            *reinterpret_cast<uint2 *>(d + p * part_stride) = w;
            if ((w.x | w.y) & 0x7FFF7FFFu) seen |= 1u << p;
        }
    }
    publish_piece_mask(mask, seen);
}
// rows x cols contiguous f32 inputs, cols a multiple of 4, 16-byte aligned bases; ST_UNSUPPORTED otherwise
int act_grad_split_launch(const float *x, const float *gy, int act, float *out32, uint16_t *dst, uint64_t ld_dst,
                          uint32_t rows, uint32_t cols, uint32_t nparts, cudaStream_t s, uint32_t *mask) {
    if (!rows || !cols) return ST_OK;
    if ((act != 1 && act != 2) || cols % 4 || ld_dst % 4 || (((uintptr_t)x | (uintptr_t)gy | (uintptr_t)out32) & 15) ||
        ((uintptr_t)dst & 7))
        return ST_UNSUPPORTED;
    if (mask && cudaMemsetAsync(mask, 0, sizeof(uint32_t), s) != cudaSuccess) { cudaGetLastError(); return ST_GEMM; }
    act_grad_split_kernel<<<grid_for((uint64_t)rows * cols / 4, 256), 256, 0, s>>>(x, gy, act, out32, dst, ld_dst, rows, cols / 4,
                                                                                  nparts, mask);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}
// the same product as f32 only (no pieces): g' = gy * act'(x), for the routes that split per product
__global__ void act_grad_kernel(const float *__restrict__ x, const float *__restrict__ gy, int act, float *__restrict__ out,
                                uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = act == 2 ? gelu_grad_f(x[i], gy[i]) : (x[i] > 0.0f ? gy[i] : 0.0f);
}
int act_grad_launch(const float *x, const float *gy, int act, float *out, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    if (act != 1 && act != 2) return ST_UNSUPPORTED;
    act_grad_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, gy, act, out, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// One warp per row: max, sum of exp(x - max), normalise (picograd ops/activations.c:22-45).
// General form: three passes over the row (it stays in L1/L2 between them).
__global__ void softmax_rows_kernel(const float *__restrict__ src, float *__restrict__ d32,
                                    unsigned short *__restrict__ d16, int dtype16, uint64_t rows, uint32_t len) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t row = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const float *s = src + row * len;
        float mx = -INFINITY;
        for (uint32_t j = lane; j < len; j += 32) mx = fmaxf(mx, s[j]);
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
        for (uint32_t j = lane; j < len; j += 32) sum += expf(s[j] - mx);
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
        for (uint32_t j = lane; j < len; j += 32) {
            const float y = expf(s[j] - mx) * inv;
            if (d32) d32[row * len + j] = y;
            if (d16) d16[row * len + j] = to16(y, dtype16);
        }
    }
}

// Fast form: the row lives in registers (VEC float4 per lane, len == 128 * VEC), read once with
// 16-byte loads, exp evaluated once per element, written with 16-byte (f32) / 8-byte (16-bit) stores.
template <int VEC>
__global__ void __launch_bounds__(256) softmax_rows_reg_kernel(const float *__restrict__ src, float *__restrict__ d32,
                                                               unsigned short *__restrict__ d16, int dtype16,
                                                               uint64_t rows) {
    constexpr uint32_t LEN = 128 * VEC;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t row = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const float4 *s = reinterpret_cast<const float4 *>(src + row * LEN);
        float4 v[VEC];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            v[i] = s[lane + 32 * i];
            mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        }
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            v[i].x = expf(v[i].x - mx); v[i].y = expf(v[i].y - mx); v[i].z = expf(v[i].z - mx); v[i].w = expf(v[i].w - mx);
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float4 y = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
            if (d32) reinterpret_cast<float4 *>(d32 + row * LEN)[lane + 32 * i] = y;
            if (d16) {
                uint2 u;
                u.x = (uint32_t)to16(y.x, dtype16) | ((uint32_t)to16(y.y, dtype16) << 16);
                u.y = (uint32_t)to16(y.z, dtype16) | ((uint32_t)to16(y.w, dtype16) << 16);
                reinterpret_cast<uint2 *>(d16 + row * LEN)[lane + 32 * i] = u;
            }
        }
    }
}

int softmax_rows_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16, uint64_t rows, uint32_t len,
                        cudaStream_t s) {
    if (!rows || !len) return ST_OK;
    const bool aligned = (((uintptr_t)src | (uintptr_t)dst_f32) & 15) == 0 && ((uintptr_t)dst_16 & 7) == 0;
    const unsigned grid = grid_for(rows * 32, 256);
    if (aligned && len == 2048) softmax_rows_reg_kernel<16><<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows);
    else if (aligned && len == 1024) softmax_rows_reg_kernel<8><<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows);
    else if (aligned && len == 512) softmax_rows_reg_kernel<4><<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows);
    else if (aligned && len == 256) softmax_rows_reg_kernel<2><<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows);
    else if (aligned && len == 128) softmax_rows_reg_kernel<1><<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows);
    else softmax_rows_kernel<<<grid, 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows, len);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

__global__ void fill_f32_kernel(float *__restrict__ dst, float v, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = v;
}
int fill_f32_launch(float *dst, float v, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    fill_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(dst, v, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

}  // namespace pgb
