// Small HBM-bound helper kernels around the GEMMs: exact f32 -> bf16-pieces
// split (feeds the tensor cores with f32 data without rounding it), split-K
// reduction, gradient accumulation, and the element-wise harness steps of the
// attention-shaped and MLP workloads (softmax rows, GELU and its gradient,
// f32 -> 16-bit casts).  All are grid-stride / one-warp-per-row kernels with
// 16-byte accesses where alignment allows.

#include "pg_internal.h"

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
__global__ void split_f32_kernel(const float *__restrict__ src, uint64_t ld_src, uint64_t src_bs,
                                 unsigned short *__restrict__ dst, uint64_t ld_dst, uint32_t rows, uint32_t cols,
                                 uint32_t batch, uint32_t nparts) {
    const uint64_t per_batch = (uint64_t)rows * cols;
    const uint64_t total = per_batch * batch;
    const uint64_t part_stride = (uint64_t)rows * ld_dst;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i / per_batch;
        const uint64_t r = (i - b * per_batch) / cols;
        const uint64_t c = i - b * per_batch - r * cols;
        float x = src[b * src_bs + r * ld_src + c];
        unsigned short *d = dst + b * nparts * part_stride + r * ld_dst + c;
        unsigned short h0 = bf16_rne(x);
        d[0] = h0;
        float r1 = x - bf16_up(h0);
        unsigned short h1 = bf16_rne(r1);
        d[part_stride] = h1;
        if (nparts > 2) {
            float r2 = r1 - bf16_up(h1);
            d[2 * part_stride] = bf16_rne(r2);
        }
    }
}

int split_f32_to_bf16_launch(const float *src, uint64_t ld_src, uint64_t src_bs, uint16_t *dst, uint64_t ld_dst,
                             uint32_t rows, uint32_t cols, uint32_t batch, uint32_t nparts, cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * cols * batch;
    if (!total) return ST_OK;
    split_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, ld_src, src_bs, dst, ld_dst, rows, cols, batch, nparts);
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

// 0.5 x (1 + erf(x / sqrt 2))   (picograd ops/activations.c:114)
__global__ void gelu_kernel(const float *__restrict__ src, float *__restrict__ d32, unsigned short *__restrict__ d16,
                            int dtype16, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float x = src[i];
        const float y = 0.5f * x * (1.0f + erff(x * 0.70710678118f));
        if (d32) d32[i] = y;
        if (d16) d16[i] = to16(y, dtype16);
    }
}
int gelu_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    gelu_kernel<<<grid_for(n, 256), 256, 0, s>>>(src, dst_f32, dst_16, dtype16, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// gy * (0.5 (1 + erf(x/sqrt 2)) + x phi(x))   (picograd autograd/autograd.c:794-801, :531-532)
__global__ void gelu_grad_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ out,
                                 uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        const float e = erff(v * 0.70710678118f);
        const float phi = expf(-0.5f * v * v) / 2.50662827463f;
        out[i] = gy[i] * (0.5f * (1.0f + e) + v * phi);
    }
}
int gelu_grad_launch(const float *x, const float *gy, float *out, uint64_t n, cudaStream_t s) {
    if (!n) return ST_OK;
    gelu_grad_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, gy, out, n);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// One warp per row: max, sum of exp(x - max), normalise (picograd ops/activations.c:22-45).
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
int softmax_rows_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16, uint64_t rows, uint32_t len,
                        cudaStream_t s) {
    if (!rows || !len) return ST_OK;
    softmax_rows_kernel<<<grid_for(rows * 32, 256), 256, 0, s>>>(src, dst_f32, dst_16, dtype16, rows, len);
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
