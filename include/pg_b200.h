/* pg_b200.h — C-ABI of libpg_b200.so, the B200 (sm_100a) device side of
 * picograd's dense matrix-multiply path.
 *
 * The library is what picograd's CUDA seat (src/backend/cuda/cuda.c) would bind
 * instead of its embedded sm_75 PTX: every entry below names the picograd
 * interface it stands behind.  Plain C types only; pointers called "device"
 * come from pg_b200_malloc (or any CUDA allocation of the current device).
 * Matrices are row-major, leading dimensions are in ELEMENTS, C is always f32
 * and is overwritten (no alpha/beta), exactly as in backend/backend.h:103-136.
 *
 * Status codes are picograd's pg_status (backend/backend.h:25-32):
 *   0 OK, -1 UNSUPPORTED, -2 ALLOC, -3 COPY, -4 SYNC, -5 GEMM.
 * Kernel launches are asynchronous on the library's stream; asynchronous
 * failures (a kernel wait that gave up) surface at pg_b200_sync().
 * The library is not thread-safe, like the backend it replaces
 * (backend/backend.c:50, backend/cuda/cuda.c:32-33).
 */
#ifndef PG_B200_H
#define PG_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PG_B200_API __attribute__((visibility("default")))
#else
#define PG_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* pg_dtype (core/dtype.h:11-16) */
#define PG_B200_F32 0
#define PG_B200_F16 1
#define PG_B200_BF16 2

/* ---- vtable entries of pg_backend_ops (backend/backend_i.h:8-34) ---------- */

/* .init — cuda.c:30-105.  Binds the calling thread to a B200 (ordinal from
 * pg_b200_set_device, default 0), creates the library's state.  Returns
 * UNSUPPORTED when no sm_100 device or driver is present. */
PG_B200_API int pg_b200_init(void);
/* .malloc / .free — cuda.c:107-121 */
PG_B200_API void *pg_b200_malloc(size_t nbytes);
PG_B200_API void pg_b200_free(void *p);
/* .copy_h2d / .copy_d2h — cuda.c:123-141 (synchronous, like cuMemcpyHtoD) */
PG_B200_API int pg_b200_copy_h2d(void *dst, const void *src, size_t nbytes);
PG_B200_API int pg_b200_copy_d2h(void *dst, const void *src, size_t nbytes);
/* .sync — cuda.c:143-148; also reports kernel-side wait failures as GEMM */
PG_B200_API int pg_b200_sync(void);
/* .gemm — cuda.c:150-174: f32 C = A*B, device pointers, any lda/ldb/ldc
 * (picograd's kernel silently returns unless lda==k, ldb==n, ldc==n). */
PG_B200_API void pg_b200_gemm(size_t m, size_t n, size_t k, const float *a, size_t lda,
                  const float *b, size_t ldb, float *c, size_t ldc);
/* .hgemm / .bgemm — NULL in picograd's CUDA seat (cuda.c:282-291) */
PG_B200_API void pg_b200_hgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda,
                   const uint16_t *b, size_t ldb, float *c, size_t ldc);
PG_B200_API void pg_b200_bgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda,
                   const uint16_t *b, size_t ldb, float *c, size_t ldc);
/* .gemm_ex — backend.c:150-177.  Accepts device pointers, or host pointers
 * (what ops/matmul.c:264-271 passes for f16/bf16), which are staged through
 * device memory inside the call: H2D, GEMM, D2H, synchronous.  All three
 * pointers must be of the same kind. */
PG_B200_API int pg_b200_gemm_ex(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                    const void *b, size_t ldb, float *c, size_t ldc);

/* ---- fused epilogues: backend/cpu/gemm.c:632-817, used by nn/nn.c:60,85 ------ */

/* pg_act of backend/cpu/gemm.h */
#define PG_B200_ACT_NONE 0
#define PG_B200_ACT_RELU 1
#define PG_B200_ACT_GELU 2   /* 0.5 x (1 + erf(x / sqrt 2)) */
/* OR-ed into `act` of pg_b200_gemm_fused_out16: the activation goes into the 16-bit copy only and C keeps
 * bias + A*B — what a training step wants from the first layer of an MLP: the pre-activation in f32 for the
 * backward pass (autograd.c:794-801 reads it) and the activated value in 16 bits for the next GEMM. */
#define PG_B200_ACT_COPY_ONLY 0x100

/* pg_cpu_gemm_fused_ex (gemm.c:806-817): C = act(bias[j] + A*B), bias of n floats or NULL.
 * In picograd each row of C starts as the bias row and the micro-kernels accumulate onto it, so
 * the sum of column j is a chain that STARTS at bias[j]; the FFMA path here does the same and
 * agrees bit for bit for ACT_NONE and ACT_RELU (ACT_GELU to the last bits of erff); the
 * tensor-core path adds the bias to the finished f32 sum.  Either way bias and activation are
 * applied in the GEMM kernel's own epilogue, on the accumulators, before C is written once.
 * Device pointers (bias too), or host pointers throughout, staged like pg_b200_gemm_ex. */
PG_B200_API int pg_b200_gemm_fused_ex(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                          const void *b, size_t ldb, float *c, size_t ldc, const float *bias, int act);
/* pg_cpu_gemm_fused (gemm.c:685-716): the f32 form; void like the entry it replaces, errors are
 * kept for pg_b200_last_error() and pg_b200_sync(). */
PG_B200_API void pg_b200_gemm_fused(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b,
                        size_t ldb, float *c, size_t ldc, const float *bias, int act);
/* No counterpart in picograd, where the next layer re-reads the f32 C and converts it
 * (ops/cast.c): the same call also writes C rounded to f16/bf16 (round-to-nearest-even) into
 * c16 (m x n, leading dimension ldc16 elements), so that a 16-bit consumer reads 2 bytes per
 * element instead of 4 and no cast kernel runs.  Device pointers only. */
PG_B200_API int pg_b200_gemm_fused_out16(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                             const void *b, size_t ldb, float *c, size_t ldc, const float *bias, int act,
                             uint16_t *c16, size_t ldc16, int dtype16);

/* ---- the callers' shapes: ops/matmul.c and autograd/autograd.c ------------- */

/* General strided-batched product behind pg_matmul / pg_bmm / pg_tensordot
 * (ops/matmul.c:186-284, :340-369, :407-490) and the two products of
 * bwd_matmul (autograd/autograd.c:659-691).  Device pointers.
 *   C[b] (f32, m x n) = op(A[b]) * op(B[b]),  b = 0..batch-1
 *   trans_a = 0: A[b] is m x k with leading dimension lda; 1: A[b] is stored k x m
 *   trans_b = 0: B[b] is k x n with leading dimension ldb; 1: B[b] is stored n x k
 *   dtype_a / dtype_b: a 16-bit operand may be paired with an f32 one (the f32
 *   gradient of the backward pass); the f32 side is then split exactly into
 *   bf16 pieces on the device, never rounded to one.
 *   stride_* are element offsets between consecutive batch elements (0 =
 *   operand shared by the whole batch).  accumulate != 0: C += (used for grads). */
PG_B200_API int pg_b200_gemm_batched(int dtype_a, int dtype_b, int trans_a, int trans_b,
                         size_t batch, size_t m, size_t n, size_t k,
                         const void *a, size_t lda, size_t stride_a,
                         const void *b, size_t ldb, size_t stride_b,
                         float *c, size_t ldc, size_t stride_c, int accumulate);

/* A column shard of C written into the full C of several devices by the GEMM kernel itself (no counterpart in
 * picograd, which has one device).  The product is pg_b200_gemm_ex's: C_shard (m x n, f32) = A (m x k) * B (k x n);
 * every tile of it is stored to dst[i] + col0 for i = 0 .. n_dst-1, each dst[i] the base of a row-major m x ldc
 * f32 matrix: this device's own full C and, typically, the other devices' full C mapped into this process
 * (pg_b200_ipc_open).  After every rank of an N-column-sharded product has made this call and the ranks have met
 * (stream synchronisation on each, then a barrier among the processes), every device holds all of C in row-major
 * order: no all-gather, no re-layout pass, and the transfer over NVLink overlaps the product tile by tile.
 * f16 / bf16 only; 1 to 8 destinations; col0, n and ldc multiples of 4, destinations 16-byte aligned (dst[0] is
 * written with TMA bulk stores, the others with 16-byte stores from the same staged chunks: put the local matrix
 * first); PG_ERR_UNSUPPORTED otherwise — the caller then gathers with NCCL.  The kernel only stores to the other
 * devices and waits for none of them. */
PG_B200_API int pg_b200_gemm_ex_scatter(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                                        const void *b, size_t ldb, float *const *dst, size_t n_dst, size_t ldc,
                                        size_t col0);
/* One process per GPU: handle of a pg_b200_malloc allocation for another process (cudaIpcGetMemHandle, 64
 * bytes), and the mapping of such a handle into this process with peer access enabled (cudaIpcOpenMemHandle).
 * pg_b200_ipc_close unmaps; the owner frees its allocation only after every process has closed it. */
PG_B200_API int pg_b200_ipc_export(const void *dev_ptr, unsigned char handle[64]);
PG_B200_API int pg_b200_ipc_open(const unsigned char handle[64], void **dev_ptr);
PG_B200_API int pg_b200_ipc_close(void *dev_ptr);

/* pg_addmm (ops/matmul.c:371-405): c = beta * input + alpha * (a * b).  a [m,k], b [k,n] in `dtype`; c f32 [m,n];
 * input f32 read at input[i * in_row_stride + j * in_col_stride] (strides in elements, 0 = broadcast along that
 * dimension, so [m,n], [n], [m,1] and scalars all fit).  The product is pg_matmul's; the tail is one kernel that
 * rounds after every step as picograd's separate scale and add passes do (same bits for f32).  Device pointers. */
PG_B200_API int pg_b200_addmm(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                  float *c, size_t ldc, const float *input, size_t in_row_stride, size_t in_col_stride,
                  float alpha, float beta);

/* permute_copy of pg_tensordot (ops/matmul.c:21-42): dst (contiguous, dimension d of size shape[perm[d]])
 * receives src (contiguous, `shape`) with its dimensions reordered; dtype gives the element size.  Device
 * pointers, ndim <= 8 (picograd's PG_MAX_NDIM).  pg_tensordot is this on both operands, then pg_matmul. */
PG_B200_API int pg_b200_permute_copy(int dtype, size_t ndim, const size_t *shape, const size_t *perm,
                         const void *src, void *dst);

/* bwd_matmul (autograd/autograd.c:561-706) for a [batch,m,k] x [batch,k,n]
 * (or shared [k,n] when b_batched == 0) product: ga += g * B^T, gb += A^T * g.
 * a, b in `dtype`; g, ga, gb f32; ga / gb may be NULL. Device pointers. */
PG_B200_API int pg_b200_matmul_backward(int dtype, size_t batch, size_t m, size_t n, size_t k,
                            const void *a, const void *b, int b_batched,
                            const float *g, float *ga, float *gb);

/* pg_conv2d (ops/conv.c:10-146, ops/conv.h:27-33): NCHW 2-D convolution, f32.  x [n,cin,h,w], wt [cout,cin,kh,kw],
 * bias [cout] or NULL -> out [n,cout,oh,ow] with oh = (h + 2 padding - kh) / stride + 1 (likewise ow).  Device
 * pointers.  Same algorithm as picograd: im2col (rows in (ci,ki,kj) order, zeros outside the image) on the
 * device, one f32 GEMM per batch element through the FFMA kernels (one fused multiply-add chain per output,
 * zeros included, so results equal picograd's bit for bit), then the bias.  UNSUPPORTED for the shapes
 * pg_conv2d returns NULL for (stride <= 0, window larger than the padded image). */
PG_B200_API int pg_b200_conv2d(size_t n, size_t cin, size_t h, size_t w, size_t cout, size_t kh, size_t kw,
                   int stride, int padding, const float *x, const float *wt, const float *bias, float *out);

/* The attention-shaped chain of picograd calls as ONE entry: O = 16bit(softmax_rows(Q * Kt)) * V, i.e.
 * pg_bmm (ops/matmul.c:340-369) -> pg_softmax over the last axis (ops/activations.c:22-45) -> cast to the
 * operand dtype -> pg_bmm.  q [batch, seq_q, d], kt [batch, d, seq_k], v [batch, seq_k, d] in `dtype`
 * (f16/bf16), contiguous, device pointers; o [batch, seq_q, d] f32.  No scaling and no mask: the chain has
 * none.  For d == 128 and 16-byte aligned operands one kernel does all of it and the f32 scores and the
 * 16-bit probabilities never reach device memory (P is still rounded to 16 bits after the division by the
 * row sum, as the chain does, so the result equals the chain's to rounding noise); other shapes run the
 * chain with the library's own kernels.  pg_b200_last_path() says which ("attn:fused_128x128" / "attn:chain"). */
PG_B200_API int pg_b200_attention_bmm(int dtype, size_t batch, size_t seq_q, size_t seq_k, size_t d,
                          const void *q, const void *kt, const void *v, float *o);

/* The same with accumulate == 0: ga = g * B^T, gb = A^T * g (overwrite).  For gradients that were just created:
 * picograd zeroes them (autograd.c:2490-2492) and adds; overwriting saves the zero fill and the read of the
 * old values, with the same result. */
PG_B200_API int pg_b200_matmul_backward_ex(int dtype, size_t batch, size_t m, size_t n, size_t k,
                               const void *a, const void *b, int b_batched,
                               const float *g, float *ga, float *gb, int accumulate);

/* The same with the backward of an activation node folded in (no counterpart as one call in picograd, whose
 * autograd runs bwd_gelu / bwd_relu, autograd.c:794-801 / :557, as a pass of its own before bwd_matmul): the
 * gradient that enters the products is g' = g * act'(act_input), act = PG_ACT_RELU or PG_ACT_GELU, act_input f32 of
 * g's shape [batch*m, n].  On the tensor-core route g' is cut into its bf16 pieces as it is computed and never
 * written as f32; pass gr_pre (f32, g's shape) to receive it as well, or NULL.  act == 0: plain
 * pg_b200_matmul_backward_ex. */
PG_B200_API int pg_b200_matmul_backward_act(int dtype, size_t batch, size_t m, size_t n, size_t k,
                                const void *a, const void *b, int b_batched, const float *g, int act,
                                const float *act_input, float *gr_pre, float *ga, float *gb, int accumulate);

/* Harness steps between the GEMMs of the attention-shaped and MLP workloads
 * (ops/activations.c:22-45 softmax rows, :114 GELU, autograd.c:794-801 GELU
 * gradient), so that those workloads stay on the device.  out16 (optional)
 * receives the result rounded to dtype16 (f16/bf16, round-to-nearest-even). */
PG_B200_API int pg_b200_softmax_rows(const float *src, float *out_f32, uint16_t *out16, int dtype16,
                         size_t rows, size_t len);
PG_B200_API int pg_b200_gelu(const float *src, float *out_f32, uint16_t *out16, int dtype16, size_t n);
PG_B200_API int pg_b200_gelu_grad(const float *x, const float *gy, float *out, size_t n);
PG_B200_API int pg_b200_cast_f32(const float *src, uint16_t *dst, int dtype16, size_t n);
PG_B200_API int pg_b200_fill_f32(float *dst, float value, size_t n);

/* ---- picograd's tensor-level callers, device-resident ------------------------ */

/* What the callers read of a pg_tensor (core/tensor.h:21-36), with a DEVICE data pointer.  Strides in elements. */
#define PG_B200_MAX_NDIM 8      /* PG_MAX_NDIM */
typedef struct pg_b200_tensor {
    int dtype;                          /* PG_DTYPE_* */
    size_t ndim;                        /* 1 .. 8 */
    size_t shape[PG_B200_MAX_NDIM];
    size_t stride[PG_B200_MAX_NDIM];
    void *data;
} pg_b200_tensor;

/* pg_matmul (ops/matmul.c:186-284), pg_bmm (:340-369), pg_tensordot (:407-490) with picograd's shape rules applied
 * in this library: 1-D operands promoted to a row / a column, batch dimensions equal or absent on one side, any
 * batch strides (picograd's odometer), operand dtypes equal, last-dimension stride 1; result always f32, of
 * picograd's result shape.  `out`: set out->data = NULL to have the result allocated with pg_b200_malloc (free it
 * with pg_b200_free), or point it at a contiguous f32 buffer of the result's size; dtype / ndim / shape / stride are
 * filled in either way.  PG_ERR_UNSUPPORTED where picograd returns NULL (reason in pg_b200_last_error()); one rule
 * is stricter: a 1-D b must have as many elements as a's last dimension (picograd does not check).  pg_bmm takes
 * contiguous operands, as picograd assumes. */
PG_B200_API int pg_b200_matmul(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out);
PG_B200_API int pg_b200_bmm(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out);
/* The shape rules alone: fill dtype / ndim / shape / stride of the result (or refuse) without touching any data,
 * for a caller that allocates the result itself before the call proper. */
PG_B200_API int pg_b200_matmul_result_shape(const pg_b200_tensor *a, const pg_b200_tensor *b, pg_b200_tensor *out);
PG_B200_API int pg_b200_tensordot_result_shape(const pg_b200_tensor *a, const pg_b200_tensor *b, size_t ndims,
                                               const size_t *axes_a, const size_t *axes_b, pg_b200_tensor *out);
PG_B200_API int pg_b200_tensordot(const pg_b200_tensor *a, const pg_b200_tensor *b, size_t ndims, const size_t *axes_a,
                                  const size_t *axes_b, pg_b200_tensor *out);
/* bwd_matmul (autograd/autograd.c:561-706) with the same operand shapes as pg_b200_matmul: grad_out has the shape
 * of the matmul's result; grad_a / grad_b (either may be NULL) have the shapes of a / b, f32, contiguous.  A
 * gradient shared by the batch (b 2-D under a batched a, or a 2-D under a batched b) sums over the batch.
 * accumulate != 0: grad += product (picograd's form); 0: the gradients are overwritten. */
PG_B200_API int pg_b200_matmul_backward_nd(const pg_b200_tensor *a, const pg_b200_tensor *b, const float *grad_out,
                                           float *grad_a, float *grad_b, int accumulate);

/* ---- more than one GPU ------------------------------------------------------- */

/* No counterpart in picograd (one device only, backend/cuda/cuda.c:49-55).  pg_gemm_ex is partitioned over the GPUs
 * of a node by N-column shards of B and C, and a caller that wants the whole C on one device all-gathers the shards
 * (NCCL).  An all-gather delivers shard g as a contiguous row-major [rows][width] block at staging + g*rows*width;
 * this kernel writes the row-major [rows][n] matrix (leading dimension ld) whose columns [g*width, (g+1)*width),
 * clipped at n, are shard g.  Device pointers; HBM-bound (each element read once, written once). */
PG_B200_API int pg_b200_gather_relayout(const float *staging, float *dst, size_t shards, size_t rows, size_t width,
                                        size_t n, size_t ld);

/* ---- for callers that must not allocate ------------------------------------- */

/* No counterpart in picograd.  pg_gemm_ex for f16/bf16 through the split-K tensor-core path, with
 * the K-slices kept in a fixed array inside the library image instead of a cudaMalloc'ed buffer, so
 * that the call allocates nothing (no cudaMalloc / cudaFree / cudaMallocHost, directly or through a
 * library, on the first call or later).  For code that runs where the allocator is off limits: a
 * service whose arena already owns all free HBM, a loop that may not take the allocator's lock or the
 * device-wide synchronisation an allocation implies, a plugin forbidden to allocate after start-up.
 *   - Device pointers only; a, b 16-byte aligned, lda and ldb multiples of 8 elements, K > 64.
 *   - k_splits: number of K slices (0 = choose, always >= 2).  k_splits * m * round_up(n,4) * 4
 *     bytes must fit in PG_B200_STATIC_SCRATCH_BYTES, else PG_ERR_UNSUPPORTED with the sizes in
 *     pg_b200_last_error().
 *   - The array costs PG_B200_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the
 *     library, until the process exits.  All calls share it: calls whose kernels overlap on the GPU
 *     (other streams, other threads) race; calls on one stream are ordered.
 *   - The first call on a device resolves the array's device address and sets kernel attributes;
 *     make that call before any stream capture begins.  It is also the call at which the driver
 *     loads this library's kernels and the array into device memory (lazy module loading): a
 *     one-time reservation of the array plus a few MiB of code, so make it at start-up, before your
 *     arena takes the remaining memory.  Later calls leave free device memory unchanged.
 *   - One caller thread, like the rest of this library (the per-device set-up is not locked).
 *   - The call synchronises its stream before returning, so a kernel-side failure is returned as
 *     PG_ERR_GEMM by the call itself. */
#define PG_B200_STATIC_SCRATCH_BYTES (16u << 20)
PG_B200_API int pg_b200_gemm_ex_static_scratch(int dtype, size_t m, size_t n, size_t k,
                                               const void *a, size_t lda, const void *b, size_t ldb,
                                               float *c, size_t ldc, int k_splits);

/* ---- control ---------------------------------------------------------------- */

/* Device ordinal used by pg_b200_init (picograd uses device 0, cuda.c:49). */
PG_B200_API int pg_b200_set_device(int ordinal);
/* Run the library's kernels and copies on this CUDA stream (a cudaStream_t /
 * CUstream handle; NULL = the default stream).  Calls are stream-ordered: the library keeps ONE scratch
 * buffer, one set of arrival counters, one set of staging buffers and one status word per process, so two
 * calls in flight on different streams would share them and return wrong sums.  Switch streams only after
 * the previous stream's work has been synchronised; one caller thread, like picograd (backend.c:50). */
PG_B200_API int pg_b200_set_stream(void *stream);
/* Text of the last error recorded by this library ("" if none). */
PG_B200_API const char *pg_b200_last_error(void);
/* Tuning / test hooks: kernel path 0 = choose, 1 = tensor-core kernel only
 * (UNSUPPORTED if it cannot take the shape), 2 = FFMA kernel only;
 * tile configuration index (-1 = choose) and its name; epilogue -1 = choose,
 * 0 = direct stores, 1 = TMA stores; K splits 0 = choose.
 * Two options change results within the stated tolerance:
 *   "k_serpentine" (default 1): large products sum K upwards in a CTA's even-numbered tiles and downwards
 *     in its odd-numbered ones (fewer DRAM reads).  Deterministic for a shape; set 0 when results must be
 *     bit-identical across shapes, shards or tile configurations (every element then sums K ascending).
 *   "f32_tensor_cores" (default 0): f32 x f32 as three exact bf16 pieces per operand on the tensor cores,
 *     K accumulated in chunks of "f32_chunk" (default 512; 0 = one accumulation) that are added to C in f32.
 *     Closer to the exact product than one f32 chain, hence not bit-identical to picograd's CPU result. */
PG_B200_API int pg_b200_set_option(const char *name, int value);
PG_B200_API int pg_b200_num_tile_configs(void);
PG_B200_API const char *pg_b200_tile_config_name(int index);
/* Failure-detection self-test (no counterpart in picograd, whose launch failure is an assert,
 * cuda.c:173): launches a kernel that waits on a barrier nothing completes, with the bounded wait the
 * GEMM kernels use and a limit of `limit_ms` (<= 1000).  The kernel returns normally after the limit
 * and the NEXT pg_b200_sync() reports PG_ERR_GEMM; the device stays usable. */
PG_B200_API int pg_b200_selftest_wait_timeout(unsigned limit_ms);
/* Diagnostics of the timing experiments (option "debug" bit 32): copies per-CTA cycle counters
 * of the last tensor-core launch, 16 per CTA, to `out`. */
PG_B200_API int pg_b200_debug_counters(uint64_t *out, size_t count);
/* Test hook (host arithmetic only, needs no GPU): how the tensor-core kernel deals the K ranges of a partly filled
 * last wave out to all SMs.  `tiles` output tiles of `k_blocks` 64-deep K blocks on `slots` resident CTA pairs;
 * part (0, 1) of CTA pair `cluster`.  out = {1 if the balanced schedule is used, whole-tile waves, index of the tail
 * tile, first K block, number of K blocks (0 = no such part), role (1 = first slice: stored, 2 = second slice: added)}. */
PG_B200_API int pg_b200_debug_tail_schedule(uint64_t tiles, unsigned slots, unsigned k_blocks, unsigned cluster,
                                            unsigned part, unsigned out[6]);
/* Test hook (host arithmetic only, needs no GPU): the i-th output tile that CTA pair `id` of `count` takes in a
 * product of m_tiles x n_tiles tiles walked in rasterisation groups of `group_m` M tiles, by the function the
 * kernel's roles call.  die_aware: the pair is number `id` of `count` on die `die` and walks that die's half of every
 * group; serpentine: odd groups walk N downwards; k_serpentine: a pair's odd-numbered tiles fetch their K blocks last
 * to first.  out = {1 if there is such a tile, M tile, N tile, 1 if K runs downwards}. */
PG_B200_API int pg_b200_debug_walk(unsigned m_tiles, unsigned n_tiles, unsigned group_m, unsigned k_blocks,
                                   unsigned die_aware, unsigned serpentine, unsigned k_serpentine, unsigned die,
                                   unsigned id, unsigned count, unsigned i, unsigned out[4]);
/* Diagnostic: the table smid -> die (0 / 1) that pg_b200_init measured on this GPU (L2 hit latency from every SM to
 * one address: the SMs of the die that holds the line answer ~70 cycles sooner) and that the die-aware tile walk of
 * the tensor-core GEMM uses; up to 256 entries.  PG_ERR_UNSUPPORTED when the SMs did not fall into two clean groups
 * (the GEMM then walks its tiles without regard to the dies). */
PG_B200_API int pg_b200_die_table(unsigned char *out, size_t count);
/* Number of kernels this library has launched since it was loaded. */
PG_B200_API uint64_t pg_b200_launch_count(void);
/* Name of the path the last GEMM call took ("tc:2cta_256x256", "simt", ...). */
PG_B200_API const char *pg_b200_last_path(void);

#ifdef __cplusplus
}
#endif
#endif
