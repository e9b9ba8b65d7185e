// pg_b200_gemm_ex_static_scratch: the split-K tensor-core GEMM for callers that must not allocate.
//
// Who that is: code that runs where the CUDA allocator is off limits — a service that has handed
// every free byte of HBM to its own arena, a control loop that may not take the allocator's lock or
// the device-wide synchronisation cudaMalloc and cudaFree imply, a plugin whose host forbids
// allocation after start-up.  The regular entry points grow a scratch buffer with cudaMalloc when a
// shape needs split-K; this one keeps the K-slices in a fixed array that is part of the library
// image, so it calls no cudaMalloc, cudaFree, cudaMallocHost or allocating library routine on any
// path.  What the first call on a device does cost: with CUDA's lazy module loading that call is when
// the driver places this library's kernels and the array itself in device memory (a one-time
// reservation the driver makes, not an allocator call), so it belongs at start-up, before an arena
// takes the remaining memory; every later call leaves free memory untouched.
//
// The price: the array is PG_B200_STATIC_SCRATCH_BYTES (16 MiB) of device memory on every GPU that
// loads the library, held until the process exits, and it is shared by all calls — two calls whose
// kernels overlap on the GPU (different streams, different host threads) race on it.  Calls on one
// stream are ordered and safe.  Like the rest of the library it expects one caller thread: the
// per-device set-up below is not guarded against two threads running it at once.

#include "../../include/pg_b200.h"
#include "pg_internal.h"

namespace pgb {

constexpr size_t STATIC_SCRATCH_BYTES = PG_B200_STATIC_SCRATCH_BYTES;

// K-slices of the product, [split][M][ld] f32.  In host code this name is only a handle for the
// runtime's symbol table, never a device address: the address is fetched once per device below.
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_BYTES / sizeof(float)];
// Wait-failure bits of the kernels launched from here (the regular status word is cudaMalloc'ed).
static __device__ __align__(256) uint32_t g_static_status[64];

struct StaticScratch {
    float *slices = nullptr;
    uint32_t *status = nullptr;
};
static StaticScratch g_dev[64];   // per device ordinal

// Set-up for the CURRENT device, done by the first call on that device: resolves the device
// addresses of the two arrays and clears the status word.  Allocates nothing.
static int setup_current_device(StaticScratch **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        set_error("static-scratch GEMM: no usable current device");
        return ST_UNSUPPORTED;
    }
    StaticScratch &s = g_dev[dev];
    if (!s.slices) {
        void *p_slices = nullptr, *p_status = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p_slices, g_static_scratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&p_status, g_static_status);
        if (e != cudaSuccess || !p_slices || !p_status) {
            set_error("static-scratch GEMM: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            cudaGetLastError();
            return ST_GEMM;
        }
        e = cudaMemsetAsync(p_status, 0, sizeof(uint32_t) * 64, current_stream());
        if (e != cudaSuccess) {
            set_error("static-scratch GEMM: clearing the status word failed: %s", cudaGetErrorString(e));
            cudaGetLastError();
            return ST_GEMM;
        }
        s.status = (uint32_t *)p_status;      // slices last: it is the "set-up done" mark
        s.slices = (float *)p_slices;
    }
    *out = &s;
    return ST_OK;
}

}  // namespace pgb

using namespace pgb;

extern "C" int pg_b200_gemm_ex_static_scratch(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda,
                                              const void *b, size_t ldb, float *c, size_t ldc, int k_splits) {
    if (dtype != DT_F16 && dtype != DT_BF16) {
        set_error("static-scratch GEMM: dtype must be f16 or bf16");
        return ST_UNSUPPORTED;
    }
    if (m == 0 || n == 0) return ST_OK;
    if (!a || !b || !c || k == 0) {
        set_error("static-scratch GEMM: null operand or k == 0");
        return ST_UNSUPPORTED;
    }
    if (m > 0x7FFFFFFFull || n > 0x7FFFFFFFull || k > 0x7FFFFFFFull) return ST_UNSUPPORTED;
    int st = ensure_device_info();
    if (st != ST_OK) return st;
    StaticScratch *ss = nullptr;
    st = setup_current_device(&ss);
    if (st != ST_OK) return st;

    // K slices: at least two (this entry point exists for the split-K path), at most one per K block
    const uint32_t k_blocks = (uint32_t)((k + 63) / 64);
    if (k_blocks < 2) {
        set_error("static-scratch GEMM: K = %zu has a single 64-deep block, nothing to split", k);
        return ST_UNSUPPORTED;
    }
    uint32_t splits;
    if (k_splits > 0) {
        splits = (uint32_t)k_splits;
    } else {
        const uint64_t tiles = ((m + 127) / 128) * ((n + 127) / 128);
        const uint64_t want = (uint64_t)device_sm_count() / (tiles ? tiles : 1);
        splits = (uint32_t)(want < 2 ? 2 : (want > 16 ? 16 : want));
    }
    if (splits < 2) splits = 2;
    if (splits > k_blocks) splits = k_blocks;
    const uint32_t per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;                      // no empty slice
    const size_t ws_ld = (n + 3) / 4 * 4;
    const size_t need = (size_t)splits * m * ws_ld * sizeof(float);
    if (need > STATIC_SCRATCH_BYTES) {
        set_error("static-scratch GEMM: %u K-slices of %zu x %zu need %zu bytes of scratch, the static array holds %zu; "
                  "use fewer slices, a smaller product, or pg_b200_gemm_ex",
                  splits, m, n, need, STATIC_SCRATCH_BYTES);
        return ST_UNSUPPORTED;
    }

    TcGemm t = {};
    t.dtype = dtype;
    t.M = (uint32_t)m; t.N = (uint32_t)n; t.K = (uint32_t)k; t.batch = 1;
    t.A.ptr = a; t.A.ld = lda; t.A.z_stride = 0; t.A.nparts = 1; t.A.mn_major = 0;
    t.B.ptr = b; t.B.ld = ldb; t.B.z_stride = 0; t.B.nparts = 1; t.B.mn_major = 1;
    t.npass = 1;
    t.C = ss->slices; t.ldc = ws_ld; t.c_stride = m * ws_ld;   // every element the reduction reads is written
    t.accumulate = 0;
    t.splits = splits;
    t.force_cfg = -1; t.force_epilogue = -1;
    t.pdl = 0;
    t.stream = current_stream();
    t.dev_status = ss->status;
    t.prof = nullptr;
    if (!tc_gemm_supported(t)) {
        set_error("static-scratch GEMM: operands must be 16-byte aligned with lda, ldb multiples of 8 elements");
        return ST_UNSUPPORTED;
    }
    st = tc_gemm_launch(t);
    if (st != ST_OK) return st;
    st = reduce_splits_launch(ss->slices, m * ws_ld, splits, c, ldc, (uint32_t)m, (uint32_t)n, ws_ld, 0, t.stream);
    if (st != ST_OK) return st;

    // Report a kernel-side wait failure now: the status word lives in static device memory, which
    // pg_b200_sync() does not read.  This makes the call synchronous on its stream.
    uint32_t bits = 0;
    cudaError_t e = cudaMemcpyAsync(&bits, ss->status, sizeof bits, cudaMemcpyDeviceToHost, t.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(t.stream);
    if (e != cudaSuccess) {
        set_error("static-scratch GEMM: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return ST_SYNC;
    }
    if (bits) {
        set_error("static-scratch GEMM: a kernel gave up waiting (status bits 0x%x)", bits);
        cudaMemsetAsync(ss->status, 0, sizeof(uint32_t), t.stream);
        cudaStreamSynchronize(t.stream);
        return ST_GEMM;
    }
    return ST_OK;
}
