// C-ABI of libpg_b200.so (declared in include/pg_b200.h) and the dispatch between
// the tensor-core kernel (gemm_tc.cu) and the FFMA kernel (gemm_simt.cu).
// There is no CPU fallback in here: when no B200 is present every entry fails.

#include "../../include/pg_b200.h"
#include "pg_internal.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace pgb {

struct DeviceBuf {
    void *ptr = nullptr;
    size_t bytes = 0;
};

struct State {
    bool tried = false;
    int init_status = ST_UNSUPPORTED;
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    uint32_t *dev_status = nullptr;
    uint32_t *host_status = nullptr;   // pinned mirror
    unsigned long long *prof = nullptr;   // per-CTA cycle counters of the timing experiments
    unsigned char *die_table = nullptr;   // smid -> die, measured at init (null when the measurement was not clean)
    uint32_t *die_claim = nullptr;        // claim counters of the die-aware walk (zero between launches)
    uint32_t *counters = nullptr;         // arrival counters of the fused split-K reduction (zero between launches)
    uint32_t num_counters = 0;
    DeviceBuf ws;                      // scratch: operand pieces, split-K slices
    DeviceBuf stage_a, stage_b, stage_c, stage_bias;  // device staging for host-pointer calls
    DeviceBuf grad_pieces;             // bf16 pieces of the f32 gradient, shared by both backward products
    // options
    int opt_path = 0;        // 0 choose, 1 tensor-core only, 2 FFMA only
    int opt_cfg = -1;
    int opt_epilogue = -1;
    int opt_splits = 0;
    int opt_f32_parts = 2;   // bf16 pieces an f32 operand is split into when paired with a 16-bit one
    int opt_f32_tc = 0;      // 1: f32 x f32 on the tensor cores as 3 bf16 pieces each (6 passes)
    int opt_f32_chunk = 512; // that route adds K into C in chunks of this many elements (0: one accumulation)
    int opt_host_pipeline = 1;   // host-pointer pg_gemm_ex: overlap copies and GEMMs block by block
    int opt_fused_splitk = 1;    // split-K slices summed by the GEMM kernel itself (else a second kernel)
    int opt_attn_q_tmem = 1;     // attention kernel: Q copied to tensor memory once per unit and read from there (0: from shared memory)
    int opt_fused_attention = 1; // 0: pg_b200_attention_bmm always runs the three-kernel chain
    DeviceBuf attn_ws;           // S and P of the chain form of pg_b200_attention_bmm
    DeviceBuf caller_ws[2];      // permuted operand copies of pg_b200_tensordot
    DeviceBuf simt_ws[2];        // row-major copies of transposed f32 operands (large products on the FFMA route)
    int opt_f32_retranspose = 1; // large f32 products with a transposed operand: transpose it once, then the row-major kernel
    int opt_cluster_splitk = 1;  // K-slices of a skinny product as one cluster (reduction through distributed shared memory)
    int opt_host_blk = 0;        // slab size of the staged host-pointer pipeline (0 = 2048)
    int opt_stream_k = 0;        // balanced last wave: the K ranges of the tiles of a partly filled last wave are dealt
                                 // out to all SMs, two slices per tile at most.  Off: on B200 it cuts the MMA cycles
                                 // of the busiest SM pair by 10 % (8192x1024x8192: 160 k -> 143 k) and the clock under
                                 // the power limit falls by as much (1.52 -> 1.39 GHz): same time to within 1 %
    int opt_pdl = 1;             // programmatic dependent launch of the tensor-core kernels
    int opt_k_serpentine = 1;    // a CTA's odd-numbered tiles run K downwards
    int opt_serpentine = 1;      // odd rasterisation groups walk N downwards
    int opt_die_aware = 1;       // large products: each die of the B200 walks its own half of every rasterisation group
    int opt_swap_skinny = 1;     // M <= 32: multiply with swapped operands (C^T = B^T A^T), narrow tiles
    int opt_l2_hints = 0;    // see TcParams::l2_hints
    int opt_group_m = 0;     // 0: choose
    int opt_stages = 0;      // 0: all smem stages of the tile configuration
    int opt_debug = 0;       // timing experiments only (see TcGemm::debug)
    char err[512] = "";
    char last_path[96] = "";
    unsigned long long launches = 0;
    EncodeTiledFn encode = nullptr;
};
static State g;

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g.err, sizeof g.err, fmt, ap);
    va_end(ap);
    if (getenv("PG_B200_DEBUG")) fprintf(stderr, "pg_b200: %s\n", g.err);
}
void set_last_path(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g.last_path, sizeof g.last_path, fmt, ap);
    va_end(ap);
}
void note_launch(int n) { g.launches += (unsigned long long)n; }
int device_sm_count() { return g.sm_count > 0 ? g.sm_count : 148; }
EncodeTiledFn get_encode_tiled() { return g.encode; }

static int do_init() {
    if (g.tried) return g.init_status;
    g.tried = true;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        set_error("no CUDA device: %s", e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
        cudaGetLastError();
        return g.init_status = ST_UNSUPPORTED;
    }
    if (g.device >= n) {
        set_error("device ordinal %d out of range (%d devices)", g.device, n);
        return g.init_status = ST_UNSUPPORTED;
    }
    if (cudaSetDevice(g.device) != cudaSuccess) {
        set_error("cudaSetDevice(%d) failed", g.device);
        cudaGetLastError();
        return g.init_status = ST_UNSUPPORTED;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, g.device) != cudaSuccess) {
        set_error("cudaGetDeviceProperties failed");
        cudaGetLastError();
        return g.init_status = ST_UNSUPPORTED;
    }
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library holds sm_100a code only", g.device, prop.major, prop.minor);
        return g.init_status = ST_UNSUPPORTED;
    }
    g.sm_count = prop.multiProcessorCount;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
    if (e != cudaSuccess || !fn || qr != cudaDriverEntryPointSuccess) {
        set_error("cuTensorMapEncodeTiled not available from the driver");
        cudaGetLastError();
        return g.init_status = ST_UNSUPPORTED;
    }
    g.encode = (EncodeTiledFn)fn;
    if (cudaMalloc((void **)&g.dev_status, 256) != cudaSuccess ||
        cudaMemset(g.dev_status, 0, 256) != cudaSuccess ||
        cudaMallocHost((void **)&g.host_status, 256) != cudaSuccess) {
        set_error("could not allocate the status word");
        cudaGetLastError();
        return g.init_status = ST_ALLOC;
    }
    *g.host_status = 0;
    if (cudaMalloc((void **)&g.prof, 512 * 16 * 8) == cudaSuccess) cudaMemset(g.prof, 0, 512 * 16 * 8);
    else { g.prof = nullptr; cudaGetLastError(); }
    g.num_counters = 1u << 16;
    if (cudaMalloc((void **)&g.counters, (size_t)g.num_counters * 4) == cudaSuccess) {
        cudaMemset(g.counters, 0, (size_t)g.num_counters * 4);
    } else {
        g.counters = nullptr; g.num_counters = 0; cudaGetLastError();
    }
    // die topology (measured once; see topology.cu): the table (256 B) and the claim words of the die-aware walk
    {
        unsigned char table[256];
        void *topo = nullptr;
        if (measure_die_table(table, nullptr) && cudaMalloc(&topo, 512) == cudaSuccess && cudaMemset(topo, 0, 512) == cudaSuccess &&
            cudaMemcpy(topo, table, 256, cudaMemcpyHostToDevice) == cudaSuccess) {
            g.die_table = (unsigned char *)topo;
            g.die_claim = (uint32_t *)((char *)topo + 256);
        }
    }
    cudaGetLastError();
    return g.init_status = ST_OK;
}

static bool ready() { return do_init() == ST_OK; }

// Device facts the kernels' launchers need (SM count, the tensor-map encoder), gathered without
// allocating anything; for entry points that must not touch the allocator.
int ensure_device_info() {
    if (g.encode && g.sm_count > 0) return ST_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); set_error("no current CUDA device"); return ST_UNSUPPORTED; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { cudaGetLastError(); set_error("cudaGetDeviceProperties failed"); return ST_UNSUPPORTED; }
    if (prop.major != 10) { set_error("device %d is sm_%d%d; this library holds sm_100a code only", dev, prop.major, prop.minor); return ST_UNSUPPORTED; }
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
    if (e != cudaSuccess || !fn || qr != cudaDriverEntryPointSuccess) { cudaGetLastError(); set_error("cuTensorMapEncodeTiled not available from the driver"); return ST_UNSUPPORTED; }
    g.sm_count = prop.multiProcessorCount;
    g.encode = (EncodeTiledFn)fn;
    return ST_OK;
}
cudaStream_t current_stream() { return g.stream; }

static int grow(DeviceBuf &b, size_t bytes) {
    if (bytes <= b.bytes) return ST_OK;
    if (b.ptr) {
        cudaStreamSynchronize(g.stream);   // nothing in flight may still use the old buffer
        cudaFree(b.ptr);
        b.ptr = nullptr;
        b.bytes = 0;
    }
    size_t want = bytes + (bytes >> 3);
    want = (want + 0xFFFFF) & ~(size_t)0xFFFFF;
    if (cudaMalloc(&b.ptr, want) != cudaSuccess) {
        cudaGetLastError();
        if (cudaMalloc(&b.ptr, bytes) != cudaSuccess) {
            cudaGetLastError();
            set_error("out of device memory for %zu bytes of scratch", bytes);
            return ST_ALLOC;
        }
        want = bytes;
    }
    b.bytes = want;
    return ST_OK;
}

void *caller_scratch(int slot, size_t bytes) {
    if (slot < 0 || slot > 1 || grow(g.caller_ws[slot], bytes ? bytes : 1) != ST_OK) return nullptr;
    return g.caller_ws[slot].ptr;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t esize(int dt) { return dt == DT_F32 ? 4 : 2; }

// One GEMM, device pointers.
struct Problem {
    int dtype_a, dtype_b, trans_a, trans_b;
    size_t batch, m, n, k;
    const void *a; size_t lda, stride_a;
    const void *b; size_t ldb, stride_b;
    float *c; size_t ldc, stride_c;
    int accumulate;
    // an f32 operand whose bf16 pieces the caller has already made ([batch][piece][rows][ld]): lets
    // the two products of a backward pass share one split of the gradient
    const uint16_t *a_pieces = nullptr, *b_pieces = nullptr;
    size_t pieces_ld = 0;
    uint32_t pieces_n = 0;
    const uint32_t *pieces_mask = nullptr;    // device word: which of those pieces hold a non-zero element
    // pg_cpu_gemm_fused_ex (backend/cpu/gemm.c:718-817): C = act(bias[col] + A*B), batch == 1, no
    // accumulate; c16 (optional) receives C rounded to dtype16
    const float *bias = nullptr;
    int act = 0;
    uint16_t *c16 = nullptr;
    size_t ld16 = 0;
    int dtype16 = DT_BF16;
    int act_copy_only = 0;       // the activation goes into c16 only; C keeps bias + A*B
    int no_split_k = 0;          // every element keeps the K order of the unsplit product (staged pieces of a large one)
    float *extra_c[7] = {};      // further destinations of C (same ldc), e.g. other devices' full C
    uint32_t n_extra = 0;
    bool has_epilogue() const { return bias != nullptr || act != 0 || c16 != nullptr; }
};

static int run_simt(const Problem &p);

// Large f32 products with a transposed operand — the two products of bwd_matmul on f32 leaves (autograd.c:659-691) —
// would take the generic strided kernel (27 TFLOP/s at 4096^3).  The transposed operand is instead copied once into
// scratch in row-major order (bandwidth-bound: 134 MB at 4096^2, ~1 % of the product's time) and the product takes
// the row-major kernel (51 TFLOP/s).  Same chain per element, same bits.
static int run_simt_retransposed(const Problem &p, bool &taken) {
    taken = false;
    if (!g.opt_f32_retranspose || p.dtype_a != DT_F32 || p.dtype_b != DT_F32 || p.batch != 1) return ST_OK;
    if (!(p.trans_a || p.trans_b) || (uint64_t)p.m * p.n < (uint64_t)512 * 512 * 4 || p.k < 64) return ST_OK;
    if ((p.trans_a && p.k % 4) || (p.trans_b && p.n % 4)) return ST_OK;          // the row-major kernel wants 16-byte rows
    Problem q = p;
    for (int which = 0; which < 2; ++which) {
        if (!(which == 0 ? p.trans_a : p.trans_b)) continue;
        // stored [rows_src][cols_src] with leading dimension ld; wanted [cols_src][rows_src], contiguous
        const uint64_t rows_src = which == 0 ? p.k : p.n, cols_src = which == 0 ? p.m : p.k;
        const uint64_t ld = which == 0 ? p.lda : p.ldb;
        int st = grow(g.simt_ws[which], rows_src * cols_src * 4);
        if (st != ST_OK) return st;
        const uint64_t shape[2] = {rows_src, cols_src}, stride[2] = {ld, 1};
        const uint32_t perm[2] = {1, 0};
        st = permute_copy_launch(which == 0 ? p.a : p.b, g.simt_ws[which].ptr, 4, 2, shape, perm, g.stream, stride);
        if (st != ST_OK) return st;
        if (which == 0) { q.a = g.simt_ws[0].ptr; q.lda = rows_src; q.trans_a = 0; }
        else { q.b = g.simt_ws[1].ptr; q.ldb = rows_src; q.trans_b = 0; }
    }
    taken = true;
    return run_simt(q);
}

static int run_simt(const Problem &p) {
    {
        bool taken = false;
        const int st = run_simt_retransposed(p, taken);
        if (taken || st != ST_OK) return st;
    }
    SimtGemm s;
    s.dtype_a = p.dtype_a; s.dtype_b = p.dtype_b;
    s.M = (uint32_t)p.m; s.N = (uint32_t)p.n; s.K = (uint32_t)p.k; s.batch = (uint32_t)p.batch;
    s.A = p.a; s.B = p.b;
    if (!p.trans_a) { s.a_rs = (int64_t)p.lda; s.a_cs = 1; } else { s.a_rs = 1; s.a_cs = (int64_t)p.lda; }
    if (!p.trans_b) { s.b_rs = (int64_t)p.ldb; s.b_cs = 1; } else { s.b_rs = 1; s.b_cs = (int64_t)p.ldb; }
    s.a_bs = (int64_t)p.stride_a; s.b_bs = (int64_t)p.stride_b;
    s.C = p.c; s.ldc = (int64_t)p.ldc; s.c_bs = (int64_t)p.stride_c;
    s.accumulate = p.accumulate;
    s.bias = p.bias; s.act = p.act; s.c16 = p.c16; s.ld16 = (int64_t)p.ld16; s.dtype16 = p.dtype16;
    s.act_copy_only = p.act_copy_only;
    s.stream = g.stream;
    s.pdl = g.opt_pdl;
    int st = simt_gemm_launch(s);
    if (st == ST_OK) set_last_path("simt");
    return st;
}

// Pieces an operand is cut into for the tensor cores, or 1 when it goes as it is.
static uint32_t parts_for(int dt, int other_dt) {
    if (dt == DT_F32) return other_dt == DT_F32 ? 3u : (uint32_t)g.opt_f32_parts;
    if (dt == DT_F16 && other_dt != DT_F16) return 2u;   // f16 = bf16 + bf16 exactly
    return 1u;
}

// Tensor-core route.  Returns ST_UNSUPPORTED when the operands break a TMA rule.
static int run_tc(const Problem &p) {
    const bool mixed = p.dtype_a != p.dtype_b || p.dtype_a == DT_F32;
    const uint32_t npa = p.a_pieces ? p.pieces_n : (mixed ? parts_for(p.dtype_a, p.dtype_b) : 1u);
    const uint32_t npb = p.b_pieces ? p.pieces_n : (mixed ? parts_for(p.dtype_b, p.dtype_a) : 1u);
    if (p.m > 0x7FFFFFFFull || p.n > 0x7FFFFFFFull || p.k > 0x7FFFFFFFull || p.batch > 0x7FFFFFFull) return ST_UNSUPPORTED;

    TcGemm t = {};
    t.dtype = mixed ? DT_BF16 : p.dtype_a;
    t.M = (uint32_t)p.m; t.N = (uint32_t)p.n; t.K = (uint32_t)p.k; t.batch = (uint32_t)p.batch;
    t.A.ptr = p.a; t.A.ld = p.lda; t.A.z_stride = p.stride_a; t.A.nparts = 1; t.A.mn_major = p.trans_a ? 1u : 0u;
    t.B.ptr = p.b; t.B.ld = p.ldb; t.B.z_stride = p.stride_b; t.B.nparts = 1; t.B.mn_major = p.trans_b ? 0u : 1u;
    t.npass = 1; t.a_sel = 0; t.b_sel = 0;
    t.C = p.c; t.ldc = p.ldc; t.c_stride = p.stride_c;
    t.accumulate = p.accumulate;
    t.n_extra = p.n_extra;
    for (uint32_t d = 0; d < p.n_extra && d < 7; ++d) t.extra_c[d] = p.extra_c[d];
    t.splits = 1;
    t.force_cfg = g.opt_cfg; t.force_epilogue = g.opt_epilogue;
    t.stages = g.opt_stages; t.debug = g.opt_debug; t.l2_hints = g.opt_l2_hints; t.group_m = g.opt_group_m;
    t.stream = g.stream; t.dev_status = g.dev_status; t.prof = g.prof;
    t.allow_stream_k = g.opt_stream_k && !p.no_split_k;
    if (g.opt_die_aware) { t.die_table = g.die_table; t.die_claim = g.die_claim; }
    t.pdl = g.opt_pdl;
    t.serpentine = g.opt_serpentine;
    t.k_serpentine = g.opt_k_serpentine;
    t.cluster_splitk = g.opt_cluster_splitk;
    t.counters = g.counters; t.num_counters = g.num_counters;

    // a batch-shared operand (stride 0) with batch > 1 cannot be a TMA dimension of stride 0
    if (p.batch > 1 && (p.stride_a == 0 || p.stride_b == 0)) {
        // fold: run the batch elements as separate launches
        int st = ST_OK;
        for (size_t s = 0; s < p.batch && st == ST_OK; ++s) {
            Problem q = p;
            q.batch = 1;
            q.a = (const char *)p.a + s * p.stride_a * esize(p.dtype_a);
            q.b = (const char *)p.b + s * p.stride_b * esize(p.dtype_b);
            q.c = p.c + s * p.stride_c;
            st = run_tc(q);
        }
        return st;
    }

    // ---- scratch layout -------------------------------------------------------
    const size_t a_rows = p.trans_a ? p.k : p.m, a_cols = p.trans_a ? p.m : p.k;
    const size_t b_rows = p.trans_b ? p.n : p.k, b_cols = p.trans_b ? p.k : p.n;
    const size_t a_ld2 = p.a_pieces ? p.pieces_ld : align_up(a_cols, 8);
    const size_t b_ld2 = p.b_pieces ? p.pieces_ld : align_up(b_cols, 8);
    size_t off = 256, off_a = 0, off_b = 0, off_k = 0;      // the first 256 bytes: the piece masks of A (word 0) and B (word 1)
    if (npa > 1 && !p.a_pieces) { off_a = off; off = align_up(off + p.batch * npa * a_rows * a_ld2 * 2, 256); }
    if (npb > 1 && !p.b_pieces) { off_b = off; off = align_up(off + p.batch * npb * b_rows * b_ld2 * 2, 256); }
    // A 16-bit operand that breaks a TMA rule (base not 16-byte aligned, leading dimension or batch
    // stride not a multiple of 8 elements) is copied once into scratch with an aligned pitch when the
    // product is large enough for the copy to be noise; small ones go to the FFMA kernel instead.
    auto misaligned = [&](const void *ptr, size_t ld, size_t stride) {
        return ((uintptr_t)ptr & 15u) != 0 || ld % 8 != 0 || (p.batch > 1 && stride % 8 != 0);
    };
    const bool big = (double)p.m * (double)p.n * (double)p.k * (double)p.batch >= (double)(1u << 27);
    const bool repitch_a = npa == 1 && !mixed && big && misaligned(p.a, p.lda, p.stride_a) && (p.batch == 1 || p.stride_a != 0);
    const bool repitch_b = npb == 1 && !mixed && big && misaligned(p.b, p.ldb, p.stride_b) && (p.batch == 1 || p.stride_b != 0);
    size_t off_ra = 0, off_rb = 0;
    if (repitch_a) { off_ra = off; off = align_up(off + p.batch * a_rows * a_ld2 * 2, 256); }
    if (repitch_b) { off_rb = off; off = align_up(off + p.batch * b_rows * b_ld2 * 2, 256); }

    // Skinny M (decode-like): multiply with the operands swapped, C^T = B^T A^T, so that N fills the
    // 128 tensor-memory lanes and M becomes a 16- or 32-wide UMMA N: a stage then holds 16 KB of B and
    // only 2-4 KB of A (12 stages in flight), and the transposed store is coalesced.
    const bool swap = g.opt_swap_skinny && g.opt_cfg < 0 && !mixed && p.batch == 1 && !p.trans_a && p.m <= 32 &&
                      p.n >= 256 && !p.n_extra;
    // split-K for shapes that would leave most SMs idle
    uint32_t splits = 1;
    const uint32_t k_blocks = (uint32_t)((p.k + 63) / 64);
    if (p.batch == 1 && npa == 1 && npb == 1 && !p.no_split_k && !p.n_extra) {
        if (g.opt_splits > 0) {
            splits = (uint32_t)g.opt_splits;
        } else {
            const uint64_t tiles = swap ? (p.n + 127) / 128 : ((p.m + 127) / 128) * ((p.n + 127) / 128);
            const uint32_t sms = (uint32_t)device_sm_count();
            if (tiles * 2 <= sms && k_blocks >= 8) {
                uint32_t want = (uint32_t)(sms / tiles);
                uint32_t maxs = k_blocks / 4;
                splits = want < maxs ? want : maxs;
                if (splits < 1) splits = 1;
            }
        }
        if (splits > k_blocks) splits = k_blocks;
        if (splits > 1) {
            uint32_t per = (k_blocks + splits - 1) / splits;
            splits = (k_blocks + per - 1) / per;
        }
    }
    const size_t ws_ld = align_up(p.n, 4);
    if (splits > 1) { off_k = off; off = align_up(off + (size_t)splits * p.m * ws_ld * 4, 256); }
    if (off > 256) {
        int st = grow(g.ws, off);
        if (st != ST_OK) return st;
    }
    char *ws = (char *)g.ws.ptr;
    uint32_t *ws_masks = (uint32_t *)ws;

    // ---- re-pitched copies ----------------------------------------------------------
    if (repitch_a || repitch_b) {
        for (int which = 0; which < 2; ++which) {
            if (!(which == 0 ? repitch_a : repitch_b)) continue;
            const char *src = (const char *)(which == 0 ? p.a : p.b);
            const size_t ld = which == 0 ? p.lda : p.ldb, stride = which == 0 ? p.stride_a : p.stride_b;
            const size_t rows = which == 0 ? a_rows : b_rows, cols = which == 0 ? a_cols : b_cols;
            const size_t ld2 = which == 0 ? a_ld2 : b_ld2;
            char *dst = ws + (which == 0 ? off_ra : off_rb);
            for (size_t bi = 0; bi < p.batch; ++bi) {
                cudaError_t e = cudaMemcpy2DAsync(dst + bi * rows * ld2 * 2, ld2 * 2, src + bi * stride * 2, ld * 2, cols * 2, rows,
                                                  cudaMemcpyDeviceToDevice, g.stream);
                if (e != cudaSuccess) { set_error("re-pitch copy failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_COPY; }
            }
            TcOperand &o = which == 0 ? t.A : t.B;
            o.ptr = dst; o.ld = ld2; o.z_stride = rows * ld2;
        }
    }

    // ---- operand pieces -----------------------------------------------------------
    if (p.a_pieces) {
        t.A.ptr = p.a_pieces; t.A.ld = a_ld2; t.A.z_stride = a_rows * a_ld2; t.A.nparts = npa;
        t.a_piece_mask = p.pieces_mask;
    } else if (npa > 1) {
        uint16_t *dst = (uint16_t *)(ws + off_a);
        int st;
        if (p.dtype_a == DT_F32) {
            st = split_f32_to_bf16_launch((const float *)p.a, p.lda, p.stride_a, dst, a_ld2, (uint32_t)a_rows,
                                          (uint32_t)a_cols, (uint32_t)p.batch, npa, g.stream, ws_masks);
            t.a_piece_mask = ws_masks;
        }
        else
            st = split_f16_to_bf16_launch((const uint16_t *)p.a, p.lda, p.stride_a, dst, a_ld2, (uint32_t)a_rows,
                                          (uint32_t)a_cols, (uint32_t)p.batch, g.stream);
        if (st != ST_OK) return st;
        t.A.ptr = dst; t.A.ld = a_ld2; t.A.z_stride = a_rows * a_ld2; t.A.nparts = npa;
    } else if (mixed && p.dtype_a == DT_F16) {
        return ST_UNSUPPORTED;
    }
    if (p.b_pieces) {
        t.B.ptr = p.b_pieces; t.B.ld = b_ld2; t.B.z_stride = b_rows * b_ld2; t.B.nparts = npb;
        t.b_piece_mask = p.pieces_mask;
    } else if (npb > 1) {
        uint16_t *dst = (uint16_t *)(ws + off_b);
        int st;
        if (p.dtype_b == DT_F32) {
            st = split_f32_to_bf16_launch((const float *)p.b, p.ldb, p.stride_b, dst, b_ld2, (uint32_t)b_rows,
                                          (uint32_t)b_cols, (uint32_t)p.batch, npb, g.stream, ws_masks + 1);
            t.b_piece_mask = ws_masks + 1;
        }
        else
            st = split_f16_to_bf16_launch((const uint16_t *)p.b, p.ldb, p.stride_b, dst, b_ld2, (uint32_t)b_rows,
                                          (uint32_t)b_cols, (uint32_t)p.batch, g.stream);
        if (st != ST_OK) return st;
        t.B.ptr = dst; t.B.ld = b_ld2; t.B.z_stride = b_rows * b_ld2; t.B.nparts = npb;
    } else if (mixed && p.dtype_b == DT_F16) {
        return ST_UNSUPPORTED;
    }
    if (npa > 1 || npb > 1) {
        // keep products whose combined order is below the larger piece count; smallest terms first
        const uint32_t maxo = (npa > npb ? npa : npb) - 1;
        uint32_t np = 0, asel = 0, bsel = 0;
        for (int order = (int)maxo; order >= 0; --order)
            for (uint32_t i = 0; i < npa; ++i) {
                int j = order - (int)i;
                if (j < 0 || j >= (int)npb) continue;
                asel |= i << (4 * np);
                bsel |= (uint32_t)j << (4 * np);
                ++np;
            }
        t.npass = np; t.a_sel = asel; t.b_sel = bsel;
    }

    bool fused = false;
    if (splits > 1) {
        t.splits = splits;
        t.C = (float *)(ws + off_k);
        t.ldc = ws_ld;
        t.c_stride = p.m * ws_ld;
        fused = g.opt_fused_splitk && g.counters != nullptr;
        if (fused) {
            t.Cout = p.c; t.ldc_out = p.ldc; t.counters = g.counters; t.num_counters = g.num_counters;
            t.accumulate = p.accumulate;           // applied by the final sum only
        } else {
            t.accumulate = 0;
        }
    }
    // f32 x f32 in pieces: the tensor cores add into their f32 accumulator without rounding to nearest,
    // so the error of one long accumulation grows in proportion to K.  K therefore goes in chunks: each
    // chunk is accumulated in tensor memory from zero and added to C in f32 (round to nearest) by the
    // store, one launch per chunk in stream order, which keeps the result deterministic.
    const size_t chunk = (size_t)g.opt_f32_chunk;
    const bool chunked = p.dtype_a == DT_F32 && p.dtype_b == DT_F32 && npa > 1 && npb > 1 && chunk >= 64 &&
                         chunk % 64 == 0 && p.k > chunk && splits == 1 && !swap;
    // Bias and activation ride in the kernel's epilogue when every tile holds finished sums; K-slices,
    // K-chunks and the swapped route finish C first and one elementwise pass follows.
    const bool epi_in_kernel = p.has_epilogue() && splits == 1 && !swap && !chunked;
    if (epi_in_kernel) { t.bias = p.bias; t.act = p.act; t.c16 = p.c16; t.ld16 = p.ld16; t.dtype16 = p.dtype16; t.act_copy_only = p.act_copy_only; }
    if (swap) {
        // A' = B (its N runs along the tile rows), B' = A, tile stored transposed into the same C
        TcOperand opa = t.A;
        t.A = t.B; t.A.mn_major = p.trans_b ? 0u : 1u;
        t.B = opa; t.B.mn_major = 0u;
        t.M = (uint32_t)p.n; t.N = (uint32_t)p.m;
        t.c_trans = 1;
        t.force_cfg = p.m <= 16 ? tc_config_index("1cta_128x16_t") : tc_config_index("1cta_128x32_t");
    }
    if (g.opt_path != 1 && !tc_gemm_supported(t)) return ST_UNSUPPORTED;
    if (chunked) {
        const char *a0 = (const char *)t.A.ptr, *b0 = (const char *)t.B.ptr;
        for (size_t k0 = 0; k0 < p.k; k0 += chunk) {
            t.K = (uint32_t)(p.k - k0 < chunk ? p.k - k0 : chunk);
            t.A.ptr = a0 + 2 * (t.A.mn_major ? k0 * t.A.ld : k0);      // pieces are 16-bit
            t.B.ptr = b0 + 2 * (t.B.mn_major ? k0 * t.B.ld : k0);
            t.accumulate = k0 ? 1 : p.accumulate;
            int st = tc_gemm_launch(t);
            if (st != ST_OK) return st;
        }
        if (p.has_epilogue())
            return bias_act_launch(p.c, p.ldc, p.bias, p.act, p.act_copy_only, p.c16, p.ld16, p.dtype16, p.m, p.n, g.stream);
        return ST_OK;
    }
    int st = tc_gemm_launch(t);
    if (st == ST_UNSUPPORTED && fused) {           // more slabs than counters: fall back to the two-kernel form
        fused = false;
        t.Cout = nullptr; t.accumulate = 0;
        st = tc_gemm_launch(t);
    }
    if (st != ST_OK) return st;
    if (splits > 1 && !fused) {
        st = reduce_splits_launch((const float *)(ws + off_k), p.m * ws_ld, splits, p.c, p.ldc, (uint32_t)p.m,
                                  (uint32_t)p.n, ws_ld, p.accumulate, g.stream);
        if (st != ST_OK) return st;
    }
    if (p.has_epilogue() && !epi_in_kernel) {
        st = bias_act_launch(p.c, p.ldc, p.bias, p.act, p.act_copy_only, p.c16, p.ld16, p.dtype16, p.m, p.n, g.stream);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

static int run_problem(const Problem &p) {
    if (!ready()) return g.init_status;
    if (p.m == 0 || p.n == 0 || p.batch == 0) return ST_OK;
    if (!p.a || !p.b || !p.c) { set_error("null operand"); return ST_GEMM; }
    if (p.has_epilogue() && (p.batch != 1 || p.accumulate)) {
        set_error("fused bias/activation takes one product and overwrites C");
        return ST_UNSUPPORTED;
    }
    const bool f32f32 = p.dtype_a == DT_F32 && p.dtype_b == DT_F32;
    bool want_tc = g.opt_path != 2 && p.k > 0;
    if (f32f32 && !g.opt_f32_tc && g.opt_path != 1) want_tc = false;
    // tiny problems: one FFMA CTA beats building three tensor maps
    if (g.opt_path == 0 && (uint64_t)p.m * p.n * p.k * p.batch <= (uint64_t)64 * 64 * 64) want_tc = false;
    if (want_tc) {
        int st = run_tc(p);
        if (st == ST_OK) return ST_OK;
        if (st != ST_UNSUPPORTED || g.opt_path == 1) return st;
    }
    if (p.n_extra) {
        set_error("several destinations of C: only the tensor-core route with a TMA-storable C takes them");
        return ST_UNSUPPORTED;
    }
    return run_simt(p);
}

static bool is_device_ptr(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// Host-pointer pg_gemm_ex: stage compact copies through device memory.
static int gemm_ex_host(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                        float *c, size_t ldc, const float *dev_bias, int act) {
    const size_t es = esize(dtype);
    const size_t k8 = align_up(k, 8), n8 = align_up(n, 8), n4 = align_up(n, 4);
    int st;
    if ((st = grow(g.stage_a, m * k8 * es + 256)) != ST_OK) return st;
    if ((st = grow(g.stage_b, k * n8 * es + 256)) != ST_OK) return st;
    if ((st = grow(g.stage_c, m * n4 * 4 + 256)) != ST_OK) return st;
    cudaError_t e;
    if (k) {
        e = cudaMemcpy2DAsync(g.stage_a.ptr, k8 * es, a, lda * es, k * es, m, cudaMemcpyHostToDevice, g.stream);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(g.stage_b.ptr, n8 * es, b, ldb * es, n * es, k, cudaMemcpyHostToDevice, g.stream);
        if (e != cudaSuccess) { set_error("H2D staging failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_COPY; }
    }
    Problem p = {dtype, dtype, 0, 0, 1, m, n, k, g.stage_a.ptr, k8, 0, g.stage_b.ptr, n8, 0,
                 (float *)g.stage_c.ptr, n4, 0, 0};
    p.bias = dev_bias; p.act = act;
    st = run_problem(p);
    if (st != ST_OK) return st;
    e = cudaMemcpy2DAsync(c, ldc * 4, g.stage_c.ptr, n4 * 4, n * 4, m, cudaMemcpyDeviceToHost, g.stream);
    if (e != cudaSuccess) { set_error("D2H staging failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_COPY; }
    if (cudaStreamSynchronize(g.stream) != cudaSuccess) { set_error("sync after staged GEMM failed"); cudaGetLastError(); return ST_SYNC; }
    return ST_OK;
}

// Large host-pointer products: the same staging, cut into blocks of C so that the copies in, the
// GEMMs and the copies out overlap (PCIe is full duplex; C is as many bytes as A and B together).
// Row slabs of A and column slabs of B are sent alternately, a block of C is multiplied as soon as
// its two slabs have landed and goes back while later slabs are still arriving.
struct HostPipe {
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t ev_a[16] = {}, ev_b[16] = {}, ev_c[256] = {};
    bool ok = false, tried = false;
};
static HostPipe g_pipe;

static bool host_pipe_ready(size_t gm, size_t gn) {
    if (gm > 16 || gn > 16) return false;
    if (!g_pipe.tried) {
        g_pipe.tried = true;
        bool ok = cudaStreamCreateWithFlags(&g_pipe.in, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&g_pipe.out, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; ok && i < 16; ++i)
            ok = cudaEventCreateWithFlags(&g_pipe.ev_a[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&g_pipe.ev_b[i], cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < 256; ++i)
            ok = cudaEventCreateWithFlags(&g_pipe.ev_c[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) cudaGetLastError();
        g_pipe.ok = ok;
    }
    return g_pipe.ok;
}

static int gemm_ex_host_pipelined(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b,
                                  size_t ldb, float *c, size_t ldc, size_t bm, size_t bn, const float *dev_bias,
                                  int act) {
    const size_t es = esize(dtype);
    const size_t k8 = align_up(k, 8), n8 = align_up(n, 8), n4 = align_up(n, 4);
    const size_t gm = (m + bm - 1) / bm, gn = (n + bn - 1) / bn;
    int st;
    if ((st = grow(g.stage_a, m * k8 * es + 256)) != ST_OK) return st;
    if ((st = grow(g.stage_b, k * n8 * es + 256)) != ST_OK) return st;
    if ((st = grow(g.stage_c, m * n4 * 4 + 256)) != ST_OK) return st;
    char *da = (char *)g.stage_a.ptr, *db = (char *)g.stage_b.ptr;
    float *dc = (float *)g.stage_c.ptr;
    cudaError_t e = cudaSuccess;
    // Slabs in, alternating A row slabs and B column slabs.  When a slab has landed, everything it completes is
    // ONE product: row slab i of A with all column slabs of B that are there (a strip of C, i blocks wide), column
    // slab j of B with all row slabs of A that are there (a strip j + 1 blocks high).  The strips grow as the
    // operands arrive, so the products stay large enough to fill the GPU while the copies out start after the
    // first two slabs and then run beside the copies in (PCIe is full duplex).
    size_t na = 0, nb = 0, strips = 0;       // slabs of A / B sent so far
    for (size_t t = 0; t < (gm > gn ? gm : gn); ++t) {
        for (int which = 0; which < 2; ++which) {
            size_t r0, rh, c0, cw;
            if (which == 0) {
                if (t >= gm) continue;
                r0 = t * bm; rh = (m - r0 < bm) ? m - r0 : bm;
                e = cudaMemcpy2DAsync(da + r0 * k8 * es, k8 * es, (const char *)a + r0 * lda * es, lda * es, k * es, rh,
                                      cudaMemcpyHostToDevice, g_pipe.in);
                if (e == cudaSuccess) e = cudaEventRecord(g_pipe.ev_a[t], g_pipe.in);
                ++na;
                c0 = 0; cw = nb * bn < n ? nb * bn : n;              // the strip this slab completes
            } else {
                if (t >= gn) continue;
                c0 = t * bn; cw = (n - c0 < bn) ? n - c0 : bn;
                e = cudaMemcpy2DAsync(db + c0 * es, n8 * es, (const char *)b + c0 * es, ldb * es, cw * es, k,
                                      cudaMemcpyHostToDevice, g_pipe.in);
                if (e == cudaSuccess) e = cudaEventRecord(g_pipe.ev_b[t], g_pipe.in);
                ++nb;
                r0 = 0; rh = na * bm < m ? na * bm : m;
            }
            if (e != cudaSuccess) {
                set_error("H2D staging failed: %s", cudaGetErrorString(e));
                cudaGetLastError();
                cudaStreamSynchronize(g_pipe.in); cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g_pipe.out);
                return ST_COPY;
            }
            if (rh == 0 || cw == 0) continue;                        // the very first slab completes nothing
            // the copy stream is in order: the newest event of each operand implies the earlier ones
            cudaStreamWaitEvent(g.stream, g_pipe.ev_a[na - 1], 0);
            cudaStreamWaitEvent(g.stream, g_pipe.ev_b[nb - 1], 0);
            Problem p = {dtype, dtype, 0, 0, 1, rh, cw, k, da + r0 * k8 * es, k8, 0, db + c0 * es, n8, 0,
                         dc + r0 * n4 + c0, n4, 0, 0};
            p.bias = dev_bias ? dev_bias + c0 : nullptr; p.act = act;
            p.no_split_k = 1;        // same K order per element as the product in one piece: same bits
            st = run_problem(p);
            if (st != ST_OK) { cudaStreamSynchronize(g_pipe.in); cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g_pipe.out); return st; }
            cudaEvent_t done = g_pipe.ev_c[strips++];
            cudaEventRecord(done, g.stream);
            cudaStreamWaitEvent(g_pipe.out, done, 0);
            e = cudaMemcpy2DAsync(c + r0 * ldc + c0, ldc * 4, dc + r0 * n4 + c0, n4 * 4, cw * 4, rh,
                                  cudaMemcpyDeviceToHost, g_pipe.out);
            if (e != cudaSuccess) {
                set_error("D2H staging failed: %s", cudaGetErrorString(e));
                cudaGetLastError();
                cudaStreamSynchronize(g_pipe.in); cudaStreamSynchronize(g.stream); cudaStreamSynchronize(g_pipe.out);
                return ST_COPY;
            }
        }
    }
    e = cudaStreamSynchronize(g_pipe.out);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g_pipe.in);
    if (e != cudaSuccess) { set_error("sync after staged GEMM failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_SYNC; }
    return ST_OK;
}

static int gemm_ex_any(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                       float *c, size_t ldc, const float *bias = nullptr, int act = 0, uint16_t *c16 = nullptr,
                       size_t ld16 = 0, int dtype16 = DT_BF16) {
    if (!ready()) return g.init_status;
    if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_BF16) { set_error("bad dtype %d", dtype); return ST_UNSUPPORTED; }
    const int copy_only = (act & 0x100) ? 1 : 0;      // PG_B200_ACT_COPY_ONLY
    act &= ~0x100;
    if (act < 0 || act > 2) { set_error("bad activation %d", act); return ST_UNSUPPORTED; }
    if (copy_only && !c16) { set_error("PG_B200_ACT_COPY_ONLY needs the 16-bit output"); return ST_UNSUPPORTED; }
    if (c16 && dtype16 != DT_F16 && dtype16 != DT_BF16) { set_error("bad 16-bit output dtype %d", dtype16); return ST_UNSUPPORTED; }
    if (m == 0 || n == 0) return ST_OK;
    const bool da = is_device_ptr(a), db = is_device_ptr(b), dc = is_device_ptr(c);
    if (da && db && dc) {
        if ((bias && !is_device_ptr(bias)) || (c16 && !is_device_ptr(c16))) {
            set_error("pg_gemm_fused_ex: bias and the 16-bit output must be device pointers like A, B and C");
            return ST_UNSUPPORTED;
        }
        Problem p = {dtype, dtype, 0, 0, 1, m, n, k, a, lda, 0, b, ldb, 0, c, ldc, 0, 0};
        p.bias = bias; p.act = act; p.c16 = c16; p.ld16 = ld16; p.dtype16 = dtype16; p.act_copy_only = copy_only;
        return run_problem(p);
    }
    if (!da && !db && !dc) {
        if (c16) { set_error("pg_gemm_fused_ex: the 16-bit output is for device pointers only"); return ST_UNSUPPORTED; }
        const float *dev_bias = nullptr;
        if (bias) {
            if (is_device_ptr(bias)) { set_error("pg_gemm_fused_ex: host operands need a host bias"); return ST_UNSUPPORTED; }
            int st = grow(g.stage_bias, n * 4 + 256);
            if (st != ST_OK) return st;
            if (cudaMemcpyAsync(g.stage_bias.ptr, bias, n * 4, cudaMemcpyHostToDevice, g.stream) != cudaSuccess) {
                set_error("H2D staging of the bias failed"); cudaGetLastError(); return ST_COPY;
            }
            dev_bias = (const float *)g.stage_bias.ptr;
        }
        // pipeline only products whose copies dominate and that cut into at least 2 x 2 blocks
        // slabs of 1024 rows / columns (2048 for products beyond 16 slabs a side)
        const size_t blk = (size_t)(g.opt_host_blk > 0 ? g.opt_host_blk : 2048);
        if (g.opt_host_pipeline && k > 0 && m >= 2 * blk && n >= 2 * blk && (m + blk - 1) / blk <= 16 &&
            (n + blk - 1) / blk <= 16 && host_pipe_ready((m + blk - 1) / blk, (n + blk - 1) / blk))
            return gemm_ex_host_pipelined(dtype, m, n, k, a, lda, b, ldb, c, ldc, blk, blk, dev_bias, act);
        return gemm_ex_host(dtype, m, n, k, a, lda, b, ldb, c, ldc, dev_bias, act);
    }
    set_error("pg_gemm_ex: A, B and C must all be device pointers or all host pointers");
    return ST_UNSUPPORTED;
}

}  // namespace pgb

using namespace pgb;

extern "C" {

int pg_b200_init(void) { return do_init(); }

int pg_b200_set_device(int ordinal) {
    if (g.tried && g.init_status == ST_OK && ordinal != g.device) {
        set_error("pg_b200_set_device after init: the library is bound to device %d", g.device);
        return ST_UNSUPPORTED;
    }
    if (ordinal < 0) return ST_UNSUPPORTED;
    g.device = ordinal;
    return ST_OK;
}

int pg_b200_set_stream(void *stream) {
    g.stream = (cudaStream_t)stream;
    return ST_OK;
}

void *pg_b200_malloc(size_t nbytes) {
    if (!ready()) return nullptr;
    void *p = nullptr;
    if (cudaMalloc(&p, nbytes ? nbytes : 1) != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc(%zu) failed", nbytes);
        return nullptr;
    }
    return p;
}

void pg_b200_free(void *p) {
    if (p && ready()) cudaFree(p);
}

int pg_b200_copy_h2d(void *dst, const void *src, size_t nbytes) {
    if (!ready()) return ST_COPY;
    if (!nbytes) return ST_OK;
    cudaError_t e = cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, g.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g.stream);
    if (e != cudaSuccess) { set_error("copy_h2d: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_COPY; }
    return ST_OK;
}

int pg_b200_copy_d2h(void *dst, const void *src, size_t nbytes) {
    if (!ready()) return ST_COPY;
    if (!nbytes) return ST_OK;
    cudaError_t e = cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, g.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g.stream);
    if (e != cudaSuccess) { set_error("copy_d2h: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_COPY; }
    return ST_OK;
}

int pg_b200_sync(void) {
    if (!ready()) return ST_SYNC;
    cudaError_t e = cudaMemcpyAsync(g.host_status, g.dev_status, 4, cudaMemcpyDeviceToHost, g.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g.stream);
    if (e != cudaSuccess) { set_error("sync: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_SYNC; }
    if (*g.host_status) {
        set_error("a GEMM kernel gave up waiting (status bits 0x%x)", *g.host_status);
        *g.host_status = 0;
        cudaMemsetAsync(g.dev_status, 0, 4, g.stream);
        if (g.counters) cudaMemsetAsync(g.counters, 0, (size_t)g.num_counters * 4, g.stream);   // an aborted kernel may leave counts
        if (g.die_claim) cudaMemsetAsync(g.die_claim, 0, 16, g.stream);
        cudaStreamSynchronize(g.stream);
        return ST_GEMM;
    }
    return ST_OK;
}

void pg_b200_gemm(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b, size_t ldb, float *c,
                  size_t ldc) {
    int st = gemm_ex_any(DT_F32, m, n, k, a, lda, b, ldb, c, ldc);
    if (st != ST_OK && getenv("PG_B200_DEBUG")) fprintf(stderr, "pg_b200_gemm failed: %d %s\n", st, g.err);
}
void pg_b200_hgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb,
                   float *c, size_t ldc) {
    int st = gemm_ex_any(DT_F16, m, n, k, a, lda, b, ldb, c, ldc);
    if (st != ST_OK && getenv("PG_B200_DEBUG")) fprintf(stderr, "pg_b200_hgemm failed: %d %s\n", st, g.err);
}
void pg_b200_bgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb,
                   float *c, size_t ldc) {
    int st = gemm_ex_any(DT_BF16, m, n, k, a, lda, b, ldb, c, ldc);
    if (st != ST_OK && getenv("PG_B200_DEBUG")) fprintf(stderr, "pg_b200_bgemm failed: %d %s\n", st, g.err);
}
int pg_b200_gemm_ex(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                    float *c, size_t ldc) {
    return gemm_ex_any(dtype, m, n, k, a, lda, b, ldb, c, ldc);
}

int pg_b200_gemm_fused_ex(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                          float *c, size_t ldc, const float *bias, int act) {
    return gemm_ex_any(dtype, m, n, k, a, lda, b, ldb, c, ldc, bias, act);
}
void pg_b200_gemm_fused(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b, size_t ldb, float *c,
                        size_t ldc, const float *bias, int act) {
    (void)gemm_ex_any(DT_F32, m, n, k, a, lda, b, ldb, c, ldc, bias, act);
}
int pg_b200_gemm_fused_out16(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b,
                             size_t ldb, float *c, size_t ldc, const float *bias, int act, uint16_t *c16, size_t ldc16,
                             int dtype16) {
    return gemm_ex_any(dtype, m, n, k, a, lda, b, ldb, c, ldc, bias, act, c16, ldc16, dtype16);
}

int pg_b200_gemm_batched(int dtype_a, int dtype_b, int trans_a, int trans_b, size_t batch, size_t m, size_t n,
                         size_t k, const void *a, size_t lda, size_t stride_a, const void *b, size_t ldb,
                         size_t stride_b, float *c, size_t ldc, size_t stride_c, int accumulate) {
    for (int dt : {dtype_a, dtype_b})
        if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) { set_error("bad dtype %d", dt); return ST_UNSUPPORTED; }
    Problem p = {dtype_a, dtype_b, trans_a ? 1 : 0, trans_b ? 1 : 0, batch, m, n, k, a, lda, stride_a,
                 b, ldb, stride_b, c, ldc, stride_c, accumulate ? 1 : 0};
    return run_problem(p);
}

int pg_b200_matmul_backward(int dtype, size_t batch, size_t m, size_t n, size_t k, const void *a, const void *b,
                            int b_batched, const float *gr, float *ga, float *gb) {
    return pg_b200_matmul_backward_ex(dtype, batch, m, n, k, a, b, b_batched, gr, ga, gb, 1);
}

int pg_b200_matmul_backward_ex(int dtype, size_t batch, size_t m, size_t n, size_t k, const void *a, const void *b,
                               int b_batched, const float *gr, float *ga, float *gb, int accumulate) {
    return pg_b200_matmul_backward_act(dtype, batch, m, n, k, a, b, b_batched, gr, 0, nullptr, nullptr, ga, gb, accumulate);
}

int pg_b200_matmul_backward_act(int dtype, size_t batch, size_t m, size_t n, size_t k, const void *a, const void *b,
                                int b_batched, const float *gr, int act, const float *act_input, float *gr_pre, float *ga,
                                float *gb, int accumulate) {
    if (!ready()) return g.init_status;
    const int acc = accumulate ? 1 : 0;
    if (batch == 0 || m == 0 || n == 0 || k == 0) return ST_OK;
    if (act < 0 || act > 2 || (act && !act_input)) { set_error("pg_b200_matmul_backward_act: activation %d needs its input", act); return ST_UNSUPPORTED; }
    if (!gr) { set_error("pg_b200_matmul_backward_act: no incoming gradient"); return ST_UNSUPPORTED; }
    int st = ST_OK;
    // The f32 gradient meets the tensor cores as exact bf16 pieces; both products read the same
    // [batch*m, n] matrix, so it is split once.  (f16 operands and tiny or unaligned shapes go
    // through the general route, which splits per product or uses the FFMA kernel.)
    const uint16_t *pieces = nullptr;
    uint32_t *pieces_mask = nullptr;
    const size_t ld2 = align_up(n, 8);
    const uint32_t np = (uint32_t)g.opt_f32_parts;
    const bool share = dtype == DT_BF16 && g.opt_path != 2 && ga && gb && (uint64_t)batch * m * n * k > (uint64_t)64 * 64 * 64 &&
                       (uint64_t)batch * m <= 0x7FFFFFFFull && (!b_batched || batch == 1);
    if (share) {
        const size_t piece_bytes = align_up((size_t)np * batch * m * ld2 * 2, 256);
        st = grow(g.grad_pieces, piece_bytes + 256);
        if (st != ST_OK) return st;
        // one "batch" of batch*m rows: pieces laid out [piece][batch*m][ld2]; behind them the word that says which
        // pieces hold anything (a gradient of bf16 values, like the ones of a sum loss, has an all-zero second piece
        // and both products then run one pass instead of two)
        pieces_mask = (uint32_t *)((char *)g.grad_pieces.ptr + piece_bytes);
        st = ST_UNSUPPORTED;
        // (only where the tensor-core route is certain to take both products: the FFMA fallback would need the f32 form)
        const bool tma_safe = n % 8 == 0 && k % 8 == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
        if (act && (gr_pre || tma_safe))   // the activation node's backward happens inside the split
            st = act_grad_split_launch(act_input, gr, act, gr_pre, (uint16_t *)g.grad_pieces.ptr, ld2, (uint32_t)(batch * m),
                                       (uint32_t)n, np, g.stream, pieces_mask);
        if (st == ST_OK && act) {
            // without gr_pre the f32 form of g' does not exist; the products below read the pieces only
            gr = gr_pre ? gr_pre : (const float *)g.grad_pieces.ptr;
            act = 0;
        } else if (!act) {
            st = split_f32_to_bf16_launch(gr, n, 0, (uint16_t *)g.grad_pieces.ptr, ld2, (uint32_t)(batch * m), (uint32_t)n, 1, np,
                                          g.stream, pieces_mask);
        }
        if (st == ST_OK) pieces = (const uint16_t *)g.grad_pieces.ptr;
        else if (st != ST_UNSUPPORTED) return st;
    }
    if (act) {
        // general route: g' = g * act'(input) as f32 (into the caller's buffer, else scratch), then as any gradient
        float *dst = gr_pre;
        if (!dst) {
            st = grow(g.caller_ws[0], batch * m * n * sizeof(float));
            if (st != ST_OK) return st;
            dst = (float *)g.caller_ws[0].ptr;
        }
        st = act_grad_launch(act_input, gr, act, dst, batch * m * n, g.stream);
        if (st != ST_OK) return st;
        gr = dst;
    }
    if (ga) {
        // ga[batch][m][k] += g[batch][m][n] * B^T : the product's "A" is g (m x n), its "B" is B (stored
        // k x n) read transposed.  A B shared by the batch folds the batch into the rows of g and ga.
        Problem p = {DT_F32, dtype, 0, 1, batch, m, k, n, gr, n, m * n, b, n, k * n, ga, k, m * k, acc};
        if (!b_batched) { p.batch = 1; p.m = batch * m; p.stride_a = p.stride_b = p.stride_c = 0; }
        if (pieces && p.batch == 1) { p.a_pieces = pieces; p.pieces_ld = ld2; p.pieces_n = np; p.pieces_mask = pieces_mask; }
        st = run_problem(p);
        if (st != ST_OK) return st;
    }
    if (gb) {
        if (b_batched && batch > 1) {
            // gb[batch][k][n] += A^T[batch][k][m] * g[batch][m][n]
            Problem p = {dtype, DT_F32, 1, 0, batch, k, n, m, a, k, m * k, gr, n, m * n, gb, n, k * n, acc};
            st = run_problem(p);
        } else {
            // B shared by the batch (or no batch): gb[k][n] += sum_b A[b]^T g[b]  ==  one product with the
            // batch folded into the contraction: A as [(batch*m)][k], g as [(batch*m)][n]
            Problem p = {dtype, DT_F32, 1, 0, 1, k, n, batch * m, a, k, 0, gr, n, 0, gb, n, 0, acc};
            if (pieces) { p.b_pieces = pieces; p.pieces_ld = ld2; p.pieces_n = np; p.pieces_mask = pieces_mask; }
            st = run_problem(p);
        }
    }
    return st;
}

int pg_b200_addmm(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb, float *c,
                  size_t ldc, const float *input, size_t in_row_stride, size_t in_col_stride, float alpha, float beta) {
    if (!ready()) return g.init_status;
    if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_BF16) { set_error("bad dtype %d", dtype); return ST_UNSUPPORTED; }
    if (m == 0 || n == 0) return ST_OK;
    if (beta != 0.0f && !input) { set_error("pg_addmm: beta != 0 needs the input"); return ST_GEMM; }
    Problem p = {dtype, dtype, 0, 0, 1, m, n, k, a, lda, 0, b, ldb, 0, c, ldc, 0, 0};
    int st = run_problem(p);
    if (st != ST_OK) return st;
    return addmm_finish_launch(c, ldc, input, in_row_stride, in_col_stride, alpha, beta, m, n, g.stream);
}

int pg_b200_permute_copy(int dtype, size_t ndim, const size_t *shape, const size_t *perm, const void *src, void *dst) {
    if (!ready()) return g.init_status;
    if (ndim == 0 || ndim > 8 || !shape || !perm) { set_error("pg_b200_permute_copy: 1 to 8 dimensions"); return ST_UNSUPPORTED; }
    uint64_t sh[8]; uint32_t pm[8];
    for (size_t d = 0; d < ndim; ++d) { sh[d] = shape[d]; pm[d] = (uint32_t)perm[d]; }
    const int st = permute_copy_launch(src, dst, esize(dtype), (uint32_t)ndim, sh, pm, g.stream);
    if (st == ST_UNSUPPORTED) set_error("pg_b200_permute_copy: perm is not a permutation of 0..ndim-1");
    return st;
}

int pg_b200_conv2d(size_t n, size_t cin, size_t h, size_t w, size_t cout, size_t kh, size_t kw, int stride, int padding,
                   const float *x, const float *wt, const float *bias, float *out) {
    if (!ready()) return g.init_status;
    if (stride <= 0 || padding < 0) { set_error("pg_conv2d: stride must be positive"); return ST_UNSUPPORTED; }
    const long vh = (long)h + 2L * padding - (long)kh, vw = (long)w + 2L * padding - (long)kw;   // ops/conv.h:19-25
    if (vh < 0 || vw < 0 || cin == 0 || kh == 0 || kw == 0) { set_error("pg_conv2d: empty output"); return ST_UNSUPPORTED; }
    if (n == 0 || cout == 0) return ST_OK;
    if (!x || !wt || !out) { set_error("null operand"); return ST_GEMM; }
    const size_t oh = (size_t)(vh / stride) + 1, ow = (size_t)(vw / stride) + 1;
    const size_t K = cin * kh * kw, ncols = oh * ow;
    if (K > 0x7FFFFFFFull || ncols > 0x7FFFFFFFull || cout > 0x7FFFFFFFull || h > 0xFFFFFFFFull || w > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    // batch elements per pass: the im2col matrices of one pass stay within 512 MiB of scratch
    const size_t per = K * ncols * 4;
    size_t nb = per ? (512ull << 20) / per : n;
    if (nb < 1) nb = 1;
    if (nb > n) nb = n;
    if (nb > 65535) nb = 65535;
    int st = grow(g.attn_ws, align_up(nb * per, 256));
    if (st != ST_OK) return st;
    float *col = (float *)g.attn_ws.ptr;
    for (size_t b0 = 0; b0 < n; b0 += nb) {
        const size_t cur = n - b0 < nb ? n - b0 : nb;
        st = im2col_launch(x + b0 * cin * h * w, col, (uint32_t)cur, (uint32_t)cin, (uint32_t)h, (uint32_t)w, (uint32_t)kh,
                           (uint32_t)kw, (uint32_t)oh, (uint32_t)ow, stride, padding, g.stream);
        if (st != ST_OK) return st;
        // out[b] (cout x ncols) = W (cout x K, shared by the batch) * col[b] (K x ncols): f32, one chain per element
        Problem p = {DT_F32, DT_F32, 0, 0, cur, cout, ncols, K, wt, K, 0, col, ncols, K * ncols,
                     out + b0 * cout * ncols, ncols, cout * ncols, 0};
        if ((st = run_problem(p)) != ST_OK) return st;
    }
    if (bias) {
        st = bias_rows_launch(out, bias, (uint32_t)cout, n * cout, ncols, g.stream);
        if (st != ST_OK) return st;
    }
    // f32 x f32: the one-chain FFMA kernels unless the caller chose the tensor-core route (option f32_tensor_cores)
    set_last_path(!strncmp(g.last_path, "tc:", 3) ? "conv:im2col+tc" : "conv:im2col+simt");
    return ST_OK;
}

int pg_b200_attention_bmm(int dtype, size_t batch, size_t seq_q, size_t seq_k, size_t d, const void *q, const void *kt,
                          const void *v, float *o) {
    if (!ready()) return g.init_status;
    if (dtype != DT_F16 && dtype != DT_BF16) { set_error("pg_b200_attention_bmm: f16 or bf16 operands"); return ST_UNSUPPORTED; }
    if (batch == 0 || seq_q == 0 || d == 0) return ST_OK;
    if (seq_k == 0) { set_error("pg_b200_attention_bmm: softmax over an empty row"); return ST_UNSUPPORTED; }
    if (!q || !kt || !v || !o) { set_error("null operand"); return ST_GEMM; }
    if (g.opt_fused_attention && batch <= 0x7FFFFFu && seq_q <= 0x7FFFFFFFu && seq_k <= 0x7FFFFFFFu) {
        AttnProblem a = {};
        a.dtype = dtype; a.batch = (uint32_t)batch; a.sq = (uint32_t)seq_q; a.sk = (uint32_t)seq_k; a.d = (uint32_t)d;
        a.q = q; a.ldq = d; a.q_stride = seq_q * d;
        a.kt = kt; a.ldk = seq_k; a.k_stride = d * seq_k;
        a.v = v; a.ldv = d; a.v_stride = seq_k * d;
        a.o = o; a.ldo = d; a.o_stride = seq_q * d;
        a.stream = g.stream; a.dev_status = g.dev_status;
        a.prof = (g.opt_debug & 32) ? g.prof : nullptr;
        a.debug = (uint32_t)g.opt_debug;
        a.q_tmem = g.opt_attn_q_tmem;
        const int st = attn_fused_launch(a);
        if (st != ST_UNSUPPORTED) return st;
    }
    // the chain, as picograd's callers would run it: pg_bmm, softmax rows + cast, pg_bmm
    const size_t s_bytes = align_up(batch * seq_q * seq_k * 4, 256), p_bytes = align_up(batch * seq_q * seq_k * 2, 256);
    int st = grow(g.attn_ws, s_bytes + p_bytes);
    if (st != ST_OK) return st;
    float *S = (float *)g.attn_ws.ptr;
    uint16_t *P = (uint16_t *)((char *)g.attn_ws.ptr + s_bytes);
    Problem p1 = {dtype, dtype, 0, 0, batch, seq_q, seq_k, d, q, d, seq_q * d, kt, seq_k, d * seq_k, S, seq_k, seq_q * seq_k, 0};
    if ((st = run_problem(p1)) != ST_OK) return st;
    if (seq_k > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    if ((st = softmax_rows_launch(S, nullptr, P, dtype, batch * seq_q, (uint32_t)seq_k, g.stream)) != ST_OK) return st;
    Problem p2 = {dtype, dtype, 0, 0, batch, seq_q, d, seq_k, P, seq_k, seq_q * seq_k, v, d, seq_k * d, o, d, seq_q * d, 0};
    if ((st = run_problem(p2)) != ST_OK) return st;
    set_last_path("attn:chain");
    return ST_OK;
}

int pg_b200_softmax_rows(const float *src, float *out_f32, uint16_t *out16, int dtype16, size_t rows, size_t len) {
    if (!ready()) return g.init_status;
    if (len > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    return softmax_rows_launch(src, out_f32, out16, dtype16, rows, (uint32_t)len, g.stream);
}
int pg_b200_gelu(const float *src, float *out_f32, uint16_t *out16, int dtype16, size_t n) {
    if (!ready()) return g.init_status;
    return gelu_launch(src, out_f32, out16, dtype16, n, g.stream);
}
int pg_b200_gelu_grad(const float *x, const float *gy, float *out, size_t n) {
    if (!ready()) return g.init_status;
    return gelu_grad_launch(x, gy, out, n, g.stream);
}
int pg_b200_cast_f32(const float *src, uint16_t *dst, int dtype16, size_t n) {
    if (!ready()) return g.init_status;
    return cast_f32_launch(src, dst, n, dtype16, g.stream);
}
int pg_b200_fill_f32(float *dst, float value, size_t n) {
    if (!ready()) return g.init_status;
    return fill_f32_launch(dst, value, n, g.stream);
}

int pg_b200_gather_relayout(const float *staging, float *dst, size_t shards, size_t rows, size_t width, size_t n, size_t ld) {
    if (!ready()) return g.init_status;
    if (shards > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    const int st = gather_relayout_launch(staging, dst, (uint32_t)shards, rows, width, n, ld, g.stream);
    if (st == ST_UNSUPPORTED) set_error("pg_b200_gather_relayout: %zu shards of %zu columns do not cover n = %zu (ld %zu)", shards, width, n, ld);
    return st;
}

int pg_b200_die_table(unsigned char *out, size_t count) {
    if (!ready()) return g.init_status;
    if (!g.die_table) return ST_UNSUPPORTED;
    if (count > 256) count = 256;
    return cudaMemcpy(out, g.die_table, count, cudaMemcpyDeviceToHost) == cudaSuccess ? ST_OK : ST_COPY;
}

int pg_b200_debug_counters(uint64_t *out, size_t count) {
    if (!ready() || !g.prof) return ST_UNSUPPORTED;
    if (count > 512 * 16) count = 512 * 16;
    cudaStreamSynchronize(g.stream);
    return cudaMemcpy(out, g.prof, count * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? ST_OK : ST_COPY;
}

int pg_b200_selftest_wait_timeout(unsigned limit_ms) {
    if (!ready()) return g.init_status;
    return wait_timeout_selftest_launch(g.dev_status, limit_ms, g.stream);
}

int pg_b200_debug_tail_schedule(uint64_t tiles, unsigned slots, unsigned k_blocks, unsigned cluster, unsigned part,
                                 unsigned out[6]) {
    return tc_tail_schedule(tiles, slots, k_blocks, cluster, part, out);
}

int pg_b200_gemm_ex_scatter(int dtype, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb,
                            float *const *dst, size_t n_dst, size_t ldc, size_t col0) {
    if (!ready()) return g.init_status;
    if (dtype != DT_F16 && dtype != DT_BF16) { set_error("pg_b200_gemm_ex_scatter: f16 or bf16 operands"); return ST_UNSUPPORTED; }
    if (!dst || n_dst == 0 || n_dst > 8) { set_error("pg_b200_gemm_ex_scatter: 1 to 8 destinations"); return ST_UNSUPPORTED; }
    if (m == 0 || n == 0) return ST_OK;
    if (col0 % 4 || ldc % 4 || n % 4 || col0 + n > ldc) {
        set_error("pg_b200_gemm_ex_scatter: col0, n and ldc must be multiples of 4 and the shard must lie inside a row of C");
        return ST_UNSUPPORTED;
    }
    for (size_t d = 0; d < n_dst; ++d)
        if (!dst[d]) { set_error("null destination"); return ST_GEMM; }
    Problem p = {dtype, dtype, 0, 0, 1, m, n, k, a, lda, 0, b, ldb, 0, dst[0] + col0, ldc, 0, 0};
    p.n_extra = (uint32_t)(n_dst - 1);
    for (size_t d = 1; d < n_dst; ++d) p.extra_c[d - 1] = dst[d] + col0;
    return run_problem(p);
}

int pg_b200_ipc_export(const void *dev_ptr, unsigned char handle[64]) {
    if (!ready()) return g.init_status;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr));
    if (e != cudaSuccess) { set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_UNSUPPORTED; }
    memcpy(handle, &h, 64);
    return ST_OK;
}

int pg_b200_ipc_open(const unsigned char handle[64], void **dev_ptr) {
    if (!ready()) return g.init_status;
    if (!dev_ptr) return ST_UNSUPPORTED;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { *dev_ptr = nullptr; set_error("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_UNSUPPORTED; }
    return ST_OK;
}

int pg_b200_ipc_close(void *dev_ptr) {
    if (!dev_ptr) return ST_OK;
    cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    if (e != cudaSuccess) { set_error("cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return ST_UNSUPPORTED; }
    return ST_OK;
}

int pg_b200_debug_walk(unsigned m_tiles, unsigned n_tiles, unsigned group_m, unsigned k_blocks, unsigned die_aware,
                       unsigned serpentine, unsigned k_serpentine, unsigned die, unsigned id, unsigned count, unsigned i,
                       unsigned out[4]) {
    return tc_walk_unit(m_tiles, n_tiles, group_m, k_blocks, die_aware, serpentine, k_serpentine, die, id, count, i, out);
}

const char *pg_b200_last_error(void) { return g.err; }
const char *pg_b200_last_path(void) { return g.last_path; }
uint64_t pg_b200_launch_count(void) { return g.launches; }
int pg_b200_num_tile_configs(void) { return tc_num_configs(); }
const char *pg_b200_tile_config_name(int index) { return tc_config_name(index); }

int pg_b200_set_option(const char *name, int value) {
    if (!name) return ST_UNSUPPORTED;
    if (!strcmp(name, "path")) { g.opt_path = value; return ST_OK; }
    if (!strcmp(name, "tile_config")) { g.opt_cfg = value; return ST_OK; }
    if (!strcmp(name, "epilogue")) { g.opt_epilogue = value; return ST_OK; }
    if (!strcmp(name, "k_splits")) { g.opt_splits = value; return ST_OK; }
    if (!strcmp(name, "f32_parts")) { if (value != 2 && value != 3) return ST_UNSUPPORTED; g.opt_f32_parts = value; return ST_OK; }
    if (!strcmp(name, "f32_tensor_cores")) { g.opt_f32_tc = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "f32_chunk")) { if (value < 0 || value % 64) return ST_UNSUPPORTED; g.opt_f32_chunk = value; return ST_OK; }
    if (!strcmp(name, "stages")) { g.opt_stages = value; return ST_OK; }
    if (!strcmp(name, "l2_promotion")) { if (value < 0 || value > 3) return ST_UNSUPPORTED; g_l2_promotion = value; return ST_OK; }
    if (!strcmp(name, "l2_hints")) { g.opt_l2_hints = value; return ST_OK; }
    if (!strcmp(name, "group_m")) { g.opt_group_m = value; return ST_OK; }
    if (!strcmp(name, "host_pipeline")) { g.opt_host_pipeline = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "fused_splitk")) { g.opt_fused_splitk = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "swap_skinny")) { g.opt_swap_skinny = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "attn_q_tmem")) { g.opt_attn_q_tmem = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "fused_attention")) { g.opt_fused_attention = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "cluster_splitk")) { g.opt_cluster_splitk = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "host_blk")) { g.opt_host_blk = value; return ST_OK; }
    if (!strcmp(name, "stream_k")) { g.opt_stream_k = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "big_f32_min_ctas")) { g_big_f32_min_ctas = value; return ST_OK; }
    if (!strcmp(name, "f32_retranspose")) { g.opt_f32_retranspose = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "big_f32_pipe")) { g_big_f32_pipe = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "small_f32_pipe")) { g_small_f32_pipe = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "k_serpentine")) { g.opt_k_serpentine = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "serpentine")) { g.opt_serpentine = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "die_aware")) { g.opt_die_aware = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "pdl")) { g.opt_pdl = value ? 1 : 0; return ST_OK; }
    if (!strcmp(name, "debug")) { g.opt_debug = value; return ST_OK; }
    set_error("unknown option %s", name);
    return ST_UNSUPPORTED;
}

}  // extern "C"
