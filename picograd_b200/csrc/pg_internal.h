// Internal declarations shared by the .cu files of libpg_b200.so.
// Nothing here is part of the C-ABI (that is include/pg_b200.h).
#pragma once

#include <cuda.h>          // CUtensorMap and its enums only; no libcuda symbol is linked
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pgb {

// pg_status values of picograd (backend/backend.h:25-32)
enum : int { ST_OK = 0, ST_UNSUPPORTED = -1, ST_ALLOC = -2, ST_COPY = -3, ST_SYNC = -4, ST_GEMM = -5 };
// pg_dtype values of picograd (core/dtype.h:11-16)
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

// Bits of the device status word a kernel ORs in when one of its bounded waits
// gives up.  The host reads the word at pg_b200_sync() and maps any bit to
// PG_ERR_GEMM.
enum : uint32_t {
    DEV_ERR_WAIT_EMPTY = 1u << 0,      // TMA producer: smem stage never freed
    DEV_ERR_WAIT_FULL = 1u << 1,       // MMA issuer: TMA bytes never landed
    DEV_ERR_WAIT_TMEM_EMPTY = 1u << 2, // MMA issuer: epilogue never drained TMEM
    DEV_ERR_WAIT_TMEM_FULL = 1u << 3,  // epilogue: accumulator never completed
    DEV_ERR_WAIT_TILE_FLAG = 1u << 4,  // epilogue: the first K-slice of a shared tile never arrived
    DEV_ERR_SELFTEST = 1u << 8,        // the wait-timeout self-test kernel ran out of time, as it must
};

// One operand of the tensor-core GEMM as it lies in HBM.
//   K-major  (mn_major = 0): element (r, k) at ptr[z*z_stride + r*ld + k]   (r = row of A / column of B)
//   MN-major (mn_major = 1): element (r, k) at ptr[z*z_stride + k*ld + r]
// z runs over batch * nparts (+ part); parts are the bf16 pieces an f32 operand
// was split into, laid out one after the other.
struct TcOperand {
    const void *ptr;
    uint64_t ld;        // elements
    uint64_t z_stride;  // elements between consecutive z slices
    uint32_t nparts;    // pieces per batch element (1 for a native 16-bit operand)
    uint32_t mn_major;
};

struct TcGemm {
    int dtype;                 // DT_F16 or DT_BF16 (both operands)
    uint32_t M, N, K, batch;
    TcOperand A, B;            // A: MN extent = M, B: MN extent = N
    uint32_t npass;            // K passes; pass p multiplies part a_sel[p] of A with part b_sel[p] of B
    uint32_t a_sel, b_sel;     // 4 bits per pass
    const uint32_t *a_piece_mask, *b_piece_mask;   // device words (or null): bit i = piece i has a non-zero element
    float *C;
    uint64_t ldc, c_stride;    // elements; c_stride between batch elements (or split-K slices)
    int accumulate;            // C += A*B instead of C = A*B
    // Further destinations of C: every tile is stored to extra_c[i] as well (same M, N, ldc; one product, no
    // accumulate, TMA-store epilogue only).  The pointers may be another device's memory mapped into this
    // process: a column shard then lands in every device's full C without a collective afterwards.
    float *extra_c[7];
    uint32_t n_extra;
    // fused epilogue: C = act(A*B + bias[col]) and an optional 16-bit copy of C ([batch][M][ld16])
    const float *bias; int act; uint16_t *c16; uint64_t ld16; int dtype16;
    int act_copy_only;         // activation applied to the 16-bit copy only
    int c_trans;               // store the tile transposed: element (row, col) -> C[col*ldc + row]
    // splits > 1 with Cout set: C holds the K-slices and the kernel itself sums them into Cout
    float *Cout;
    uint64_t ldc_out;
    uint32_t *counters;        // zeroed device words, one per (tile, CTA, epilogue warp)
    uint32_t num_counters;
    int cluster_splitk;        // may run the K-slices of a narrow tile as one cluster, summed through distributed shared memory
    int allow_stream_k;        // may deal the K ranges of a partly filled last wave out to all clusters (two slices per tile)
    const unsigned char *die_table;   // device table smid -> die (or null: die-oblivious walk); see topology.cu
    uint32_t *die_claim;              // three zeroed device words (claims per die, pairs finished)
    int pdl;                   // launch with programmatic stream serialisation: the prologue overlaps the previous kernel's tail
    uint32_t splits;           // >1: split-K, slice s goes to C + s*c_stride (batch must be 1)
    int force_cfg;             // -1 = choose; else index into the config table
    int force_epilogue;        // -1 = choose; 0 = direct stores; 1 = TMA stores
    int stages;                // 0 = all the configuration has; else use this many smem stages
    int l2_hints;              // L2 eviction priorities of the bulk copies (see TcParams::l2_hints)
    int group_m;               // 0 = choose; else M tiles per rasterisation group
    int serpentine;            // 1: odd rasterisation groups walk N downwards
    int k_serpentine;          // 1: a CTA's odd-numbered tiles run K downwards
    int debug;                 // timing experiments: 1 = no TMA loads, 2 = no C stores (results are garbage)
    cudaStream_t stream;
    uint32_t *dev_status;      // device status word
    unsigned long long *prof;  // 16 counters per CTA for debug bit 32 (may be null)
};

// Returns ST_OK if launched, ST_UNSUPPORTED if the shape/alignment cannot go
// through TMA (caller then uses the SIMT kernel), ST_GEMM on a launch error.
int tc_gemm_launch(const TcGemm &g);
// true if operands satisfy the TMA rules (16-byte aligned bases and strides)
bool tc_gemm_supported(const TcGemm &g);
int wait_timeout_selftest_launch(uint32_t *status, unsigned limit_ms, cudaStream_t stream);
extern int g_l2_promotion;   // CUtensorMapL2promotion of the operand tensor maps
int tc_tail_schedule(uint64_t tiles, uint32_t slots, uint32_t k_blocks, uint32_t c, uint32_t j, uint32_t out[6]);
int tc_walk_unit(uint32_t m_tiles, uint32_t n_tiles, uint32_t group_m, uint32_t k_blocks, uint32_t die_aware, uint32_t serpentine,
                 uint32_t k_serpentine, uint32_t die, uint32_t id, uint32_t count, uint32_t i, uint32_t out[4]);
// topology.cu: measures which SMs share a die; false when the SMs do not fall into two clean groups
bool measure_die_table(unsigned char table[256], cudaStream_t stream);
int tc_num_configs();
const char *tc_config_name(int cfg);
int tc_config_index(const char *name);   // -1 if unknown

// Q Kt -> softmax -> 16-bit P -> P V in one kernel (attn_tc.cu).  Q [b][sq][d], Kt [b][d][sk], V [b][sk][d]
// in `dtype` (f16/bf16), O [b][sq][d] f32; leading dimensions and batch strides in elements.
// ST_UNSUPPORTED when d != 128 or an operand breaks the TMA alignment rules.
struct AttnProblem {
    int dtype;
    uint32_t batch, sq, sk, d;
    const void *q; uint64_t ldq, q_stride;
    const void *kt; uint64_t ldk, k_stride;
    const void *v; uint64_t ldv, v_stride;
    float *o; uint64_t ldo, o_stride;
    cudaStream_t stream;
    uint32_t *dev_status;
    unsigned long long *prof;   // 16 cycle counters per CTA, for the timing experiments (may be null)
    uint32_t debug;             // timing experiments: 1 = no TMA loads, 16 = no MMAs (results are garbage)
    int q_tmem;                 // keep Q in tensor memory (A operand of the Q Kt products read from there)
};
int attn_fused_launch(const AttnProblem &a);

// Generic FFMA fallback: any dtype (per operand), any strides.
struct SimtGemm {
    int dtype_a, dtype_b;      // DT_*
    uint32_t M, N, K, batch;
    const void *A; int64_t a_rs, a_cs, a_bs;   // element strides: row (m), column (k), batch
    const void *B; int64_t b_rs, b_cs, b_bs;   // row (k), column (n), batch
    float *C; int64_t ldc, c_bs;
    int accumulate;            // C += instead of C =
    const float *bias; int act;   // fused epilogue: the chain of column j starts at bias[j]; act applied at the store
    uint16_t *c16; int64_t ld16; int dtype16;
    int act_copy_only;         // activation applied to the 16-bit copy only
    int pdl;                   // small f32 kernel: launch with programmatic stream serialisation
    cudaStream_t stream;
};
int simt_gemm_launch(const SimtGemm &g);
extern int g_big_f32_min_ctas; // the 128 x 128 f32 kernel is used from this many CTAs on
extern int g_big_f32_pipe;     // large f32 x f32 products: cp.async-pipelined 128 x 128 kernel (1) or the register-staged one (0)
extern int g_small_f32_pipe;   // small f32 x f32 products: cp.async-pipelined 32 x 64 kernel (1) or the 64 x 64 one (0)

// Helper kernels (aux_kernels.cu)
// mask (device word, may be null; cleared by the launch): bit i is set when piece i holds a non-zero element
int split_f32_to_bf16_launch(const float *src, uint64_t ld_src, uint64_t src_bs,
                             uint16_t *dst, uint64_t ld_dst, uint32_t rows, uint32_t cols,
                             uint32_t batch, uint32_t nparts, cudaStream_t s, uint32_t *mask = nullptr);
int split_f16_to_bf16_launch(const uint16_t *src, uint64_t ld_src, uint64_t src_bs,
                             uint16_t *dst, uint64_t ld_dst, uint32_t rows, uint32_t cols,
                             uint32_t batch, cudaStream_t s);
int reduce_splits_launch(const float *ws, uint64_t slice_stride, uint32_t splits,
                         float *c, uint64_t ldc, uint32_t M, uint32_t N, uint64_t ws_ld,
                         int accumulate, cudaStream_t s);
int add_inplace_launch(float *dst, const float *src, uint64_t n, cudaStream_t s);
int cast_f32_launch(const float *src, uint16_t *dst, uint64_t n, int dtype, cudaStream_t s);
int gelu_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16, uint64_t n, cudaStream_t s);
int gelu_grad_launch(const float *x, const float *gy, float *out, uint64_t n, cudaStream_t s);
int act_grad_split_launch(const float *x, const float *gy, int act, float *out32, uint16_t *dst, uint64_t ld_dst,
                          uint32_t rows, uint32_t cols, uint32_t nparts, cudaStream_t s, uint32_t *mask);
int act_grad_launch(const float *x, const float *gy, int act, float *out, uint64_t n, cudaStream_t s);
int softmax_rows_launch(const float *src, float *dst_f32, uint16_t *dst_16, int dtype16,
                        uint64_t rows, uint32_t len, cudaStream_t s);
int bias_act_launch(float *c, uint64_t ldc, const float *bias, int act, int act_copy_only, uint16_t *c16, uint64_t ld16,
                    int dtype16, uint64_t rows, uint64_t n, cudaStream_t s);
int im2col_launch(const float *x, float *col, uint32_t batch, uint32_t cin, uint32_t h, uint32_t w, uint32_t kh, uint32_t kw,
                  uint32_t oh, uint32_t ow, int stride, int pad, cudaStream_t s);
int bias_rows_launch(float *out, const float *bias, uint32_t cout, uint64_t rows, uint64_t n, cudaStream_t s);
// src_stride (elements, per source dimension) = nullptr: the source is contiguous
int permute_copy_launch(const void *src, void *dst, size_t elem_size, uint32_t ndim, const uint64_t *shape, const uint32_t *perm,
                        cudaStream_t s, const uint64_t *src_stride = nullptr);
// grow-only device scratch of the tensor-level callers (two slots: the permuted copies of pg_tensordot)
void *caller_scratch(int slot, size_t bytes);
int addmm_finish_launch(float *c, uint64_t ldc, const float *input, uint64_t in_rs, uint64_t in_cs, float alpha, float beta,
                        uint64_t rows, uint64_t n, cudaStream_t s);
int fill_f32_launch(float *dst, float v, uint64_t n, cudaStream_t s);
int gather_relayout_launch(const float *staging, float *dst, uint32_t shards, uint64_t rows, uint64_t width, uint64_t n,
                           uint64_t ld, cudaStream_t s);

void set_error(const char *fmt, ...);
void set_last_path(const char *fmt, ...);
void note_launch(int n = 1);   // counts kernels launched by this library

// cuTensorMapEncodeTiled, fetched through the runtime (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

int device_sm_count();
int ensure_device_info();        // fills the above without allocating; ST_OK or ST_UNSUPPORTED
cudaStream_t current_stream();   // the stream set with pg_b200_set_stream

}  // namespace pgb
