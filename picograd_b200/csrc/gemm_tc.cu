// Dense GEMM on the Blackwell tensor cores (sm_100a): C[f32] = A * B with 16-bit
// (f16 / bf16) operands and f32 accumulation in tensor memory.
//
//   * tcgen05.mma (kind::f16) issued by one thread per CTA (or per CTA pair with
//     cta_group::2), accumulators in TMEM, double-buffered so that the epilogue of
//     one tile overlaps the main loop of the next.
//   * Operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle, no
//     cluster multicast) into a ring of shared-memory stages guarded by mbarriers.
//   * Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
//     warps 2..5 = epilogue (tcgen05.ld -> swizzled smem -> TMA store, or direct
//     predicated stores when C does not satisfy the TMA alignment rules).
//   * Persistent: each CTA (pair) walks a strided list of work units
//     (batch x M-tile x N-tile x K-split) in an L2-friendly grouped order:
//     rasterisation groups of M tiles, each die of the GPU on its own half of a
//     group, odd groups walking N downwards and a CTA's odd-numbered tiles
//     fetching K last to first, so that a wave starts on what the one before it
//     has just read.
//   * A tile of C can be stored to several matrices at once (other devices' C
//     mapped into this process): a column shard then lands in every device's full
//     C while the next tiles are multiplied, with no collective afterwards.
//   * Either operand may be K-major or MN-major in memory (that is how the
//     row-major NN product and the two transposed products of the backward pass
//     are served without materialising a transpose), and the K loop may run
//     several "passes" over different bf16 pieces of an operand that was split
//     from f32 (used by the backward pass and by the f32 GEMM).
//   * Every mbarrier wait is bounded: after ~2 s it records a bit in the device
//     status word, raises a CTA-wide abort flag and the CTA drains and exits.
//
// This implements the device side of pg_gemm_ex for f16/bf16
// (picograd backend/backend.c:150-177; the CUDA seat backend/cuda/cuda.c:282-291
// leaves hgemm/bgemm/gemm_ex NULL — this kernel is what fills them).

#include "pg_internal.h"
#include "tc_ptx.cuh"
#include "fast_math.cuh"

#include <stdio.h>
#include <string.h>

// Timing experiments (TcParams::debug: loads / stores / MMAs switched off, in-kernel cycle counters) exist only in
// builds made with -DPG_TC_EXPERIMENTS=1.  In the product build the switches are compile-time false, so the role
// loops hold no experiment branch and the "debug" option does nothing.
#ifndef PG_TC_EXPERIMENTS
#define PG_TC_EXPERIMENTS 0
#endif

namespace pgb {

constexpr bool kExperiments = PG_TC_EXPERIMENTS != 0;
#define PG_DBG(bits) (kExperiments && (p.debug & (bits)))

// ---------------------------------------------------------------------------------------------
// Tile constants
// ---------------------------------------------------------------------------------------------
constexpr uint32_t BM_CTA = 128;                 // C rows per CTA == TMEM lanes
constexpr uint32_t BK = 64;                      // 64 x 16-bit = one 128-byte swizzle row
constexpr uint32_t UMMA_K = 16;                  // K of one tcgen05.mma for 16-bit inputs
constexpr uint32_t A_TILE_BYTES = BM_CTA * BK * 2;
constexpr uint32_t EPI_COLS = 32;                // columns per tcgen05.ld / per TMA-store box
constexpr uint32_t EPI_BUF_BYTES = 32 * EPI_COLS * 4;
constexpr uint32_t SMEM_LIMIT = 232448;          // 227 KB opt-in maximum per CTA

// CG      CTAs per tile (1, or 2 = cta_group::2 pair)
// BN      columns of the tile (UMMA N)
// SUB     64-deep K blocks per pipeline stage
// STAGING epilogue goes through shared memory and TMA stores (else straight from registers)
// EW      epilogue warps (4, or 8: two per TMEM lane quadrant, alternating column chunks)
// EB      staging buffers per epilogue warp
template <int CG, int BN, int SUB, bool STAGING, int EW, int EB>
struct Cfg {
    static constexpr uint32_t BN_CTA = BN / CG;                      // B columns loaded by one CTA
    static constexpr uint32_t B_TILE_BYTES = BN_CTA * BK * 2;
    static constexpr uint32_t SUB_BYTES = A_TILE_BYTES + B_TILE_BYTES;  // one 64-deep K block of A and B
    static constexpr uint32_t STAGE_BYTES = SUB * SUB_BYTES;            // SUB K blocks share one barrier round
    static constexpr uint32_t EPI_BYTES = STAGING ? EW * EB * EPI_BUF_BYTES : 0;
    static constexpr uint32_t BAR_BYTES = 512;
    static constexpr uint32_t STAGES_RAW = (SMEM_LIMIT - 1024 - EPI_BYTES - BAR_BYTES) / STAGE_BYTES;
    static constexpr uint32_t STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
    static constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators
    static constexpr uint32_t THREADS = 32 * (2 + EW);
    static constexpr uint32_t EPI_W = BN < 32 ? BN : 32;             // columns per epilogue chunk
    static_assert(EW == 4 || EW == 8, "epilogue warps");
    static_assert(STAGES >= 2, "pipeline too shallow");
    static_assert(TMEM_COLS >= 32 && TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns");
    static_assert(SUB_BYTES % 1024 == 0, "tiles must keep the 1024-byte swizzle alignment");
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
    static_assert(STAGING ? BN >= 16 : true, "staging area: TMA-store chunks (BN >= 32) or the cluster reduction (BN <= 32)");
};

struct TcParams {
    uint32_t M, N, K;
    uint32_t batch, splits;
    uint32_t m_tiles, n_tiles;
    uint32_t k_blocks, kb_per_split;
    uint32_t npass, a_sel, b_sel, a_nparts, b_nparts;
    // Piece masks (device words, may be null): bit i set = piece i of that operand has a non-zero element.  Passes
    // over an all-zero piece are skipped (they would add exact zeros): a gradient whose values are bf16 numbers —
    // the ones of a sum loss, for one — costs one pass instead of two.
    const uint32_t *a_piece_mask, *b_piece_mask;
    uint32_t a_mn, b_mn;          // operand is MN-major in memory
    uint32_t idesc;               // tcgen05 instruction descriptor
    uint32_t group_m;             // M tiles per rasterisation group
    uint32_t n_extra;             // further destinations of every C tile
    float *extra_c[7];            // their bases (same ldc as C)
    uint32_t serpentine;          // odd groups walk N downwards: the B panels a group ends on are the next one's first
    uint32_t k_serpentine;        // a CTA's odd-numbered tiles run K downwards: the K blocks a wave ends on are the next one's first
    uint32_t epilogue_tma;        // 1: TMA-store epilogue, 0: direct stores
    uint32_t accumulate;          // C += instead of C = (TMA reduce-add / read-modify-write)
    uint32_t c_vec4;              // direct stores may use 16-byte vectors
    uint32_t stages;              // smem stages in use (<= the configuration's maximum)
    uint32_t debug;               // timing experiments only (results are garbage): 1 = no TMA loads, 2 = no C
                                  // stores, 4 = no TMEM reads, 8 = alternate accumulators, 16 = no MMAs
    uint32_t l2_hints;            // 2 bits each for A loads, B loads, C stores: 0 normal, 1 evict_first, 2 evict_last
    uint32_t c_trans;             // element (row, col) of the tile goes to C[col*ldc + row] (swapped operands)
    uint32_t cluster_k;           // > 1: the K-slices of a tile are the CTAs of one cluster of this size; their partial
                                  // tiles meet in the leader's shared memory and the leader writes Cout (BN <= 32)
    // fused epilogue (picograd pg_cpu_gemm_fused_ex): C = act(A*B + bias[col]); optional 16-bit copy of C
    const float *bias;
    uint32_t act;                 // 0 none, 1 relu, 2 gelu (erf form)
    uint32_t act_copy_only;       // the activation goes into the 16-bit copy only; C keeps bias + A*B
    unsigned short *c16;
    uint64_t ld16;
    uint32_t dtype16;
    uint32_t bias_vec4, c16_vec;  // bias 16-byte aligned; c16 rows 16-byte aligned
    float *C;                     // splits > 1: the K-slices [split][rows][ldc]; else the result
    uint64_t ldc, c_stride;
    // fused split-K reduction: the last warp to finish a slab sums the slices (in slice order) into Cout
    float *Cout;
    uint64_t ldc_out;
    uint32_t *counters;           // one per (tile, CTA of the pair, epilogue warp); zero between launches
    // Balanced last wave (sk_on): with T tiles on S resident clusters, the first sk_full = T / S waves are whole
    // tiles; the K ranges of the remaining T % S tiles are dealt out so that every cluster gets the same share
    // and no tile has more than two K-slices (see tail_unit).  `counters` then holds one hand-over flag per
    // (tail tile, CTA of the pair, epilogue warp).
    uint32_t sk_on, sk_full, sk_q, sk_r;
    // Die-aware walk (die_table != nullptr): the two dies of a B200 each have their own half of the L2, and a line
    // read by SMs of both dies occupies both halves.  Each rasterisation group of group_m M-tiles is cut in two:
    // the CTA pairs of die 0 walk the upper group_m / 2 M-tiles, those of die 1 the lower ones, both along N in
    // step.  The A panel of a group then lives in ONE half of the L2 (half the footprint per half, so it survives
    // from wave to wave) and only B is shared across the link.  die_table[smid] is measured once per process;
    // die_claim = {pairs of die 0 so far, of die 1, pairs finished} gives every pair a rank on its die.
    const unsigned char *die_table;
    uint32_t *die_claim;
    uint32_t *status;
    unsigned long long *prof;     // debug & 32: 16 cycle counters per CTA
};

struct WorkUnit {
    uint32_t m_blk, n_blk, batch, split;
    uint32_t kb_begin, kb_count;
    uint32_t role;        // 0: the tile's whole K range (or a K-split slice with its own output)
                          // 1: first K-slice of a shared tail tile: written to C, then the hand-over flag is raised
                          // 2: second K-slice of a shared tail tile: added to C once the flag is up
    uint32_t flag_tile;   // roles 1, 2: index of the tail tile (selects the flags)
    uint32_t k_down;      // the producer fetches this unit's K blocks last to first
};

__host__ __device__ __forceinline__ WorkUnit decode_unit(const TcParams &p, uint32_t u) {
    WorkUnit w;
    uint32_t t = u / p.splits;
    w.split = u - t * p.splits;
    uint32_t per_batch = p.m_tiles * p.n_tiles;
    w.batch = t / per_batch;
    uint32_t r = t - w.batch * per_batch;
    uint32_t gsz = p.group_m * p.n_tiles;
    uint32_t g = r / gsz;
    uint32_t first_m = g * p.group_m;
    uint32_t gm = p.m_tiles - first_m < p.group_m ? p.m_tiles - first_m : p.group_m;
    uint32_t in_g = r - g * gsz;
    w.m_blk = first_m + in_g % gm;
    w.n_blk = in_g / gm;
    if (p.serpentine && (g & 1u)) w.n_blk = p.n_tiles - 1 - w.n_blk;
    w.kb_begin = w.split * p.kb_per_split;
    uint32_t kb_end = w.kb_begin + p.kb_per_split;
    if (kb_end > p.k_blocks) kb_end = p.k_blocks;
    w.kb_count = kb_end - w.kb_begin;
    w.role = 0; w.flag_tile = 0; w.k_down = 0;
    return w;
}

// Balanced last wave.  R = T % S tail tiles (R < S) are handled by S clusters in G = S - R groups; a group of k
// tiles has k + 1 clusters (R = q G + r: the first r groups have k = q + 1 tiles, the others k = q).  Inside a group,
// tile t is shared by clusters t and t + 1 only:
//     cluster t + 1 computes K blocks [0, s_t)  first  (role 1: stores the partial tile, raises the flag),
//     cluster t     computes K blocks [s_t, KB) second (role 2: waits for the flag, adds its partial tile),
// with s_t = KB (t + 1) / (k + 1), so that every cluster multiplies KB k / (k + 1) blocks.  A cluster does its
// role-1 part before its role-2 part, so the part a role-2 unit waits for was started a whole role-1 part earlier
// than the role-2 unit itself: the wait is over before it begins, except for one pair per group whose two parts end
// together.  Each element of a shared tile is (slice 0) + (slice 1): two terms, one order, deterministic.
// j = 0, 1 enumerates the parts of cluster c; false when there is none.
__host__ __device__ inline bool tail_part(uint32_t q, uint32_t r, uint32_t KB, uint32_t c, uint32_t j, uint32_t &tile,
                                          uint32_t &kb_begin, uint32_t &kb_count, uint32_t &role) {
    const uint32_t big = r * (q + 2);
    uint32_t pos, k, tile0;
    if (c < big) {
        const uint32_t g = c / (q + 2);
        pos = c - g * (q + 2); k = q + 1; tile0 = g * (q + 1);
    } else {
        const uint32_t c2 = c - big, g = c2 / (q + 1);
        pos = c2 - g * (q + 1); k = q; tile0 = r * (q + 1) + g * q;
    }
    if (k == 0) return false;
    const bool has0 = pos >= 1, has1 = pos + 1 <= k;
    uint32_t which;
    if (j == 0) which = has0 ? 0u : 1u;
    else if (j == 1 && has0 && has1) which = 1u;
    else return false;
    const uint32_t t = which == 0 ? pos - 1 : pos;
    uint32_t split = (uint32_t)(((uint64_t)KB * (t + 1) + (k + 1) / 2) / (k + 1));
    split = split < 1 ? 1 : (split > KB - 1 ? KB - 1 : split);
    tile = tile0 + t;
    if (which == 0) { kb_begin = 0; kb_count = split; role = 1; }
    else { kb_begin = split; kb_count = KB - split; role = 2; }
    return true;
}
__host__ __device__ __noinline__ bool tail_unit(const TcParams &p, uint32_t c, uint32_t S, uint32_t j, WorkUnit &w) {
    uint32_t tile, kb_begin, kb_count, role;
    if (!tail_part(p.sk_q, p.sk_r, p.k_blocks, c, j, tile, kb_begin, kb_count, role)) return false;
    w = decode_unit(p, p.sk_full * S + tile);
    w.kb_begin = kb_begin; w.kb_count = kb_count; w.role = role; w.flag_tile = tile;
    return true;
}

// The i-th work unit of a cluster (i = 0, 1, ...); false past the last one.  Every role of the CTA (pair) walks the
// same sequence.
struct Walk { uint32_t id, count, die; };    // this CTA pair's position: id of count (on its die when die-aware)

__host__ __device__ __forceinline__ bool get_unit(const TcParams &p, const Walk &wk, uint32_t total_units, uint32_t i, WorkUnit &w) {
    if (p.die_table) {
        // this die's half of every group: h = group_m / 2 M-tiles x n_tiles, M fastest
        const uint32_t h = p.group_m >> 1, per_g = h * p.n_tiles;
        const uint32_t j = wk.id + i * wk.count;
        if (j >= (p.m_tiles >> 1) * p.n_tiles) return false;
        const uint32_t g = j / per_g, in_g = j - g * per_g;
        w.n_blk = in_g / h;
        w.m_blk = g * p.group_m + wk.die * h + (in_g - w.n_blk * h);
        if (p.serpentine && (g & 1u)) w.n_blk = p.n_tiles - 1 - w.n_blk;
        w.batch = 0; w.split = 0; w.kb_begin = 0; w.kb_count = p.k_blocks; w.role = 0; w.flag_tile = 0;
        w.k_down = p.k_serpentine & i;
        return true;
    }
    if (!p.sk_on) {
        const uint64_t u = (uint64_t)wk.id + (uint64_t)i * wk.count;
        if (u >= total_units) return false;
        w = decode_unit(p, (uint32_t)u);
        w.k_down = p.k_serpentine & i;
        return true;
    }
    if (i < p.sk_full) {
        w = decode_unit(p, wk.id + i * wk.count);
        return true;
    }
    return tail_unit(p, wk.id, wk.count, i - p.sk_full, w);
}

// Hand-over flag of a shared tail tile (global memory, gpu scope).
__device__ __forceinline__ void flag_raise(uint32_t *flag) {
    asm volatile("fence.proxy.async;" ::: "memory");      // the partial tile was written by bulk copies
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
}
// Whole warp; false when the wait ran out of time (2 s) or the CTA is aborting.
__device__ __noinline__ bool flag_wait(uint32_t *flag, volatile uint32_t *abort_flag, uint32_t *status) {
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (__all_sync(0xffffffffu, v != 0)) break;
        __nanosleep(128);
        uint32_t give_up = *abort_flag;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) give_up = 1;
        if (__any_sync(0xffffffffu, give_up)) {
            if ((threadIdx.x & 31) == 0) { *abort_flag = 1; atomicOr(status, DEV_ERR_WAIT_TILE_FLAG); }
            return false;
        }
    }
    asm volatile("fence.proxy.async;" ::: "memory");      // the add that follows is a bulk copy
    return true;
}

__device__ __forceinline__ uint32_t pack_bf16(uint32_t lo, uint32_t hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16(uint32_t lo, uint32_t hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
    return r;
}
__device__ __forceinline__ unsigned short f32_to_16(float v, uint32_t dtype16) {
    if (dtype16 == (uint32_t)DT_BF16) {
        uint32_t u = __float_as_uint(v);
        if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (unsigned short)(0x7FC0u | ((u >> 16) & 1u));
        u += 0x7FFFu + ((u >> 16) & 1u);
        return (unsigned short)(u >> 16);
    }
    unsigned short h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
    return h;
}

// Fused split-K reduction of one chunk (32 tile rows x `w` tile columns) by one warp: the K-slices
// are summed in slice order into Cout.  Each lane owns up to 32 elements; the loads of one slice are
// all issued before any is used.
//   transposed tile: lane = tile row (consecutive addresses of C), e = tile column
//   plain tile:      lane = tile column of the chunk,              e = tile row of the slab
// Kept out of line so that its registers do not weigh on the main loops.
__device__ __noinline__ void sum_slices_chunk(const TcParams &p, uint32_t row0, uint32_t col, uint32_t w, uint32_t lane) {
    constexpr uint32_t E = 16;
    const uint32_t row = row0 + lane;
    uint32_t n_e;
    bool lane_ok;
    uint64_t base, obase;
    if (p.c_trans) {
        n_e = (p.N - col) < w ? (p.N - col) : w;
        lane_ok = row < p.M;
        base = (uint64_t)col * p.ldc + row;
        obase = (uint64_t)col * p.ldc_out + row;
    } else {
        n_e = (p.M - row0) < 32u ? (p.M - row0) : 32u;
        lane_ok = lane < w && col + lane < p.N;
        base = (uint64_t)row0 * p.ldc + col + lane;
        obase = (uint64_t)row0 * p.ldc_out + col + lane;
    }
    if (!lane_ok) return;
    for (uint32_t e0 = 0; e0 < n_e; e0 += E) {
        float sum[E];
#pragma unroll
        for (uint32_t e = 0; e < E; ++e) sum[e] = e0 + e < n_e ? __ldcg(p.C + base + (uint64_t)(e0 + e) * p.ldc) : 0.0f;
        for (uint32_t sidx = 1; sidx < p.splits; ++sidx) {
            const float *sl = p.C + (uint64_t)sidx * p.c_stride + base;
#pragma unroll
            for (uint32_t e = 0; e < E; ++e)
                if (e0 + e < n_e) sum[e] += __ldcg(sl + (uint64_t)(e0 + e) * p.ldc);
        }
#pragma unroll
        for (uint32_t e = 0; e < E; ++e) {
            if (e0 + e < n_e) {
                float *d = p.Cout + obase + (uint64_t)(e0 + e) * p.ldc_out;
                *d = p.accumulate ? *d + sum[e] : sum[e];
            }
        }
    }
}

// The K passes this launch really runs: those of the host's list whose pieces both hold a non-zero element.  The
// list ends with the pass over the leading pieces (0, 0); it is kept when nothing else is, so that C is still
// written.  Every role computes the same answer from the same two device words.
struct PassList { uint32_t n, a_sel, b_sel; };
__device__ __forceinline__ PassList effective_passes(const TcParams &p) {
    PassList l = {p.npass, p.a_sel, p.b_sel};
    if (!p.a_piece_mask && !p.b_piece_mask) return l;
    const uint32_t ma = p.a_piece_mask ? *reinterpret_cast<const volatile uint32_t *>(p.a_piece_mask) : 0xFFFFFFFFu;
    const uint32_t mb = p.b_piece_mask ? *reinterpret_cast<const volatile uint32_t *>(p.b_piece_mask) : 0xFFFFFFFFu;
    l.n = 0; l.a_sel = 0; l.b_sel = 0;
    for (uint32_t pass = 0; pass < p.npass; ++pass) {
        const uint32_t ai = (p.a_sel >> (4 * pass)) & 0xF, bi = (p.b_sel >> (4 * pass)) & 0xF;
        if (((ma >> ai) & 1u) && ((mb >> bi) & 1u)) {
            l.a_sel |= ai << (4 * l.n); l.b_sel |= bi << (4 * l.n); ++l.n;
        }
    }
    if (l.n == 0) {
        l.n = 1;
        l.a_sel = (p.a_sel >> (4 * (p.npass - 1))) & 0xF;
        l.b_sel = (p.b_sel >> (4 * (p.npass - 1))) & 0xF;
    }
    return l;
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int CG, int BN, int SUB, bool STAGING, int EW, int EB>
__global__ void __launch_bounds__(32 * (2 + EW), 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const TcParams p) {
    using C_ = Cfg<CG, BN, SUB, STAGING, EW, EB>;
    constexpr uint32_t EPI_WARPS = EW, EPI_BUFS = EB;
    constexpr uint32_t STAGES = C_::STAGES;     // allocated; p.stages of them are cycled through
    const uint32_t nstages = p.stages;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // timing experiments: wall-clock nanoseconds at which this CTA started / set up / ended (counters 14, 15, 7)
    if (PG_DBG(32u) && p.prof && threadIdx.x == 0) p.prof[(size_t)blockIdx.x * 16 + 14] = globaltimer_ns();

    const uint32_t stage_base = smem_base;
    const uint32_t epi_base = smem_base + STAGES * C_::STAGE_BYTES;
    const uint32_t bar_base = epi_base + C_::EPI_BYTES;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](uint32_t s) { return bar_base + 8u * (2 * STAGES + s); };
    auto tmem_empty_bar = [&](uint32_t s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
    const uint32_t abort_off = (bar_base - smem_base) + 8u * (2 * STAGES + 4) + 8u;
    const uint32_t red_bar = bar_base + 8u * (2 * STAGES + 4) + 16u;   // cluster reduction: partial tiles have landed
    const uint32_t die_slot = bar_base + 8u * (2 * STAGES + 4) + 24u;  // die-aware walk: this pair's (die, rank)
    volatile uint32_t *tmem_slot_gen = (volatile uint32_t *)(smem_gen + (tmem_slot - smem_base));
    volatile uint32_t *abort_flag = (volatile uint32_t *)(smem_gen + abort_off);

    // warp index through a shuffle, so that the compiler knows it is the same in all lanes
    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0;
    const uint32_t cluster_id = blockIdx.x / CG;
    const uint32_t num_clusters = gridDim.x / CG;
    const uint32_t total_units = p.batch * p.m_tiles * p.n_tiles * p.splits;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        prefetch_tmap(&map_a);
        prefetch_tmap(&map_b);
        if (p.epilogue_tma) prefetch_tmap(&map_c);
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(tmem_full_bar(s), 1);
            mbar_init(tmem_empty_bar(s), EPI_WARPS * CG);
        }
        mbar_init(red_bar, p.cluster_k > 1 ? (p.cluster_k - 1) * EPI_WARPS * 32 : 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<CG>(tmem_slot, C_::TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tc_fence_before();
    // (a cluster of K-slices: every CTA must be running and its barriers initialised before a peer touches them)
    if (CG == 2 || p.cluster_k > 1) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;
    // Programmatic dependent launch: everything above touched no global memory, so it may run while the previous
    // kernel of the stream is still finishing; from here on its results (and its hand-over flags) are needed.  The
    // next kernel of the stream may be scheduled as soon as SMs become free (its own prologue then waits here).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const PassList passes = effective_passes(p);
    Walk walk = {cluster_id, num_clusters, 0};
    if (p.die_table) {
        // Which die is this CTA pair on, and the how-manieth pair of that die is it?  A die with more than half of
        // the pairs hands its surplus to the ranks the other die leaves unclaimed (exactly as many: the grid is
        // num_clusters pairs), so every (die, rank) is taken once whatever the placement.
        volatile uint32_t *slot = (volatile uint32_t *)(smem_gen + (die_slot - smem_base));
        if (threadIdx.x == 0 && cta_rank == 0) {
            uint32_t smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            uint32_t d = p.die_table[smid & 255u] & 1u;
            uint32_t r = atomicAdd(p.die_claim + d, 1u);
            const uint32_t half = num_clusters >> 1;
            if (r >= half) { d ^= 1u; r = 2u * half - 1u - r; }
            const uint32_t word = d | (r << 8);
            *slot = word;
            if constexpr (CG == 2) {
                asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa(die_slot, 1)), "r"(word) : "memory");
            }
        }
        if (CG == 2) cluster_sync_all(); else __syncthreads();
        const uint32_t word = *slot;
        walk.die = word & 1u;
        walk.id = word >> 8;
        walk.count = num_clusters >> 1;
    }
    if (PG_DBG(32u) && p.prof && threadIdx.x == 0) p.prof[(size_t)blockIdx.x * 16 + 7] = globaltimer_ns();

    // Each role loop below is executed by its whole warp with warp-uniform state; the instructions
    // that must come from one thread (TMA, tcgen05.mma, tcgen05.commit, barrier arrives) sit under
    // elect_one().
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        const bool prof = PG_DBG(32u);
        long long tp_wait = 0, tp_issue = 0;
        const uint64_t pol_a = l2_policy((int)(p.l2_hints & 3u)), pol_b = l2_policy((int)((p.l2_hints >> 2) & 3u));
        for (uint32_t ui = 0; ok; ++ui) {
            WorkUnit w;
            if (!get_unit(p, walk, total_units, ui, w)) break;
            const int32_t m0 = (int32_t)(w.m_blk * BM_CTA * CG + cta_rank * BM_CTA);
            const int32_t n0 = (int32_t)(w.n_blk * BN + cta_rank * C_::BN_CTA);
            const uint32_t rounds = (w.kb_count + SUB - 1) / SUB;
            for (uint32_t pass = 0; pass < passes.n && ok; ++pass) {
                // a unit that runs K downwards also takes its passes last to first: it begins on the very
                // blocks (same pieces, same K) the unit before it ended on
                const uint32_t ps = w.k_down ? passes.n - 1 - pass : pass;
                const int32_t za = (int32_t)(w.batch * p.a_nparts + ((passes.a_sel >> (4 * ps)) & 0xF));
                const int32_t zb = (int32_t)(w.batch * p.b_nparts + ((passes.b_sel >> (4 * ps)) & 0xF));
                for (uint32_t r = 0; r < rounds; ++r) {
                    long long c0 = prof ? clock64() : 0;
                    ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY);
                    if (!ok) break;
                    long long c1 = prof ? clock64() : 0;
                    // the barrier that counts this stage's bytes: the leader CTA's when paired
                    uint32_t bar = full_bar(stage);
                    if constexpr (CG == 2) bar = mapa(bar, 0);
                    const uint32_t sbase = stage_base + stage * C_::STAGE_BYTES;
                    const int32_t kbase = (int32_t)((w.kb_begin + (w.k_down ? rounds - 1 - r : r) * SUB) * BK);
                    if (elect_one()) {
                        if PG_DBG(1u) {
                            if (cta_rank == 0) mbar_arrive(full_bar(stage));
                        } else {
                            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), C_::STAGE_BYTES * CG);
#pragma unroll
                            for (uint32_t j = 0; j < (uint32_t)SUB; ++j) {
                                // a K block past the end of K is all zero fill (and still counts its bytes)
                                const int32_t k0 = kbase + (int32_t)(j * BK);
                                const uint32_t sa = sbase + j * C_::SUB_BYTES;
                                const uint32_t sb = sa + A_TILE_BYTES;
                                if (!p.a_mn) {
                                    tma_load_3d<CG>(sa, &map_a, bar, k0, m0, za, pol_a);
                                } else {
#pragma unroll
                                    for (uint32_t c = 0; c < BM_CTA / 64; ++c)
                                        tma_load_3d<CG>(sa + c * (BK * 128), &map_a, bar, m0 + (int32_t)(c * 64), k0, za, pol_a);
                                }
                                if (!p.b_mn) {
                                    tma_load_3d<CG>(sb, &map_b, bar, k0, n0, zb, pol_b);
                                } else if constexpr (C_::BN_CTA >= 64) {   // narrower tiles take a K-major B only
#pragma unroll
                                    for (uint32_t c = 0; c < C_::BN_CTA / 64; ++c)
                                        tma_load_3d<CG>(sb + c * (BK * 128), &map_b, bar, n0 + (int32_t)(c * 64), k0, zb, pol_b);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (prof) { tp_wait += c1 - c0; tp_issue += clock64() - c1; }
                    if (++stage == nstages) { stage = 0; phase ^= 1; }
                }
            }
        }
        if (prof && lane == 0) {
            unsigned long long *o = p.prof + (size_t)blockIdx.x * 16;
            o[8] = (unsigned long long)tp_wait; o[9] = (unsigned long long)tp_issue;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA) ------------------------------
        // The tensor core queues only about two MMAs ahead of the one it executes (measured: the
        // issue of a third blocks), so whatever happens between MMAs must fit in the time two of
        // them take.  Hence the order inside a round: issue the first half of the round's MMAs,
        // THEN wait for the next round's bytes, then issue the second half and release this
        // round's stage (a tcgen05.commit costs ~100 cycles) while those are still executing.
        if (cta_rank == 0) {
            constexpr uint32_t MMAS = SUB * (BK / UMMA_K);        // per round
            constexpr uint32_t HALF = MMAS / 2;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            const uint32_t a_lbo = p.a_mn ? BK * 128 : 0;
            const uint32_t b_lbo = p.b_mn ? BK * 128 : 0;
            const uint32_t a_k1 = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4, a_k2 = 2 * a_k1, a_k3 = 3 * a_k1;
            const uint32_t b_k1 = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4, b_k2 = 2 * b_k1, b_k3 = 3 * b_k1;
            const uint64_t desc_a0 = make_desc(stage_base, a_lbo);
            const uint64_t desc_b0 = make_desc(stage_base + A_TILE_BYTES, b_lbo);
            const uint32_t a_hi = (uint32_t)(desc_a0 >> 32), b_hi = (uint32_t)(desc_b0 >> 32);
            const uint32_t a_lo0 = (uint32_t)desc_a0, b_lo0 = (uint32_t)desc_b0;
            const uint32_t idesc = p.idesc;
            bool ok = true;
            bool ready = false;             // full_bar(stage) has already been seen complete
            const bool prof = PG_DBG(32u);
            long long t_wait = 0, t_issue = 0, t_commit = 0, t_tmem = 0, t_all = prof ? clock64() : 0, n_rounds = 0;

            auto issue = [&](uint32_t m, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t nsub, uint32_t accum) {
                const uint32_t j = m / (BK / UMMA_K), kk = m % (BK / UMMA_K);
                if (SUB > 1 && j >= nsub) return;
                const uint32_t ak = kk == 0 ? 0u : (kk == 1 ? a_k1 : (kk == 2 ? a_k2 : a_k3));
                const uint32_t bk = kk == 0 ? 0u : (kk == 1 ? b_k1 : (kk == 2 ? b_k2 : b_k3));
                umma_lohi<CG>(d_tmem, a_lo + j * (C_::SUB_BYTES >> 4) + ak, a_hi, b_lo + j * (C_::SUB_BYTES >> 4) + bk,
                              b_hi, idesc, accum);
            };

            WorkUnit w, w_next;
            bool have = get_unit(p, walk, total_units, 0, w);
            for (uint32_t ui = 0; have && ok; ++ui, w = w_next) {
                const bool more_units = get_unit(p, walk, total_units, ui + 1, w_next);
                have = more_units;
                long long c0 = prof ? clock64() : 0;
                ok = mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                if (prof) t_tmem += clock64() - c0;
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t rounds = (w.kb_count + SUB - 1) / SUB;
                const uint32_t iters = passes.n * rounds;
                uint32_t r = 0;
                for (uint32_t it = 0; it < iters; ++it) {
                    long long c1 = prof ? clock64() : 0;
                    if (!ready) {
                        ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, DEV_ERR_WAIT_FULL);
                        if (!ok) break;
                    }
                    long long c2 = prof ? clock64() : 0;
                    const uint32_t soff = stage * (C_::STAGE_BYTES >> 4);
                    const uint32_t a_lo = a_lo0 + soff, b_lo = b_lo0 + soff;
                    uint32_t nsub = SUB;
                    if (SUB > 1 && w.kb_count - r * SUB < (uint32_t)SUB) nsub = w.kb_count - r * SUB;  // rest belongs to the next split
                    const bool do_mma = !PG_DBG(16u);
                    if (elect_one()) {
                        if (do_mma) {
#pragma unroll
                            for (uint32_t m = 0; m < HALF; ++m) issue(m, d_tmem, a_lo, b_lo, nsub, (it | m) ? 1u : 0u);
                        }
                    }
                    __syncwarp();
                    long long c3 = prof ? clock64() : 0;
                    uint32_t ns = stage + 1, np = phase;
                    if (ns == nstages) { ns = 0; np ^= 1; }
                    if (it + 1 < iters || more_units) {
                        ok = mbar_wait(full_bar(ns), np, abort_flag, p.status, DEV_ERR_WAIT_FULL);
                        if (!ok) break;
                        ready = true;
                    } else {
                        ready = false;
                    }
                    long long c4 = prof ? clock64() : 0;
                    const bool last = it + 1 == iters;
                    if (elect_one()) {
                        if (do_mma) {
#pragma unroll
                            for (uint32_t m = HALF; m < MMAS; ++m) issue(m, d_tmem, a_lo, b_lo, nsub, 1u);
                        }
                        umma_commit<CG>(empty_bar(stage));                  // frees this round's stage
                        if (last) umma_commit<CG>(tmem_full_bar(acc));      // accumulator complete
                    }
                    __syncwarp();
                    if (prof) {
                        long long c5 = clock64();
                        t_wait += (c2 - c1) + (c4 - c3); t_issue += (c3 - c2) + (c5 - c4); ++n_rounds;
                    }
                    if (++r == rounds) r = 0;
                    stage = ns; phase = np;
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
            if (prof && lane == 0) {
                unsigned long long *o = p.prof + (size_t)blockIdx.x * 16;
                o[0] = (unsigned long long)(clock64() - t_all); o[1] = (unsigned long long)t_wait;
                o[2] = (unsigned long long)t_issue; o[3] = (unsigned long long)t_commit;
                o[4] = (unsigned long long)t_tmem; o[5] = (unsigned long long)n_rounds;
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        constexpr uint32_t W = C_::EPI_W;               // columns per chunk
        constexpr uint32_t CHUNKS = BN / W;
        const uint32_t q = warp & 3;                    // TMEM lane quadrant this warp may read
        const uint32_t ew = warp - 2;                   // 0 .. EW-1
        const uint32_t half = ew >> 2;                  // with 8 warps: which of the alternating chunks
        constexpr uint32_t CSTEP = EW / 4;
        const uint32_t my_epi = epi_base + ew * EPI_BUFS * EPI_BUF_BYTES;
        uint8_t *my_epi_gen = smem_gen + (my_epi - smem_base);
        uint32_t acc = 0, acc_phase = 0;
        uint32_t buf = 0;
        bool ok = true;
        const bool cluster_mode = CG == 1 && BN <= 32 && STAGING && p.cluster_k > 1;
        const bool fused = p.splits > 1 && p.Cout != nullptr && !cluster_mode;
        const uint64_t pol_c = l2_policy((int)((p.l2_hints >> 4) & 3u)), pol_keep = l2_policy(0);
        const bool prof = PG_DBG(32u) && ew == 0;
        long long te_wait = 0, te_ld = 0, te_math = 0, te_store = 0, last_e3 = 0;
        for (uint32_t ui = 0; ok; ++ui) {
            WorkUnit w;
            if (!get_unit(p, walk, total_units, ui, w)) break;
            // Bias of a chunk: lane l holds bias[col + l], fetched one chunk ahead (the first one before the
            // wait for the accumulator) and handed round by shuffles, so no chunk waits for a load.
            auto bias_fetch = [&](uint32_t c) -> float {
                const uint32_t bc = w.n_blk * BN + c * W + lane;
                return (p.bias && c < CHUNKS && lane < W && bc < p.N) ? __ldg(p.bias + bc) : 0.0f;
            };
            float bias_next = bias_fetch(half);
            long long e0 = prof ? clock64() : 0;
            ok = mbar_wait_patient(tmem_full_bar(acc), acc_phase, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            if (prof) te_wait += clock64() - e0;
            const uint32_t row0 = w.m_blk * BM_CTA * CG + cta_rank * BM_CTA + q * 32;  // first row of this warp
            const uint32_t col0 = w.n_blk * BN;
            const uint32_t zc = p.splits > 1 ? w.split : w.batch;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * BN;
            const uint32_t row = row0 + lane;
            float *cbase = p.C + (uint64_t)zc * p.c_stride;
            const bool accum = p.accumulate && !fused;      // K-slices are plain stores; only the final sum accumulates
            // shared tail tile: hand-over flag of this warp's slab; the second slice is added to the first
            uint32_t *tile_flag = w.role ? p.counters + ((w.flag_tile * CG + cta_rank) * EPI_WARPS + ew) : nullptr;
            bool flag_pending = w.role == 2;
            if constexpr (CG == 1 && BN <= 32 && STAGING) {
                if (cluster_mode) {
                    // Split-K inside a cluster: CTA r of the cluster holds K-slice r of this tile (one chunk of
                    // W = BN columns per warp).  Slices 1.. write their 32 x W partial sums into the leader's
                    // staging area through distributed shared memory and arrive on its barrier; the leader adds
                    // them to its own registers in slice order and writes C.  No global round trip, no atomics.
                    static_assert(CHUNKS == 1, "one chunk per warp");
                    const uint32_t rank = cluster_ctarank();
                    uint32_t v[32];
                    if constexpr (W == 32) tmem_ld32(taddr, v); else tmem_ld16(taddr, v);
                    tmem_ld_wait();
                    constexpr uint32_t SLOT = 32 * W * 4;                 // one warp's partial of one slice
                    if (rank != 0) {
                        const uint32_t dst = mapa(epi_base + ((rank - 1) * 4 + q) * SLOT + lane * (W * 4), 0);
#pragma unroll
                        for (uint32_t j = 0; j < W / 4; ++j) st_cluster_v4(dst + 16 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        mbar_arrive_release_cluster(mapa(red_bar, 0));
                    } else {
                        const uint64_t t0 = globaltimer_ns();
                        bool landed = true;
                        while (!__all_sync(0xffffffffu, mbar_try_acquire_cluster(red_bar, 0))) {
                            uint32_t give_up = *abort_flag;
                            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) give_up = 1;
                            if (__any_sync(0xffffffffu, give_up)) {
                                if (lane == 0) { *abort_flag = 1; atomicOr(p.status, DEV_ERR_WAIT_TMEM_FULL); }
                                landed = false;
                                break;
                            }
                        }
                        if (landed && !PG_DBG(2u)) {
                            for (uint32_t r = 1; r < p.cluster_k; ++r) {
                                const uint4 *src = reinterpret_cast<const uint4 *>(smem_gen + (epi_base - smem_base) + ((r - 1) * 4 + q) * SLOT + lane * (W * 4));
#pragma unroll
                                for (uint32_t j = 0; j < W / 4; ++j) {
                                    const uint4 t4 = src[j];
                                    v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + __uint_as_float(t4.x));
                                    v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + __uint_as_float(t4.y));
                                    v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + __uint_as_float(t4.z));
                                    v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + __uint_as_float(t4.w));
                                }
                            }
                            if (row < p.M) {
                                float *out = p.Cout + (uint64_t)w.batch * p.M * p.ldc_out;
#pragma unroll
                                for (uint32_t j = 0; j < W; ++j) {
                                    if (col0 + j < p.N) {
                                        float *d = p.c_trans ? out + (uint64_t)(col0 + j) * p.ldc_out + row : out + (uint64_t)row * p.ldc_out + col0 + j;
                                        *d = p.accumulate ? *d + __uint_as_float(v[j]) : __uint_as_float(v[j]);
                                    }
                                }
                            }
                        }
                        if (!landed) ok = false;
                    }
                }
            }
#pragma unroll 1
            for (uint32_t c = half; c < CHUNKS && !cluster_mode; c += CSTEP) {
                const uint32_t col = col0 + c * W;
                if (col >= p.N || row0 >= p.M) break;   // nothing of this warp's slab is inside C
                if PG_DBG(4u) break;
                uint32_t v[32];
                const float bias_cur = bias_next;
                bias_next = bias_fetch(c + CSTEP);
                long long e1 = prof ? clock64() : 0;
                if (prof && last_e3) te_store += e1 - last_e3;
                if constexpr (W == 32) tmem_ld32(taddr + c * W, v); else tmem_ld16(taddr + c * W, v);
                tmem_ld_wait();
                long long e2 = prof ? clock64() : 0;
                if PG_DBG(2u) continue;
                if (p.bias || p.act || p.c16) {
                    // bias and activation on the f32 accumulators, in registers (no split/partial route reaches here)
                    if (p.bias) {
#pragma unroll
                        for (uint32_t j = 0; j < W; ++j)
                            v[j] = __float_as_uint(__uint_as_float(v[j]) + __shfl_sync(0xffffffffu, bias_cur, j));
                    }
                    // u: what the 16-bit copy receives.  Normally C gets the same; with act_copy_only C keeps the
                    // value before the activation (a training step needs it for the backward pass) and only the
                    // copy is activated.
                    uint32_t u[32];
#pragma unroll
                    for (uint32_t j = 0; j < W; ++j) u[j] = v[j];
                    if (p.act == 1) {
#pragma unroll
                        for (uint32_t j = 0; j < W; ++j) u[j] = __float_as_uint(fmaxf(__uint_as_float(u[j]), 0.0f));
                    } else if (p.act == 2) {
#pragma unroll
                        for (uint32_t j = 0; j < W; ++j) u[j] = __float_as_uint(gelu_erf(__uint_as_float(u[j])));
                    }
                    if (!p.act_copy_only) {
#pragma unroll
                        for (uint32_t j = 0; j < W; ++j) v[j] = u[j];
                    }
                    if (p.c16 && row < p.M) {
                        unsigned short *d16 = p.c16 + (uint64_t)zc * p.M * p.ld16 + (uint64_t)row * p.ld16 + col;
                        if (p.c16_vec && col + W <= p.N && row0 + 32 <= p.M) {
                            // A lane's W values are W/8 16-byte pieces of its row.  Neighbouring lanes swap
                            // every other piece, so that each store instruction writes whole 32-byte sectors:
                            // the even lane's row in one instruction, the odd lane's row in the next.
                            const bool odd = lane & 1u;
                            unsigned short *pair_row = p.c16 + (uint64_t)zc * p.M * p.ld16 + (uint64_t)(row & ~1u) * p.ld16 + col;
#pragma unroll
                            for (uint32_t j = 0; j < W; j += 16) {
                                uint4 lo, hi;           // pieces j/8 and j/8 + 1 of this lane's row
                                if (p.dtype16 == (uint32_t)DT_BF16) {
                                    lo = make_uint4(pack_bf16(u[j], u[j + 1]), pack_bf16(u[j + 2], u[j + 3]),
                                                    pack_bf16(u[j + 4], u[j + 5]), pack_bf16(u[j + 6], u[j + 7]));
                                    hi = make_uint4(pack_bf16(u[j + 8], u[j + 9]), pack_bf16(u[j + 10], u[j + 11]),
                                                    pack_bf16(u[j + 12], u[j + 13]), pack_bf16(u[j + 14], u[j + 15]));
                                } else {
                                    lo = make_uint4(pack_f16(u[j], u[j + 1]), pack_f16(u[j + 2], u[j + 3]),
                                                    pack_f16(u[j + 4], u[j + 5]), pack_f16(u[j + 6], u[j + 7]));
                                    hi = make_uint4(pack_f16(u[j + 8], u[j + 9]), pack_f16(u[j + 10], u[j + 11]),
                                                    pack_f16(u[j + 12], u[j + 13]), pack_f16(u[j + 14], u[j + 15]));
                                }
                                uint4 give = odd ? lo : hi, got;
                                got.x = __shfl_xor_sync(0xffffffffu, give.x, 1);
                                got.y = __shfl_xor_sync(0xffffffffu, give.y, 1);
                                got.z = __shfl_xor_sync(0xffffffffu, give.z, 1);
                                got.w = __shfl_xor_sync(0xffffffffu, give.w, 1);
                                // even row: even lane writes its lo, odd lane the even lane's hi
                                *reinterpret_cast<uint4 *>(pair_row + j + (odd ? 8 : 0)) = odd ? got : lo;
                                // odd row: even lane writes the odd lane's lo, odd lane its own hi
                                *reinterpret_cast<uint4 *>(pair_row + p.ld16 + j + (odd ? 8 : 0)) = odd ? hi : got;
                            }
                        } else if (p.c16_vec && col + W <= p.N) {
                            if (p.dtype16 == (uint32_t)DT_BF16) {
#pragma unroll
                                for (uint32_t j = 0; j < W; j += 8)
                                    *reinterpret_cast<uint4 *>(d16 + j) =
                                        make_uint4(pack_bf16(u[j], u[j + 1]), pack_bf16(u[j + 2], u[j + 3]),
                                                   pack_bf16(u[j + 4], u[j + 5]), pack_bf16(u[j + 6], u[j + 7]));
                            } else {
#pragma unroll
                                for (uint32_t j = 0; j < W; j += 8)
                                    *reinterpret_cast<uint4 *>(d16 + j) =
                                        make_uint4(pack_f16(u[j], u[j + 1]), pack_f16(u[j + 2], u[j + 3]),
                                                   pack_f16(u[j + 4], u[j + 5]), pack_f16(u[j + 6], u[j + 7]));
                            }
                        } else {
#pragma unroll
                            for (uint32_t j = 0; j < W; ++j)
                                if (col + j < p.N) d16[j] = f32_to_16(__uint_as_float(u[j]), p.dtype16);
                        }
                    }
                }
                long long e3 = prof ? clock64() : 0;
                if (prof) { te_ld += e2 - e1; te_math += e3 - e2; last_e3 = e3; }
                if (STAGING && p.epilogue_tma) {
                    // the store issued EPI_BUFS chunks ago must have finished reading this buffer
                    if (lane == 0) tma_store_wait_read<EPI_BUFS - 1>();
                    __syncwarp();
                    uint8_t *dst = my_epi_gen + buf * EPI_BUF_BYTES + lane * 128;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        uint4 val = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        *reinterpret_cast<uint4 *>(dst + ((j ^ (lane & 7)) << 4)) = val;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (flag_pending) {
                        // the first K-slice of this slab must be in C before anything is added to it
                        ok = flag_wait(tile_flag, abort_flag, p.status);
                        flag_pending = false;
                        if (!ok) break;
                    }
                    if (lane == 0) {
                        if (accum || w.role == 2)
                            tma_reduce_add_3d(&map_c, my_epi + buf * EPI_BUF_BYTES, (int32_t)col, (int32_t)row0, (int32_t)zc);
                        else   // a slab that a second slice will be added to should not leave L2 first
                            tma_store_3d(&map_c, my_epi + buf * EPI_BUF_BYTES, (int32_t)col, (int32_t)row0, (int32_t)zc,
                                         w.role == 1 ? pol_keep : pol_c);
                        tma_store_commit();
                    }
                    if (p.n_extra) {
                        // Further destinations (other devices' C): while the bulk store above reads the staged chunk,
                        // the warp reads it back row-wise and writes it with plain 16-byte stores, 8 lanes per
                        // 128-byte row piece, 4 rows per instruction.  (One more bulk store per destination was
                        // measured slower over NVLink: 0.434 against 0.410 ms for product + exchange at 4 GPUs.)
                        const uint32_t piece = lane & 7u;
                        const uint8_t *src = my_epi_gen + buf * EPI_BUF_BYTES;
                        const bool col_ok = col + piece * 4 < p.N;            // N is a multiple of 4 on this route
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) {
                            const uint32_t r = 4 * i + (lane >> 3);
                            const uint4 val = *reinterpret_cast<const uint4 *>(src + r * 128 + ((piece ^ (r & 7u)) << 4));
                            if (col_ok && row0 + r < p.M) {
                                const uint64_t off = (uint64_t)(row0 + r) * p.ldc + col + piece * 4;
                                for (uint32_t d = 0; d < p.n_extra; ++d)
                                    *reinterpret_cast<uint4 *>(p.extra_c[d] + off) = val;
                            }
                        }
                    }
                    if (++buf == EPI_BUFS) buf = 0;
                } else if (p.c_trans) {
                    // swapped operands: this lane's row is a COLUMN of C, so for each j the warp writes
                    // 32 consecutive floats
                    if (row < p.M) {
#pragma unroll
                        for (uint32_t j = 0; j < W; ++j) {
                            if (col + j < p.N) {
                                float *d = cbase + (uint64_t)(col + j) * p.ldc + row;
                                *d = accum ? *d + __uint_as_float(v[j]) : __uint_as_float(v[j]);
                            }
                        }
                    }
                } else {
                    if (row < p.M) {
                        float *crow = cbase + (uint64_t)row * p.ldc + col;
                        if (accum) {
#pragma unroll
                            for (uint32_t j = 0; j < W; ++j)
                                if (col + j < p.N) crow[j] += __uint_as_float(v[j]);
                        } else if (p.c_vec4 && col + W <= p.N) {
#pragma unroll
                            for (uint32_t j = 0; j < W / 4; ++j)
                                *reinterpret_cast<uint4 *>(crow + 4 * j) =
                                    make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        } else {
#pragma unroll
                            for (uint32_t j = 0; j < W; ++j)
                                if (col + j < p.N) crow[j] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            // all TMEM reads of this accumulator are done: hand it back to the MMA issuer
            if (prof && last_e3) { te_store += clock64() - last_e3; last_e3 = 0; }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                uint32_t bar = tmem_empty_bar(acc);
                if constexpr (CG == 2) {
                    mbar_arrive_cluster(mapa(bar, 0));
                } else {
                    mbar_arrive(bar);
                }
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }

            if (w.role == 1) {
                // first slice: once this warp's stores have completed, raise the flag of its slab
                if (lane == 0) {
                    tma_store_wait_all();
                    flag_raise(tile_flag);
                }
                __syncwarp();
            } else if (w.role == 2 && ok) {
                // second slice: consume the flag (also when no chunk of this slab lay inside C) and re-arm it
                if (flag_pending) ok = flag_wait(tile_flag, abort_flag, p.status);
                if (lane == 0) *tile_flag = 0;
            }
            if (fused && row0 < p.M && !PG_DBG(6u)) {
                // Fused split-K reduction.  This warp's slab of slice `split` is in global memory
                // (plain stores); publish it and count.  The warp that finds all other slices already
                // counted sums the slab over the slices in slice order — the result does not depend on
                // which warp arrives last — writes it to Cout and re-arms the counter.
                const uint32_t slab = (((w.m_blk * p.n_tiles + w.n_blk) * CG + cta_rank) * EPI_WARPS) + ew;
                __threadfence();
                __syncwarp();
                uint32_t old = 0;
                if (lane == 0) old = atomicAdd(p.counters + slab, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == p.splits - 1) {
                    __threadfence();
                    for (uint32_t c = half; c < CHUNKS; c += CSTEP) {
                        const uint32_t col = col0 + c * W;
                        if (col >= p.N) break;
                        sum_slices_chunk(p, row0, col, W, lane);
                    }
                    __syncwarp();
                    if (lane == 0) p.counters[slab] = 0;
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
        if (prof && lane == 0) {
            unsigned long long *o = p.prof + (size_t)blockIdx.x * 16;
            o[10] = (unsigned long long)te_wait; o[11] = (unsigned long long)te_ld;
            o[12] = (unsigned long long)te_math; o[13] = (unsigned long long)te_store;
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    // (K-slices as a cluster: no CTA may leave while a peer can still write into its shared memory)
    if (CG == 2 || p.cluster_k > 1) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CG>(tmem_base, C_::TMEM_COLS);
    }
    if (p.die_table && threadIdx.x == 0 && cta_rank == 0) {
        // the last pair to finish re-arms the claim counters for the next launch
        __threadfence();
        if (atomicAdd(p.die_claim + 2, 1u) == num_clusters - 1) {
            p.die_claim[0] = 0; p.die_claim[1] = 0; p.die_claim[2] = 0;
            __threadfence();
        }
    }
    if (PG_DBG(32u) && p.prof && threadIdx.x == 0) p.prof[(size_t)blockIdx.x * 16 + 15] = globaltimer_ns();
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait: a barrier that nothing will ever complete.  The warp polls it with
// the same spin primitive as the GEMM roles, gives up after `limit_ns`, records DEV_ERR_SELFTEST in
// the status word and returns normally — no trap, no fault, the context stays usable.
// ---------------------------------------------------------------------------------------------
__global__ void wait_timeout_selftest_kernel(uint32_t *status, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncthreads();
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        const uint32_t done = mbar_spin(b, 0, 64);
        if (__all_sync(0xffffffffu, done)) return;          // cannot happen: nobody arrives
        if (globaltimer_ns() - t0 > limit_ns) break;
    }
    if (threadIdx.x == 0) atomicOr(status, DEV_ERR_SELFTEST);
}

int wait_timeout_selftest_launch(uint32_t *status, unsigned limit_ms, cudaStream_t stream) {
    if (limit_ms > 1000) limit_ms = 1000;                   // a second at most
    wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(status, (unsigned long long)limit_ms * 1000000ull);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_GEMM;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct TcConfig {
    const char *name;
    int cg, bn, sub;
    bool staging;
    int ew;
    bool auto_ok;          // may be picked by the cost model (others only by hand or by a dedicated route)
    uint32_t smem, stages, threads;
    const void *fn;
};

#define PG_TC_CFG(NAME, CG_, BN_, SUB_, STG_, EW_, EB_, AUTO_) \
    {NAME, CG_, BN_, SUB_, STG_, EW_, AUTO_, Cfg<CG_, BN_, SUB_, STG_, EW_, EB_>::SMEM_BYTES, \
     Cfg<CG_, BN_, SUB_, STG_, EW_, EB_>::STAGES, Cfg<CG_, BN_, SUB_, STG_, EW_, EB_>::THREADS, \
     (const void *)tc_gemm_kernel<CG_, BN_, SUB_, STG_, EW_, EB_>}
static const TcConfig g_cfgs[] = {
    PG_TC_CFG("1cta_128x256", 1, 256, 1, true, 4, 2, true),
    PG_TC_CFG("1cta_128x128", 1, 128, 1, true, 4, 2, true),
    PG_TC_CFG("1cta_128x64", 1, 64, 1, true, 4, 2, true),
    PG_TC_CFG("2cta_256x256", 2, 256, 1, true, 4, 2, true),
    PG_TC_CFG("2cta_256x128", 2, 128, 1, true, 4, 2, true),
    PG_TC_CFG("1cta_128x16_t", 1, 16, 1, true, 4, 2, false),      // swapped operands for M <= 16 (staging area = cluster reduction)
    PG_TC_CFG("1cta_128x32_t", 1, 32, 1, true, 4, 2, false),      // swapped operands for M <= 32
};
constexpr int NUM_CFGS = sizeof(g_cfgs) / sizeof(g_cfgs[0]);

int tc_num_configs() { return NUM_CFGS; }
const char *tc_config_name(int cfg) { return (cfg >= 0 && cfg < NUM_CFGS) ? g_cfgs[cfg].name : "?"; }

int tc_config_index(const char *name) {
    for (int i = 0; i < NUM_CFGS; ++i)
        if (!strcmp(g_cfgs[i].name, name)) return i;
    return -1;
}

static bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

bool tc_gemm_supported(const TcGemm &g) {
    if (g.dtype != DT_F16 && g.dtype != DT_BF16) return false;
    if (g.M == 0 || g.N == 0 || g.K == 0 || g.batch == 0) return false;
    const TcOperand *ops[2] = {&g.A, &g.B};
    for (const TcOperand *o : ops) {
        if (!aligned16(o->ptr)) return false;
        if (o->ld % 8) return false;
        if ((uint64_t)g.batch * o->nparts > 1 && (o->z_stride % 8)) return false;
        if (o->ld * 2 >= (1ull << 40)) return false;
    }
    if ((uint64_t)g.batch * g.A.nparts > 0x7FFFFFFFull || (uint64_t)g.batch * g.B.nparts > 0x7FFFFFFFull) return false;
    if (g.splits > 1 && g.batch != 1) return false;
    if (g.npass < 1 || g.npass > 8) return false;
    return true;
}

// L2 promotion of the operand loads (CUtensorMapL2promotion: 0 none, 1 64 B, 2 128 B, 3 256 B); a tuning hook.
// Measured at 8192^3, three interleaved rounds on one GPU: none 1536.1-1537.5, 64 B 1535.0-1536.2, 128 B
// 1534.8-1536.9, 256 B 1531.5-1533.9 TFLOP/s.
int g_l2_promotion = (int)CU_TENSOR_MAP_L2_PROMOTION_NONE;
static int encode_operand(CUtensorMap *map, const TcOperand &o, int dtype, uint32_t mn_extent, uint32_t K,
                          uint32_t z, uint32_t mn_box_rows) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return ST_UNSUPPORTED;
    CUtensorMapDataType dt = dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3], strides[2];
    cuuint32_t box[3], estr[3] = {1, 1, 1};
    if (!o.mn_major) {
        dims[0] = K; dims[1] = mn_extent; dims[2] = z;
        box[0] = BK; box[1] = mn_box_rows; box[2] = 1;
    } else {
        dims[0] = mn_extent; dims[1] = K; dims[2] = z;
        box[0] = 64; box[1] = BK; box[2] = 1;
    }
    strides[0] = o.ld * 2;
    strides[1] = (z > 1 ? o.z_stride : o.ld * dims[1]) * 2;   // a single slice gets a harmless stride
    CUresult r = enc(map, dt, 3, const_cast<void *>(o.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, (CUtensorMapL2promotion)g_l2_promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(operand) failed: %d", (int)r);
        return ST_GEMM;
    }
    return ST_OK;
}

static int encode_c(CUtensorMap *map, const TcGemm &g, uint32_t z) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return ST_UNSUPPORTED;
    cuuint64_t dims[3] = {g.N, g.M, z};
    uint64_t zs = z > 1 ? g.c_stride : g.ldc * g.M;
    cuuint64_t strides[2] = {g.ldc * 4, zs * 4};
    cuuint32_t box[3] = {EPI_COLS, 32, 1}, estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, g.C, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(C) failed: %d", (int)r);
        return ST_GEMM;
    }
    return ST_OK;
}

struct CfgRuntime {
    bool ready = false;
    bool usable = false;
    int max_clusters = 0;   // co-resident clusters (CG == 2) or CTAs (CG == 1)
};
static CfgRuntime g_rt[8][NUM_CFGS];   // per device

static const CfgRuntime &prepare_cfg(int cfg) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 8) dev = 0;
    CfgRuntime &rt = g_rt[dev][cfg];
    if (rt.ready) return rt;
    rt.ready = true;
    const TcConfig &c = g_cfgs[cfg];
    cudaError_t e = cudaFuncSetAttribute(c.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem);
    if (e != cudaSuccess) {
        set_error("cudaFuncSetAttribute(%s, smem=%u): %s", c.name, c.smem, cudaGetErrorString(e));
        cudaGetLastError();
        return rt;
    }
    int sms = device_sm_count();
    if (c.cg == 1) {
        rt.max_clusters = sms;
    } else {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3((unsigned)(sms / 2 * 2), 1, 1);
        lc.blockDim = dim3(c.threads, 1, 1);
        lc.dynamicSmemBytes = c.smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        lc.attrs = at;
        lc.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, c.fn, &lc);
        if (e != cudaSuccess || n <= 0) {
            set_error("cudaOccupancyMaxActiveClusters(%s): %s", c.name, cudaGetErrorString(e));
            cudaGetLastError();
            return rt;
        }
        rt.max_clusters = n < sms / 2 ? n : sms / 2;
    }
    rt.usable = rt.max_clusters > 0;
    return rt;
}

static uint32_t cdiv(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------------
// Balanced last wave (see tail_unit).  With T tiles on S resident clusters and R = T % S != 0, the plain
// schedule runs R clusters for a whole tile while S - R wait; here every cluster gets k / (k + 1) of a tile,
// k = ceil(R / (S - R)) tiles per group.  Worth it when that is clearly less than the plain last wave
// (a partly filled wave already runs faster than a full one: more clock and more L2 per CTA, measured as
// 0.5 + 0.5 * occupancy of a full wave's time).
// ---------------------------------------------------------------------------------------------
static bool balanced_tail(uint64_t tiles, uint32_t slots, uint32_t k_blocks, uint32_t &full, uint32_t &q, uint32_t &r,
                          double *last_wave = nullptr) {
    full = (uint32_t)(tiles / slots);
    const uint32_t rem = (uint32_t)(tiles % slots);
    if (last_wave) *last_wave = rem ? 0.5 + 0.5 * (double)rem / slots : 0.0;
    if (rem == 0 || k_blocks < 16) return false;
    const uint32_t groups = slots - rem;
    q = rem / groups; r = rem % groups;
    const uint32_t kmax = q + (r ? 1 : 0);
    if (kmax + 1 > k_blocks / 4) return false;             // slices shorter than 4 K blocks are not worth a hand-over
    const double share = kmax ? (double)kmax / (kmax + 1) : 0.0;
    const double plain = 0.5 + 0.5 * (double)rem / slots;
    // hand-over and a second epilogue cost about 3 % of a tile; products of many waves gain too little to give up
    // "every element is one accumulation over K in order" (which makes all tile configurations agree bit for bit)
    if ((plain - (share + 0.03)) / ((double)full + plain) < 0.02) return false;
    if (last_wave) *last_wave = share + 0.03;
    return true;
}

// Pick a tile configuration.  Cost model fitted to measurements on B200 (bf16, K = 8192):
// relative throughput per configuration at full occupancy, and a last partial wave that costs
// 0.5 + 0.5 * occupancy of a full one (fewer CTAs run faster: more clock and more L2 each).
static int choose_cfg(const TcGemm &g) {
    if (g.force_cfg >= 0 && g.force_cfg < NUM_CFGS) return g.force_cfg;
    int best = 0;
    double best_cost = 1e300;
    for (int i = 0; i < NUM_CFGS; ++i) {
        const TcConfig &c = g_cfgs[i];
        if (!c.auto_ok) continue;
        const CfgRuntime &rt = prepare_cfg(i);
        if (!rt.usable) continue;
        const uint64_t tiles = (uint64_t)g.batch * cdiv(g.M, BM_CTA * c.cg) * cdiv(g.N, c.bn) * (g.splits ? g.splits : 1);
        const uint64_t slots = (uint64_t)rt.max_clusters;
        uint32_t full = 0, q = 0, r = 0;
        double last = 0.0;
        const bool may_balance = g.allow_stream_k && !g.bias && !g.act && !g.c16 && (g.splits ? g.splits : 1) == 1 &&
                                 g.npass == 1 && !g.c_trans && g.counters;
        if (!may_balance || !balanced_tail(tiles, (uint32_t)slots, cdiv(g.K, BK), full, q, r, &last)) {
            full = (uint32_t)(tiles / slots);
            const uint64_t tail = tiles % slots;
            last = tail ? 0.5 + 0.5 * (double)tail / (double)slots : 0.0;
        }
        const double waves = (double)full + last;
        double eff;
        if (c.cg == 2) eff = c.bn >= 256 ? 1.0 : 0.75;
        else eff = c.bn >= 256 ? 0.885 : (c.bn == 128 ? 0.71 : 0.45);
        // time ~ waves * tile area per SM / efficiency
        const double cost = waves * (double)BM_CTA * c.bn / eff;
        if (cost < best_cost) { best_cost = cost; best = i; }
    }
    return best;
}

// Host view of the balanced last wave, for tests: part j (0, 1) of cluster c when `tiles` tiles of `k_blocks` K
// blocks run on `slots` clusters.  out = {used, whole-tile waves, tail tile, first K block, K blocks, role}.
int tc_tail_schedule(uint64_t tiles, uint32_t slots, uint32_t k_blocks, uint32_t c, uint32_t j, uint32_t out[6]) {
    uint32_t full = 0, q = 0, r = 0;
    for (int i = 0; i < 6; ++i) out[i] = 0;
    if (slots == 0 || c >= slots) return ST_UNSUPPORTED;
    if (!balanced_tail(tiles, slots, k_blocks, full, q, r)) return ST_OK;       // out[0] == 0: plain schedule
    out[0] = 1; out[1] = full;
    uint32_t tile, b, n, role;
    if (tail_part(q, r, k_blocks, c, j, tile, b, n, role)) { out[2] = tile; out[3] = b; out[4] = n; out[5] = role; }
    return ST_OK;
}

// The i-th unit of CTA pair `id` of `count` (on die `die` when the walk is die-aware), by the function the kernel's
// roles call: out = {1 if there is one, M tile, N tile, 1 if its K blocks are fetched last to first}.
int tc_walk_unit(uint32_t m_tiles, uint32_t n_tiles, uint32_t group_m, uint32_t k_blocks, uint32_t die_aware, uint32_t serpentine,
                 uint32_t k_serpentine, uint32_t die, uint32_t id, uint32_t count, uint32_t i, uint32_t out[4]) {
    for (int j = 0; j < 4; ++j) out[j] = 0;
    if (!m_tiles || !n_tiles || !group_m || !count || id >= count) return ST_UNSUPPORTED;
    if (die_aware && (group_m % 2 || m_tiles % group_m || die > 1)) return ST_UNSUPPORTED;
    TcParams p = {};
    p.batch = 1; p.splits = 1; p.m_tiles = m_tiles; p.n_tiles = n_tiles; p.group_m = group_m;
    p.k_blocks = k_blocks; p.kb_per_split = k_blocks;
    p.serpentine = serpentine ? 1u : 0u; p.k_serpentine = k_serpentine ? 1u : 0u;
    static const unsigned char some_table[1] = {0};
    if (die_aware) p.die_table = some_table;          // only its presence selects the walk
    Walk wk = {id, count, die};
    WorkUnit w;
    if (!get_unit(p, wk, m_tiles * n_tiles, i, w)) return ST_OK;
    out[0] = 1; out[1] = w.m_blk; out[2] = w.n_blk; out[3] = w.k_down;
    return ST_OK;
}

int tc_gemm_launch(const TcGemm &g) {
    if (!tc_gemm_supported(g)) return ST_UNSUPPORTED;
    const int cfg = choose_cfg(g);
    const TcConfig &c = g_cfgs[cfg];
    const CfgRuntime &rt = prepare_cfg(cfg);
    if (!rt.usable) return ST_GEMM;

    if (g.B.mn_major && c.bn / c.cg < 64) {
        set_error("tc_gemm: tile %s cannot take an MN-major B operand", c.name);
        return ST_UNSUPPORTED;
    }
    const uint32_t splits = g.splits ? g.splits : 1;
    TcParams p = {};
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.batch = g.batch;
    p.m_tiles = cdiv(g.M, BM_CTA * c.cg);
    p.n_tiles = cdiv(g.N, c.bn);
    p.k_blocks = cdiv(g.K, BK);
    p.kb_per_split = cdiv(p.k_blocks, splits);
    p.splits = cdiv(p.k_blocks, p.kb_per_split);     // no empty slice
    if (p.splits != splits) {
        set_error("tc_gemm: %u K-splits leave an empty slice (k_blocks=%u)", splits, p.k_blocks);
        return ST_GEMM;
    }
    p.npass = g.npass; p.a_sel = g.a_sel; p.b_sel = g.b_sel;
    p.a_piece_mask = g.a_piece_mask; p.b_piece_mask = g.b_piece_mask;
    p.a_nparts = g.A.nparts; p.b_nparts = g.B.nparts;
    p.a_mn = g.A.mn_major; p.b_mn = g.B.mn_major;
    const uint32_t fmt = g.dtype == DT_BF16 ? 1u : 0u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
              ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(c.bn >> 3) << 17) |
              ((uint32_t)((BM_CTA * c.cg) >> 4) << 24);
    p.group_m = 8;
    {
        // keep one wave's footprint roughly square in elements: group_m * BM ~ slots/group_m * BN
        uint32_t slots = (uint32_t)rt.max_clusters;
        uint32_t bm = BM_CTA * c.cg;
        uint32_t best = 1;
        double best_cost = 1e300;
        for (uint32_t gm = 1; gm <= 32 && gm <= p.m_tiles; ++gm) {
            double cols = (double)slots / gm;
            double cost = gm * (double)bm + cols * (double)c.bn;
            // a group height that does not divide the M tiles leaves a flatter last group, whose waves touch more
            // columns of B (measured at 8192^3: 9 rows -> 1.11 GB of DRAM reads, 8 rows -> 1.04 GB, and 1.3 % faster)
            if (p.m_tiles % gm) cost *= 1.05;
            if (cost < best_cost) { best_cost = cost; best = gm; }
        }
        p.group_m = best;
    }
    p.C = g.C; p.ldc = g.ldc; p.c_stride = g.c_stride;
    p.c_trans = g.c_trans ? 1u : 0u;
    // K-slices as the CTAs of a cluster, reduced through distributed shared memory: narrow tiles whose partial
    // sums of all slices fit in the leader's 32 KB staging area (128 x BN x 4 bytes per slice beyond the first)
    p.cluster_k = 0;
    if (g.cluster_splitk && c.cg == 1 && c.staging && c.bn <= 32 && g.Cout && g.batch == 1 && splits >= 2 && splits <= 8 &&
        (splits - 1) * BM_CTA * c.bn * 4 <= c.ew * 2 * EPI_BUF_BYTES && !(g.debug & 5))
        p.cluster_k = splits;
    p.act_copy_only = g.act_copy_only ? 1u : 0u;
    p.bias = g.bias; p.act = (uint32_t)g.act; p.c16 = (unsigned short *)g.c16; p.ld16 = g.ld16; p.dtype16 = (uint32_t)g.dtype16;
    p.bias_vec4 = aligned16(g.bias) ? 1u : 0u;
    p.c16_vec = (g.c16 && aligned16(g.c16) && g.ld16 % 8 == 0) ? 1u : 0u;
    if ((g.bias || g.act || g.c16) && (splits > 1 || g.c_trans || g.accumulate)) {
        set_error("tc_gemm: the fused bias/activation epilogue does not combine with split-K, swapped operands or accumulate");
        return ST_UNSUPPORTED;
    }
    p.Cout = (splits > 1) ? g.Cout : nullptr; p.ldc_out = g.ldc_out; p.counters = g.counters;
    if (p.Cout && !p.cluster_k) {
        const uint64_t slabs = (uint64_t)p.m_tiles * p.n_tiles * c.cg * c.ew;
        if (!g.counters || slabs > g.num_counters) {
            set_error("tc_gemm: %llu slab counters needed for the fused split-K reduction, %u available",
                      (unsigned long long)slabs, g.num_counters);
            return ST_UNSUPPORTED;
        }
    }
    p.accumulate = g.accumulate ? 1u : 0u;
    p.stages = (g.stages >= 2 && (uint32_t)g.stages < c.stages) ? (uint32_t)g.stages : c.stages;
    p.debug = (uint32_t)g.debug;
    if (g.l2_hints > 0) {
        p.l2_hints = (uint32_t)g.l2_hints;
    } else if (g.l2_hints < 0) {
        p.l2_hints = 0;
    } else {
        // C is written once: let it leave the L2 first, and nothing of the operands (both evict-last).  Measured
        // interleaved against B at normal priority: 1271.0 -> 1294.6 and 1312.8 -> 1334.0 TFLOP/s at 8192^3 on two GPUs,
        // 1295.0 -> 1312.7 at 8192 x 4096 x 8192, 1293.8 -> 1308.9 at 8192 x 16384 x 4096, 1150.6 -> 1159.0 at 4096^3;
        // against A at normal priority where a group's A panel is larger than the L2 keeps (K = 16384): 1292.9 -> 1307.6.
        p.l2_hints = (1u << 4) | (2u << 2) | 2u;
        if (g.c_trans) p.l2_hints = (1u << 4) | 2u;          // swapped skinny route (one stream through B): as before
        // A narrow product (all of its N tiles inside one wave: the N-column shard of a multi-GPU run) turns the
        // roles round: every wave multiplies new rows of A by ALL of B, so B is what should stay and A is read once
        // (measured at 8192 x 1024 x 8192, interleaved: 1092.9 -> 1130.3 and 1111.8 -> 1154.1 TFLOP/s, +3.4-3.8 %; with
        // a B of 33.5 MB, 8192 x 2048 x 8192, the same hints lose 1.6 % and the general rule above is the best
        // of those tried: 1212.9 against 1201.3 with A at normal priority; so the rule stops at 24 MB).
        const uint32_t wave_n = (uint32_t)rt.max_clusters / (p.group_m ? p.group_m : 1);
        const uint64_t b_all = (uint64_t)g.N * g.K * 2;
        if (g.batch == 1 && p.n_tiles <= wave_n && b_all <= (24ull << 20)) p.l2_hints = (1u << 4) | (2u << 2) | 1u;
    }
    if (g.group_m > 0) p.group_m = (uint32_t)g.group_m;
    p.serpentine = g.serpentine ? 1u : 0u;
    p.prof = g.prof;
    if (!p.prof) p.debug &= ~32u;
    p.status = g.dev_status;
    const uint32_t zc = splits > 1 ? splits : g.batch;
    const bool c_vec_ok = aligned16(g.C) && (g.ldc % 4 == 0) && (zc == 1 || g.c_stride % 4 == 0);
    // A TMA store clips the innermost extent in 16-byte units (measured on B200: with N % 4 != 0
    // it wrote up to the next multiple of four columns), so it is used only when N is one.
    const bool c_tma_ok = c_vec_ok && (g.N % 4 == 0);
    p.epilogue_tma = (g.force_epilogue >= 0) ? (uint32_t)(g.force_epilogue && c_tma_ok) : (c_tma_ok ? 1u : 0u);
    if (!c.staging || p.c_trans || p.Cout) p.epilogue_tma = 0;   // K-slices of a fused reduction are plain stores
    p.c_vec4 = c_vec_ok ? 1u : 0u;

    CUtensorMap ma, mb, mc;
    int st = encode_operand(&ma, g.A, g.dtype, g.M, g.K, g.batch * g.A.nparts, BM_CTA);
    if (st != ST_OK) return st;
    st = encode_operand(&mb, g.B, g.dtype, g.N, g.K, g.batch * g.B.nparts, (uint32_t)(c.bn / c.cg));
    if (st != ST_OK) return st;
    if (p.epilogue_tma) {
        st = encode_c(&mc, g, zc);
        if (st != ST_OK) return st;
    } else {
        mc = ma;  // unused by the kernel
    }

    if (g.n_extra) {
        if (g.n_extra > 7 || !p.epilogue_tma || p.accumulate || p.splits > 1 || g.batch != 1) {
            set_error("tc_gemm: further destinations of C need one product, no accumulate and a C that TMA can store "
                      "(16-byte aligned base, ldc and N multiples of 4)");
            return ST_UNSUPPORTED;
        }
        for (uint32_t d = 0; d < g.n_extra; ++d) {
            if (!aligned16(g.extra_c[d])) { set_error("tc_gemm: destination %u of C is not 16-byte aligned", d + 1); return ST_UNSUPPORTED; }
            p.extra_c[d] = g.extra_c[d];
        }
        p.n_extra = g.n_extra;
    }

    const uint64_t units = (uint64_t)g.batch * p.m_tiles * p.n_tiles * p.splits;
    if (units > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    uint32_t clusters = (uint32_t)(units < (uint64_t)rt.max_clusters ? units : (uint64_t)rt.max_clusters);
    bool stream_k = false;
    if (g.allow_stream_k && !g.n_extra && !g.bias && !g.act && !g.c16 && p.splits == 1 && p.npass == 1 && !p.c_trans && p.epilogue_tma &&
        g.counters && !(kExperiments && (p.debug & 31u))) {
        uint32_t full = 0, q = 0, r = 0;
        const uint32_t slots = (uint32_t)rt.max_clusters;
        if (balanced_tail(units, slots, p.k_blocks, full, q, r) &&
            (units % slots) * c.cg * c.ew <= (uint64_t)g.num_counters) {
            p.sk_on = 1; p.sk_full = full; p.sk_q = q; p.sk_r = r;
            p.counters = g.counters;
            clusters = slots;
            stream_k = true;
        }
    }

    if (p.cluster_k) clusters = (uint32_t)units;      // one unit per CTA; consecutive CTAs = the slices of one tile
    // die-aware walk: large single products that fill every SM pair for several waves, groups that halve evenly
    bool die_aware = false;
    if (g.die_table && g.die_claim && !stream_k && !p.cluster_k && p.batch == 1 && p.splits == 1 &&
        clusters == (uint32_t)rt.max_clusters && clusters % 2 == 0 && p.group_m % 2 == 0 && p.m_tiles % p.group_m == 0 &&
        units >= 4ull * clusters && !(kExperiments && (p.debug & 31u))) {
        p.die_table = g.die_table; p.die_claim = g.die_claim;
        die_aware = true;
    }
    // K up and down: where the operands are more than the L2 keeps from one wave to the next, a CTA's odd-numbered
    // tiles fetch their K blocks last to first, so that a wave begins on the blocks the wave before it ended on
    // (the rows of A are the same within a rasterisation group).  Measured at 8192^3: 0.98 -> 0.88 GB of DRAM reads
    // per launch and +1.4 % under the power cap.  The sum of an element then runs over K in an order that depends
    // on where its tile falls in the walk: results stay deterministic for a shape but are not bit-identical
    // between shapes or shards (option k_serpentine = 0 restores ascending K everywhere).
    if (g.k_serpentine && c.sub == 1 && p.splits == 1 && g.batch == 1 && !stream_k && !p.cluster_k && units > clusters &&
        ((uint64_t)g.M + g.N) * g.K * 2 >= (64ull << 20) && !(kExperiments && (p.debug & 31u)))
        p.k_serpentine = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(clusters * c.cg, 1, 1);
    lc.blockDim = dim3(c.threads, 1, 1);
    lc.dynamicSmemBytes = c.smem;
    lc.stream = g.stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = p.cluster_k ? p.cluster_k : (unsigned)c.cg;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    if (g.pdl) {
        // the kernel's prologue (barriers, tensor memory, descriptor prefetch) may overlap the tail of the kernel
        // before it in the stream; it waits (griddepcontrol.wait) before its first global access
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        lc.numAttrs = 2;
    }
    void *args[4] = {(void *)&ma, (void *)&mb, (void *)&mc, (void *)&p};
    cudaError_t e = cudaLaunchKernelExC(&lc, c.fn, args);
    if (e != cudaSuccess) {
        set_error("launch %s failed: %s", c.name, cudaGetErrorString(e));
        cudaGetLastError();
        return ST_GEMM;
    }
    note_launch();
    char more[24] = "";
    if (p.n_extra) snprintf(more, sizeof more, ":to%u", p.n_extra + 1);
    set_last_path("tc:%s%s%s%s%s%s%s", c.name, p.epilogue_tma ? "" : ":direct", p.splits > 1 ? ":splitk" : "",
                  p.cluster_k ? ":cluster" : (p.Cout ? ":fused" : ""), stream_k ? ":balanced_tail" : (die_aware ? ":die_aware" : ""),
                  p.k_serpentine ? ":k_up_down" : "", more);
    return ST_OK;
}

}  // namespace pgb
