// Attention-shaped chain of picograd's pg_bmm calls, fused into one kernel (sm_100a):
//
//     S = Q * Kt                (pg_bmm, ops/matmul.c:340-369; f32 [B, Sq, Sk])
//     P = 16-bit(softmax(S))    (pg_softmax over the last axis, ops/activations.c:22-45, then a cast)
//     O = P * V                 (pg_bmm; f32 [B, Sq, D])
//
// without S or P ever reaching HBM.  The arithmetic follows the chain, not the usual "online
// softmax": P is rounded to 16 bits AFTER the division by the row sum, exactly as the separate
// kernels do, so the result agrees with the chain to rounding noise.  That needs the row maximum and
// row sum before the first P exists, hence two passes over the keys per 128 query rows:
//
//     pass 1:  S_blk = Q Kt_blk (tensor cores) -> running max m and sum l of exp(s - m)
//     pass 2:  S_blk again -> p = exp(s - m) / l -> 16-bit -> shared memory -> O += P_blk V_blk
//
// Q Kt is computed twice (3 instead of 2 GEMM-equivalents); what is saved is the 1 GiB write and read of
// S and the 0.5 GiB write and read of P at picograd's attention-shaped configuration (B=64, Sq=Sk=2048,
// D=128).  The kernel is bound by the exponentials (two per element of S), not by HBM or the MMAs.
//
// Roles (384 threads, one CTA per SM, persistent over (batch, 128-row query block) units).  The softmax
// warps keep the schedulers busy, so whatever else runs on them must be a short instruction stream: the two
// kinds of product have an issuing warp each, and so have their operands.
//   warp 0      K producer: Q, then the 128 x 128 blocks of Kt into a two-entry ring (TMA, MN-major B operand)
//   warp 11     V producer: the 128 x 128 blocks of V into a two-entry ring
//   warp 1      S issuer: S[e] = Q Kt_blk into one of two TMEM buffers (8 MMAs, one commit)
//   warp 10     PV issuer: O += P[pb] V_blk into a third TMEM buffer
//   warps 2-5   softmax group 0, warps 6-9 group 1: the groups take alternate S buffers; a thread owns one
//               query row (TMEM lane), pulls its 128 scores into registers with tcgen05.ld, hands the buffer
//               straight back, and in pass 2 writes its row of P into the 128-byte-swizzled K-major layout
//               the MMA reads.  In pass 2 the S products run ahead of the P V products by themselves.
// Ring entry e of Kt belongs to S buffer e and ring entry pb of V to P tile pb, so "entry free again" is the
// same event as "product completed" (s_full / p_empty): one commit per product.
// All waits are bounded mbarrier waits (status word + CTA abort flag), no named barriers.

#include "pg_internal.h"
#include "tc_ptx.cuh"

namespace pgb {

constexpr uint32_t AT_ROWS = 128;                 // query rows per unit == TMEM lanes
constexpr uint32_t AT_KEYS = 128;                 // keys per block
constexpr uint32_t AT_D = 128;                    // head dimension
constexpr uint32_t AT_ATOM = 128 * 64 * 2;        // [128 rows x 64 elements] K-major, or [64 k x 128 n] MN-major
constexpr uint32_t AT_ENTRY = 2 * AT_ATOM;        // one ring entry: a 128 x 128 block of Kt or V
constexpr uint32_t AT_ENTRIES = 4;
constexpr uint32_t AT_SLOTS = AT_ENTRIES;         // (barrier pairs of the ring)
constexpr uint32_t AT_Q_BYTES = 2 * AT_ATOM;      // one Q tile (two d-halves)
constexpr uint32_t AT_P_BYTES = 2 * AT_ATOM;      // one P tile (two key-halves)
constexpr uint32_t AT_BAR_BYTES = 1024;
constexpr uint32_t AT_SMEM = 1024 + AT_Q_BYTES + 2 * AT_P_BYTES + AT_ENTRIES * AT_ENTRY + AT_BAR_BYTES;
constexpr uint32_t AT_THREADS = 384;
constexpr uint32_t AT_TMEM_COLS = 512;            // S0 at 0, S1 at 128, O at 256, Q at 384, row statistics at 448
static_assert(AT_SMEM <= 232448, "shared memory budget");

struct AttnParams {
    uint32_t batch, sq, sk;
    uint32_t q_tiles, nkb;        // 128-row query blocks per batch element, 128-key blocks
    uint32_t idesc;
    uint32_t dtype;               // DT_F16 / DT_BF16: operands and the 16-bit P
    float *O;
    uint64_t ldo, o_stride;       // elements
    uint32_t *status;
    unsigned long long *prof;     // timing experiments: 16 cycle counters per CTA (may be null)
    uint32_t debug;               // timing experiments (results are garbage): 1 = no TMA loads, 16 = no MMAs
    uint32_t q_tmem;              // Q is copied to tensor memory once per unit and read from there by the MMAs
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t a, uint32_t b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, uint32_t &a, uint32_t &b) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(taddr) : "memory");
}
__device__ __forceinline__ uint32_t at_pack16(float lo, float hi, uint32_t dtype) {
    uint32_t r;
    if (dtype == (uint32_t)DT_BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (128 rows = lanes, 16 K-elements = 8 columns per MMA) read
// from tensor memory, so that only B crosses the shared-memory port.
__device__ __forceinline__ void umma_ta(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// Shared memory -> tensor memory: 128 rows x 256 bits (16 16-bit elements of each row of a K-major tile) into 8
// columns; asynchronous, ordered before later tcgen05.mma of the same thread.
__device__ __forceinline__ void tmem_cp_128x256b(uint32_t taddr, uint32_t s_lo, uint32_t s_hi) {
    asm volatile(
        "{\n\t.reg .b64 ds;\n\tmov.b64 ds, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::1.128x256b [%0], ds;\n\t}"
        ::"r"(taddr), "r"(s_lo), "r"(s_hi) : "memory");
}
// Waits for this thread's outstanding tcgen05.ld and ties the wait to the registers just loaded, so that the
// compiler cannot schedule arithmetic on them above it (loads of the next chunk are issued before the
// arithmetic of the current one).
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                   "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#define AT_F(i) __uint_as_float(v[i])
// Columns col0 .. col0+31 of a block whose first `valid` columns exist: the others count as -inf.
__device__ __forceinline__ void at_mask(uint32_t (&v)[32], uint32_t col0, uint32_t valid) {
#pragma unroll
    for (uint32_t j = 0; j < 32; ++j)
        if (col0 + j >= valid) v[j] = __float_as_uint(-INFINITY);
}
// Pass 1 pieces on 32 scores of a row: their maximum, and the sum of 2^(s log2 e + nmc).
__device__ __forceinline__ float at_max32(const uint32_t (&v)[32]) {
    float a[10];
#pragma unroll
    for (uint32_t k = 0; k < 10; ++k) a[k] = fmax3(AT_F(3 * k), AT_F(3 * k + 1), AT_F(3 * k + 2));
    const float r0 = fmax3(a[0], a[1], a[2]), r1 = fmax3(a[3], a[4], a[5]), r2 = fmax3(a[6], a[7], a[8]);
    return fmax3(fmax3(r0, r1, r2), fmax3(a[9], AT_F(30), AT_F(31)), -INFINITY);
}
__device__ __forceinline__ float at_sum32(const uint32_t (&v)[32], float nmc) {
    const float LOG2E = 1.4426950408889634f;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < 32; j += 4) {
        s0 += ex2_approx(fmaf(AT_F(j), LOG2E, nmc));
        s1 += ex2_approx(fmaf(AT_F(j + 1), LOG2E, nmc));
        s2 += ex2_approx(fmaf(AT_F(j + 2), LOG2E, nmc));
        s3 += ex2_approx(fmaf(AT_F(j + 3), LOG2E, nmc));
    }
    return (s0 + s1) + (s2 + s3);
}
// Pass 2 on 32 scores: p = 2^(s log2 e + off) with off = -(M log2 e + log2 L), i.e. exp(s - M) / L, rounded to
// 16 bits, two per word.
__device__ __forceinline__ void at_probs32(const uint32_t (&v)[32], float off, uint32_t dtype, uint32_t (&w)[16]) {
    const float LOG2E = 1.4426950408889634f;
#pragma unroll
    for (uint32_t j = 0; j < 32; j += 2)
        w[j >> 1] = at_pack16(ex2_approx(fmaf(AT_F(j), LOG2E, off)), ex2_approx(fmaf(AT_F(j + 1), LOG2E, off)), dtype);
}
// The 32 probabilities as four 16-byte pieces of the row's 128-byte line of the swizzled P tile.
__device__ __forceinline__ void at_store32(const uint32_t (&w)[16], uint8_t *line, uint32_t first_piece, uint32_t row7) {
#pragma unroll
    for (uint32_t jj = 0; jj < 4; ++jj)
        *reinterpret_cast<uint4 *>(line + (((first_piece + jj) ^ row7) << 4)) =
            make_uint4(w[4 * jj], w[4 * jj + 1], w[4 * jj + 2], w[4 * jj + 3]);
}
#undef AT_F

#ifndef PG_ATTN_HINT_NS
#define PG_ATTN_HINT_NS 32
#endif
// every hand-over in this kernel is latency-critical: short suspend hint
__device__ __forceinline__ bool at_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t *status,
                                        uint32_t err_bit) {
    return mbar_wait_quick(bar, parity, abort_flag, status, err_bit, PG_ATTN_HINT_NS);
}

// Timing experiments (debug bit 64): CTA 0 records (tag << 32 | low 32 bits of the clock) into the counter
// buffer from entry 2400 on, 1400 entries per role (S issuer, softmax group 0, group 1, PV issuer), plain stores.
__device__ __forceinline__ void at_trace(const AttnParams &p, uint32_t role, uint32_t &n, uint32_t tag) {
    if ((p.debug & 64u) && p.prof && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && n < 1400)
        p.prof[2400 + role * 1400 + n++] = ((unsigned long long)tag << 32) | (unsigned long long)(uint32_t)clock64();
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kt,
                  const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t q_base = smem_base;                                   // 32 KB
    const uint32_t p_base = q_base + AT_Q_BYTES;                         // 2 x 32 KB
    const uint32_t ring_base = p_base + 2 * AT_P_BYTES;                  // AT_ENTRIES x 32 KB
    const uint32_t bar_base = ring_base + AT_ENTRIES * AT_ENTRY;
    uint32_t nb = 0;
    auto take = [&](uint32_t n) { uint32_t b = bar_base + 8u * nb; nb += n; return b; };
    const uint32_t kfull0 = take(2), vfull0 = take(2);
    const uint32_t q_full0 = take(1), q_empty0 = take(1);
    const uint32_t s_full0 = take(2), s_empty0 = take(2);
    const uint32_t p_full0 = take(2), p_empty0 = take(2);
    const uint32_t o_full = take(1), o_empty = take(1);
    const uint32_t stat0 = take(2);
    const uint32_t tmem_slot = take(1);
    const uint32_t abort_off = (take(1) - smem_base);
    volatile uint32_t *tmem_slot_gen = (volatile uint32_t *)(smem_gen + (tmem_slot - smem_base));
    volatile uint32_t *abort_flag = (volatile uint32_t *)(smem_gen + abort_off);
    static_assert(8 * (4 + 5 * 2 + 2 + 2 + 2) <= AT_BAR_BYTES, "barrier block");

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total_units = p.batch * p.q_tiles;
    const uint32_t nkb = p.nkb;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_kt);
        prefetch_tmap(&map_v);
        for (uint32_t s = 0; s < 2; ++s) { mbar_init(kfull0 + 8 * s, 1); mbar_init(vfull0 + 8 * s, 1); }
        mbar_init(q_full0, 1);
        mbar_init(q_empty0, 1);
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 4);
            mbar_init(p_full0 + 8 * s, 4); mbar_init(p_empty0 + 8 * s, 1);
            mbar_init(stat0 + 8 * s, 8);
        }
        mbar_init(o_full, 1);
        mbar_init(o_empty, 8);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, AT_TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;

    // Use number n (0, 1, 2, ...) of a barrier completes its phase n & 1; "free again after use n - 1" is a
    // wait for parity (n & 1) ^ 1, which a fresh barrier passes at once.
    if (warp == 0) {
        // ------------------------------ K producer: Q, then the blocks of Kt ------------------------------
        // K-ring entry e holds the operand of the product into S buffer e, so "entry free" is the very event
        // "that product has completed" = s_full[e]: no separate empty barrier, no extra commit.
        bool ok = true;
        uint32_t n_unit = 0;
        const uint64_t pol = l2_policy(0);
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            const int32_t b = (int32_t)(u / p.q_tiles), row0 = (int32_t)((u % p.q_tiles) * AT_ROWS);
            // the single Q buffer is free once the last Q Kt product of the previous unit has completed
            ok = at_wait(q_empty0, (n_unit & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY);
            if (!ok) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(q_full0, AT_Q_BYTES);
                tma_load_3d<1>(q_base, &map_q, q_full0, 0, row0, b, pol);
                tma_load_3d<1>(q_base + AT_ATOM, &map_q, q_full0, 64, row0, b, pol);
            }
            __syncwarp();
            for (uint32_t t = 0; t < 2 * nkb && ok; ++t) {
                const uint32_t e = t & 1, n = n_unit * nkb + (t >> 1);
                ok = at_wait(s_full0 + 8 * e, (n & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t bar = kfull0 + 8 * e, dst = ring_base + e * AT_ENTRY;
                    const int32_t key0 = (int32_t)((t < nkb ? t : t - nkb) * AT_KEYS);
                    if (p.debug & 1u) {
                        mbar_arrive(bar);
                    } else {    // K of the MMA = d (all 128 rows of Kt), N = the block's keys, two 64-key halves
                        mbar_arrive_expect_tx(bar, AT_ENTRY);
                        tma_load_3d<1>(dst, &map_kt, bar, key0, 0, b, pol);
                        tma_load_3d<1>(dst + AT_ATOM, &map_kt, bar, key0 + 64, 0, b, pol);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 11) {
        // ------------------------------ V producer ------------------------------
        // V-ring entry pb holds the operand of the product that reads P tile pb: "entry free" = p_empty[pb].
        bool ok = true;
        uint32_t cnt0 = 0, cnt1 = 0;
        const uint64_t pol = l2_policy(0);
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
            const int32_t b = (int32_t)(u / p.q_tiles);
            for (uint32_t j = 0; j < nkb && ok; ++j) {
                const uint32_t pb = (nkb + j) & 1, n = pb ? cnt1 : cnt0;
                ok = at_wait(p_empty0 + 8 * pb, (n & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                if (pb) ++cnt1; else ++cnt0;
                if (elect_one()) {
                    const uint32_t bar = vfull0 + 8 * pb, dst = ring_base + (2 + pb) * AT_ENTRY;
                    const int32_t key0 = (int32_t)(j * AT_KEYS);
                    if (p.debug & 1u) {
                        mbar_arrive(bar);
                    } else {    // K of the MMA = the block's keys, N = d, two 64-column halves
                        mbar_arrive_expect_tx(bar, AT_ENTRY);
                        tma_load_3d<1>(dst, &map_v, bar, 0, key0, b, pol);
                        tma_load_3d<1>(dst + AT_ATOM, &map_v, bar, 64, key0, b, pol);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------ S issuer: S[e] = Q Kt_blk ------------------------------
        // Eight MMAs (k = 16 each) per product: the K-major A operand Q advances 32 bytes per step inside a
        // 64-element half and 16 KB to the other half; the MN-major B operand advances 16 k-rows = 2048 bytes.
        bool ok = true;
        uint32_t n_unit = 0, ntr = 0;
        const bool prof = p.prof != nullptr;
        long long w_data = 0, w_role = 0, t_all = prof ? clock64() : 0;
        const uint32_t idesc = p.idesc;
        const uint64_t dq = make_desc(q_base, 0), dr = make_desc(ring_base, 128 * 128);
        const uint32_t q_hi = (uint32_t)(dq >> 32), r_hi = (uint32_t)(dr >> 32), q_lo = (uint32_t)dq, r_lo0 = (uint32_t)dr;
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            ok = at_wait(q_full0, n_unit & 1, abort_flag, p.status, DEV_ERR_WAIT_FULL);
            if (ok && p.q_tmem) {
                // Q: shared memory -> TMEM columns 384..447 (8 columns per 16 elements of d).  The copies queue
                // behind the previous unit's last product, which was the last reader of those columns; after
                // them the shared-memory tile is free for the next unit's Q.
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < 8; ++kk)
                        tmem_cp_128x256b(tmem_base + 384 + kk * 8, q_lo + (kk >> 2) * (AT_ATOM >> 4) + (kk & 3) * 2, q_hi);
                    umma_commit<1>(q_empty0);
                }
                __syncwarp();
            }
            for (uint32_t t = 0; t < 2 * nkb && ok; ++t) {
                const uint32_t e = t & 1, n = n_unit * nkb + (t >> 1);
                long long c0 = prof ? clock64() : 0;
                ok = at_wait(kfull0 + 8 * e, n & 1, abort_flag, p.status, DEV_ERR_WAIT_FULL);
                if (!ok) break;
                long long c1 = prof ? clock64() : 0;
                ok = at_wait(s_empty0 + 8 * e, (n & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                if (prof) { w_data += c1 - c0; w_role += clock64() - c1; }
                at_trace(p, 0, ntr, 0x100000u | t);
                if (elect_one()) {
                    const uint32_t d_tmem = tmem_base + e * 128, b_lo = r_lo0 + e * (AT_ENTRY >> 4);
                    if (p.debug & 16u) {
                    } else if (p.q_tmem) {
#pragma unroll
                        for (uint32_t kk = 0; kk < 8; ++kk)
                            umma_ta(d_tmem, tmem_base + 384 + kk * 8, b_lo + kk * 128, r_hi, idesc, kk ? 1u : 0u);
                    } else {
#pragma unroll
                        for (uint32_t kk = 0; kk < 8; ++kk)
                            umma_lohi<1>(d_tmem, q_lo + (kk >> 2) * (AT_ATOM >> 4) + (kk & 3) * 2, q_hi, b_lo + kk * 128, r_hi, idesc,
                                         kk ? 1u : 0u);
                    }
                    umma_commit<1>(s_full0 + 8 * e);
                    if (t == 2 * nkb - 1 && !p.q_tmem) umma_commit<1>(q_empty0);       // Q is not read again in this unit
                }
                __syncwarp();
                at_trace(p, 0, ntr, 0x200000u | t);
            }
        }
        if (prof && lane == 0) {
            unsigned long long *o = p.prof + (size_t)blockIdx.x * 16;
            o[0] = (unsigned long long)(clock64() - t_all); o[1] = (unsigned long long)w_data; o[2] = (unsigned long long)w_role;
        }
    } else if (warp == 10) {
        // ------------------------------ PV issuer: O += P[pb] V_blk ------------------------------
        bool ok = true;
        uint32_t n_unit = 0, cnt0 = 0, cnt1 = 0, ntr = 0;
        const bool prof = p.prof != nullptr;
        long long w_data = 0, w_role = 0;
        const uint32_t idesc = p.idesc;
        const uint64_t dp = make_desc(p_base, 0), dr = make_desc(ring_base + 2 * AT_ENTRY, 128 * 128);
        const uint32_t p_hi = (uint32_t)(dp >> 32), r_hi = (uint32_t)(dr >> 32), p_lo0 = (uint32_t)dp, r_lo0 = (uint32_t)dr;
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            for (uint32_t j = 0; j < nkb && ok; ++j) {
                const uint32_t pb = (nkb + j) & 1, n = pb ? cnt1 : cnt0;
                long long c0 = prof ? clock64() : 0;
                ok = at_wait(vfull0 + 8 * pb, n & 1, abort_flag, p.status, DEV_ERR_WAIT_FULL);
                if (!ok) break;
                long long c1 = prof ? clock64() : 0;
                ok = at_wait(p_full0 + 8 * pb, n & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                if (!ok) break;
                // the previous unit's O must have been read out before the first product overwrites it
                if (j == 0) ok = at_wait(o_empty, (n_unit & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                if (pb) ++cnt1; else ++cnt0;
                tc_fence_after();
                if (prof) { w_data += c1 - c0; w_role += clock64() - c1; }
                at_trace(p, 3, ntr, 0x300000u | j);
                if (elect_one()) {
                    const uint32_t d_tmem = tmem_base + 256, a_lo = p_lo0 + pb * (AT_P_BYTES >> 4), b_lo = r_lo0 + pb * (AT_ENTRY >> 4);
                    if (!(p.debug & 16u)) {
#pragma unroll
                        for (uint32_t kk = 0; kk < 8; ++kk)
                            umma_lohi<1>(d_tmem, a_lo + (kk >> 2) * (AT_ATOM >> 4) + (kk & 3) * 2, p_hi, b_lo + kk * 128, r_hi, idesc,
                                         (j | kk) ? 1u : 0u);
                    }
                    umma_commit<1>(p_empty0 + 8 * pb);
                    if (j == nkb - 1) umma_commit<1>(o_full);
                }
                __syncwarp();
                at_trace(p, 3, ntr, 0x400000u | j);
            }
        }
        if (prof && lane == 0) {
            unsigned long long *o = p.prof + (size_t)blockIdx.x * 16;
            o[3] = (unsigned long long)w_data; o[4] = (unsigned long long)w_role;
        }
    } else if (warp < 10) {
        // ------------------------------ softmax groups ------------------------------
        const uint32_t sw = warp - 2, g = sw >> 2, q = warp & 3;
        const uint32_t row_in_tile = q * 32 + lane;
        const uint32_t t_lane = (q * 32u) << 16;
        const float LOG2E = 1.4426950408889634f;
        uint32_t s_cnt = 0, p_cnt = 0, n_unit = 0, ntr = 0;
        bool ok = true;
        const bool prof = p.prof != nullptr && (sw & 3) == 0;
        long long x_sfull1 = 0, x_sfull2 = 0, x_pempty = 0, x_stat = 0, x_ofull = 0;
        // O of a finished unit: this group's 64 columns of the accumulator, straight from TMEM to global
        // memory.  It is read out AFTER pass 1 of the following unit (which does not touch O), when its last
        // P V product has long completed: nobody waits for it, and only pass 2 of that unit needs O free.
        bool have_prev = false;
        uint32_t prev_b = 0, prev_row0 = 0, prev_unit = 0;
        auto drain_o = [&](uint32_t ob, uint32_t orow0, uint32_t ounit) -> bool {
            long long co = prof ? clock64() : 0;
            if (!mbar_wait_patient(o_full, ounit & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL)) return false;
            tc_fence_after();
            if (prof) x_ofull += clock64() - co;
            const uint32_t row = orow0 + row_in_tile;
            float *orow = p.O + (uint64_t)ob * p.o_stride + (uint64_t)row * p.ldo + g * 64;
#pragma unroll 1
            for (uint32_t c = 0; c < 2; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + t_lane + 256 + g * 64 + c * 32, v);
                tmem_ld_wait();
                if (row < p.sq) {
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4 *>(orow + c * 32 + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_empty);
            return true;
        };
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            const uint32_t b = u / p.q_tiles, row0 = (u % p.q_tiles) * AT_ROWS;
            float m = -INFINITY, l = 0.0f;
            // ---- pass 1: row maximum and sum of exp over the blocks of this group ----
            for (uint32_t t = g; t < nkb && ok; t += 2) {
                long long c0 = prof ? clock64() : 0;
                ok = at_wait(s_full0 + 8 * g, s_cnt & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after();
                if (prof) x_sfull1 += clock64() - c0;
                if ((sw & 3) == 0) at_trace(p, 1 + g, ntr, (0x800000u + g * 0x400000u) | t);
                const uint32_t valid = p.sk - t * AT_KEYS;          // >= 128 except in a ragged last block
                const bool ragged = valid < AT_KEYS;
                const uint32_t ts = tmem_base + t_lane + g * 128;
                // all 128 scores of the row into registers, then the buffer goes straight back to the MMA
                // warp: the next product into it overlaps the arithmetic below
                uint32_t v0[32], v1[32], v2[32], v3[32];
                tmem_ld32(ts, v0); tmem_ld32(ts + 32, v1); tmem_ld32(ts + 64, v2); tmem_ld32(ts + 96, v3);
                tmem_ld_wait_on(v0); tmem_ld_wait_on(v1); tmem_ld_wait_on(v2); tmem_ld_wait_on(v3);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty0 + 8 * g);
                if (ragged) { at_mask(v0, 0, valid); at_mask(v1, 32, valid); at_mask(v2, 64, valid); at_mask(v3, 96, valid); }
                const float mx = fmax3(fmax3(at_max32(v0), at_max32(v1), at_max32(v2)), at_max32(v3), m);
                const float nmc = -mx * LOG2E;          // the first 32 columns of a block always exist: mx is finite
                l = l * ex2_approx(fmaf(m, LOG2E, nmc)) + ((at_sum32(v0, nmc) + at_sum32(v1, nmc)) + (at_sum32(v2, nmc) + at_sum32(v3, nmc)));
                m = mx;
                if ((sw & 3) == 0) at_trace(p, 1 + g, ntr, (0x900000u + g * 0x400000u) | t);
            }
            if (!ok) break;
            if (have_prev) {
                ok = drain_o(prev_b, prev_row0, prev_unit);
                if (!ok) break;
            }
            // ---- exchange (m, l) with the other group: both groups have a warp on every TMEM lane
            //      quadrant, so a row's two partial results meet in two spare TMEM columns of its lane
            //      (columns 448.., alternating with the unit so that a fast group cannot overwrite
            //      what a slow one has not read yet) ----
            const uint32_t par = n_unit & 1;
            const uint32_t t_stat = tmem_base + t_lane + 448 + par * 4;
            tmem_st2(t_stat + g * 2, __float_as_uint(m), __float_as_uint(l));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(stat0 + 8 * par);
            long long cs = prof ? clock64() : 0;
            ok = at_wait(stat0 + 8 * par, (n_unit >> 1) & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            if (prof) x_stat += clock64() - cs;
            uint32_t om, ol;
            tmem_ld2(t_stat + (g ^ 1) * 2, om, ol);
            tmem_ld_wait();
            const float other_m = __uint_as_float(om), other_l = __uint_as_float(ol);
            const float M = fmaxf(m, other_m);
            const float nMc = -M * LOG2E;
            const float L = l * ex2_approx(fmaf(m, LOG2E, nMc)) + other_l * ex2_approx(fmaf(other_m, LOG2E, nMc));
            const float off = nMc - lg2_approx(L);      // p = 2^(s log2 e + off) = exp(s - M) / L
            // ---- pass 2: P blocks ----
            for (uint32_t t = nkb + ((nkb + g) & 1); t < 2 * nkb && ok; t += 2) {
                const uint32_t kb = t - nkb;
                long long c0 = prof ? clock64() : 0;
                ok = at_wait(s_full0 + 8 * g, s_cnt & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after();
                if (prof) x_sfull2 += clock64() - c0;
                if ((sw & 3) == 0) at_trace(p, 1 + g, ntr, (0x800000u + g * 0x400000u) | t);
                const uint32_t valid = p.sk - kb * AT_KEYS;
                const bool ragged = valid < AT_KEYS;
                const uint32_t ts = tmem_base + t_lane + g * 128;
                // this row's two 128-byte lines of the P tile: keys 0..63 and 64..127 of the block
                uint8_t *line0 = smem_gen + (p_base - smem_base) + g * AT_P_BYTES + row_in_tile * 128, *line1 = line0 + AT_ATOM;
                const uint32_t row7 = row_in_tile & 7;
                uint32_t v0[32], v1[32], v2[32], v3[32];
                tmem_ld32(ts, v0); tmem_ld32(ts + 32, v1); tmem_ld32(ts + 64, v2); tmem_ld32(ts + 96, v3);
                tmem_ld_wait_on(v0); tmem_ld_wait_on(v1); tmem_ld_wait_on(v2); tmem_ld_wait_on(v3);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty0 + 8 * g);
                if (ragged) { at_mask(v0, 0, valid); at_mask(v1, 32, valid); at_mask(v2, 64, valid); at_mask(v3, 96, valid); }
                uint32_t w0[16], w1[16], w2[16], w3[16];
                at_probs32(v0, off, p.dtype, w0);
                at_probs32(v1, off, p.dtype, w1);
                at_probs32(v2, off, p.dtype, w2);
                at_probs32(v3, off, p.dtype, w3);
                // only now is the P tile needed: the product that read its previous contents has had the whole
                // of the arithmetic above to complete
                long long c1 = prof ? clock64() : 0;
                ok = at_wait(p_empty0 + 8 * g, (p_cnt & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                ++p_cnt;
                if (prof) x_pempty += clock64() - c1;
                at_store32(w0, line0, 0, row7);
                at_store32(w1, line0, 4, row7);
                at_store32(w2, line1, 0, row7);
                at_store32(w3, line1, 4, row7);
                fence_proxy_async_smem();      // generic-proxy writes -> visible to the MMA's async-proxy reads
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full0 + 8 * g);
                if ((sw & 3) == 0) at_trace(p, 1 + g, ntr, (0x900000u + g * 0x400000u) | t);
            }
            if (!ok) break;
            have_prev = true; prev_b = b; prev_row0 = row0; prev_unit = n_unit;
        }
        if (ok && have_prev) ok = drain_o(prev_b, prev_row0, prev_unit);
        if (prof && lane == 0) {
            unsigned long long *o = p.prof + (size_t)blockIdx.x * 16 + 6 + g * 5;
            o[0] = (unsigned long long)x_sfull1; o[1] = (unsigned long long)x_sfull2; o[2] = (unsigned long long)x_pempty;
            o[3] = (unsigned long long)x_stat; o[4] = (unsigned long long)x_ofull;
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, AT_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int encode_3d(CUtensorMap *map, int dtype, const void *ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld,
                     uint64_t z_stride, uint32_t box0, uint32_t box1) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return ST_UNSUPPORTED;
    CUtensorMapDataType dt = dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {ld * 2, (d2 > 1 ? z_stride : ld * d1) * 2};
    cuuint32_t box[3] = {box0, box1, 1}, estr[3] = {1, 1, 1};
    CUresult r = enc(map, dt, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(attention operand) failed: %d", (int)r);
        return ST_GEMM;
    }
    return ST_OK;
}

static bool al16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

int attn_fused_launch(const AttnProblem &a) {
    if (a.dtype != DT_F16 && a.dtype != DT_BF16) return ST_UNSUPPORTED;
    if (a.d != AT_D || a.batch == 0 || a.sq == 0 || a.sk == 0) return ST_UNSUPPORTED;
    if (a.batch > 0x7FFFFFu || a.sq > 0x7FFFFFFFu || a.sk > 0x7FFFFFFFu) return ST_UNSUPPORTED;
    if (!al16(a.q) || !al16(a.kt) || !al16(a.v) || !al16(a.o)) return ST_UNSUPPORTED;
    if (a.ldq % 8 || a.ldk % 8 || a.ldv % 8 || a.ldo % 4) return ST_UNSUPPORTED;
    if (a.batch > 1 && (a.q_stride % 8 || a.k_stride % 8 || a.v_stride % 8 || a.o_stride % 4)) return ST_UNSUPPORTED;
    if (ensure_device_info() != ST_OK) return ST_UNSUPPORTED;

    static bool attr_done[8] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 8) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM);
        if (e != cudaSuccess) {
            set_error("cudaFuncSetAttribute(attn_fused_kernel, smem=%u): %s", AT_SMEM, cudaGetErrorString(e));
            cudaGetLastError();
            return ST_GEMM;
        }
        attr_done[dev] = true;
    }

    CUtensorMap mq, mk, mv;
    int st;
    // Q [b][sq][d] as a K-major A operand: boxes of 64 d-elements x 128 rows
    if ((st = encode_3d(&mq, a.dtype, a.q, a.d, a.sq, a.batch, a.ldq, a.q_stride, 64, 128)) != ST_OK) return st;
    // Kt [b][d][sk]: MN-major B with N = keys (contiguous), K = d: boxes of 64 keys x 128 d-rows
    if ((st = encode_3d(&mk, a.dtype, a.kt, a.sk, a.d, a.batch, a.ldk, a.k_stride, 64, 128)) != ST_OK) return st;
    // V [b][sk][d]: MN-major B with N = d (contiguous), K = keys: boxes of 64 d x 128 key-rows
    if ((st = encode_3d(&mv, a.dtype, a.v, a.d, a.sk, a.batch, a.ldv, a.v_stride, 64, 128)) != ST_OK) return st;

    AttnParams p = {};
    p.batch = a.batch; p.sq = a.sq; p.sk = a.sk;
    p.q_tiles = (a.sq + AT_ROWS - 1) / AT_ROWS;
    p.nkb = (a.sk + AT_KEYS - 1) / AT_KEYS;
    const uint32_t fmt = a.dtype == DT_BF16 ? 1u : 0u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (1u << 16) | ((AT_KEYS >> 3) << 17) | ((AT_ROWS >> 4) << 24);
    p.dtype = (uint32_t)a.dtype;
    p.O = a.o; p.ldo = a.ldo; p.o_stride = a.o_stride;
    p.status = a.dev_status;
    p.prof = a.prof;
    p.debug = a.debug;
    p.q_tmem = a.q_tmem ? 1u : 0u;
    const uint64_t units = (uint64_t)p.batch * p.q_tiles;
    if (units > 0xFFFFFFFFull) return ST_UNSUPPORTED;
    const uint32_t sms = (uint32_t)device_sm_count();
    const uint32_t grid = (uint32_t)(units < sms ? units : sms);
    attn_fused_kernel<<<grid, AT_THREADS, AT_SMEM, a.stream>>>(mq, mk, mv, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("attn_fused_kernel launch: %s", cudaGetErrorString(e));
        return ST_GEMM;
    }
    note_launch();
    set_last_path("attn:fused_128x128");
    return ST_OK;
}

}  // namespace pgb
