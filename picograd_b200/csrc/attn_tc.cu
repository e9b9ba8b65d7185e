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
// Roles (320 threads, one CTA per SM, persistent over (batch, 128-row query block) units):
//   warp 0      TMA producer: Q (double-buffered) and a ring of 16 KB slots, each a [64 x 128] slice of
//               Kt or V as an MN-major B operand, in exactly the order the MMA warp consumes them
//   warp 1      MMA issuer: S = Q Kt_blk into one of two TMEM buffers; O += P V_blk into a third
//   warps 2-5   softmax group 0, warps 6-9 group 1: the groups take alternate S buffers; a thread owns one
//               query row (TMEM lane), reads its 128 scores with tcgen05.ld, and in pass 2 writes its row
//               of P into the 128-byte-swizzled K-major layout the MMA reads
// All waits are bounded mbarrier waits (status word + CTA abort flag), no named barriers.

#include "pg_internal.h"
#include "tc_ptx.cuh"

namespace pgb {

constexpr uint32_t AT_ROWS = 128;                 // query rows per unit == TMEM lanes
constexpr uint32_t AT_KEYS = 128;                 // keys per block
constexpr uint32_t AT_D = 128;                    // head dimension
constexpr uint32_t AT_ATOM = 128 * 64 * 2;        // [128 rows x 64 elements] K-major, or [64 k x 128 n] MN-major
constexpr uint32_t AT_SLOTS = 6;
constexpr uint32_t AT_Q_BYTES = 2 * AT_ATOM;      // one Q tile (two d-halves)
constexpr uint32_t AT_P_BYTES = 2 * AT_ATOM;      // one P tile (two key-halves)
constexpr uint32_t AT_BAR_BYTES = 1024;
constexpr uint32_t AT_SMEM = 1024 + 2 * AT_Q_BYTES + 2 * AT_P_BYTES + AT_SLOTS * AT_ATOM + AT_BAR_BYTES;
constexpr uint32_t AT_THREADS = 320;
constexpr uint32_t AT_TMEM_COLS = 512;            // S0 at 0, S1 at 128, O at 256
static_assert(AT_SMEM <= 232448, "shared memory budget");

struct AttnParams {
    uint32_t batch, sq, sk;
    uint32_t q_tiles, nkb;        // 128-row query blocks per batch element, 128-key blocks
    uint32_t idesc;
    uint32_t dtype;               // DT_F16 / DT_BF16: operands and the 16-bit P
    float *O;
    uint64_t ldo, o_stride;       // elements
    uint32_t *status;
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

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kt,
                  const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t q_base = smem_base;                                   // 2 x 32 KB
    const uint32_t p_base = q_base + 2 * AT_Q_BYTES;                     // 2 x 32 KB
    const uint32_t ring_base = p_base + 2 * AT_P_BYTES;                  // AT_SLOTS x 16 KB
    const uint32_t bar_base = ring_base + AT_SLOTS * AT_ATOM;
    uint32_t nb = 0;
    auto take = [&](uint32_t n) { uint32_t b = bar_base + 8u * nb; nb += n; return b; };
    const uint32_t full0 = take(AT_SLOTS), empty0 = take(AT_SLOTS);
    const uint32_t q_full0 = take(2), q_empty0 = take(2);
    const uint32_t s_full0 = take(2), s_empty0 = take(2);
    const uint32_t p_full0 = take(2), p_empty0 = take(2);
    const uint32_t o_full = take(1), o_empty = take(1);
    const uint32_t stat0 = take(2);
    const uint32_t tmem_slot = take(1);
    const uint32_t abort_off = (take(1) - smem_base);
    volatile uint32_t *tmem_slot_gen = (volatile uint32_t *)(smem_gen + (tmem_slot - smem_base));
    volatile uint32_t *abort_flag = (volatile uint32_t *)(smem_gen + abort_off);
    static_assert(8 * (2 * AT_SLOTS + 7 * 2 + 2 + 2) <= AT_BAR_BYTES, "barrier block");

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total_units = p.batch * p.q_tiles;
    const uint32_t nkb = p.nkb;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_kt);
        prefetch_tmap(&map_v);
        for (uint32_t s = 0; s < AT_SLOTS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(q_full0 + 8 * s, 1); mbar_init(q_empty0 + 8 * s, 1);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        uint32_t slot = 0, slot_phase = 0, n_unit = 0;
        bool ok = true;
        const uint64_t pol = l2_policy(0);
        // one 16 KB slot: rows k0..k0+63 (the MMA's K) by columns n0..n0+127 of an MN-major operand
        auto load_slot = [&](const CUtensorMap *map, int32_t n0, int32_t k0, int32_t z) -> bool {
            if (!mbar_wait(empty0 + 8 * slot, slot_phase ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY)) return false;
            if (elect_one()) {
                const uint32_t bar = full0 + 8 * slot, dst = ring_base + slot * AT_ATOM;
                mbar_arrive_expect_tx(bar, AT_ATOM);
                tma_load_3d<1>(dst, map, bar, n0, k0, z, pol);
                tma_load_3d<1>(dst + 8192, map, bar, n0 + 64, k0, z, pol);
            }
            __syncwarp();
            if (++slot == AT_SLOTS) { slot = 0; slot_phase ^= 1; }
            return true;
        };
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            const int32_t b = (int32_t)(u / p.q_tiles), row0 = (int32_t)((u % p.q_tiles) * AT_ROWS);
            const uint32_t qb = n_unit & 1, q_phase = (n_unit >> 1) & 1;
            ok = mbar_wait(q_empty0 + 8 * qb, q_phase ^ 1, abort_flag, p.status, DEV_ERR_WAIT_EMPTY);
            if (!ok) break;
            if (elect_one()) {
                const uint32_t bar = q_full0 + 8 * qb, dst = q_base + qb * AT_Q_BYTES;
                mbar_arrive_expect_tx(bar, AT_Q_BYTES);
                tma_load_3d<1>(dst, &map_q, bar, 0, row0, b, pol);
                tma_load_3d<1>(dst + AT_ATOM, &map_q, bar, 64, row0, b, pol);
            }
            __syncwarp();
            auto load_kt = [&](uint32_t kb) {     // K of this MMA = d: halves 0..63, 64..127; N = keys
                return load_slot(&map_kt, (int32_t)(kb * AT_KEYS), 0, b) && load_slot(&map_kt, (int32_t)(kb * AT_KEYS), 64, b);
            };
            auto load_v = [&](uint32_t kb) {      // K of this MMA = keys: halves of the block; N = d
                return load_slot(&map_v, 0, (int32_t)(kb * AT_KEYS), b) && load_slot(&map_v, 0, (int32_t)(kb * AT_KEYS + 64), b);
            };
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) ok = load_kt(kb);
            for (uint32_t i = 0; i <= nkb && ok; ++i) {
                if (i < nkb) ok = load_kt(i);
                if (ok && i >= 1) ok = load_v(i - 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        uint32_t slot = 0, slot_phase = 0, n_unit = 0;
        uint32_t s_cnt[2] = {0, 0}, p_cnt[2] = {0, 0};
        bool ok = true;
        const uint32_t idesc = p.idesc;
        const uint64_t dq = make_desc(q_base, 0), dp = make_desc(p_base, 0), dr = make_desc(ring_base, 64 * 128);
        const uint32_t q_hi = (uint32_t)(dq >> 32), p_hi = (uint32_t)(dp >> 32), r_hi = (uint32_t)(dr >> 32);
        const uint32_t q_lo0 = (uint32_t)dq, p_lo0 = (uint32_t)dp, r_lo0 = (uint32_t)dr;
        // 4 MMAs (k = 16 each) of one slot: A advances 32 bytes per step inside its 128-byte rows, the
        // MN-major B advances 16 k-rows = 2048 bytes
        auto mma_slot = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, bool first) -> bool {
            if (!mbar_wait(full0 + 8 * slot, slot_phase, abort_flag, p.status, DEV_ERR_WAIT_FULL)) return false;
            tc_fence_after();
            const uint32_t b_lo = r_lo0 + slot * (AT_ATOM >> 4);
            if (elect_one()) {
#pragma unroll
                for (uint32_t kk = 0; kk < 4; ++kk)
                    umma_lohi<1>(d_tmem, a_lo + kk * 2, a_hi, b_lo + kk * 128, r_hi, idesc, (first && kk == 0) ? 0u : 1u);
                umma_commit<1>(empty0 + 8 * slot);
            }
            __syncwarp();
            if (++slot == AT_SLOTS) { slot = 0; slot_phase ^= 1; }
            return true;
        };
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            const uint32_t qb = n_unit & 1, q_phase = (n_unit >> 1) & 1;
            ok = mbar_wait(q_full0 + 8 * qb, q_phase, abort_flag, p.status, DEV_ERR_WAIT_FULL);
            if (!ok) break;
            const uint32_t q_lo = q_lo0 + qb * (AT_Q_BYTES >> 4);
            // S block number t of this unit (0 .. 2 nkb - 1) goes to S buffer t % 2
            auto s_block = [&](uint32_t t) -> bool {
                const uint32_t sb = t & 1;
                if (!mbar_wait(s_empty0 + 8 * sb, (s_cnt[sb] & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY)) return false;
                tc_fence_after();
                ++s_cnt[sb];
                const uint32_t d_tmem = tmem_base + sb * 128;
                if (!mma_slot(d_tmem, q_lo, q_hi, true)) return false;
                if (!mma_slot(d_tmem, q_lo + (AT_ATOM >> 4), q_hi, false)) return false;
                if (elect_one()) umma_commit<1>(s_full0 + 8 * sb);
                __syncwarp();
                return true;
            };
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) ok = s_block(kb);
            for (uint32_t i = 0; i <= nkb && ok; ++i) {
                if (i < nkb) ok = s_block(nkb + i);
                if (ok && i >= 1) {
                    const uint32_t j = i - 1, pb = (nkb + j) & 1;
                    ok = mbar_wait(p_full0 + 8 * pb, p_cnt[pb] & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                    if (!ok) break;
                    ++p_cnt[pb];
                    if (j == 0) {   // the previous unit's O must have been read out
                        ok = mbar_wait(o_empty, (n_unit & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + 256, pl = p_lo0 + pb * (AT_P_BYTES >> 4);
                    ok = mma_slot(d_tmem, pl, p_hi, j == 0) && mma_slot(d_tmem, pl + (AT_ATOM >> 4), p_hi, false);
                    if (!ok) break;
                    if (elect_one()) {
                        umma_commit<1>(p_empty0 + 8 * pb);
                        if (j == nkb - 1) {
                            umma_commit<1>(o_full);
                            umma_commit<1>(q_empty0 + 8 * qb);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ------------------------------ softmax groups ------------------------------
        const uint32_t sw = warp - 2, g = sw >> 2, q = warp & 3;
        const uint32_t row_in_tile = q * 32 + lane;
        const uint32_t t_lane = (q * 32u) << 16;
        const float LOG2E = 1.4426950408889634f;
        uint32_t s_cnt = 0, p_cnt = 0, n_unit = 0;
        bool ok = true;
        for (uint32_t u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++n_unit) {
            const uint32_t b = u / p.q_tiles, row0 = (u % p.q_tiles) * AT_ROWS;
            float m = -INFINITY, l = 0.0f;
            // ---- pass 1: row maximum and sum of exp over the blocks of this group ----
            for (uint32_t t = g; t < nkb && ok; t += 2) {
                ok = mbar_wait(s_full0 + 8 * g, s_cnt & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after();
                const uint32_t valid = p.sk - t * AT_KEYS;          // >= 128 except in a ragged last block
#pragma unroll 1
                for (uint32_t c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + t_lane + g * 128 + c * 32, v);
                    tmem_ld_wait();
                    if (c == 3) {       // every score of the block is in registers or consumed: free the buffer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(s_empty0 + 8 * g);
                    }
                    if (valid < AT_KEYS) {
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            if (c * 32 + j >= valid) v[j] = __float_as_uint(-INFINITY);
                    }
                    float mx = m;
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
                    if (mx != -INFINITY) {
                        const float nmc = -mx * LOG2E;
                        float a0 = l * ex2_approx(fmaf(m, LOG2E, nmc)), a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 4) {
                            a0 += ex2_approx(fmaf(__uint_as_float(v[j]), LOG2E, nmc));
                            a1 += ex2_approx(fmaf(__uint_as_float(v[j + 1]), LOG2E, nmc));
                            a2 += ex2_approx(fmaf(__uint_as_float(v[j + 2]), LOG2E, nmc));
                            a3 += ex2_approx(fmaf(__uint_as_float(v[j + 3]), LOG2E, nmc));
                        }
                        l = (a0 + a1) + (a2 + a3);
                        m = mx;
                    }
                }
            }
            if (!ok) break;
            // ---- exchange (m, l) with the other group: both groups have a warp on every TMEM lane
            //      quadrant, so a row's two partial results meet in two spare TMEM columns of its lane
            //      (columns 384.., alternating with the unit so that a fast group cannot overwrite
            //      what a slow one has not read yet) ----
            const uint32_t par = n_unit & 1;
            const uint32_t t_stat = tmem_base + t_lane + 384 + par * 4;
            tmem_st2(t_stat + g * 2, __float_as_uint(m), __float_as_uint(l));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(stat0 + 8 * par);
            ok = mbar_wait(stat0 + 8 * par, (n_unit >> 1) & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            uint32_t om, ol;
            tmem_ld2(t_stat + (g ^ 1) * 2, om, ol);
            tmem_ld_wait();
            const float other_m = __uint_as_float(om), other_l = __uint_as_float(ol);
            const float M = fmaxf(m, other_m);
            const float nMc = -M * LOG2E;
            const float L = l * ex2_approx(fmaf(m, LOG2E, nMc)) + other_l * ex2_approx(fmaf(other_m, LOG2E, nMc));
            const float inv = 1.0f / L;
            // ---- pass 2: P blocks ----
            for (uint32_t t = nkb + ((nkb + g) & 1); t < 2 * nkb && ok; t += 2) {
                const uint32_t kb = t - nkb;
                ok = mbar_wait(s_full0 + 8 * g, s_cnt & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
                if (!ok) break;
                ++s_cnt;
                ok = mbar_wait(p_empty0 + 8 * g, (p_cnt & 1) ^ 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                ++p_cnt;
                tc_fence_after();
                const uint32_t valid = p.sk - kb * AT_KEYS;
                uint8_t *prow = smem_gen + (p_base - smem_base) + g * AT_P_BYTES + row_in_tile * 128;
#pragma unroll 1
                for (uint32_t c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + t_lane + g * 128 + c * 32, v);
                    tmem_ld_wait();
                    if (c == 3) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(s_empty0 + 8 * g);
                    }
                    if (valid < AT_KEYS) {
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            if (c * 32 + j >= valid) v[j] = __float_as_uint(-INFINITY);
                    }
                    uint32_t w[16];
#pragma unroll
                    for (uint32_t j = 0; j < 32; j += 2) {
                        const float p0 = ex2_approx(fmaf(__uint_as_float(v[j]), LOG2E, nMc)) * inv;
                        const float p1 = ex2_approx(fmaf(__uint_as_float(v[j + 1]), LOG2E, nMc)) * inv;
                        w[j >> 1] = at_pack16(p0, p1, p.dtype);
                    }
                    // keys c*32 .. c*32+31 of this row: key-half (atom) c / 2, 16-byte chunks (c % 2) * 4 .. + 3
                    uint8_t *dst = prow + (c >> 1) * AT_ATOM;
#pragma unroll
                    for (uint32_t jj = 0; jj < 4; ++jj)
                        *reinterpret_cast<uint4 *>(dst + (((((c & 1) * 4 + jj)) ^ (row_in_tile & 7)) << 4)) =
                            make_uint4(w[4 * jj], w[4 * jj + 1], w[4 * jj + 2], w[4 * jj + 3]);
                }
                fence_proxy_async_smem();      // generic-proxy writes -> visible to the MMA's async-proxy reads
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full0 + 8 * g);
            }
            if (!ok) break;
            // ---- O: this group's 64 columns of the finished accumulator ----
            ok = mbar_wait_patient(o_full, n_unit & 1, abort_flag, p.status, DEV_ERR_WAIT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            const uint32_t row = row0 + row_in_tile;
            float *orow = p.O + (uint64_t)b * p.o_stride + (uint64_t)row * p.ldo + g * 64;
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
    // Kt [b][d][sk]: MN-major B with N = keys (contiguous), K = d: boxes of 64 keys x 64 d-rows
    if ((st = encode_3d(&mk, a.dtype, a.kt, a.sk, a.d, a.batch, a.ldk, a.k_stride, 64, 64)) != ST_OK) return st;
    // V [b][sk][d]: MN-major B with N = d (contiguous), K = keys: boxes of 64 d x 64 key-rows
    if ((st = encode_3d(&mv, a.dtype, a.v, a.d, a.sk, a.batch, a.ldv, a.v_stride, 64, 64)) != ST_OK) return st;

    AttnParams p = {};
    p.batch = a.batch; p.sq = a.sq; p.sk = a.sk;
    p.q_tiles = (a.sq + AT_ROWS - 1) / AT_ROWS;
    p.nkb = (a.sk + AT_KEYS - 1) / AT_KEYS;
    const uint32_t fmt = a.dtype == DT_BF16 ? 1u : 0u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (1u << 16) | ((AT_KEYS >> 3) << 17) | ((AT_ROWS >> 4) << 24);
    p.dtype = (uint32_t)a.dtype;
    p.O = a.o; p.ldo = a.ldo; p.o_stride = a.o_stride;
    p.status = a.dev_status;
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
