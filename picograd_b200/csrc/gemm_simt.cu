// FFMA GEMM for everything the tensor-core kernel does not take: f32 operands
// (picograd's pg_gemm, backend/backend.c:134-148, whose CUDA kernel is
// backend/cuda/kernels/kernel_sgemm.c:50-111), leading dimensions or pointers
// that break the TMA alignment rules, and tiny shapes.
//
// Every C element is one fused-multiply-add chain over k ascending on exactly
// upcast operands — the same arithmetic as picograd's CPU micro-kernels
// (backend/cpu/asm/sgemm_avx512.S:126-154), so results agree with them bit for
// bit, not merely within tolerance.  No TF32, no reordering.
//
// Tiling: 256 threads, a TILE x TILE block of C per CTA, (TILE/16)^2 outputs per
// thread, K in slabs of 16 staged through shared memory with register prefetch.  Operands are read
// through generic (row, column, batch) element strides, so transposed views and
// mixed dtypes need no separate kernel.

#include "pg_internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace pgb {

struct SimtParams {
    uint32_t M, N, K, batch;
    const void *A; long long a_rs, a_cs, a_bs;
    const void *B; long long b_rs, b_cs, b_bs;
    float *C; long long ldc, c_bs;
    int dtype_a, dtype_b, accumulate;
    // fused epilogue of pg_cpu_gemm_fused_ex (backend/cpu/gemm.c:718-817): each row of C starts as the
    // bias row, the micro-kernels accumulate onto it, the activation runs over the finished row
    const float *bias; int act;
    unsigned short *c16; long long ld16, c16_bs; int dtype16;
    int act_copy_only;          // the activation goes into the 16-bit copy only
};

__device__ __forceinline__ float simt_act(float x, int act) {
    if (act == 1) return x > 0.0f ? x : 0.0f;
    if (act == 2) return 0.5f * x * (1.0f + erff(x * 0.70710678118f));
    return x;
}
__device__ __forceinline__ unsigned short simt_to16(float v, int dtype16) {
    if (dtype16 == DT_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    return __half_as_ushort(__float2half_rn(v));
}

__device__ __forceinline__ float load_as_f32(const void *base, long long idx, int dtype) {
    if (dtype == DT_F32) return reinterpret_cast<const float *>(base)[idx];
    const unsigned short raw = reinterpret_cast<const unsigned short *>(base)[idx];
    if (dtype == DT_BF16) return __uint_as_float((unsigned)raw << 16);
    return __half2float(__ushort_as_half(raw));
}

constexpr int SK = 16;

// The next K slab is fetched into registers while the current one is multiplied out of shared
// memory, so the global-load latency overlaps the FFMA work; each thread owns a T x T block of
// contiguous rows and columns and reads its operands from shared memory as 16-byte vectors.
template <int TILE>
__global__ void __launch_bounds__(256) simt_gemm_kernel(const SimtParams p) {
    constexpr int T = TILE / 16;              // outputs per thread per dimension
    constexpr int PER = TILE * SK / 256;      // elements of each operand a thread stages per slab
    constexpr int LD = TILE + 4;              // row pitch: keeps 16-byte alignment, spreads banks
    __shared__ __align__(16) float As[SK][LD];
    __shared__ __align__(16) float Bs[SK][LD];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const uint32_t bz = blockIdx.z;
    const long long m0 = (long long)blockIdx.y * TILE, n0 = (long long)blockIdx.x * TILE;
    const long long a_off = (long long)bz * p.a_bs, b_off = (long long)bz * p.b_bs;

    // the chain of column gn starts at bias[gn], as in picograd, where the micro-kernel accumulates onto
    // a C row that was initialised with the bias
    float2 acc2[T][T / 2];                    // columns in pairs: what fma.rn.f32x2 (sm_100) reads and writes
#define ACC(i, j) (((j) & 1) ? acc2[i][(j) >> 1].y : acc2[i][(j) >> 1].x)
#pragma unroll
    for (int j = 0; j < T; ++j) {
        const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
        const float b0 = (p.bias && gn < p.N) ? p.bias[gn] : 0.0f;
#pragma unroll
        for (int i = 0; i < T; ++i) ACC(i, j) = b0;
    }

    // walk the contiguous dimension of each operand with consecutive threads
    const bool a_k_contig = (p.a_cs == 1);
    const bool b_n_contig = (p.b_cs == 1);
    int a_kk[PER], a_mm[PER], b_kk[PER], b_nn[PER];
#pragma unroll
    for (int r = 0; r < PER; ++r) {
        const int idx = tid + r * 256;
        if (a_k_contig) { a_kk[r] = idx % SK; a_mm[r] = idx / SK; } else { a_mm[r] = idx % TILE; a_kk[r] = idx / TILE; }
        if (b_n_contig) { b_nn[r] = idx % TILE; b_kk[r] = idx / TILE; } else { b_kk[r] = idx % SK; b_nn[r] = idx / SK; }
    }
    // D K-slabs are kept in flight in registers: the loads of slab i + D are issued while slab i is being
    // multiplied, so a load has D slabs of arithmetic to arrive (a 64-wide tile leaves one CTA of 8 warps per
    // SM on small products: nothing else hides the latency of L2).
    constexpr int D = TILE == 64 ? 4 : 1;
    float ra[D][PER], rb[D][PER];
    auto fetch = [&](float (&qa)[PER], float (&qb)[PER], uint32_t k0) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const long long gm = m0 + a_mm[r], gka = (long long)k0 + a_kk[r];
            qa[r] = (gm < p.M && gka < p.K) ? load_as_f32(p.A, a_off + gm * p.a_rs + gka * p.a_cs, p.dtype_a) : 0.0f;
            const long long gn = n0 + b_nn[r], gkb = (long long)k0 + b_kk[r];
            qb[r] = (gn < p.N && gkb < p.K) ? load_as_f32(p.B, b_off + gkb * p.b_rs + gn * p.b_cs, p.dtype_b) : 0.0f;
        }
    };

#pragma unroll
    for (int d = 0; d < D; ++d)
        if ((uint32_t)(d * SK) < p.K) fetch(ra[d], rb[d], d * SK);
    for (uint32_t kbase = 0; kbase < p.K; kbase += D * SK) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const uint32_t k0 = kbase + d * SK;
            if (k0 >= p.K) break;
#pragma unroll
            for (int r = 0; r < PER; ++r) {
                As[a_kk[r]][a_mm[r]] = ra[d][r];
                Bs[b_kk[r]][b_nn[r]] = rb[d][r];
            }
            __syncthreads();
            if (k0 + D * SK < p.K) fetch(ra[d], rb[d], k0 + D * SK);
            // stop at the true K so that the chain of each element is exactly its K fused multiply-adds
            const int kmax = (p.K - k0) < (uint32_t)SK ? (int)(p.K - k0) : SK;
#pragma unroll 4
            for (int kk = 0; kk < kmax; ++kk) {
                // a thread's T rows (columns) are groups of four, 64 apart: the 16 threads of a half-warp
                // then read 256 contiguous bytes per 16-byte load — no shared-memory bank conflict
                float a[T], b[T];
#pragma unroll
                for (int i = 0; i < T; i += 4) {
                    const float4 va = *reinterpret_cast<const float4 *>(&As[kk][ty * 4 + i * 16]);
                    a[i] = va.x; a[i + 1] = va.y; a[i + 2] = va.z; a[i + 3] = va.w;
                    const float4 vb = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4 + i * 16]);
                    b[i] = vb.x; b[i + 1] = vb.y; b[i + 2] = vb.z; b[i + 3] = vb.w;
                }
                // two columns per instruction; each lane is the same fused multiply-add as the scalar form
#pragma unroll
                for (int i = 0; i < T; ++i) {
                    const float2 aa = make_float2(a[i], a[i]);
#pragma unroll
                    for (int j = 0; j < T; j += 2) acc2[i][j >> 1] = __ffma2_rn(aa, make_float2(b[j], b[j + 1]), acc2[i][j >> 1]);
                }
            }
            __syncthreads();
        }
    }

    float *Cb = p.C + (long long)bz * p.c_bs;
#pragma unroll
    for (int i = 0; i < T; ++i) {
        const long long gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < T; ++j) {
            const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
            if (gn >= p.N) continue;
            float *dst = Cb + gm * p.ldc + gn;
            const float r = simt_act(ACC(i, j), p.act), rc = p.act_copy_only ? ACC(i, j) : r;
            *dst = p.accumulate ? (*dst + rc) : rc;
            if (p.c16) p.c16[(long long)bz * p.c16_bs + gm * p.ld16 + gn] = simt_to16(r, p.dtype16);
        }
    }
}
#undef ACC

// ---------------------------------------------------------------------------------------------
// f32 x f32, both operands row-major with unit column stride and 16-byte aligned rows (the shape of
// pg_gemm): 128 x 128 tile (64 x 64 for small products, which then fill more SMs), K slabs of 16, 16-byte global loads, double-buffered shared memory (one
// barrier per slab), 8 x 8 outputs per thread.  Same arithmetic as above: one fmaf chain per element,
// k ascending (zero-filled slab tails add exact zeros).
// ---------------------------------------------------------------------------------------------
template <int TILE>
__global__ void __launch_bounds__(256, 2) sgemm_nn_kernel(const SimtParams p) {
    constexpr int LD = TILE + 4, T = TILE / 16, NV = TILE / 64;     // NV 16-byte vectors of each operand per thread and slab
    __shared__ __align__(16) float As[2][SK][LD];
    __shared__ __align__(16) float Bs[2][SK][LD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const uint32_t bz = blockIdx.z;
    const long long m0 = (long long)blockIdx.y * TILE, n0 = (long long)blockIdx.x * TILE;
    const float *A = reinterpret_cast<const float *>(p.A) + (long long)bz * p.a_bs;
    const float *B = reinterpret_cast<const float *>(p.B) + (long long)bz * p.b_bs;

    float acc[T][T];
#pragma unroll
    for (int j = 0; j < T; ++j) {
        const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
        const float b0 = (p.bias && gn < p.N) ? p.bias[gn] : 0.0f;
#pragma unroll
        for (int i = 0; i < T; ++i) acc[i][j] = b0;
    }

    // staging roles: A as float4 along k (rows a_r, a_r + 64), B as float4 along n (k rows b_k, b_k + BKS)
    constexpr int BROW = TILE / 4;                 // float4 per k-row of B
    constexpr int BKS = 256 / BROW;                // k-rows of B covered by one pass of the CTA
    const int a_r = tid >> 2, a_kq = (tid & 3) * 4;
    const int b_k = tid / BROW, b_nq = (tid % BROW) * 4;
    // R register sets: the loads of slab s + R are issued while slab s is multiplied and slab s + 1 already sits
    // in the other shared-memory buffer.  R = 2 measured slower than R = 1 on the 64-wide tile (29.2 vs 25.0 us
    // at 512^3), so one set it is.
    constexpr int R = 1;
    float4 ra[R][NV], rb[R][NV];
    auto fetch = [&](float4 (&qa)[NV], float4 (&qb)[NV], uint32_t k0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const long long gm = m0 + a_r + 64 * i, gk = (long long)k0 + a_kq;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gm < p.M && gk < p.K) {
                const float *src = A + gm * p.a_rs + gk;
                if (gk + 3 < p.K) v = *reinterpret_cast<const float4 *>(src);
                else {
                    v.x = src[0];
                    if (gk + 1 < p.K) v.y = src[1];
                    if (gk + 2 < p.K) v.z = src[2];
                }
            }
            qa[i] = v;
            const long long gkb = (long long)k0 + b_k + BKS * i, gn = n0 + b_nq;
            float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gkb < p.K && gn < p.N) {
                const float *src = B + gkb * p.b_rs + gn;
                if (gn + 3 < p.N) w = *reinterpret_cast<const float4 *>(src);
                else {
                    w.x = src[0];
                    if (gn + 1 < p.N) w.y = src[1];
                    if (gn + 2 < p.N) w.z = src[2];
                }
            }
            qb[i] = w;
        }
    };
    auto stash = [&](const float4 (&qa)[NV], const float4 (&qb)[NV], int buf) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            As[buf][a_kq + 0][a_r + 64 * i] = qa[i].x;
            As[buf][a_kq + 1][a_r + 64 * i] = qa[i].y;
            As[buf][a_kq + 2][a_r + 64 * i] = qa[i].z;
            As[buf][a_kq + 3][a_r + 64 * i] = qa[i].w;
            *reinterpret_cast<float4 *>(&Bs[buf][b_k + BKS * i][b_nq]) = qb[i];
        }
    };
    auto multiply = [&](int buf) {
#pragma unroll
        for (int kk = 0; kk < SK; ++kk) {
            float a[T], b[T];
#pragma unroll
            for (int i = 0; i < T; i += 4) {
                const float4 va = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4 + i * 16]);
                a[i] = va.x; a[i + 1] = va.y; a[i + 2] = va.z; a[i + 3] = va.w;
                const float4 vb = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4 + i * 16]);
                b[i] = vb.x; b[i + 1] = vb.y; b[i + 2] = vb.z; b[i + 3] = vb.w;
            }
#pragma unroll
            for (int i = 0; i < T; ++i)
#pragma unroll
                for (int j = 0; j < T; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
    };

    // slab s is multiplied out of shared buffer s % 2; register set (s + 1) % R holds slab s + 1 on entry to
    // iteration s, is stored to the other buffer and refilled with slab s + 1 + R
    if (p.K) {
        fetch(ra[0], rb[0], 0);
        stash(ra[0], rb[0], 0);
#pragma unroll
        for (int r = 0; r < R; ++r)
            if ((uint32_t)((r + 1) * SK) < p.K) fetch(ra[(r + 1) % R], rb[(r + 1) % R], (r + 1) * SK);
    }
    __syncthreads();
    for (uint32_t k0 = 0; k0 < p.K; k0 += R * SK) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t ks = k0 + r * SK;                 // slab s = ks / SK, s % R == r
            if (ks >= p.K) break;
            const int buf = (ks / SK) & 1, set = (r + 1) % R;
            const bool more = ks + SK < p.K;
            if (more) stash(ra[set], rb[set], buf ^ 1);
            if (ks + (1 + R) * SK < p.K) fetch(ra[set], rb[set], ks + (1 + R) * SK);
            multiply(buf);
            __syncthreads();
        }
    }

    float *Cb = p.C + (long long)bz * p.c_bs;
    const bool vec = (p.ldc % 4 == 0) && (((uintptr_t)Cb & 15) == 0) && !p.accumulate;
    if (p.act && !p.act_copy_only) {
#pragma unroll
        for (int i = 0; i < T; ++i)
#pragma unroll
            for (int j = 0; j < T; ++j) acc[i][j] = simt_act(acc[i][j], p.act);
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
        const long long gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
        if (p.c16) {
#pragma unroll
            for (int j = 0; j < T; ++j) {
                const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
                const float y = p.act_copy_only ? simt_act(acc[i][j], p.act) : acc[i][j];
                if (gn < p.N) p.c16[(long long)bz * p.c16_bs + gm * p.ld16 + gn] = simt_to16(y, p.dtype16);
            }
        }
#pragma unroll
        for (int jh = 0; jh < T / 4; ++jh) {
            const long long gn = n0 + tx * 4 + jh * 64;
            float *dst = Cb + gm * p.ldc + gn;
            if (vec && gn + 3 < p.N) {
                *reinterpret_cast<float4 *>(dst) = make_float4(acc[i][jh * 4], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gn + j < p.N) dst[j] = p.accumulate ? dst[j] + acc[i][jh * 4 + j] : acc[i][jh * 4 + j];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same product for SMALL f32 shapes (the 512^3 of pg_matmul's test configuration): 32 x 64 tile and 128
// threads, so that 512^3 is 128 CTAs on the 148 SMs (a 64 x 64 tile fills 64), each thread a 4 x 4 block; K slabs
// of 16 go from global to shared memory with 16-byte cp.async copies, four slabs in flight, one barrier per slab,
// so the L2 latency that bounded the register-staged kernel (~0.8 us per slab, 32 slabs) is hidden behind the
// arithmetic.  Rows of A stay rows in shared memory ([m][k], read as 16-byte vectors along k); tails in M, N and K
// are zero-filled by the copy itself (source size < 16).  One fmaf chain per element, k ascending: the bits of
// picograd's CPU kernels, as above.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gsrc, int src_bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int PM = 32, PN = 64, PK = 32, PSTAGES = 3;
int g_small_f32_pipe = 1;      // small f32 products take the cp.async kernel (0: the register-staged 64 x 64 one)
__global__ void __launch_bounds__(128) sgemm_nn_pipe_kernel(const SimtParams p) {
    constexpr int LDA = PK + 4, LDB = PN + 4;
    __shared__ __align__(16) float As[PSTAGES][PM][LDA];
    __shared__ __align__(16) float Bs[PSTAGES][PK][LDB];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;                 // 16 x 8 threads, each 4 columns x 4 rows
    const uint32_t bz = blockIdx.z;
    const long long m0 = (long long)blockIdx.y * PM, n0 = (long long)blockIdx.x * PN;
    const float *A = reinterpret_cast<const float *>(p.A) + (long long)bz * p.a_bs;
    const float *B = reinterpret_cast<const float *>(p.B) + (long long)bz * p.b_bs;
    // Launched with programmatic stream serialisation: this CTA may have been started while the kernel before it in
    // the stream was still draining.  Nothing of global memory is touched before that kernel has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    float2 acc2[4][2];                   // columns in pairs: what fma.rn.f32x2 reads and writes
#define ACC(i, j) (((j) & 1) ? acc2[i][(j) >> 1].y : acc2[i][(j) >> 1].x)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const long long gn = n0 + tx * 4 + j;
        const float b0 = (p.bias && gn < p.N) ? p.bias[gn] : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ACC(i, j) = b0;
    }

    // copy roles: A 32 rows x 8 vectors = two per thread; B 32 k-rows x 16 vectors = four per thread
    const int a_r = tid >> 3, a_kq = (tid & 7) * 4;
    const int b_k = tid >> 4, b_nq = (tid & 15) * 4;
    auto issue = [&](int stage, uint32_t k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long gm = m0 + a_r + 16 * h, gk = (long long)k0 + a_kq;
            int bytes = 0;
            if (gm < p.M && gk < p.K) bytes = (int)((p.K - gk) < 4 ? (p.K - gk) : 4) * 4;
            cp_async_16(&As[stage][a_r + 16 * h][a_kq], bytes ? A + gm * p.a_rs + gk : A, bytes);
        }
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const long long gk = (long long)k0 + b_k + 8 * h, gn = n0 + b_nq;
            int bytes = 0;
            if (gk < p.K && gn < p.N) bytes = (int)((p.N - gn) < 4 ? (p.N - gn) : 4) * 4;
            cp_async_16(&Bs[stage][b_k + 8 * h][b_nq], bytes ? B + gk * p.b_rs + gn : B, bytes);
        }
    };
    // the operands of four k steps in registers; the next four are fetched while these are multiplied, so that the
    // one warp a scheduler has does not wait for shared memory between its multiply-adds
    struct Frag { float4 a[4], b[4]; };
    auto fetch = [&](Frag &f, int st, int kq) {
#pragma unroll
        for (int i = 0; i < 4; ++i) f.a[i] = *reinterpret_cast<const float4 *>(&As[st][ty * 4 + i][kq]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) f.b[kk] = *reinterpret_cast<const float4 *>(&Bs[st][kq + kk][tx * 4]);
    };
    auto multiply = [&](const Frag &f) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = kk == 0 ? f.a[i].x : (kk == 1 ? f.a[i].y : (kk == 2 ? f.a[i].z : f.a[i].w));
                const float2 aa = make_float2(a, a);      // fma.rn.f32x2: two columns per instruction, same arithmetic per lane
                acc2[i][0] = __ffma2_rn(aa, make_float2(f.b[kk].x, f.b[kk].y), acc2[i][0]);
                acc2[i][1] = __ffma2_rn(aa, make_float2(f.b[kk].z, f.b[kk].w), acc2[i][1]);
            }
        }
    };

    const uint32_t slabs = (p.K + PK - 1) / PK;
#pragma unroll
    for (int s = 0; s < PSTAGES - 1; ++s) {
        if ((uint32_t)s < slabs) issue(s, s * PK);
        cp_async_commit();
    }
    for (uint32_t s = 0; s < slabs; ++s) {
        cp_async_wait<PSTAGES - 2>();          // slab s has landed (this thread's copies) ...
        __syncthreads();                       // ... and everyone's; the stage read in iteration s - 1 is free again
        if (s + PSTAGES - 1 < slabs) issue((s + PSTAGES - 1) % PSTAGES, (s + PSTAGES - 1) * PK);
        cp_async_commit();
        const int st = s % PSTAGES;
        Frag f0, f1;
        fetch(f0, st, 0);
#pragma unroll
        for (int kq = 0; kq < PK; kq += 8) {
            fetch(f1, st, kq + 4);
            multiply(f0);
            if (kq + 8 < PK) fetch(f0, st, kq + 8);
            multiply(f1);
        }
    }

    float *Cb = p.C + (long long)bz * p.c_bs;
    const bool vec = (p.ldc % 4 == 0) && (((uintptr_t)Cb & 15) == 0) && !p.accumulate;
    const long long gn = n0 + tx * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long gm = m0 + ty * 4 + i;
        if (gm >= p.M) continue;
        float y[4], c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            y[j] = simt_act(ACC(i, j), p.act);
            c[j] = p.act_copy_only ? ACC(i, j) : y[j];
        }
        if (p.c16) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (gn + j < p.N) p.c16[(long long)bz * p.c16_bs + gm * p.ld16 + gn + j] = simt_to16(y[j], p.dtype16);
        }
        float *dst = Cb + gm * p.ldc + gn;
        if (vec && gn + 3 < p.N) {
            *reinterpret_cast<float4 *>(dst) = make_float4(c[0], c[1], c[2], c[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (gn + j < p.N) dst[j] = p.accumulate ? dst[j] + c[j] : c[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
#undef ACC

// The same product for LARGE f32 shapes: 128 x 128 tile, 256 threads, 8 x 8 outputs per thread (rows ty*4.. and
// 64 + ty*4.., columns tx*4.. and 64 + tx*4..), K slabs of 32 brought in by 16-byte cp.async copies with three slabs
// in flight (106 KB of dynamic shared memory, two CTAs per SM: 16 warps hide each other's shared-memory latency).
// A stays [m][k] in shared memory; a thread reads two k steps of its eight rows as 8-byte vectors and two k rows of
// B as 16-byte vectors, then issues the 128 multiply-adds of those two steps as 64 fma.rn.f32x2 (sm_100: two
// columns per instruction, each lane the same fused multiply-add as the scalar form; measured 48.1 against 43.5
// TFLOP/s at 4096^3 for scalar fmaf in the same kernel with 16-deep slabs, 50.7 with 32-deep ones, 38.6 for the
// register-staged kernel).  One fmaf chain per
// element, k ascending, tails zero-filled by the copies: the bits of picograd's CPU kernels.
// ---------------------------------------------------------------------------------------------
constexpr int GM = 128, GN = 128, GK = 32, GSTAGES = 3;
constexpr int G_LDA = GK + 4, G_LDB = GN + 4;
constexpr int G_SMEM = GSTAGES * (GM * G_LDA + GK * G_LDB) * 4;
int g_big_f32_pipe = 1;        // large f32 products take this kernel (0: the register-staged 128 x 128 one)
int g_big_f32_min_ctas = 140;  // ... when its grid has at least this many CTAs (measured: 144 CTAs 44.1 vs 40.2 TFLOP/s for the small kernel, 128 CTAs 38.7 vs 40.0, 64 CTAs 19.3 vs 27.5)
__global__ void __launch_bounds__(256, 2) sgemm_nn_big_kernel(const SimtParams p) {
    extern __shared__ __align__(16) float g_smem[];
    float (*As)[GM][G_LDA] = reinterpret_cast<float (*)[GM][G_LDA]>(g_smem);
    float (*Bs)[GK][G_LDB] = reinterpret_cast<float (*)[GK][G_LDB]>(g_smem + GSTAGES * GM * G_LDA);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const uint32_t bz = blockIdx.z;
    const long long m0 = (long long)blockIdx.y * GM, n0 = (long long)blockIdx.x * GN;
    const float *A = reinterpret_cast<const float *>(p.A) + (long long)bz * p.a_bs;
    const float *B = reinterpret_cast<const float *>(p.B) + (long long)bz * p.b_bs;

    float2 acc2[8][4];                                  // columns in pairs: what fma.rn.f32x2 reads and writes
#define ACC(i, j) (((j) & 1) ? acc2[i][(j) >> 1].y : acc2[i][(j) >> 1].x)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
        const float b0 = (p.bias && gn < p.N) ? p.bias[gn] : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ACC(i, j) = b0;
    }

    // copy roles per slab: A 128 rows x GK/4 vectors and B GK k-rows x 32 vectors, GK/8 of each per thread
    constexpr int AV = GK / 4;                       // 16-byte vectors per row of A in a slab
    auto issue = [&](int stage, uint32_t k0) {
#pragma unroll
        for (int h = 0; h < GK / 8; ++h) {
            const int idx = tid + 256 * h;
            const int r = idx / AV, kq = (idx % AV) * 4;
            const long long gm = m0 + r, gk = (long long)k0 + kq;
            int bytes = 0;
            if (gm < p.M && gk < p.K) bytes = (int)((p.K - gk) < 4 ? (p.K - gk) : 4) * 4;
            cp_async_16(&As[stage][r][kq], bytes ? A + gm * p.a_rs + gk : A, bytes);
        }
#pragma unroll
        for (int h = 0; h < GK / 8; ++h) {
            const int idx = tid + 256 * h;
            const int k = idx >> 5, nq = (idx & 31) * 4;
            const long long gk = (long long)k0 + k, gn = n0 + nq;
            int bytes = 0;
            if (gk < p.K && gn < p.N) bytes = (int)((p.N - gn) < 4 ? (p.N - gn) : 4) * 4;
            cp_async_16(&Bs[stage][k][nq], bytes ? B + gk * p.b_rs + gn : B, bytes);
        }
    };

    const uint32_t slabs = (p.K + GK - 1) / GK;
#pragma unroll
    for (int s = 0; s < GSTAGES - 1; ++s) {
        if ((uint32_t)s < slabs) issue(s, s * GK);
        cp_async_commit();
    }
    for (uint32_t s = 0; s < slabs; ++s) {
        cp_async_wait<GSTAGES - 2>();
        __syncthreads();
        if (s + GSTAGES - 1 < slabs) issue((s + GSTAGES - 1) % GSTAGES, (s + GSTAGES - 1) * GK);
        cp_async_commit();
        const int st = s % GSTAGES;
#pragma unroll 1
        for (int k2 = 0; k2 < GK; k2 += 2) {      // (not unrolled: unrolling costs registers that two CTAs per SM do not have)
            float2 a[8];
            float4 b[2][2];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float2 *>(&As[st][ty * 4 + (i / 4) * 64 + (i % 4)][k2]);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                b[kk][0] = *reinterpret_cast<const float4 *>(&Bs[st][k2 + kk][tx * 4]);
                b[kk][1] = *reinterpret_cast<const float4 *>(&Bs[st][k2 + kk][64 + tx * 4]);
            }
            // two columns per instruction: fma.rn.f32x2 (sm_100) on {a, a} x {b[j], b[j+1]} + {acc[i][j], acc[i][j+1]};
            // each lane of it is the same fused multiply-add as the scalar instruction
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float av = kk == 0 ? a[i].x : a[i].y;
                    const float2 aa = make_float2(av, av);
                    acc2[i][0] = __ffma2_rn(aa, make_float2(b[kk][0].x, b[kk][0].y), acc2[i][0]);
                    acc2[i][1] = __ffma2_rn(aa, make_float2(b[kk][0].z, b[kk][0].w), acc2[i][1]);
                    acc2[i][2] = __ffma2_rn(aa, make_float2(b[kk][1].x, b[kk][1].y), acc2[i][2]);
                    acc2[i][3] = __ffma2_rn(aa, make_float2(b[kk][1].z, b[kk][1].w), acc2[i][3]);
                }
            }
        }
    }

    float *Cb = p.C + (long long)bz * p.c_bs;
    const bool vec = (p.ldc % 4 == 0) && (((uintptr_t)Cb & 15) == 0) && !p.accumulate;
    if (p.act && !p.act_copy_only) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) ACC(i, j) = simt_act(ACC(i, j), p.act);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
        if (p.c16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const long long gn = n0 + tx * 4 + (j / 4) * 64 + (j % 4);
                const float y = p.act_copy_only ? simt_act(ACC(i, j), p.act) : ACC(i, j);
                if (gn < p.N) p.c16[(long long)bz * p.c16_bs + gm * p.ld16 + gn] = simt_to16(y, p.dtype16);
            }
        }
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const long long gn = n0 + tx * 4 + jh * 64;
            float *dst = Cb + gm * p.ldc + gn;
            if (vec && gn + 3 < p.N) {
                *reinterpret_cast<float4 *>(dst) = make_float4(ACC(i, jh * 4), ACC(i, jh * 4 + 1), ACC(i, jh * 4 + 2), ACC(i, jh * 4 + 3));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gn + j < p.N) dst[j] = p.accumulate ? dst[j] + ACC(i, jh * 4 + j) : ACC(i, jh * 4 + j);
            }
        }
    }
}

#undef ACC

int simt_gemm_launch(const SimtGemm &g) {
    if (g.M == 0 || g.N == 0 || g.batch == 0) return ST_OK;
    SimtParams p;
    p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.batch;
    p.A = g.A; p.a_rs = g.a_rs; p.a_cs = g.a_cs; p.a_bs = g.a_bs;
    p.B = g.B; p.b_rs = g.b_rs; p.b_cs = g.b_cs; p.b_bs = g.b_bs;
    p.C = g.C; p.ldc = g.ldc; p.c_bs = g.c_bs;
    p.dtype_a = g.dtype_a; p.dtype_b = g.dtype_b; p.accumulate = g.accumulate;
    p.bias = g.bias; p.act = g.act; p.c16 = (unsigned short *)g.c16; p.ld16 = g.ld16;
    p.c16_bs = (long long)g.M * g.ld16; p.dtype16 = g.dtype16; p.act_copy_only = g.act_copy_only;
    // grid.z is limited to 65535: launch the batch in slices
    const bool big = (uint64_t)g.M * g.N >= (uint64_t)512 * 512 * 4;
    const int tile = big ? 128 : 64;
    uint32_t done = 0;
    while (done < g.batch) {
        uint32_t nb = g.batch - done < 65535u ? g.batch - done : 65535u;
        SimtParams q = p;
        q.batch = nb;
        const size_t esa = g.dtype_a == DT_F32 ? 4 : 2, esb = g.dtype_b == DT_F32 ? 4 : 2;
        q.A = (const char *)g.A + (long long)done * g.a_bs * (long long)esa;
        q.B = (const char *)g.B + (long long)done * g.b_bs * (long long)esb;
        q.C = g.C + (long long)done * g.c_bs;
        if (q.c16) q.c16 = p.c16 + (long long)done * p.c16_bs;
        dim3 grid((g.N + tile - 1) / tile, (g.M + tile - 1) / tile, nb);
        if (grid.y > 65535u) { set_error("simt gemm: M too large for one launch"); return ST_UNSUPPORTED; }
        const bool nn_f32 = g.dtype_a == DT_F32 && g.dtype_b == DT_F32 && g.a_cs == 1 && g.b_cs == 1 &&
                            g.a_rs % 4 == 0 && g.b_rs % 4 == 0 && g.a_bs % 4 == 0 && g.b_bs % 4 == 0 &&
                            (((uintptr_t)g.A | (uintptr_t)g.B) & 15) == 0;
        // the 128 x 128 kernel needs a grid that fills the SMs; below that the 32 x 64 tiles of the small kernel do better
        const bool big_grid = (uint64_t)grid.x * grid.y * grid.z >= (uint64_t)g_big_f32_min_ctas;
        if (nn_f32 && big && g_big_f32_pipe && big_grid) {
            static bool attr_set[8] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev >= 0 && dev < 8 && !attr_set[dev]) {
                cudaFuncSetAttribute((const void *)sgemm_nn_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM);
                attr_set[dev] = true;
            }
            sgemm_nn_big_kernel<<<grid, 256, G_SMEM, g.stream>>>(q);
        } else if (nn_f32 && big && !g_big_f32_pipe) sgemm_nn_kernel<128><<<grid, 256, 0, g.stream>>>(q);
        else if (nn_f32 && g_small_f32_pipe) {
            dim3 pgrid((g.N + PN - 1) / PN, (g.M + PM - 1) / PM, nb);
            cudaLaunchConfig_t lc = {};
            lc.gridDim = pgrid; lc.blockDim = dim3(128, 1, 1); lc.stream = g.stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            lc.attrs = at; lc.numAttrs = g.pdl ? 1 : 0;
            void *args[1] = {(void *)&q};
            cudaLaunchKernelExC(&lc, (const void *)sgemm_nn_pipe_kernel, args);
        } else if (nn_f32) {
            dim3 grid64((g.N + 63) / 64, (g.M + 63) / 64, nb);
            if (grid64.y > 65535u) { set_error("simt gemm: M too large for one launch"); return ST_UNSUPPORTED; }
            sgemm_nn_kernel<64><<<grid64, 256, 0, g.stream>>>(q);
        }
        else if (big) simt_gemm_kernel<128><<<grid, 256, 0, g.stream>>>(q);
        else simt_gemm_kernel<64><<<grid, 256, 0, g.stream>>>(q);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { set_error("simt gemm launch: %s", cudaGetErrorString(e)); return ST_GEMM; }
        note_launch();
        done += nb;
    }
    return ST_OK;
}

}  // namespace pgb
