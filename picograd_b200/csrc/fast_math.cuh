// Branch-free single-precision erf / GELU / GELU gradient for the kernels' epilogues and element-wise passes:
// few instructions, no slow path (CUDA's erff and expf branch), accuracy far inside the path's tolerances.
#pragma once

namespace pgb {

// 0.5 x (1 + erf(x / sqrt 2)), picograd's act_apply (backend/cpu/gemm.c:632-636), with
// erf(a) = sign(a) (1 - 2^(t Q(t))), t = min(|a|, 4): one piece, no branch, 13 instructions, so the
// epilogue warps take few issue slots from the MMA and producer warps they share schedulers with.
// Q is a weighted least-squares fit of log2(erfc(t)) / t on [0, 4.05]; tests/test_erf_coefficients.py refits it
// and checks these numbers (erf to 8e-8 absolute, GELU to 5e-7 at |x| = 6).
__device__ __forceinline__ float erf_nodiv(float a) {
    const float t = fminf(fabsf(a), 4.0f);
    float r = fmaf(-4.477160110e-05f, t, 4.406937805e-04f);
    r = fmaf(r, t, -1.474020537e-03f);
    r = fmaf(r, t, -7.993229083e-04f);
    r = fmaf(r, t, 2.827465348e-02f);
    r = fmaf(r, t, -1.484908313e-01f);
    r = fmaf(r, t, -9.184145331e-01f);
    r = fmaf(r, t, -1.627908707e+00f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(r * t));     // argument in [-25, 0]: no denormal result
    return copysignf(1.0f - e, a);
}
__device__ __forceinline__ float gelu_erf(float x) {
    const float h = 0.5f * x;
    return fmaf(h, erf_nodiv(x * 0.70710678118f), h);
}
// d/dx gelu(x) = 0.5 (1 + erf(x / sqrt 2)) + x phi(x), phi(x) = exp(-x^2 / 2) / sqrt(2 pi)
// (picograd autograd/autograd.c:794-801, :531-532); the exponential as one ex2.approx.
__device__ __forceinline__ float gelu_grad_fast(float x, float gy) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * x * -0.72134752044f));       // exp(-x^2/2) = 2^(-x^2/2 log2 e)
    const float cdf = fmaf(0.5f, erf_nodiv(x * 0.70710678118f), 0.5f);
    return gy * fmaf(x * 0.3989422804f, e, cdf);
}

}  // namespace pgb
