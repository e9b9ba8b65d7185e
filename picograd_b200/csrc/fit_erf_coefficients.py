"""Derives the coefficients of erf_nodiv() in gemm_tc.cu and checks them.

    erf(a) = sign(a) * (1 - 2^(t * Q(t))),   t = min(|a|, 4)

Q has degree 7 and is a least-squares fit of log2(erfc(t)) / t on Chebyshev nodes of [0, 4.05], weighted by
t * erfc(t) (the sensitivity of the result to an error in Q); beyond 4, erf rounds to 1 in single precision.
One piece and no branch: 1 - 2^(...) loses RELATIVE accuracy near zero, but the absolute error stays below
1e-7, and GELU multiplies erf by x/2, so its absolute error is below 5e-7 at |x| = 6 and shrinks with |x|.

Prints the coefficients (highest degree first) and the maximum absolute errors of the single-precision
evaluation against scipy's erf over [-6, 6].  Needs numpy and scipy; nothing at run time depends on it.
"""
import numpy as np
from scipy.special import erf, erfc

DEGREE = 7


def horner32(coeffs, x):
    r = np.full_like(x, np.float32(coeffs[0]))
    for c in coeffs[1:]:
        r = (r.astype(np.float64) * x + np.float32(c)).astype(np.float32)     # one fused multiply-add
    return r


def erf_nodiv(a, q):
    a = a.astype(np.float32)
    t = np.minimum(np.abs(a), np.float32(4.0))
    r = (horner32(q, t).astype(np.float64) * t).astype(np.float32)
    return np.copysign((1.0 - np.exp2(r.astype(np.float64))).astype(np.float32), a)


def main():
    nodes = np.cos(np.pi * (np.arange(6000) + 0.5) / 6000)
    t = (nodes + 1) / 2 * 4.05
    q = np.polyfit(t, np.log2(erfc(t)) / t, DEGREE, w=erfc(t) * t)
    x = np.linspace(-6, 6, 2000001).astype(np.float32)
    print("Q:", ", ".join("%.9ef" % np.float32(c) for c in q))
    print("erf  max abs error: %.3e" % np.abs(erf_nodiv(x, q) - erf(x.astype(np.float64))).max())
    g = 0.5 * x.astype(np.float64) * (1 + erf(x.astype(np.float64) / np.sqrt(2)))
    xs = (x * np.float32(0.70710678118)).astype(np.float32)
    mine = (np.float32(0.5) * x * (np.float32(1.0) + erf_nodiv(xs, q))).astype(np.float32)
    print("GELU max abs error: %.3e" % np.abs(mine - g).max())


if __name__ == "__main__":
    main()
