"""The branch-free erf of the tensor-core epilogue (erf_nodiv in picograd_b200/csrc/fast_math.cuh) checked on the CPU.

    erf(a) = sign(a) * (1 - 2^(t * Q(t))),   t = min(|a|, 4)

Q (degree 7) is a least-squares fit of log2(erfc(t)) / t on Chebyshev nodes of [0, 4.05], weighted by t * erfc(t);
beyond 4, erf rounds to 1 in single precision.  The test reads the coefficients out of the CUDA source, evaluates
the same single-precision Horner form with numpy, and holds it to the accuracy the fused GELU epilogue relies on
(picograd's act_apply, backend/cpu/gemm.c:632-636, uses erff): erf to 1e-7 absolute, GELU to 5e-7 over [-6, 6].
It also refits Q and checks that the source holds the fitted values.
"""
import os
import re

import numpy as np
from scipy.special import erf, erfc

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "picograd_b200", "csrc", "fast_math.cuh")


def coefficients_in_source():
    text = open(SRC).read()
    body = text[text.index("float erf_nodiv(float a)"):]
    body = body[:body.index("ex2.approx")]
    nums = re.findall(r"(-?\d\.\d+e[+-]\d+)f", body)
    assert len(nums) == 8, nums
    return [float(x) for x in nums]          # highest degree first


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


def test_erf_and_gelu_accuracy_of_the_coefficients_in_the_source():
    q = coefficients_in_source()
    x = np.linspace(-6, 6, 400001).astype(np.float32)
    assert np.abs(erf_nodiv(x, q) - erf(x.astype(np.float64))).max() < 1e-7
    g = 0.5 * x.astype(np.float64) * (1 + erf(x.astype(np.float64) / np.sqrt(2)))
    xs = (x * np.float32(0.70710678118)).astype(np.float32)
    mine = (np.float32(0.5) * x * (np.float32(1.0) + erf_nodiv(xs, q))).astype(np.float32)
    assert np.abs(mine - g).max() < 5e-7


def test_source_holds_the_fitted_polynomial():
    nodes = np.cos(np.pi * (np.arange(6000) + 0.5) / 6000)
    t = (nodes + 1) / 2 * 4.05
    fit = np.polyfit(t, np.log2(erfc(t)) / t, 7, w=erfc(t) * t)
    q = np.array(coefficients_in_source())
    # the polynomials agree as functions on the fitted interval (coefficients of a degree-7 fit are ill-conditioned
    # one by one)
    tt = np.linspace(0, 4, 2001)
    assert np.abs(np.polyval(fit, tt) - np.polyval(q, tt)).max() < 1e-6
