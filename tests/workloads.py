"""Seeded synthetic inputs of the five benchmark configurations (test + bench harness).

No dataset stands behind these: shapes, distributions and seeds are the whole
specification.  16-bit tensors are returned as uint16 bit patterns (numpy), rounded
from float32 with IEEE round-to-nearest-even; the same bytes go to the CPU checker
and to the GPU.
"""
import numpy as np

F32, F16, BF16 = 0, 1, 2


def to_bf16_bits(x):
    """float32 -> bf16 bit pattern, round-to-nearest-even (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_f16_bits(x):
    return np.ascontiguousarray(x, np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b):
    return b.view(np.float16).astype(np.float32)


def bits_to_f32(dtype, b):
    if dtype == F32:
        return b
    return bf16_bits_to_f32(b) if dtype == BF16 else f16_bits_to_f32(b)


def config1(n=512):
    """f32 sgemm via pg_matmul: A, B [n,n] i.i.d. U[-1,1], seed 0."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    return a, b


def config2(m=8192, n=None, k=None):
    """bf16 pg_gemm_ex: A [m,k], B [k,n] ~ N(0,1) in f32, rounded to bf16; seed 1."""
    n = m if n is None else n
    k = m if k is None else k
    rng = np.random.default_rng(1)
    a = to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    b = to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32))
    return a, b


def config3(m, n, k):
    """f16 pg_gemm_ex: U[-0.5,0.5] rounded to f16; seed 2 (full sizes 4096x14336x4096, 16x4096x4096)."""
    rng = np.random.default_rng(2)
    a = to_f16_bits(rng.uniform(-0.5, 0.5, (m, k)).astype(np.float32))
    b = to_f16_bits(rng.uniform(-0.5, 0.5, (k, n)).astype(np.float32))
    return a, b


def config4(batch=64, seq=2048, d=128):
    """attention-shaped bf16 bmm: Q, V [b,s,d], K^T [b,d,s] ~ N(0, 1/sqrt(d)); seed 3."""
    rng = np.random.default_rng(3)
    # N(0, 1/sqrt(d)) read as variance 1/sqrt(d): standard deviation d^(-1/4), which gives the
    # scores Q K^T unit variance
    sd = float(d) ** -0.25
    q = to_bf16_bits(rng.standard_normal((batch, seq, d), dtype=np.float32) * np.float32(sd))
    kt = to_bf16_bits(rng.standard_normal((batch, d, seq), dtype=np.float32) * np.float32(sd))
    v = to_bf16_bits(rng.standard_normal((batch, seq, d), dtype=np.float32) * np.float32(sd))
    return q, kt, v


def config5(rows=8192, d_in=4096, d_hidden=16384):
    """MLP step: x [rows,d_in] ~ N(0,1) bf16; W1 [d_in,d_hidden] ~ U[+-1/sqrt(d_in)],
    W2 [d_hidden,d_in] ~ U[+-1/sqrt(d_hidden)], bf16; seed 4."""
    rng = np.random.default_rng(4)
    x = to_bf16_bits(rng.standard_normal((rows, d_in), dtype=np.float32))
    b1 = 1.0 / np.sqrt(d_in)
    b2 = 1.0 / np.sqrt(d_hidden)
    w1 = to_bf16_bits(rng.uniform(-b1, b1, (d_in, d_hidden)).astype(np.float32))
    w2 = to_bf16_bits(rng.uniform(-b2, b2, (d_hidden, d_in)).astype(np.float32))
    return x, w1, w2


def dyadic(n):
    """picograd's own exact-in-f32 test data ((i*37+11)%19 - 9)/8 (benchmarks/bench_gemm_cuda.c:16-20)."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 37 + 11) % 19).astype(np.float32) - 9.0) / 8.0


def seeded_uniform(rows, cols, seed, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, (rows, cols)).astype(np.float32)


def tolerance(dtype, k):
    """Normwise relative error bound: 1e-6 for f32, 1e-5*sqrt(K) for f16/bf16."""
    return 1e-6 if dtype == F32 else 1e-5 * float(np.sqrt(max(k, 1)))


def relerr(c, ref):
    c = np.asarray(c, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(c - ref) / den) if den > 0 else float(np.linalg.norm(c))
