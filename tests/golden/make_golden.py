"""Generates tests/golden/reference_outputs.npz from the UNMODIFIED picograd CPU library.

Run in a container that holds picograd's sources: `make -C oracle ref` compiles them into
oracle/_ref/libpicograd_ref.so, then `python tests/golden/make_golden.py` calls its
pg_gemm / pg_gemm_ex on small seeded inputs and stores inputs' seeds + outputs.  The committed
.npz is what travels; the tests re-create the inputs from the seeds and compare our oracle
(and, on a GPU, the CUDA path) with these reference outputs.

The host CPU matters for one case: on AVX512-FP16 hosts picograd's f16 micro-kernel
(backend/cpu/hgemm_avx512fp16.c:31-41) resets the accumulators of columns 0..15 of every
32-column block at each 256-deep K block, so for K > 256 only columns 16..31 (mod 32) of its
f16 output are an f32 accumulation over all of K.  In pg_cpu_gemm_fused_ex the same reset throws
away the bias row those columns were initialised with, whatever K is.  `<case>_valid_cols`
records which columns of each f16 case are usable as golden values on the host that generated
the file.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib  # noqa: E402
import workloads as wl  # noqa: E402

CASES = [
    # (name, dtype, m, n, k, seed)
    ("f32_13x9x7", wl.F32, 13, 9, 7, 10),
    ("f32_16x16x300", wl.F32, 16, 16, 300, 11),       # crosses the 256-deep K block (tests/test_ops.c:78-102)
    ("f32_37x53x129", wl.F32, 37, 53, 129, 12),
    ("f32_96x80x520", wl.F32, 96, 80, 520, 13),
    ("bf16_13x9x7", wl.BF16, 13, 9, 7, 20),
    ("bf16_40x72x256", wl.BF16, 40, 72, 256, 21),
    ("bf16_64x96x600", wl.BF16, 64, 96, 600, 22),
    ("f16_13x9x7", wl.F16, 13, 9, 7, 30),
    ("f16_40x72x256", wl.F16, 40, 72, 256, 31),
    ("f16_64x96x600", wl.F16, 64, 96, 600, 32),
]


# pg_cpu_gemm_fused_ex (backend/cpu/gemm.c:718-817): (name, dtype, m, n, k, seed, with_bias, act).
# f16 cases keep K <= 256 so that the accumulator reset described above cannot touch them.
FUSED_CASES = [
    ("fused_f32_13x9x7_bias_none", wl.F32, 13, 9, 7, 40, True, 0),
    ("fused_f32_37x53x300_bias_relu", wl.F32, 37, 53, 300, 41, True, 1),
    ("fused_f32_37x53x300_bias_gelu", wl.F32, 37, 53, 300, 42, True, 2),
    ("fused_f32_24x40x64_nobias_relu", wl.F32, 24, 40, 64, 43, False, 1),
    ("fused_bf16_40x72x520_bias_relu", wl.BF16, 40, 72, 520, 44, True, 1),
    ("fused_bf16_40x72x520_bias_gelu", wl.BF16, 40, 72, 520, 45, True, 2),
    ("fused_f16_40x72x256_bias_relu", wl.F16, 40, 72, 256, 46, True, 1),
    ("fused_f16_13x48x7_bias_none", wl.F16, 13, 48, 7, 47, True, 0),
]


# pg_conv2d (ops/conv.c:10-146): (name, N, Cin, H, W, Cout, kh, kw, stride, padding, with_bias, seed)
CONV_CASES = [
    ("conv_2x3x7x7_k3_s1_p1_bias", 2, 3, 7, 7, 2, 3, 3, 1, 1, True, 60),       # the shape of tests/test_nn_layers.c:87-92
    ("conv_1x4x19x23_k5x3_s2_p2_bias", 1, 4, 19, 23, 6, 5, 3, 2, 2, True, 61),
    ("conv_3x2x40x40_k3_s1_p0_nobias", 3, 2, 40, 40, 5, 3, 3, 1, 0, False, 62),  # 1444 output pixels: two column chunks
    ("conv_2x8x9x9_k1_s1_p0_bias", 2, 8, 9, 9, 4, 1, 1, 1, 0, True, 63),
]


def make_conv_inputs(case):
    _, n, cin, h, w, cout, kh, kw, _, _, with_bias, seed = case
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (n, cin, h, w)).astype(np.float32)
    wt = rng.uniform(-1, 1, (cout, cin, kh, kw)).astype(np.float32)
    b = rng.uniform(-1, 1, cout).astype(np.float32) if with_bias else None
    return x, wt, b


# pg_addmm (ops/matmul.c:371-405), f32: (name, m, n, k, input shape, alpha, beta, seed)
ADDMM_CASES = [
    ("addmm_3x5x4_full_2_0.5", 3, 5, 4, (3, 5), 2.0, 0.5, 80),                 # tests/test_ops.c:442-448
    ("addmm_37x53x129_rowvec_1_1", 37, 53, 129, (53,), 1.0, 1.0, 81),
    ("addmm_24x40x300_colvec_-0.75_3", 24, 40, 300, (24, 1), -0.75, 3.0, 82),
    ("addmm_16x16x64_beta0", 16, 16, 64, (16, 16), 1.5, 0.0, 83),
]


def make_addmm_inputs(case):
    _, m, n, k, ishape, _, _, seed = case
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    inp = rng.uniform(-1, 1, ishape).astype(np.float32)
    return inp, a, b


# bwd_matmul through pg_backward (autograd/autograd.c:561-706, :2483-2533).
# The six shape modes of picograd's tests/test_autograd.c:288-332 (2-D x 2-D, vector x 2-D, 2-D x vector,
# vector x vector, batched x batched, batched x shared 2-D), loss = sum(matmul): (name, a shape, b shape, seed)
BWD_MODE_CASES = [
    ("bwd_mode_2d2d", (3, 4), (4, 2), 90),
    ("bwd_mode_v2d", (4,), (4, 2), 91),
    ("bwd_mode_2dv", (3, 4), (4,), 92),
    ("bwd_mode_vv", (4,), (4,), 93),
    ("bwd_mode_bmm", (2, 3, 4), (2, 4, 5), 94),
    ("bwd_mode_bcast_batch", (2, 3, 4), (4, 5), 95),
]
# Products large enough for the GEMM route of bwd_matmul (m*n*k > 4096, autograd.c:635), with a seeded
# upstream gradient (loss = sum(y * upstream)): (name, dtype, a shape, b shape, seed)
BWD_CASES = [
    ("bwd_f32_40x72x56", wl.F32, (40, 56), (56, 72), 100),
    ("bwd_f32_72x136x100", wl.F32, (72, 100), (100, 136), 101),
    ("bwd_bf16_40x72x56", wl.BF16, (40, 56), (56, 72), 102),
    ("bwd_bf16_136x264x200", wl.BF16, (136, 200), (200, 264), 103),
    ("bwd_bf16_128x64x264", wl.BF16, (128, 264), (264, 64), 104),
    ("bwd_f16_200x264x136", wl.F16, (200, 136), (136, 264), 105),
    ("bwd_bf16_batched_3x72x136x64", wl.BF16, (3, 72, 64), (3, 64, 136), 106),
    ("bwd_bf16_shared_b_3x72x136x64", wl.BF16, (3, 72, 64), (64, 136), 107),
    ("bwd_f32_shared_b_2x48x40x96", wl.F32, (2, 48, 96), (96, 40), 108),
]


def make_bwd_inputs(dtype, ashape, bshape, seed, with_upstream=True):
    """Seeded operands (f32 values or 16-bit patterns) and the upstream gradient of the matmul's output."""
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, ashape).astype(np.float32)
    b = rng.uniform(-1, 1, bshape).astype(np.float32)
    if dtype == wl.BF16:
        a, b = wl.to_bf16_bits(a), wl.to_bf16_bits(b)
    elif dtype == wl.F16:
        a, b = wl.to_f16_bits(a), wl.to_f16_bits(b)
    yshape = tuple(ashape[:-1]) + tuple(bshape[-1:]) if len(bshape) > 1 else tuple(ashape[:-1])
    if len(ashape) == 1:
        yshape = tuple(bshape[1:]) if len(bshape) > 1 else (1,)
    g = rng.standard_normal(yshape).astype(np.float32) if with_upstream else None
    return a, b, g


def make_bias(n, seed):
    return np.random.default_rng(seed + 1000).uniform(-1, 1, n).astype(np.float32)


def make_inputs(dtype, m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    if dtype == wl.BF16:
        return wl.to_bf16_bits(a), wl.to_bf16_bits(b)
    if dtype == wl.F16:
        return wl.to_f16_bits(a), wl.to_f16_bits(b)
    return a, b


def main():
    ref = oracle_lib.reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libpicograd_ref.so not built: run `make -C oracle ref` first")
    out = {}
    for name, dt, m, n, k, seed in CASES:
        a, b = make_inputs(dt, m, n, k, seed)
        c = ref.gemm_ex(dt, a, b)
        out[name] = c
        if dt == wl.F16:
            # detect the accumulator-reset columns by comparing with an f64 product
            exact = wl.f16_bits_to_f32(a).astype(np.float64) @ wl.f16_bits_to_f32(b).astype(np.float64)
            good = np.abs(c - exact).max(axis=0) < 1e-3
            out[name + "_valid_cols"] = good
    for name, dt, m, n, k, seed, with_bias, act in FUSED_CASES:
        a, b = make_inputs(dt, m, n, k, seed)
        bias = make_bias(n, seed) if with_bias else None
        out[name] = ref.gemm_fused_ex(dt, a, b, bias, act)
        if dt == wl.F16:
            # the same accumulator reset also drops the bias row the kernel should have started from
            exact = wl.f16_bits_to_f32(a).astype(np.float64) @ wl.f16_bits_to_f32(b).astype(np.float64)
            exact = exact + (bias if with_bias else 0.0)
            if act == 1:
                exact = np.maximum(exact, 0)
            out[name + "_valid_cols"] = np.abs(out[name] - exact).max(axis=0) < 1e-3
    # the f32 entry nn/nn.c:60,85 calls (Linear forward with and without ReLU)
    a, b = make_inputs(wl.F32, 20, 33, 300, 48)
    out["fused_f32_plain_entry_relu"] = ref.gemm_fused_ex(wl.F32, a, b, make_bias(33, 48), 1, plain_f32_entry=True)
    for case in ADDMM_CASES:
        inp, a, b = make_addmm_inputs(case)
        out[case[0]] = ref.addmm(inp, a, b, case[5], case[6])
    for case in CONV_CASES:
        x, wt, b = make_conv_inputs(case)
        out[case[0]] = ref.conv2d(x, wt, b, case[8], case[9])
    # the matmul node of the autograd, driven through picograd's public pg_ag_matmul / pg_backward
    for name, ash, bsh, seed in BWD_MODE_CASES:
        a, b, _ = make_bwd_inputs(wl.F32, ash, bsh, seed, with_upstream=False)
        y, ga, gb = ref.matmul_backward(wl.F32, a, b, None)
        out[name + "_y"], out[name + "_ga"], out[name + "_gb"] = y, ga, gb
    for name, dt, ash, bsh, seed in BWD_CASES:
        a, b, g = make_bwd_inputs(dt, ash, bsh, seed)
        y, ga, gb = ref.matmul_backward(dt, a, b, g)
        y2, ga2, gb2 = ref.matmul_backward(dt, a, b, g, jit=False)      # the eager route gives the same bits
        assert np.array_equal(ga, ga2) and np.array_equal(gb, gb2) and np.array_equal(y, y2), name
        out[name + "_ga"], out[name + "_gb"] = ga, gb
    # leaves drawn the way picograd's own tests draw them (tests/test_autograd.c:319-330: pg_seed(11), then
    # pg_var_uniform per leaf), kept in the file because only picograd's generator can reproduce them
    ba, bb, ba2, bw = ref.uniform(11, [(2, 3, 4), (2, 4, 5), (2, 3, 4), (4, 5)])
    for name, a, b in (("bwd_pgseed11_bmm", ba, bb), ("bwd_pgseed11_bcast_batch", ba2, bw)):
        y, ga, gb = ref.matmul_backward(wl.F32, a, b, None)
        out[name + "_a"], out[name + "_b"] = a, b
        out[name + "_y"], out[name + "_ga"], out[name + "_gb"] = y, ga, gb
    # the two-layer network of tests/test_autograd.c:393-421 (pg_seed(55)); zero biases as there
    x, = ref.uniform(55, [(2, 3)])
    w1, w2 = ref.uniform(56, [(3, 8), (8, 2)], -0.5, 0.5)
    mlp = ref.mlp_backward(x, w1, np.zeros(8, np.float32), w2, np.zeros(2, np.float32))
    out["bwd_mlp_x"], out["bwd_mlp_w1"], out["bwd_mlp_w2"] = x, w1, w2
    for key, v in mlp.items():
        out["bwd_mlp_" + key] = v
    # picograd's own dyadic correctness data (benchmarks/bench_gemm_cuda.c:16-65), exact in f32
    s = 64
    d = wl.dyadic(s * s).reshape(s, s)
    out["f32_dyadic64"] = ref.gemm_ex(wl.F32, d, d)
    np.savez_compressed(os.path.join(HERE, "reference_outputs.npz"), **out)
    print("wrote", len(out), "arrays; threads", ref.threads())
    for kname in out:
        if kname.endswith("_valid_cols"):
            print(kname, int(out[kname].sum()), "of", out[kname].size)


if __name__ == "__main__":
    main()
