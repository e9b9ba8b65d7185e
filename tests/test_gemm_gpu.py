"""Parity of the CUDA path with the CPU oracle, through the C-ABI, on the same seeded bytes.

Tolerances are the ones the path is specified with: normwise relative error <= 1e-6 for f32
and <= 1e-5 * sqrt(K) for f16/bf16 inputs.  The FFMA kernel is additionally bit-exact.
"""
import os

import numpy as np
import pytest
import torch

import workloads as wl
from golden.make_golden import ADDMM_CASES, CASES, make_addmm_inputs, make_inputs
from gpu_util import bits_to_host, gemm_dev, to_dev, to_host

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz")


def test_library_is_the_cuda_one(pg):
    from picograd_b200 import _lib
    assert os.path.basename(_lib.LIB_PATH) == "libpg_b200.so"
    n0 = pg.launch_count()
    a = torch.ones(64, 64, device="cuda").bfloat16()
    pg.pg_matmul(a, a); pg.pg_dev_sync()
    assert pg.launch_count() > n0, "no kernel of ours was launched"


def test_exact_case_from_test_backend(pg):
    # tests/test_backend.c:91-95
    v = torch.tensor([[1., 2.], [3., 4.]], device="cuda")
    w = torch.tensor([[5.], [6.]], device="cuda")
    r = pg.pg_matmul(v, w); pg.pg_dev_sync()
    assert r.flatten().tolist() == [17.0, 39.0]


def test_config1_f32_512_bit_exact(pg, oracle):
    a, b = wl.config1(512)
    want = oracle.gemm_ex(wl.F32, a, b)
    got = to_host(pg.pg_matmul(to_dev(a, wl.F32), to_dev(b, wl.F32)))
    pg.pg_dev_sync()
    assert pg.last_path() == "simt"
    assert wl.relerr(got, want) <= 1e-6
    assert np.array_equal(got, want), "FFMA path: same fused chain over k as the CPU kernels"


def test_f32_dyadic_exact_like_bench_gemm_cuda(pg):
    # benchmarks/bench_gemm_cuda.c:16-65: max abs err 0 on dyadic data
    s = 512
    d = wl.dyadic(s * s).reshape(s, s)
    got = gemm_dev(pg, wl.F32, d, d)
    assert np.array_equal(got.astype(np.float64), d.astype(np.float64) @ d.astype(np.float64))


@pytest.mark.parametrize("pipe", [1, 0], ids=["cp.async-packed-fma", "register-staged"])
@pytest.mark.parametrize("lds", [(336, 1200, 1200), (333, 1203, 1201)], ids=["aligned", "odd-ld"])
def test_f32_large_bit_exact(pg, oracle, lds, pipe):
    """Large f32 products (the 128x128 FFMA kernels: cp.async slabs and two columns per fma.rn.f32x2 when rows are
    16-byte aligned, the generic kernel otherwise) keep the one-chain-per-element arithmetic: equal to the CPU result
    bit for bit, ragged edges in M, N and K included."""
    m, n, k = 1100, 1200, 333
    rng = np.random.default_rng(20)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    pg.set_option("big_f32_pipe", pipe)
    got = gemm_dev(pg, wl.F32, a, b, lda=lds[0], ldb=lds[1], ldc=lds[2])
    assert pg.last_path() == "simt"
    assert np.array_equal(got, oracle.gemm_ex(wl.F32, a, b))


@pytest.mark.parametrize("pipe", [1, 0], ids=["cp.async-32x64", "register-staged-64x64"])
@pytest.mark.parametrize("shape", [(512, 512, 512, 0), (97, 203, 301, 0), (33, 65, 17, 4), (1, 4, 1, 0), (250, 120, 1000, 8)])
def test_f32_small_kernels_bit_exact(pg, oracle, shape, pipe):
    """Both kernels that serve small f32 products (pg_matmul's 512^3 among them) keep one fused-multiply-add chain
    per element over k ascending: the CPU result bit for bit, with ragged edges in M, N and K (K not a multiple of
    the 16-deep slab, N not a multiple of 4) and padded leading dimensions."""
    m, n, k, pad = shape
    rng = np.random.default_rng(21)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    pg.set_option("small_f32_pipe", pipe)
    r4 = lambda v: (v + 3) // 4 * 4
    got = gemm_dev(pg, wl.F32, a, b, lda=r4(k) + pad, ldb=r4(n) + pad, ldc=r4(n) + pad)
    assert pg.last_path() == "simt"
    assert np.array_equal(got, oracle.gemm_ex(wl.F32, a, b))


def test_f32_on_tensor_cores_within_1e6(pg, oracle):
    """f32 x f32 as three exact bf16 pieces per operand, six tensor-core passes."""
    a, b = wl.config1(512)
    want = oracle.gemm_ex(wl.F32, a, b)
    pg.set_option("f32_tensor_cores", 1)
    got = to_host(pg.pg_matmul(to_dev(a, wl.F32), to_dev(b, wl.F32)))
    pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:")
    assert wl.relerr(got, want) <= 1e-6


def test_f32_on_tensor_cores_long_k_goes_in_chunks(pg, oracle):
    """The tensor cores add into their f32 accumulator without rounding to nearest, so one long accumulation drifts
    in proportion to K.  The f32 route therefore accumulates K in chunks of 512 and adds each chunk to C in f32: its
    distance to the exact product stays below 5e-7 at every K — closer than the one-chain f32 result itself, which
    is why beyond K of a few thousand it cannot also stay within 1e-6 of that chain."""
    m, n, k = 256, 384, 8192
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    chain = oracle.gemm_ex(wl.F32, a, b)
    pg.set_option("f32_tensor_cores", 1)
    got = gemm_dev(pg, wl.F32, a, b)
    assert pg.last_path().startswith("tc:")
    e_tc, e_chain = wl.relerr(got, exact), wl.relerr(chain, exact)
    assert e_tc <= 5e-7 and e_tc < e_chain, (e_tc, e_chain)
    assert wl.relerr(got, chain) <= 2.5e-6
    pg.set_option("f32_chunk", 0)                    # one accumulation over all of K
    assert wl.relerr(gemm_dev(pg, wl.F32, a, b), exact) > 4 * e_tc
    pg.set_option("f32_chunk", 512)
    # bias + activation after the last chunk, ragged K (last chunk shorter)
    k2 = 1000
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    ad, bd, biasd = to_dev(a[:, :k2].copy(), wl.F32), to_dev(b[:k2].copy(), wl.F32), to_dev(bias, wl.F32)
    c = torch.empty((m, n), device="cuda")
    pg.pg_gemm_fused(m, n, k2, ad, k2, bd, n, c, n, bias=biasd, act=pg.PG_ACT_RELU)
    pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:")
    want = oracle.gemm_fused_ex(wl.F32, a[:, :k2].copy(), b[:k2].copy(), bias, pg.PG_ACT_RELU)
    assert wl.relerr(to_host(c), want) <= 1e-6


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_against_reference_outputs(pg, case):
    """The committed outputs of the unmodified picograd CPU library."""
    name, dt, m, n, k, seed = case
    gold = np.load(GOLDEN)
    a, b = make_inputs(dt, m, n, k, seed)
    got = gemm_dev(pg, dt, a, b)
    ref = gold[name]
    cols = gold[name + "_valid_cols"] if dt == wl.F16 else np.ones(n, bool)
    assert wl.relerr(got[:, cols], ref[:, cols]) <= wl.tolerance(dt, k)
    if pg.last_path() == "simt" and dt != wl.BF16:
        assert np.array_equal(got[:, cols], ref[:, cols])


@pytest.mark.parametrize("dt", [wl.BF16, wl.F16])
@pytest.mark.parametrize("shape", [(1024, 768, 512), (384, 1000, 1096), (130, 70, 4096)])
@pytest.mark.parametrize("path", [1, 2], ids=["tensor", "ffma"])
def test_gemm_ex_vs_oracle(pg, oracle, dt, shape, path):
    m, n, k = shape
    a, b = (wl.config2(m, n, k) if dt == wl.BF16 else wl.config3(m, n, k))
    pad = lambda v: (v + 7) // 8 * 8
    pg.set_option("path", path)
    got = gemm_dev(pg, dt, a, b, lda=pad(k), ldb=pad(n), ldc=pad(n) + 4)
    want = oracle.gemm_ex(dt, a, b)
    assert pg.last_path().startswith("tc:" if path == 1 else "simt")
    assert wl.relerr(got, want) <= wl.tolerance(dt, k)
    if path == 2:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("cfg", range(5))
@pytest.mark.parametrize("epi", [0, 1])
def test_every_tile_config(pg, oracle, cfg, epi):
    a, b = wl.config2(520, 776, 328)
    pg.set_option("path", 1); pg.set_option("tile_config", cfg); pg.set_option("epilogue", epi)
    got = gemm_dev(pg, wl.BF16, a, b)
    assert pg.last_path().startswith("tc:")
    assert wl.relerr(got, oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, 328)


def test_config3b_skinny_split_k(pg, oracle):
    """M = 16 decode-like shape at full size: one M tile, K split across CTAs, slices reduced."""
    a, b = wl.config3(16, 4096, 4096)
    got = gemm_dev(pg, wl.F16, a, b)
    assert "splitk" in pg.last_path()
    assert wl.relerr(got, oracle.gemm_ex(wl.F16, a, b)) <= wl.tolerance(wl.F16, 4096)


@pytest.mark.parametrize("m", [1, 5, 16, 17, 32])
@pytest.mark.parametrize("dt", [wl.BF16, wl.F16])
def test_skinny_m_swapped_operands(pg, oracle, m, dt):
    """M <= 32 goes through C^T = B^T A^T with narrow tiles; with and without K splits, ragged N."""
    for n, k in ((4096, 1024), (1000, 520), (256, 64)):
        a, b = (wl.config2(m, n, k) if dt == wl.BF16 else wl.config3(m, n, k))
        want = oracle.gemm_ex(dt, a, b)
        got = gemm_dev(pg, dt, a, b)
        if m * n * k > 64 ** 3:                     # tinier products go to the FFMA kernel
            assert "_t" in pg.last_path(), pg.last_path()
        assert wl.relerr(got, want) <= wl.tolerance(dt, k), (m, n, k, pg.last_path())
        pg.set_option("swap_skinny", 0)
        plain = gemm_dev(pg, dt, a, b)
        pg.set_option("swap_skinny", 1)
        assert wl.relerr(got, plain) <= 1e-6


def test_fused_split_k_equals_two_kernel_form(pg, oracle):
    """The slices are summed in slice order either way, so the two forms agree bit for bit."""
    a, b = wl.config2(200, 520, 2056)
    outs = {}
    for fused in (1, 0):
        pg.set_option("fused_splitk", fused); pg.set_option("k_splits", 5); pg.set_option("path", 1)
        outs[fused] = gemm_dev(pg, wl.BF16, a, b, lda=2056, ldb=520, ldc=524)
        assert ("fused" in pg.last_path()) == bool(fused), pg.last_path()
    assert np.array_equal(outs[0], outs[1])
    assert wl.relerr(outs[1], oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, 2056)
    # twice more: the arrival counters re-arm themselves
    for _ in range(2):
        pg.set_option("fused_splitk", 1); pg.set_option("k_splits", 5); pg.set_option("path", 1)
        assert np.array_equal(gemm_dev(pg, wl.BF16, a, b, lda=2056, ldb=520, ldc=524), outs[1])


@pytest.mark.parametrize("shape", [(8192, 1024, 2048), (2048, 3000, 1096), (1304, 1800, 8192)])
def test_stream_k_schedule(pg, oracle, shape):
    """A partly filled last wave is dealt out over all SMs by K ranges, two slices per tile at most: the first slice
    is stored, the second added once the first has landed.  Must agree with the plain schedule and with the
    oracle, and give the same bits every time (two terms per element, one order)."""
    m, n, k = shape
    a, b = wl.config2(m, n, k)
    ad, bd = to_dev(a, wl.BF16), to_dev(b, wl.BF16)
    outs = {}
    for sk in (1, 0):
        pg.set_option("stream_k", sk); pg.set_option("path", 1); pg.set_option("tile_config", 3)
        c = torch.full((m, n), 5.0, device="cuda")
        for _ in range(2):                      # second call: re-armed hand-over flags
            pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n)
        pg.pg_dev_sync()
        assert ("balanced_tail" in pg.last_path()) == bool(sk), pg.last_path()
        if sk:
            for _ in range(3):
                c2 = torch.full((m, n), -1.0, device="cuda")
                pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c2, n)
                pg.pg_dev_sync()
                assert torch.equal(c, c2)
        outs[sk] = c
    assert wl.relerr(to_host(outs[1]), to_host(outs[0])) <= wl.tolerance(wl.BF16, k) / 10   # other K cuts, other rounding
    for r0, r1, c0, c1 in ((0, 40, 0, 64), (m - 24, m, n - 40, n), (m // 2, m // 2 + 16, n // 3, n // 3 + 48)):
        want = oracle.gemm_ex_panel(wl.BF16, a, b, r0, r1, c0, c1)
        assert wl.relerr(to_host(outs[1][r0:r1, c0:c1]), want) <= wl.tolerance(wl.BF16, k)
    from gpu_util import freivalds
    assert freivalds(outs[1], ad.double(), bd.double()) <= wl.tolerance(wl.BF16, k) / 10


SIZES = [1, 2, 3, 7, 8, 9, 16, 17, 127, 128, 129, 255, 256, 257]


@pytest.mark.parametrize("path", [1, 2], ids=["tensor", "ffma"])
def test_edge_shape_sweep(pg, oracle, path):
    """Tile-edge sizes in each of M, N, K (the others held at an awkward size)."""
    pg.set_option("path", path)
    rng = np.random.default_rng(11)
    pad = lambda v: (v + 7) // 8 * 8
    for axis in range(3):
        for s in SIZES:
            shp = [72, 40, 136]
            shp[axis] = s
            m, n, k = shp
            a = wl.to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
            b = wl.to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32))
            if path == 1:
                got = gemm_dev(pg, wl.BF16, a, b, lda=pad(k), ldb=pad(n), ldc=pad(n))
                assert pg.last_path().startswith("tc:"), (shp, pg.last_path())
            else:
                got = gemm_dev(pg, wl.BF16, a, b, lda=k + 1, ldb=n + 3, ldc=n + 1)
            want = oracle.gemm_ex(wl.BF16, a, b)
            assert wl.relerr(got, want) <= wl.tolerance(wl.BF16, k), shp


def test_random_shapes_whatever_path_the_library_picks(pg, oracle):
    """Sixty seeded random problems: dtype, sizes, leading dimensions (aligned or not), bias / activation on or
    off.  Whatever route the library takes (tensor cores, split-K, cluster, swapped, re-pitched, FFMA), the
    result is within the path's tolerance and nothing is written outside the n columns of C."""
    rng = np.random.default_rng(2024)
    routes = set()
    for it in range(60):
        dt = [wl.F32, wl.F16, wl.BF16][rng.integers(3)]
        m = int(rng.choice([1, 3, 16, 31, 64, 130, 257, 600, 1500]))
        n = int(rng.choice([1, 5, 32, 100, 128, 264, 513, 1100]))
        k = int(rng.choice([1, 7, 64, 65, 200, 512, 1111, 2304]))
        aligned = bool(rng.integers(2))
        lda = (k + 7) // 8 * 8 if aligned else k + int(rng.integers(0, 4))
        ldb = (n + 7) // 8 * 8 if aligned else n + int(rng.integers(0, 4))
        ldc = n + int(rng.integers(0, 5))
        a32 = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        b32 = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        conv = {wl.F32: lambda x: x, wl.F16: wl.to_f16_bits, wl.BF16: wl.to_bf16_bits}[dt]
        a, b = conv(a32), conv(b32)
        act = int(rng.integers(3))
        bias = rng.uniform(-1, 1, n).astype(np.float32) if rng.integers(2) else None
        abuf = np.zeros((m, lda), a.dtype); abuf[:, :k] = a
        bbuf = np.zeros((k, ldb), b.dtype); bbuf[:, :n] = b
        ad, bd = to_dev(abuf, dt), to_dev(bbuf, dt)
        c = torch.full((m, ldc), float(0xAB), dtype=torch.float32, device="cuda")
        bt = torch.from_numpy(bias).cuda() if bias is not None else None
        pg.pg_gemm_fused_ex(dt, m, n, k, ad, lda, bd, ldb, c, ldc, bt, act)
        pg.pg_dev_sync()
        routes.add(pg.last_path().split(":")[0] + (":" + pg.last_path().split(":")[-1] if ":" in pg.last_path() else ""))
        out = c.cpu().numpy()
        assert np.all(out[:, n:] == np.float32(0xAB)), (it, dt, m, n, k, pg.last_path())
        want = oracle.gemm_fused_ex(dt, a, b, bias, act)
        tol = max(wl.tolerance(dt, k), 2e-6)            # GELU's erf differs in the last bits between libm and the GPU
        assert wl.relerr(out[:, :n], want) <= tol, (it, dt, m, n, k, lda, ldb, act, pg.last_path())
    assert "simt" in routes and any(r.startswith("tc") for r in routes), routes


def test_unaligned_operands_fall_to_ffma_not_to_garbage(pg, oracle):
    a, b = wl.config2(100, 90, 77)
    got = gemm_dev(pg, wl.BF16, a, b)          # ld = 77 / 90: breaks the 16-byte stride rule of TMA
    assert pg.last_path() == "simt"
    assert np.array_equal(got, oracle.gemm_ex(wl.BF16, a, b))
    pg.set_option("path", 1)
    with pytest.raises(pg.PgError) as e:
        gemm_dev(pg, wl.BF16, a, b)
    assert e.value.status == -1                # PG_ERR_UNSUPPORTED: the dispatcher may then go elsewhere


def test_large_unaligned_operands_are_repitched_for_the_tensor_cores(pg, oracle):
    """Odd leading dimensions on a large product: operands are copied once to an aligned pitch instead
    of sending a teraflop-sized problem to the FFMA kernel."""
    m, n, k = 520, 1031, 777
    a, b = wl.config2(m, n, k)
    got = gemm_dev(pg, wl.BF16, a, b, lda=k + 1, ldb=n, ldc=n + 2)     # lda 778, ldb 1031: both break the 16-byte rule
    assert pg.last_path().startswith("tc:"), pg.last_path()
    assert wl.relerr(got, oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, k)
    # batched, odd batch stride
    q = wl.to_bf16_bits(np.random.default_rng(18).standard_normal((5, 200, 136), dtype=np.float32))
    kt = wl.to_bf16_bits(np.random.default_rng(19).standard_normal((5, 136, 1001), dtype=np.float32))
    s = pg.pg_bmm(to_dev(q, wl.BF16), to_dev(kt, wl.BF16)); pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:"), pg.last_path()
    assert wl.relerr(to_host(s), oracle.bmm(wl.BF16, q, kt)) <= wl.tolerance(wl.BF16, 136)


def test_empty_and_k0(pg):
    c = torch.full((4, 4), 3.0, device="cuda")
    a = torch.zeros(4, 8, device="cuda").bfloat16()
    pg.pg_gemm_ex(wl.BF16, 0, 4, 8, a, 8, a, 4, c, 4)
    pg.pg_gemm_ex(wl.BF16, 4, 0, 8, a, 8, a, 4, c, 4)
    pg.pg_dev_sync()
    assert torch.all(c == 3.0)
    pg.pg_gemm_ex(wl.BF16, 4, 4, 0, a, 8, a, 4, c, 4)      # k = 0: C rows are zeroed (gemm.c:539)
    pg.pg_dev_sync()
    assert torch.all(c == 0.0)


def test_bounded_wait_reports_and_leaves_the_device_usable(pg, oracle):
    """Failure detection without a fault: a kernel waits (bounded, 20 ms) on a barrier nothing sets,
    returns normally with a status bit, pg_dev_sync raises PG_ERR_GEMM once, and the next GEMM is fine."""
    from picograd_b200._lib import lib
    pg.pg_dev_sync()
    assert lib.pg_b200_selftest_wait_timeout(20) == 0
    with pytest.raises(pg.PgError) as e:
        pg.pg_dev_sync()
    assert e.value.status == -5 and "gave up waiting" in str(e.value)
    pg.pg_dev_sync()                                        # the status word was cleared
    a, b = wl.config2(256, 256, 256)
    assert wl.relerr(gemm_dev(pg, wl.BF16, a, b), oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, 256)


def test_host_pointer_gemm_ex(pg, oracle):
    """pg_gemm_ex as ops/matmul.c:264-271 calls it: host buffers in, host buffer out."""
    a, b = wl.config2(300, 200, 264)
    c = np.full((300, 204), 0xAB, np.float32)
    pg.pg_gemm_ex_host(wl.BF16, 300, 200, 264, a, 264, b, 200, c, 204)
    assert np.all(c[:, 200:] == np.float32(0xAB))
    assert wl.relerr(c[:, :200], oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, 264)


def test_host_pointer_gemm_ex_pipelined_blocks(pg):
    """Large host-pointer products are staged block by block (copies overlap the GEMMs); the result
    must be the one the plain staging gives, bit for bit, including ragged last blocks and ld slack."""
    m, n, k = 4096 + 136, 4096 + 72, 264
    a, b = wl.config2(m, n, k)
    abuf = np.zeros((m, k + 8), np.uint16); abuf[:, :k] = a
    bbuf = np.zeros((k, n + 16), np.uint16); bbuf[:, :n] = b
    outs = []
    for pipelined in (1, 0):
        pg.set_option("host_pipeline", pipelined)
        c = np.full((m, n + 4), 0xAB, np.float32)
        pg.pg_gemm_ex_host(wl.BF16, m, n, k, abuf, k + 8, bbuf, n + 16, c, n + 4)
        assert np.all(c[:, n:] == np.float32(0xAB))
        outs.append(c[:, :n].copy())
    pg.set_option("host_pipeline", 1)
    assert np.array_equal(outs[0], outs[1])
    ad, bd = to_dev(a, wl.BF16), to_dev(b, wl.BF16)
    want = pg.pg_matmul(ad, bd); pg.pg_dev_sync()
    assert wl.relerr(outs[0], to_host(want)) <= 1e-6


def test_matmul_shape_modes(pg):
    """tests/test_ops.c:368-492: 2-D, vec.vec, vec.mat, mat.vec, bmm, batched.unbatched; 1e-4*(1+|y|)."""
    rng = np.random.default_rng(12)
    f = lambda *s: rng.uniform(-1, 1, s).astype(np.float32)
    cases = [(f(5, 7), f(7, 3)), (f(7), f(7)), (f(7), f(7, 4)), (f(6, 7), f(7)), (f(3, 5, 7), f(3, 7, 2)),
             (f(2, 3, 5, 7), f(7, 4)), (f(5, 7), f(4, 7, 6)), (f(2, 3, 4, 5), f(2, 3, 5, 6))]
    for a, b in cases:
        y = pg.pg_matmul(to_dev(a, wl.F32), to_dev(b, wl.F32)); pg.pg_dev_sync()
        ref = np.matmul(a.astype(np.float64), b.astype(np.float64))
        ref = ref.reshape(y.shape)
        assert np.all(np.abs(to_host(y) - ref) <= 1e-4 * (1 + np.abs(ref))), (a.shape, b.shape)
    # rejected like picograd does (ops/matmul.c:191-200)
    assert pg.pg_matmul(to_dev(f(4, 5), wl.F32), to_dev(f(6, 4), wl.F32)) is None
    assert pg.pg_matmul(to_dev(f(4, 5), wl.F32), to_dev(f(5, 4), wl.F32).bfloat16()) is None
    assert pg.pg_bmm(to_dev(f(2, 4, 5), wl.F32), to_dev(f(3, 5, 4), wl.F32)) is None


def test_matmul_bf16_batch_broadcast_on_tensor_cores(pg, oracle):
    """Batched x unbatched (and the reverse) for 16-bit operands: ops/matmul.c:209-225 broadcasting."""
    rng = np.random.default_rng(17)
    a3 = wl.to_bf16_bits(rng.standard_normal((3, 136, 72), dtype=np.float32))
    b2 = wl.to_bf16_bits(rng.standard_normal((72, 264), dtype=np.float32))
    y = pg.pg_matmul(to_dev(a3, wl.BF16), to_dev(b2, wl.BF16)); pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:")
    for i in range(3):
        assert wl.relerr(to_host(y[i]), oracle.gemm_ex(wl.BF16, a3[i], b2)) <= wl.tolerance(wl.BF16, 72)
    a2 = wl.to_bf16_bits(rng.standard_normal((136, 72), dtype=np.float32))
    b4 = wl.to_bf16_bits(rng.standard_normal((2, 2, 72, 264), dtype=np.float32))
    y = pg.pg_matmul(to_dev(a2, wl.BF16), to_dev(b4, wl.BF16)); pg.pg_dev_sync()
    assert tuple(y.shape) == (2, 2, 136, 264)
    for i in range(2):
        for j in range(2):
            assert wl.relerr(to_host(y[i, j]), oracle.gemm_ex(wl.BF16, a2, b4[i, j])) <= wl.tolerance(wl.BF16, 72)


def test_tensordot(pg):
    """tests/test_ops.c:451-484 shapes: contraction over one and over two axes."""
    rng = np.random.default_rng(13)
    a = rng.uniform(-1, 1, (3, 4, 5)).astype(np.float32)
    b = rng.uniform(-1, 1, (5, 4, 6)).astype(np.float32)
    y = pg.pg_tensordot(to_dev(a, wl.F32), to_dev(b, wl.F32), [2], [0]); pg.pg_dev_sync()
    ref = np.tensordot(a.astype(np.float64), b.astype(np.float64), axes=([2], [0]))
    assert np.all(np.abs(to_host(y) - ref) <= 1e-4 * (1 + np.abs(ref)))
    y = pg.pg_tensordot(to_dev(a, wl.F32), to_dev(b, wl.F32), [1, 2], [1, 0]); pg.pg_dev_sync()
    ref = np.tensordot(a.astype(np.float64), b.astype(np.float64), axes=([1, 2], [1, 0]))
    assert np.all(np.abs(to_host(y) - ref) <= 1e-4 * (1 + np.abs(ref)))
    ab = to_dev(wl.to_bf16_bits(a), wl.BF16); bb = to_dev(wl.to_bf16_bits(b), wl.BF16)
    y = pg.pg_tensordot(ab, bb, [2], [0]); pg.pg_dev_sync()
    ref = np.tensordot(ab.double().cpu().numpy(), bb.double().cpu().numpy(), axes=([2], [0]))
    assert np.all(np.abs(to_host(y) - ref) <= 1e-4 * (1 + np.abs(ref)))


@pytest.mark.parametrize("shape,perm", [((3, 4, 5), (2, 0, 1)), ((7, 33), (1, 0)), ((2, 3, 4, 5, 6), (4, 0, 3, 1, 2)),
                                        ((5, 1, 9), (1, 2, 0)), ((64, 130), (0, 1))])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_permute_copy_is_the_librarys_own_kernel(pg, shape, perm, dt):
    """permute_copy of pg_tensordot (ops/matmul.c:21-42): bytes moved, nothing computed -> equality."""
    from picograd_b200 import backend
    x = torch.arange(int(np.prod(shape)), device="cuda", dtype=torch.float32).reshape(shape).to(dt)
    n0 = pg.launch_count()
    y = backend._permute_copy(x, list(perm)); pg.pg_dev_sync()
    if list(perm) != list(range(len(shape))):
        assert pg.launch_count() == n0 + 1
    assert y.is_contiguous() and torch.equal(y, x.permute(perm))


@pytest.mark.parametrize("case", ADDMM_CASES, ids=[c[0] for c in ADDMM_CASES])
def test_addmm_against_reference_outputs(pg, case):
    """pg_addmm (ops/matmul.c:371-405): the f32 product is the bit-exact FFMA one and the tail rounds after every
    step like picograd's separate passes -> equality with the compiled reference."""
    inp, a, b = make_addmm_inputs(case)
    y = pg.pg_addmm(to_dev(inp, wl.F32), to_dev(a, wl.F32), to_dev(b, wl.F32), case[5], case[6]); pg.pg_dev_sync()
    assert np.array_equal(to_host(y), np.load(GOLDEN)[case[0]])


def test_addmm_bf16_on_tensor_cores(pg, oracle):
    rng = np.random.default_rng(84)
    a = wl.to_bf16_bits(rng.uniform(-1, 1, (300, 512)).astype(np.float32))
    b = wl.to_bf16_bits(rng.uniform(-1, 1, (512, 264)).astype(np.float32))
    inp = rng.uniform(-1, 1, (264,)).astype(np.float32)
    y = pg.pg_addmm(to_dev(inp, wl.F32), to_dev(a, wl.BF16), to_dev(b, wl.BF16), 0.5, 2.0); pg.pg_dev_sync()
    assert wl.relerr(to_host(y), oracle.addmm(wl.BF16, inp, a, b, 0.5, 2.0)) <= wl.tolerance(wl.BF16, 512)


def test_launches_can_be_captured_in_a_cuda_graph(pg, oracle):
    """Launch-bound loops (decode-like GEMMs) replay from a CUDA graph: after a warm-up call has sized the
    library's scratch, a call enqueues kernels only (the tensor maps travel by value as kernel parameters)."""
    from picograd_b200 import _lib
    m, n, k = 16, 1024, 2048
    rng = np.random.default_rng(85)
    a = wl.to_bf16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    bs = [wl.to_bf16_bits(rng.uniform(-1, 1, (k, n)).astype(np.float32)) for _ in range(3)]
    ad, bds = to_dev(a, wl.BF16), [to_dev(b, wl.BF16) for b in bs]
    outs = [torch.zeros((m, n), dtype=torch.float32, device="cuda") for _ in bs]
    bias = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda()
    side = torch.cuda.Stream()
    try:
        with torch.cuda.stream(side):
            _lib.lib.pg_b200_set_stream(side.cuda_stream)
            pg.pg_gemm_fused_ex(wl.BF16, m, n, k, ad, k, bds[0], n, outs[0], n, bias, pg.PG_ACT_RELU)      # warm-up
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for bd, out in zip(bds, outs):
                    pg.pg_gemm_fused_ex(wl.BF16, m, n, k, ad, k, bd, n, out, n, bias, pg.PG_ACT_RELU)
            for out in outs:
                out.zero_()
            graph.replay(); side.synchronize()
    finally:
        _lib.lib.pg_b200_set_stream(None)
    pg.pg_dev_sync()
    for b, out in zip(bs, outs):
        want = oracle.gemm_fused_ex(wl.BF16, a, b, bias.cpu().numpy(), 1)
        assert wl.relerr(to_host(out), want) <= wl.tolerance(wl.BF16, k)


def test_config4_attention_shaped_bmm(pg, oracle):
    """Reduced config 4 (batch 4, seq 256, d 128).  Each GEMM is checked on identical input bytes:
    P = bf16(softmax(S)) is produced once (on the device) and fed to both sides."""
    q, kt, v = wl.config4(4, 256, 128)
    qd, ktd, vd = (to_dev(x, wl.BF16) for x in (q, kt, v))
    s = pg.pg_bmm(qd, ktd); pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:")
    s_ref = oracle.bmm(wl.BF16, q, kt)
    assert wl.relerr(to_host(s), s_ref) <= wl.tolerance(wl.BF16, 128)
    from picograd_b200 import ops
    p32, p16 = ops.softmax_rows(s, out16=torch.bfloat16); pg.pg_dev_sync()
    assert np.abs(to_host(p32) - oracle.softmax_rows(to_host(s))).max() < 1e-6
    p_bits = bits_to_host(p16)
    assert np.array_equal(p_bits, wl.to_bf16_bits(to_host(p32)))
    o = pg.pg_bmm(p16, vd); pg.pg_dev_sync()
    o_ref = oracle.bmm(wl.BF16, p_bits, v)
    assert wl.relerr(to_host(o), o_ref) <= wl.tolerance(wl.BF16, 256)


@pytest.mark.parametrize("parts", [2, 3])
def test_config5_mlp_forward_backward(pg, oracle, parts):
    """Reduced config 5 (rows 256, 128 -> 512 -> 128), loss = sum.  gelu(h) is rounded to bf16 once
    and the same bytes feed layer 2 on both sides; every GEMM is compared in isolation."""
    from picograd_b200 import ops
    pg.set_option("f32_parts", parts)
    x, w1, w2 = wl.config5(256, 128, 512)
    xd, w1d, w2d = (to_dev(t, wl.BF16) for t in (x, w1, w2))
    # forward
    h = pg.pg_matmul(xd, w1d); pg.pg_dev_sync()
    h_ref = oracle.gemm_ex(wl.BF16, x, w1)
    assert wl.relerr(to_host(h), h_ref) <= wl.tolerance(wl.BF16, 128)
    a32, a16 = ops.gelu(h, out16=torch.bfloat16); pg.pg_dev_sync()
    assert np.abs(to_host(a32) - oracle.gelu(to_host(h))).max() < 1e-5
    a_bits = bits_to_host(a16)
    y = pg.pg_matmul(a16, w2d); pg.pg_dev_sync()
    assert wl.relerr(to_host(y), oracle.gemm_ex(wl.BF16, a_bits, w2)) <= wl.tolerance(wl.BF16, 512)
    # backward of loss = sum(y): dY = 1
    dy = torch.ones_like(y)
    da, dw2 = pg.pg_matmul_backward(a16, w2d, dy); pg.pg_dev_sync()
    da_ref, dw2_ref = oracle.matmul_backward(wl.BF16, a_bits, w2, np.ones(y.shape, np.float32))
    assert wl.relerr(to_host(da), da_ref) <= wl.tolerance(wl.BF16, 128)      # contraction over n = 128
    assert wl.relerr(to_host(dw2), dw2_ref) <= wl.tolerance(wl.BF16, 256)    # contraction over rows = 256
    dh = ops.gelu_grad(h, da); pg.pg_dev_sync()
    dh_host = to_host(dh)
    assert np.abs(dh_host - oracle.gelu_grad(to_host(h), to_host(da))).max() < 1e-4
    dx, dw1 = pg.pg_matmul_backward(xd, w1d, dh); pg.pg_dev_sync()
    dx_ref, dw1_ref = oracle.matmul_backward(wl.BF16, x, w1, dh_host)
    assert wl.relerr(to_host(dx), dx_ref) <= wl.tolerance(wl.BF16, 512)
    assert wl.relerr(to_host(dw1), dw1_ref) <= wl.tolerance(wl.BF16, 256)


def test_backward_accumulates_into_existing_grads(pg, oracle):
    """autograd/autograd.c:669-670, :690-691: grad += product."""
    rng = np.random.default_rng(14)
    m, n, k = 136, 264, 200
    a = wl.to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    b = wl.to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32))
    g = rng.standard_normal((m, n), dtype=np.float32)
    ga0 = rng.standard_normal((m, k), dtype=np.float32)
    gb0 = rng.standard_normal((k, n), dtype=np.float32)
    ga, gb = pg.pg_matmul_backward(to_dev(a, wl.BF16), to_dev(b, wl.BF16), to_dev(g, wl.F32),
                                   ga=to_dev(ga0, wl.F32), gb=to_dev(gb0, wl.F32))
    pg.pg_dev_sync()
    ga_ref, gb_ref = oracle.matmul_backward(wl.BF16, a, b, g)
    assert wl.relerr(to_host(ga) - ga0, ga_ref) <= wl.tolerance(wl.BF16, n)
    assert wl.relerr(to_host(gb) - gb0, gb_ref) <= wl.tolerance(wl.BF16, m)


@pytest.mark.parametrize("retranspose", [1, 0], ids=["transposed-once", "strided-kernel"])
def test_backward_large_f32_leaves_bit_exact(pg, oracle, retranspose):
    """bwd_matmul on f32 leaves (autograd.c:659-691: f32 GEMMs with a transposed operand).  Large products copy the
    transposed operand into row-major order once and take the row-major FFMA kernel; either way every gradient element
    is one fused multiply-add chain in picograd's order: the CPU result bit for bit."""
    rng = np.random.default_rng(15)
    m, n, k = 1100, 1200, 1000
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    g = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    pg.set_option("f32_retranspose", retranspose)
    ga, gb = pg.pg_matmul_backward(to_dev(a, wl.F32), to_dev(b, wl.F32), to_dev(g, wl.F32))
    pg.pg_dev_sync()
    assert pg.last_path() == "simt"
    ga_ref, gb_ref = oracle.matmul_backward(wl.F32, a, b, g)
    assert np.array_equal(to_host(ga), ga_ref)
    assert np.array_equal(to_host(gb), gb_ref)


def test_backward_f16_operands(pg, oracle):
    """f16 A and B with the f32 gradient: both sides meet the tensor cores as exact bf16 pieces."""
    rng = np.random.default_rng(16)
    m, n, k = 200, 264, 136
    a = wl.to_f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = wl.to_f16_bits(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    g = rng.standard_normal((m, n), dtype=np.float32)
    ga, gb = pg.pg_matmul_backward(to_dev(a, wl.F16), to_dev(b, wl.F16), to_dev(g, wl.F32))
    pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:"), pg.last_path()
    ga_ref, gb_ref = oracle.matmul_backward(wl.F16, a, b, g)
    assert wl.relerr(to_host(ga), ga_ref) <= wl.tolerance(wl.F16, n)
    assert wl.relerr(to_host(gb), gb_ref) <= wl.tolerance(wl.F16, m)


def test_backward_batched_and_shared_b(pg, oracle):
    rng = np.random.default_rng(15)
    bt, m, n, k = 3, 72, 136, 64
    a = wl.to_bf16_bits(rng.standard_normal((bt, m, k), dtype=np.float32))
    b = wl.to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32))
    g = rng.standard_normal((bt, m, n), dtype=np.float32)
    ga, gb = pg.pg_matmul_backward(to_dev(a, wl.BF16), to_dev(b, wl.BF16), to_dev(g, wl.F32))
    pg.pg_dev_sync()
    ga_ref = np.zeros((bt, m, k), np.float32); gb_ref = np.zeros((k, n), np.float32)
    for s in range(bt):
        x, y = oracle.matmul_backward(wl.BF16, a[s], b, g[s])
        ga_ref[s] = x; gb_ref += y
    assert wl.relerr(to_host(ga), ga_ref) <= wl.tolerance(wl.BF16, n)
    assert wl.relerr(to_host(gb), gb_ref) <= wl.tolerance(wl.BF16, bt * m)


@pytest.mark.parametrize("act", [1, 2], ids=["relu", "gelu"])
@pytest.mark.parametrize("shape", [(256, 512, 128, True), (136, 264, 200, False), (72, 100, 50, False)],
                         ids=["tma-safe", "want-pre", "odd-sizes"])
def test_backward_with_folded_activation_gradient(pg, oracle, act, shape):
    """pg_b200_matmul_backward_act: the activation node's backward inside the split that feeds bwd_matmul.  Against the
    CPU chain: g' = g * act'(h) (autograd.c:794-801 / :557), then ga = g' B^T, gb = A^T g' on identical g' bytes where
    the f32 form is returned, within the path tolerance otherwise."""
    m, n, k, drop_pre = shape
    rng = np.random.default_rng(33)
    a = wl.to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    b = wl.to_bf16_bits(rng.uniform(-0.1, 0.1, (k, n)).astype(np.float32))
    h = rng.standard_normal((m, n), dtype=np.float32) * 2
    g = rng.standard_normal((m, n), dtype=np.float32)
    ga, gb, pre = pg.pg_matmul_backward_act(to_dev(a, wl.BF16), to_dev(b, wl.BF16), to_dev(g, wl.F32), act, to_dev(h, wl.F32),
                                            want_pre=not drop_pre)
    pg.pg_dev_sync()
    want_pre = oracle.gelu_grad(h, g) if act == 2 else np.where(h > 0, g, 0).astype(np.float32)
    if pre is not None:
        assert np.abs(to_host(pre) - want_pre).max() < 1e-4
        want_pre = to_host(pre)               # identical bytes feed both sides
    ga_ref, gb_ref = oracle.matmul_backward(wl.BF16, a, b, want_pre)
    slack = 1.0 if pre is not None else 2.0   # without the f32 form the two sides' g' differ by erf rounding
    assert wl.relerr(to_host(ga), ga_ref) <= slack * wl.tolerance(wl.BF16, n)
    assert wl.relerr(to_host(gb), gb_ref) <= slack * wl.tolerance(wl.BF16, m)


def test_die_aware_walk_changes_no_bit(pg, oracle):
    """Large products are walked die by die (each half of the L2 keeps its own half of a group's A panel).  Only the
    order of the tiles changes: same bits as the die-oblivious walk, launch after launch (the claim counters re-arm
    themselves), also when the launches are replayed from a CUDA graph."""
    m, n, k = 8192, 4096, 512
    a, b = wl.config2(m, n, k)
    ad, bd = to_dev(a, wl.BF16), to_dev(b, wl.BF16)
    pg.set_option("die_aware", 0)
    ref = torch.empty((m, n), device="cuda")
    pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, ref, n); pg.pg_dev_sync()
    assert "die_aware" not in pg.last_path()
    pg.set_option("die_aware", 1)
    c = torch.zeros((m, n), device="cuda")
    pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n); pg.pg_dev_sync()
    if "die_aware" not in pg.last_path():
        pytest.skip("the SMs of this GPU did not fall into two clean latency groups: " + pg.last_path())
    assert torch.equal(c, ref)
    for _ in range(3):
        c.zero_()
        pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n); pg.pg_dev_sync()
        assert torch.equal(c, ref)
    want = oracle.gemm_ex_panel(wl.BF16, a, b, 4000, 4040, 1000, 1064)
    assert wl.relerr(to_host(c[4000:4040, 1000:1064]), want) <= wl.tolerance(wl.BF16, k)
    # the same launch replayed from a graph: every replay claims, walks and re-arms again
    from picograd_b200 import _lib
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        _lib.lib.pg_b200_set_stream(side.cuda_stream)
        pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n); side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n)
            pg.pg_gemm_ex(wl.BF16, m, n, k, ad, k, bd, n, c, n)
        for _ in range(3):
            c.zero_()
            graph.replay(); side.synchronize()
            assert torch.equal(c, ref)
    _lib.lib.pg_b200_set_stream(None)
    pg.pg_dev_sync()
