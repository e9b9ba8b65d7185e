"""The five configurations at FULL size on the GPU.

The CPU oracle cannot produce a full 8192^3 product in test time, so full-size results are checked
through (1) panels of C against the oracle (rows/columns chosen to straddle tile borders), and
(2) a size-independent property that touches every element: C x == A (B x) in float64 for a random
+-1 vector x (a Freivalds check; a wrong tile, a dropped K block or a misplaced store shows up as
an O(1) relative error, f32 accumulation over K as ~1e-5: measured 9e-6 at K = 8192).  The bound
used is a tenth of the path's tolerance 1e-5*sqrt(K).
"""
import numpy as np
import pytest
import torch

import workloads as wl
from gpu_util import bits_to_host, freivalds, to_dev, to_host

pytestmark = pytest.mark.gpu


def _panels(oracle, dtype, a_bits, b_bits, c_dev, k, rows=((0, 40), (120, 136), (-24, None)), cols=((0, 72), (248, 264), (-40, None))):
    m, n = c_dev.shape
    worst = 0.0
    for r0, r1 in rows:
        r0 = r0 % m; r1 = m if r1 is None else r1
        for c0, c1 in cols:
            c0 = c0 % n; c1 = n if c1 is None else c1
            want = oracle.gemm_ex_panel(dtype, a_bits, b_bits, r0, r1, c0, c1)
            got = c_dev[r0:r1, c0:c1].cpu().numpy()
            worst = max(worst, wl.relerr(got, want))
    assert worst <= wl.tolerance(dtype, k), worst
    return worst


def test_config2_bf16_8192(pg, oracle):
    a, b = wl.config2(8192)
    ad, bd = to_dev(a, wl.BF16), to_dev(b, wl.BF16)
    c = torch.empty((8192, 8192), dtype=torch.float32, device="cuda")
    pg.pg_gemm_ex(wl.BF16, 8192, 8192, 8192, ad, 8192, bd, 8192, c, 8192)
    pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:2cta")
    _panels(oracle, wl.BF16, a, b, c, 8192)
    assert freivalds(c, ad.double(), bd.double()) < wl.tolerance(wl.BF16, 8192) / 10
    # by default a CTA's odd-numbered tiles sum K downwards (a wave starts on the K blocks the one before ended on):
    # deterministic, launch after launch
    assert pg.last_path().endswith(":k_up_down")
    again = torch.empty_like(c)
    pg.pg_gemm_ex(wl.BF16, 8192, 8192, 8192, ad, 8192, bd, 8192, again, 8192)
    pg.pg_dev_sync()
    assert torch.equal(c, again)
    # with K ascending everywhere every tile configuration must produce the same product (same K order per element)
    pg.set_option("k_serpentine", 0)
    pg.pg_gemm_ex(wl.BF16, 8192, 8192, 8192, ad, 8192, bd, 8192, c, 8192)
    pg.pg_dev_sync()
    assert "k_up_down" not in pg.last_path()
    assert 0 < wl.relerr(again.cpu().numpy(), c.cpu().numpy()) <= wl.tolerance(wl.BF16, 8192) / 10
    _panels(oracle, wl.BF16, a, b, c, 8192)
    for cfg in (0, 1, 4):
        pg.set_option("tile_config", cfg)
        c2 = torch.empty_like(c)
        pg.pg_gemm_ex(wl.BF16, 8192, 8192, 8192, ad, 8192, bd, 8192, c2, 8192)
        pg.pg_dev_sync()
        assert torch.equal(c, c2), pg.last_path()


def test_config3a_f16_rectangular(pg, oracle):
    m, n, k = 4096, 14336, 4096
    a, b = wl.config3(m, n, k)
    ad, bd = to_dev(a, wl.F16), to_dev(b, wl.F16)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    pg.pg_gemm_ex(wl.F16, m, n, k, ad, k, bd, n, c, n)
    pg.pg_dev_sync()
    _panels(oracle, wl.F16, a, b, c, k)
    assert freivalds(c, ad.double(), bd.double()) < wl.tolerance(wl.F16, k) / 10


def test_config3b_f16_decode_like(pg, oracle):
    m, n, k = 16, 4096, 4096
    a, b = wl.config3(m, n, k)
    ad, bd = to_dev(a, wl.F16), to_dev(b, wl.F16)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    pg.pg_gemm_ex(wl.F16, m, n, k, ad, k, bd, n, c, n)
    pg.pg_dev_sync()
    assert wl.relerr(to_host(c), oracle.gemm_ex(wl.F16, a, b)) <= wl.tolerance(wl.F16, k)


def test_config4_attention_bmm_full(pg, oracle):
    from picograd_b200 import ops
    q, kt, v = wl.config4()                       # [64,2048,128], [64,128,2048], [64,2048,128]
    qd, ktd, vd = (to_dev(x, wl.BF16) for x in (q, kt, v))
    s = pg.pg_bmm(qd, ktd); pg.pg_dev_sync()      # 1 GiB of f32 scores
    assert freivalds(s, qd.double(), ktd.double()) < wl.tolerance(wl.BF16, 128) / 10
    for bi in (0, 37, 63):                        # whole batch elements against the oracle
        want = oracle.gemm_ex(wl.BF16, q[bi], kt[bi])
        assert wl.relerr(to_host(s[bi]), want) <= wl.tolerance(wl.BF16, 128)
    p32, p16 = ops.softmax_rows(s, out16=torch.bfloat16); pg.pg_dev_sync()
    del s
    rows = to_host(p32[5, 100:164])
    assert np.abs(rows.sum(axis=1) - 1).max() < 1e-5
    del p32
    o = pg.pg_bmm(p16, vd); pg.pg_dev_sync()
    assert freivalds(o, p16.double(), vd.double()) < wl.tolerance(wl.BF16, 2048) / 10
    p_bits = bits_to_host(p16[11])
    assert wl.relerr(to_host(o[11]), oracle.gemm_ex(wl.BF16, p_bits, v[11])) <= wl.tolerance(wl.BF16, 2048)
    # the same chain as ONE kernel (scores and probabilities never leave the SM): against the three-kernel
    # result above, and one batch element against the oracle running the chain on the CPU, both within the
    # stated tolerance of the second product, 1e-5 * sqrt(2048) = 4.5e-4 (measured: 4-6e-5).
    fused = pg.pg_attention_bmm(qd, ktd, vd); pg.pg_dev_sync()
    assert pg.last_path() == "attn:fused_128x128"
    e2e = wl.tolerance(wl.BF16, 2048)
    assert wl.relerr(to_host(fused), to_host(o)) <= e2e
    sc = oracle.gemm_ex(wl.BF16, q[37], kt[37])
    pc = wl.to_bf16_bits(oracle.softmax_rows(sc))
    assert wl.relerr(to_host(fused[37]), oracle.gemm_ex(wl.BF16, pc, v[37])) <= e2e
    # rows of P sum to one: with V all ones every output is one up to the rounding of P
    ones = torch.ones_like(vd)
    o1 = pg.pg_attention_bmm(qd, ktd, ones); pg.pg_dev_sync()
    assert (o1 - 1.0).abs().max().item() < 2e-3


def test_config5_mlp_step_full(pg, oracle):
    """x[8192,4096] -> Linear(4096->16384) -> gelu -> Linear(16384->4096) -> sum; forward and backward, through the
    very calls bench.py --config 5 times: first layer fused (h in f32 and bf16(gelu(h)) from one kernel), gradients
    overwritten, the GELU node's backward folded into the split that feeds the first layer's backward.  Each of the six
    GEMMs is checked with the Freivalds property on its own inputs, and panels against the oracle."""
    import math
    from picograd_b200 import ops
    from bench import mlp_step
    x, w1, w2 = wl.config5()
    xd, w1d, w2d = (to_dev(t, wl.BF16) for t in (x, w1, w2))
    dy = torch.ones((8192, 4096), dtype=torch.float32, device="cuda")
    h = torch.empty((8192, 16384), dtype=torch.float32, device="cuda")
    a16 = torch.empty((8192, 16384), dtype=torch.bfloat16, device="cuda")
    y, da, dw2, dx, dw1 = mlp_step(pg, ops, wl, xd, w1d, w2d, dy, h, a16)
    pg.pg_dev_sync()
    # forward
    _panels(oracle, wl.BF16, x, w1, h, 4096, rows=((0, 24), (-16, None)), cols=((0, 48), (-32, None)))
    assert freivalds(h, xd.double(), w1d.double()) < wl.tolerance(wl.BF16, 4096) / 10
    hp = to_host(h[:64, :256])
    assert np.array_equal(bits_to_host(a16[:64, :256]), wl.to_bf16_bits(oracle.gelu(hp))) or \
        np.abs(to_host(a16[:64, :256]) - oracle.gelu(hp)).max() < 2.0 ** -8 * np.abs(oracle.gelu(hp)).max()
    assert freivalds(y, a16.double(), w2d.double()) < wl.tolerance(wl.BF16, 16384) / 10
    # backward of the second layer: dA = dY W2^T ; dW2 = A^T dY (dY = 1: its second bf16 piece is empty, one pass each)
    assert freivalds(da, dy.double(), w2d.double(), transb=True) < wl.tolerance(wl.BF16, 4096) / 10
    assert freivalds(dw2, a16.double(), dy.double(), transa=True) < wl.tolerance(wl.BF16, 8192) / 10
    del y, dy
    # the GELU node: dH = dA * gelu'(h), here in float64 from the same h and dA
    h64 = h.double()
    dh = da.double() * (0.5 * (1 + torch.erf(h64 / math.sqrt(2))) + h64 * torch.exp(-0.5 * h64 * h64) / math.sqrt(2 * math.pi))
    del h64
    assert freivalds(dx, dh, w1d.double(), transb=True) < wl.tolerance(wl.BF16, 16384) / 10
    assert freivalds(dw1, xd.double(), dh, transa=True) < wl.tolerance(wl.BF16, 8192) / 10
    # one panel of a gradient against the oracle's f32 definition dW1 = X^T dH
    dh_h = dh[:, :64].float().cpu().numpy()
    xt = np.ascontiguousarray(wl.bf16_bits_to_f32(x).T)          # [4096, 8192] f32, exact upcast
    want = oracle.gemm_ex(wl.F32, xt[:32], dh_h)                 # rows 0..31 of dW1[:, :64]
    assert wl.relerr(to_host(dw1[:32, :64]), want) <= wl.tolerance(wl.BF16, 8192)
