"""The matmul node of the autograd on the GPU against gradients produced by picograd's own
pg_ag_matmul -> pg_backward (tests/golden/reference_outputs.npz, made by tests/golden/make_golden.py
from the unmodified library; bwd_matmul is autograd/autograd.c:561-706).

picograd multiplies the f32 gradient exactly (operands upcast to f32, f32 GEMM).  The device path cuts the
f32 gradient into bf16 pieces for the tensor cores (2 by default, 3 with option f32_parts); both settings
are held to the bound of the path, 1e-5 * sqrt(K) for 16-bit operands and 1e-6 for f32, and the measured
margins are printed (pytest -s) so that they can be quoted.
"""
import os

import numpy as np
import pytest
import torch

import workloads as wl
from golden.make_golden import BWD_CASES, BWD_MODE_CASES, make_bwd_inputs
from gpu_util import to_dev, to_host

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz")


def _as_matrices(a, b, g):
    """picograd's 1-D promotion (ops/matmul.c:186-206): a vector a is a row, a vector b a column."""
    a2 = a.reshape(1, -1) if a.ndim == 1 else a
    b2 = b.reshape(-1, 1) if b.ndim == 1 else b
    g2 = np.ascontiguousarray(g, np.float32).reshape(a2.shape[:-1] + (b2.shape[-1],))
    return a2, b2, g2


def _gpu_backward(pg, dt, a, b, g):
    a2, b2, g2 = _as_matrices(a, b, g)
    ga, gb = pg.pg_matmul_backward(to_dev(a2, dt), to_dev(b2, dt), to_dev(g2, wl.F32), dtype=dt)
    pg.pg_dev_sync()
    return to_host(ga).reshape(a.shape), to_host(gb).reshape(b.shape)


@pytest.mark.parametrize("case", BWD_MODE_CASES, ids=[c[0] for c in BWD_MODE_CASES])
def test_shape_modes_against_picograd(pg, case):
    name, ash, bsh, seed = case
    gold = np.load(GOLDEN)
    a, b, _ = make_bwd_inputs(wl.F32, ash, bsh, seed, with_upstream=False)
    ga, gb = _gpu_backward(pg, wl.F32, a, b, np.ones(gold[name + "_y"].shape, np.float32))
    assert wl.relerr(ga, gold[name + "_ga"]) <= 1e-6
    assert wl.relerr(gb, gold[name + "_gb"]) <= 1e-6


@pytest.mark.parametrize("parts", [2, 3])
@pytest.mark.parametrize("case", BWD_CASES, ids=[c[0] for c in BWD_CASES])
def test_gradients_against_picograd(pg, case, parts):
    name, dt, ash, bsh, seed = case
    gold = np.load(GOLDEN)
    pg.set_option("f32_parts", parts)
    a, b, g = make_bwd_inputs(dt, ash, bsh, seed)
    ga, gb = _gpu_backward(pg, dt, a, b, g)
    n = bsh[-1]                                             # ga contracts over n
    rows = int(np.prod(ash[:-1])) if len(bsh) == 2 else ash[-2]   # gb contracts over m (times batch when B is shared)
    ea, eb = wl.relerr(ga, gold[name + "_ga"]), wl.relerr(gb, gold[name + "_gb"])
    print(f"{name} f32_parts={parts} path={pg.last_path()}: ga {ea:.3e} (bound {wl.tolerance(dt, n):.1e}), "
          f"gb {eb:.3e} (bound {wl.tolerance(dt, rows):.1e})")
    assert ea <= wl.tolerance(dt, n)
    assert eb <= wl.tolerance(dt, rows)
    if dt == wl.F32 and len(ash) == 2:
        # f32 operands run the one-chain FFMA kernel: picograd's bits.  (With a batch that shares B picograd adds
        # one product per batch element into gb, the device folds the batch into one chain: same sum, other rounding.)
        assert np.array_equal(ga, gold[name + "_ga"]) and np.array_equal(gb, gold[name + "_gb"])


def test_picograd_drawn_leaves_and_mlp_nodes(pg):
    """Leaves drawn by picograd's generator (tests/test_autograd.c:319-330) and both matmul nodes of its
    two-layer network (:393-421)."""
    gold = np.load(GOLDEN)
    for name in ("bwd_pgseed11_bmm", "bwd_pgseed11_bcast_batch"):
        a, b, y = gold[name + "_a"], gold[name + "_b"], gold[name + "_y"]
        ga, gb = _gpu_backward(pg, wl.F32, a, b, np.ones(y.shape, np.float32))
        assert wl.relerr(ga, gold[name + "_ga"]) <= 1e-6 and wl.relerr(gb, gold[name + "_gb"]) <= 1e-6
    x, w1, w2, h = (gold["bwd_mlp_" + k] for k in ("x", "w1", "w2", "h"))
    gh, gw2 = _gpu_backward(pg, wl.F32, h, w2, gold["bwd_mlp_g_mm2"])
    assert wl.relerr(gh, gold["bwd_mlp_g_h"]) <= 1e-6 and wl.relerr(gw2, gold["bwd_mlp_g_w2"]) <= 1e-6
    gx, gw1 = _gpu_backward(pg, wl.F32, x, w1, gold["bwd_mlp_g_mm1"])
    assert wl.relerr(gx, gold["bwd_mlp_g_x"]) <= 1e-6 and wl.relerr(gw1, gold["bwd_mlp_g_w1"]) <= 1e-6


def test_tensor_core_route_is_taken_for_16_bit_leaves(pg):
    """The larger bf16 case must run on the tensor cores (the bound above would also pass on the FFMA kernel)."""
    name, dt, ash, bsh, seed = next(c for c in BWD_CASES if c[0] == "bwd_bf16_136x264x200")
    a, b, g = make_bwd_inputs(dt, ash, bsh, seed)
    _gpu_backward(pg, dt, a, b, g)
    assert pg.last_path().startswith("tc:"), pg.last_path()


@pytest.mark.parametrize("kind", ["ones", "bf16-valued", "zeros", "one-row-f32"])
def test_gradients_whose_second_piece_is_empty(pg, oracle, kind):
    """The f32 gradient meets the tensor cores as bf16 pieces; a piece without a non-zero element is skipped on the
    device (the split kernel reports which pieces hold something).  Gradients made of bf16 numbers — the ones of a
    sum loss — therefore take one pass, a zero gradient still writes zeros, and one f32-valued row brings the second
    pass back.  All must equal the CPU result."""
    rng = np.random.default_rng(31)
    m, n, k = 264, 200, 136
    a = wl.to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    b = wl.to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32))
    if kind == "ones":
        g = np.ones((m, n), np.float32)
    elif kind == "zeros":
        g = np.zeros((m, n), np.float32)
    else:
        g = wl.bf16_bits_to_f32(wl.to_bf16_bits(rng.standard_normal((m, n), dtype=np.float32)))
        if kind == "one-row-f32":
            g[17] = rng.standard_normal(n, dtype=np.float32)
    ga0 = torch.full((m, k), 3.0, device="cuda")          # overwritten, not added to
    gb0 = torch.full((k, n), 3.0, device="cuda")
    from picograd_b200._lib import lib
    pg.pg_dev_sync()
    ad, bd, gd = to_dev(a, wl.BF16), to_dev(b, wl.BF16), to_dev(g, wl.F32)      # held until the call has run
    st = lib.pg_b200_matmul_backward_ex(wl.BF16, 1, m, n, k, ad.data_ptr(), bd.data_ptr(), 0, gd.data_ptr(), ga0.data_ptr(),
                                        gb0.data_ptr(), 0)
    assert st == 0
    pg.pg_dev_sync()
    assert pg.last_path().startswith("tc:"), pg.last_path()
    ga_ref, gb_ref = oracle.matmul_backward(wl.BF16, a, b, g)
    if kind == "zeros":
        assert not ga0.any().item() and not gb0.any().item()
    else:
        assert wl.relerr(to_host(ga0), ga_ref) <= wl.tolerance(wl.BF16, n)
        assert wl.relerr(to_host(gb0), gb_ref) <= wl.tolerance(wl.BF16, m)
