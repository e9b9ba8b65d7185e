"""pg_b200_attention_bmm: the chain pg_bmm -> pg_softmax -> cast -> pg_bmm (ops/matmul.c:340-369,
ops/activations.c:22-45) as one call, against the CPU oracle running the chain step by step.

The fused kernel rounds P to 16 bits after the division by the row sum, as the chain does, so its O
differs from the chain's only where a last-bit difference in S or exp() flips a 16-bit rounding of P:
far inside the tolerance of the second product (1e-5 * sqrt(Sk))."""
import numpy as np
import pytest
import torch

import workloads as wl
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


# Normwise error of the whole chain measured on B200 where the second product's own bound is smallest (short rows):
# a last-bit difference in a score or in exp() flips the 16-bit rounding of a few probabilities, which shows as an
# error of O that does not shrink with the row length.  The floors are twice the largest value measured over the
# shapes of this file.
E2E_FLOOR = {wl.BF16: 3.2e-4, wl.F16: 5e-5}     # measured maxima: 1.55e-4 (bf16, Sk = 160, D = 64), 2.5e-5 (f16)


def e2e_tolerance(dt, sk):
    """End-to-end bound for the whole chain: the stated tolerance of the second product, 1e-5 * sqrt(Sk) (each product
    alone meets it on identical input bytes, tests/test_gemm_gpu.py), with the measured rounding-flip floor for short
    rows."""
    return max(wl.tolerance(dt, sk), E2E_FLOOR[dt])


def within(err, dt, sk, what=""):
    print(f"attention e2e {what} dt={dt} sk={sk}: {err:.3e} (bound {e2e_tolerance(dt, sk):.2e})")
    return err <= e2e_tolerance(dt, sk)


def make_qkv(bt, sq, sk, d, dt, seed):
    rng = np.random.default_rng(seed)
    conv = wl.to_bf16_bits if dt == wl.BF16 else wl.to_f16_bits
    s = 1.0 / np.sqrt(np.sqrt(d))        # scores ~ N(0, 1), as in picograd's attention-shaped configuration
    q = conv((rng.standard_normal((bt, sq, d)) * s).astype(np.float32))
    kt = conv((rng.standard_normal((bt, d, sk)) * s).astype(np.float32))
    v = conv(rng.standard_normal((bt, sk, d)).astype(np.float32))
    return q, kt, v


def oracle_chain(oracle, dt, q, kt, v):
    s = oracle.bmm(dt, q, kt)
    p = oracle.softmax_rows(s)
    # IEEE round-to-nearest-even (picograd's own f32->f16 converter mishandles subnormals, core/convert.h:33-44,
    # and small probabilities are subnormal in f16)
    p16 = wl.to_bf16_bits(p) if dt == wl.BF16 else wl.to_f16_bits(p)
    return oracle.bmm(dt, p16, v)


@pytest.mark.parametrize("dt", [wl.BF16, wl.F16], ids=["bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 256, 256), (1, 128, 128), (3, 200, 328), (1, 50, 104), (2, 384, 1152), (1, 130, 2048)],
                         ids=["even", "one-block", "ragged", "tiny", "odd-block-count", "long-row"])
def test_fused_equals_the_chain_on_the_cpu(pg, oracle, dt, shape):
    bt, sq, sk = shape
    q, kt, v = make_qkv(bt, sq, sk, 128, dt, 90)
    want = oracle_chain(oracle, dt, q, kt, v)
    got = pg.pg_attention_bmm(to_dev(q, dt), to_dev(kt, dt), to_dev(v, dt))
    pg.pg_dev_sync()
    assert pg.last_path() == "attn:fused_128x128"
    assert within(wl.relerr(got.cpu().numpy(), want), dt, sk, str(shape))


def test_q_from_shared_memory_and_from_tensor_memory_agree_bit_for_bit(pg):
    """The Q Kt products read Q from tensor memory by default (copied there once per unit) or from shared memory
    (option attn_q_tmem = 0): same operands, same MMAs, identical bits."""
    q, kt, v = make_qkv(3, 400, 776, 128, wl.BF16, 94)
    qd, ktd, vd = to_dev(q, wl.BF16), to_dev(kt, wl.BF16), to_dev(v, wl.BF16)
    a = pg.pg_attention_bmm(qd, ktd, vd); pg.pg_dev_sync()
    pg.set_option("attn_q_tmem", 0)
    b = pg.pg_attention_bmm(qd, ktd, vd); pg.pg_dev_sync()
    assert pg.last_path() == "attn:fused_128x128"
    assert torch.equal(a, b)


def test_many_units_per_cta_and_both_paths_agree(pg):
    """More work units than SMs (each CTA loops) and odd counts everywhere; the chain form of the same
    entry (the library's own three kernels) is the second opinion."""
    bt, sq, sk = 5, 4096 + 77, 640 + 8
    q, kt, v = make_qkv(bt, sq, sk, 128, wl.BF16, 91)
    qd, ktd, vd = to_dev(q, wl.BF16), to_dev(kt, wl.BF16), to_dev(v, wl.BF16)
    fused = pg.pg_attention_bmm(qd, ktd, vd); pg.pg_dev_sync()
    assert pg.last_path() == "attn:fused_128x128"
    pg.set_option("fused_attention", 0)
    chain = pg.pg_attention_bmm(qd, ktd, vd); pg.pg_dev_sync()
    pg.set_option("fused_attention", 1)
    assert pg.last_path() == "attn:chain"
    assert within(wl.relerr(fused.cpu().numpy(), chain.cpu().numpy()), wl.BF16, sk, 'fused vs chain')
    # rows of P sum to one: with V all ones every output is 1 up to the 16-bit rounding of P
    ones = torch.ones_like(vd)
    o = pg.pg_attention_bmm(qd, ktd, ones); pg.pg_dev_sync()
    assert (o - 1.0).abs().max().item() < 4e-3


@pytest.mark.parametrize("shape", [(2, 96, 160, 64), (2, 96, 333, 128)], ids=["d64", "keys-not-multiple-of-8"])
def test_shapes_the_fused_kernel_does_not_take_run_the_chain(pg, oracle, shape):
    bt, sq, sk, d = shape
    q, kt, v = make_qkv(bt, sq, sk, d, wl.BF16, 92)
    want = oracle_chain(oracle, wl.BF16, q, kt, v)
    got = pg.pg_attention_bmm(to_dev(q, wl.BF16), to_dev(kt, wl.BF16), to_dev(v, wl.BF16)); pg.pg_dev_sync()
    assert pg.last_path() == "attn:chain"
    assert within(wl.relerr(got.cpu().numpy(), want), wl.BF16, sk)


def test_large_scores_do_not_overflow(pg, oracle):
    """Row maxima far from zero: the subtraction of the maximum happens before the exponential."""
    bt, sq, sk = 1, 128, 256
    q, kt, v = make_qkv(bt, sq, sk, 128, wl.BF16, 93)
    q = wl.to_bf16_bits(wl.bf16_bits_to_f32(q) * 16.0)
    want = oracle_chain(oracle, wl.BF16, q, kt, v)
    got = pg.pg_attention_bmm(to_dev(q, wl.BF16), to_dev(kt, wl.BF16), to_dev(v, wl.BF16)); pg.pg_dev_sync()
    assert np.isfinite(got.cpu().numpy()).all()
    assert within(wl.relerr(got.cpu().numpy(), want), wl.BF16, sk)
