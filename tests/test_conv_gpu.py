"""pg_conv2d (ops/conv.c:10-146) on the GPU: device im2col + the bit-exact FFMA GEMM + bias, against picograd's
golden outputs and the CPU oracle.  Every output is the same fused multiply-add chain as on the CPU (zeros of the
padding included), so the comparison is for equality."""
import os

import numpy as np
import pytest
import torch

from golden.make_golden import CONV_CASES, make_conv_inputs

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz")


def dev(a):
    return torch.from_numpy(a).cuda() if a is not None else None


def test_case_from_test_nn_layers(pg):
    # tests/test_nn_layers.c:57-72
    x = torch.arange(1, 10, dtype=torch.float32, device="cuda").reshape(1, 1, 3, 3)
    y = pg.pg_conv2d(x, torch.full((1, 1, 1, 1), 2.0, device="cuda"), torch.tensor([1.0], device="cuda"))
    pg.pg_dev_sync()
    assert torch.equal(y, x * 2 + 1)


@pytest.mark.parametrize("case", CONV_CASES, ids=[c[0] for c in CONV_CASES])
def test_against_reference_outputs(pg, case):
    x, w, b = make_conv_inputs(case)
    y = pg.pg_conv2d(dev(x), dev(w), dev(b), stride=case[8], padding=case[9]); pg.pg_dev_sync()
    assert pg.last_path() == "conv:im2col+simt"
    assert np.array_equal(y.cpu().numpy(), np.load(GOLDEN)[case[0]])


@pytest.mark.parametrize("shape", [(4, 16, 56, 56, 32, 3, 3, 1, 1), (2, 3, 224, 224, 16, 7, 7, 2, 3), (9, 5, 17, 31, 7, 2, 4, 3, 0)],
                         ids=["resnet-block", "stem-7x7-s2", "odd"])
def test_larger_shapes_bit_exact(pg, oracle, shape):
    n, cin, h, w, cout, kh, kw, s, p = shape
    rng = np.random.default_rng(70)
    x = rng.uniform(-1, 1, (n, cin, h, w)).astype(np.float32)
    wt = rng.uniform(-1, 1, (cout, cin, kh, kw)).astype(np.float32)
    b = rng.uniform(-1, 1, cout).astype(np.float32)
    y = pg.pg_conv2d(dev(x), dev(wt), dev(b), stride=s, padding=p); pg.pg_dev_sync()
    assert np.array_equal(y.cpu().numpy(), oracle.conv2d(x, wt, b, s, p))


def test_tensor_core_route_by_option(pg, oracle):
    """With option f32_tensor_cores the convolution's GEMM takes the f32 tensor-core route (three exact bf16 pieces per
    operand, K in chunks): no longer the CPU's bits, within the f32 tolerance of them."""
    n, cin, h, w, cout, kh, kw, s, p = 4, 64, 56, 56, 128, 3, 3, 1, 1
    rng = np.random.default_rng(71)
    x = rng.uniform(-1, 1, (n, cin, h, w)).astype(np.float32)
    wt = rng.uniform(-1, 1, (cout, cin, kh, kw)).astype(np.float32)
    b = rng.uniform(-1, 1, cout).astype(np.float32)
    pg.set_option("f32_tensor_cores", 1)
    y = pg.pg_conv2d(dev(x), dev(wt), dev(b), stride=s, padding=p); pg.pg_dev_sync()
    assert pg.last_path() == "conv:im2col+tc"
    want = oracle.conv2d(x, wt, b, s, p)
    got = y.cpu().numpy()
    assert np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)) <= 1e-6


def test_rejects_what_pg_conv2d_rejects(pg):
    x = torch.zeros(1, 2, 4, 4, device="cuda")
    with pytest.raises(ValueError):
        pg.pg_conv2d(x, torch.zeros(3, 2, 5, 5, device="cuda"))              # window larger than the image
    with pytest.raises(ValueError):
        pg.pg_conv2d(x, torch.zeros(3, 1, 3, 3, device="cuda"))              # channel mismatch
    with pytest.raises(ValueError):
        pg.pg_conv2d(x, torch.zeros(3, 2, 3, 3, device="cuda"), stride=0)
