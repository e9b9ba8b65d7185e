"""pg_cpu_gemm_fused_ex (backend/cpu/gemm.c:718-817) on the GPU: bias and activation applied in the
GEMM kernels' own epilogues, against the CPU oracle and picograd's golden outputs.

FFMA path: the chain of column j starts at bias[j] as on the CPU, so NONE and RELU are bit-exact
and GELU differs only by erff's last bits.  Tensor-core path: bias added to the finished f32 sum,
within the path's tolerance (1e-5 * sqrt(K) for 16-bit inputs).
"""
import os

import numpy as np
import pytest
import torch

import workloads as wl
from golden.make_golden import FUSED_CASES, make_bias, make_inputs
from gpu_util import bits_to_host, to_dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz")
ACT_NAMES = {0: "none", 1: "relu", 2: "gelu"}


def fused_dev(pg, dt, a_bits, b_bits, bias, act, ldc=None, want16=None):
    m, k = a_bits.shape
    n = b_bits.shape[1]
    ldc = n if ldc is None else ldc
    ldb = (n + 7) // 8 * 8                       # the tensor-core path needs 16-byte aligned rows of B
    bbuf = np.zeros((max(k, 1), ldb), b_bits.dtype); bbuf[:k, :n] = b_bits
    a = to_dev(a_bits if k else np.zeros((m, 1), a_bits.dtype), dt)
    b = to_dev(bbuf, dt)
    c = torch.full((m, ldc), float(0xAB), dtype=torch.float32, device="cuda")
    bt = torch.from_numpy(bias).cuda() if bias is not None else None
    c16 = torch.zeros((m, n), dtype=want16, device="cuda") if want16 is not None else None
    pg.pg_gemm_fused_ex(dt, m, n, k, a, max(k, 1), b, ldb, c, ldc, bt, act, c16, n if c16 is not None else 0)
    pg.pg_dev_sync()
    out = c.cpu().numpy()
    assert np.all(out[:, n:] == np.float32(0xAB)), "wrote outside the n columns of C"
    return (out[:, :n], c16) if want16 is not None else out[:, :n]


@pytest.mark.parametrize("case", FUSED_CASES, ids=[c[0] for c in FUSED_CASES])
def test_against_reference_outputs(pg, case):
    name, dt, m, n, k, seed, with_bias, act = case
    gold = np.load(GOLDEN)
    ref = gold[name]
    a, b = make_inputs(dt, m, n, k, seed)
    bias = make_bias(n, seed) if with_bias else None
    cols = gold[name + "_valid_cols"] if dt == wl.F16 else np.ones(n, bool)
    got = fused_dev(pg, dt, a, b, bias, act)                       # whichever path the library picks
    assert wl.relerr(got[:, cols], ref[:, cols]) <= wl.tolerance(dt, k)
    pg.set_option("path", 2)
    got = fused_dev(pg, dt, a, b, bias, act)
    assert pg.last_path() == "simt"
    if dt == wl.BF16 or act == 2:
        assert wl.relerr(got[:, cols], ref[:, cols]) <= 2e-6
    else:
        assert np.array_equal(got[:, cols], ref[:, cols]), "FFMA path: chain from bias[j], bit for bit"


@pytest.mark.parametrize("act", [0, 1, 2], ids=ACT_NAMES.values())
@pytest.mark.parametrize("shape", [(1100, 1200, 333), (70, 50, 129)], ids=["sgemm128", "tile64"])
def test_f32_ffma_kernels(pg, oracle, shape, act):
    """Both f32 kernels (vectorised 128x128 and generic): bit-exact for NONE/RELU."""
    m, n, k = shape
    rng = np.random.default_rng(31)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    want = oracle.gemm_fused_ex(wl.F32, a, b, bias, act)
    got = fused_dev(pg, wl.F32, a, b, bias, act, ldc=n + 4)
    assert pg.last_path() == "simt"
    if act == 2:
        assert np.abs(got - want).max() <= 4e-7 * max(1.0, np.abs(want).max())
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [wl.BF16, wl.F16], ids=["bf16", "f16"])
@pytest.mark.parametrize("act", [0, 1, 2], ids=ACT_NAMES.values())
@pytest.mark.parametrize("shape", [(512, 768, 1024), (300, 1000, 520), (257, 130, 200)],
                         ids=["tma-epilogue", "ragged", "n-not-multiple-of-4"])
def test_tensor_core_epilogue(pg, oracle, dt, act, shape):
    m, n, k = shape
    a32, b32 = wl.seeded_uniform(m, k, 40), wl.seeded_uniform(k, n, 41)
    conv = wl.to_bf16_bits if dt == wl.BF16 else wl.to_f16_bits
    a, b = conv(a32), conv(b32)
    bias = np.random.default_rng(42).uniform(-2, 2, n).astype(np.float32)
    want = oracle.gemm_fused_ex(dt, a, b, bias, act)
    pg.set_option("path", 1)
    got = fused_dev(pg, dt, a, b, bias, act, ldc=n if n % 4 == 0 else n + 3)
    assert pg.last_path().startswith("tc:"), pg.last_path()
    assert wl.relerr(got, want) <= wl.tolerance(dt, k)
    if act == 1:
        assert got.min() >= 0.0


@pytest.mark.parametrize("cfg_name", ["1cta_128x256", "1cta_128x128", "1cta_128x64", "2cta_256x256", "2cta_256x128"])
def test_every_auto_tile_config(pg, oracle, cfg_name):
    from picograd_b200 import _lib
    names = [_lib.lib.pg_b200_tile_config_name(i).decode() for i in range(_lib.lib.pg_b200_num_tile_configs())]
    m, n, k = 384, 640, 256
    a, b = wl.to_bf16_bits(wl.seeded_uniform(m, k, 50)), wl.to_bf16_bits(wl.seeded_uniform(k, n, 51))
    bias = np.random.default_rng(52).uniform(-2, 2, n).astype(np.float32)
    want = oracle.gemm_fused_ex(wl.BF16, a, b, bias, 2)
    pg.set_option("path", 1)
    pg.set_option("tile_config", names.index(cfg_name))
    for epi in (0, 1):
        pg.set_option("epilogue", epi)
        got, c16 = fused_dev(pg, wl.BF16, a, b, bias, 2, want16=torch.bfloat16)
        assert cfg_name in pg.last_path()
        assert wl.relerr(got, want) <= wl.tolerance(wl.BF16, k)
        assert np.array_equal(bits_to_host(c16), wl.to_bf16_bits(got)), "16-bit copy = C rounded to nearest even"


@pytest.mark.parametrize("dt16", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("shape,path", [((256, 512, 512), 1), ((130, 77, 304), 1), ((130, 77, 300), 2),
                                        ((1100, 1200, 64), 2)], ids=["tc-vec", "tc-ragged", "ffma64", "ffma128"])
def test_16bit_copy_of_c(pg, oracle, dt16, shape, path):
    """The same call writes C rounded to f16/bf16, so a 16-bit consumer needs no cast pass."""
    m, n, k = shape
    a, b = wl.to_bf16_bits(wl.seeded_uniform(m, k, 60)), wl.to_bf16_bits(wl.seeded_uniform(k, n, 61))
    bias = np.random.default_rng(62).uniform(-1, 1, n).astype(np.float32)
    pg.set_option("path", path)
    got, c16 = fused_dev(pg, wl.BF16, a, b, bias, 1, want16=dt16)
    want = oracle.gemm_fused_ex(wl.BF16, a, b, bias, 1)
    assert wl.relerr(got, want) <= wl.tolerance(wl.BF16, k)
    conv = wl.to_bf16_bits if dt16 == torch.bfloat16 else wl.to_f16_bits
    assert np.array_equal(bits_to_host(c16), conv(got))


@pytest.mark.parametrize("shape,path", [((256, 512, 512), 1), ((130, 77, 304), 1), ((130, 77, 300), 2), ((1100, 1200, 64), 2),
                                        ((16, 4096, 1024), 0)], ids=["tc-vec", "tc-ragged", "ffma64", "ffma128", "skinny-post-pass"])
def test_activation_on_the_16bit_copy_only(pg, oracle, shape, path):
    """PG_ACT_COPY_ONLY: C keeps bias + A*B (the pre-activation a backward pass reads), the 16-bit copy gets
    the activation of it: the first layer of a training MLP in one kernel."""
    m, n, k = shape
    a, b = wl.to_bf16_bits(wl.seeded_uniform(m, k, 65)), wl.to_bf16_bits(wl.seeded_uniform(k, n, 66))
    bias = np.random.default_rng(67).uniform(-1, 1, n).astype(np.float32)
    pg.set_option("path", path)
    got, c16 = fused_dev(pg, wl.BF16, a, b, bias, pg.PG_ACT_GELU | pg.PG_ACT_COPY_ONLY, want16=torch.bfloat16)
    pre = oracle.gemm_fused_ex(wl.BF16, a, b, bias, 0)
    assert wl.relerr(got, pre) <= wl.tolerance(wl.BF16, k)
    want16 = oracle.gelu(got)                                 # activation of what C actually holds
    got16 = wl.bf16_bits_to_f32(bits_to_host(c16))
    assert np.abs(got16 - want16).max() <= 2.0 ** -8 * max(1.0, np.abs(want16).max())   # one bf16 rounding


def test_skinny_and_split_k_routes_apply_the_epilogue_after_the_sum(pg, oracle):
    """K-slices and the swapped-operand route finish C first; one elementwise pass follows."""
    for (m, n, k) in [(16, 4096, 4096), (128, 128, 8192)]:
        a, b = wl.to_bf16_bits(wl.seeded_uniform(m, k, 70)), wl.to_bf16_bits(wl.seeded_uniform(k, n, 71))
        bias = np.random.default_rng(72).uniform(-3, 3, n).astype(np.float32)
        want = oracle.gemm_fused_ex(wl.BF16, a, b, bias, 1)
        got, c16 = fused_dev(pg, wl.BF16, a, b, bias, 1, want16=torch.bfloat16)
        assert pg.last_path().startswith("tc:")
        assert wl.relerr(got, want) <= wl.tolerance(wl.BF16, k)
        assert np.array_equal(bits_to_host(c16), wl.to_bf16_bits(got))


def test_no_bias_no_act_equals_gemm_ex(pg):
    a = torch.randn(300, 200, device="cuda").bfloat16()
    b = torch.randn(200, 260, device="cuda").bfloat16()
    c0 = torch.empty(300, 260, device="cuda"); c1 = torch.empty_like(c0)
    pg.pg_gemm_ex(pg.PG_DTYPE_BF16, 300, 260, 200, a, 200, b, 260, c0, 260)
    pg.pg_gemm_fused_ex(pg.PG_DTYPE_BF16, 300, 260, 200, a, 200, b, 260, c1, 260)
    pg.pg_dev_sync()
    assert torch.equal(c0, c1)


def test_k0_gives_act_of_bias(pg):
    bias = np.array([-1.0, 0.5, 2.0, -0.25, 3.0], np.float32)
    got = fused_dev(pg, wl.F32, np.zeros((3, 0), np.float32), np.zeros((0, 5), np.float32), bias, 1)
    assert np.array_equal(got, np.tile(np.maximum(bias, 0), (3, 1)))


def test_host_pointers_like_nn_linear(pg, oracle):
    """nn/nn.c:46-96: Linear forward calls pg_cpu_gemm_fused on host tensors (with and without ReLU)."""
    rng = np.random.default_rng(80)
    x = rng.uniform(-1, 1, (64, 300)).astype(np.float32)
    w = rng.uniform(-0.1, 0.1, (300, 150)).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, 150).astype(np.float32)
    for act in (0, 1):
        out = np.full((64, 150), np.nan, np.float32)
        pg.pg_gemm_fused(64, 150, 300, x, 300, w, 150, out, 150, bias, act)
        assert np.array_equal(out, oracle.gemm_fused_ex(wl.F32, x, w, bias, act))
    # the pipelined block route of large host products carries the bias slice of each block
    m = n = 4096; k = 64
    a = wl.to_bf16_bits(wl.seeded_uniform(m, k, 81)); b = wl.to_bf16_bits(wl.seeded_uniform(k, n, 82))
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    out = np.empty((m, n), np.float32)
    pg.pg_gemm_fused_ex(wl.BF16, m, n, k, a, k, b, n, out, n, bias, 1)
    assert wl.relerr(out, oracle.gemm_fused_ex(wl.BF16, a, b, bias, 1)) <= wl.tolerance(wl.BF16, k)


def test_linear_forward_mirror(pg, oracle):
    x = torch.randn(200, 512, device="cuda").bfloat16()
    w = (torch.randn(512, 384, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(384, device="cuda")
    y16 = torch.empty(200, 384, device="cuda", dtype=torch.bfloat16)
    y = pg.pg_linear_forward(x, w, bias, relu=True, out16=y16)
    pg.pg_dev_sync()
    want = oracle.gemm_fused_ex(wl.BF16, bits_to_host(x), bits_to_host(w), bias.cpu().numpy(), 1)
    assert wl.relerr(y.cpu().numpy(), want) <= wl.tolerance(wl.BF16, 512)
    assert torch.equal(y16, y.bfloat16())


def test_rejects_what_the_entry_cannot_do(pg):
    a = torch.zeros(8, 8, device="cuda"); c = torch.zeros(8, 8, device="cuda")
    with pytest.raises(pg.PgError):
        pg.pg_gemm_fused_ex(pg.PG_DTYPE_F32, 8, 8, 8, a, 8, a, 8, c, 8, None, 7)            # unknown activation
    with pytest.raises(pg.PgError):
        pg.pg_gemm_fused_ex(pg.PG_DTYPE_F32, 8, 8, 8, a, 8, a, 8, c, 8, np.zeros(8, np.float32), 0)  # host bias, device operands
