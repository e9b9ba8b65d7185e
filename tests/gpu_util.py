"""Helpers shared by the -m gpu tests: move bit patterns to the device, bring results back."""
import numpy as np
import torch

import workloads as wl

_TORCH16 = {wl.F16: torch.float16, wl.BF16: torch.bfloat16}


def to_dev(arr, dtype):
    """numpy array (float32, or uint16 bit patterns of f16/bf16) -> CUDA tensor of the torch dtype."""
    if dtype == wl.F32:
        return torch.from_numpy(np.ascontiguousarray(arr, np.float32)).cuda()
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).cuda()
    return t.view(_TORCH16[dtype])


def to_host(t):
    return t.detach().float().cpu().numpy() if t.dtype != torch.float32 else t.detach().cpu().numpy()


def bits_to_host(t):
    """CUDA f16/bf16 tensor -> numpy uint16 bit patterns."""
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def gemm_dev(pg, dtype, a_bits, b_bits, lda=None, ldb=None, ldc=None):
    """pg_gemm_ex on device copies of a, b (optionally embedded in wider-ld buffers); returns numpy C."""
    m, k = a_bits.shape
    n = b_bits.shape[1]
    lda = k if lda is None else lda
    ldb = n if ldb is None else ldb
    ldc = n if ldc is None else ldc
    abuf = np.zeros((m, lda), a_bits.dtype); abuf[:, :k] = a_bits
    bbuf = np.zeros((max(k, 1), ldb), b_bits.dtype); bbuf[:k, :n] = b_bits
    a = to_dev(abuf, dtype); b = to_dev(bbuf, dtype)
    c = torch.full((m, ldc), float(0xAB), dtype=torch.float32, device="cuda")
    pg.pg_gemm_ex(dtype, m, n, k, a, lda, b, ldb, c, ldc)
    pg.pg_dev_sync()
    out = c.cpu().numpy()
    assert np.all(out[:, n:] == np.float32(0xAB)), "wrote outside the n columns of C"
    return out[:, :n]


def freivalds(c, a_f64, b_f64, transa=False, transb=False, seed=0):
    """Normwise relative error of C x against op(A) (op(B) x) in float64, x a random +-1 vector:
    a check of every element of a full-size C that costs O(n^2)."""
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    n = c.shape[-1]
    x = (torch.randint(0, 2, (n, 1), generator=g, device="cuda").double() * 2 - 1)
    bx = (b_f64.transpose(-1, -2) if transb else b_f64) @ x
    ref = (a_f64.transpose(-1, -2) if transa else a_f64) @ bx
    got = c.double() @ x
    return (torch.linalg.norm(got - ref) / torch.linalg.norm(ref)).item()
