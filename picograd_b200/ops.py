"""Device-resident harness steps between the GEMMs of the attention-shaped and MLP workloads.

These mirror picograd's pg_softmax (ops/activations.c:22-45), pg_gelu (:114) and the GELU
gradient (autograd/autograd.c:794-801) so that a whole workload stays in HBM; they are
HBM-bound element-wise kernels, not part of the contraction itself.
"""
import torch

from . import backend as _b
from ._lib import lib

_CODE16 = {torch.float16: _b.PG_DTYPE_F16, torch.bfloat16: _b.PG_DTYPE_BF16}


def softmax_rows(x, out16=None, want_f32=True):
    """Row softmax over the last axis of a float32 tensor; also returns the result rounded to
    `out16` (torch.float16 / torch.bfloat16) when asked.  want_f32=False skips the float32 copy
    (returns (None, y16)), which is what a P = bf16(softmax(S)) step needs."""
    _b._ready()
    x = x.contiguous()
    y = torch.empty_like(x) if want_f32 else None
    y16 = torch.empty(x.shape, dtype=out16, device=x.device) if out16 is not None else None
    _b._check(lib.pg_b200_softmax_rows(x.data_ptr(), y.data_ptr() if y is not None else None,
                                       y16.data_ptr() if y16 is not None else None,
                                       _CODE16.get(out16, 0), x.numel() // x.shape[-1], x.shape[-1]),
              "pg_b200_softmax_rows")
    return (y, y16) if out16 is not None else y


def gelu(x, out16=None, want_f32=True):
    _b._ready()
    x = x.contiguous()
    y = torch.empty_like(x) if want_f32 else None
    y16 = torch.empty(x.shape, dtype=out16, device=x.device) if out16 is not None else None
    _b._check(lib.pg_b200_gelu(x.data_ptr(), y.data_ptr() if y is not None else None,
                               y16.data_ptr() if y16 is not None else None,
                               _CODE16.get(out16, 0), x.numel()), "pg_b200_gelu")
    return (y, y16) if out16 is not None else y


def gelu_grad(x, gy):
    _b._ready()
    x, gy = x.contiguous(), gy.contiguous()
    out = torch.empty_like(x)
    _b._check(lib.pg_b200_gelu_grad(x.data_ptr(), gy.data_ptr(), out.data_ptr(), x.numel()), "pg_b200_gelu_grad")
    return out


def cast16(x, dtype16):
    _b._ready()
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=dtype16, device=x.device)
    _b._check(lib.pg_b200_cast_f32(x.data_ptr(), out.data_ptr(), _CODE16[dtype16], x.numel()), "pg_b200_cast_f32")
    return out
