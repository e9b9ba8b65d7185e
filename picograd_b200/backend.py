"""Python mirror of picograd's operator interface for the matrix-multiply path.

Same names, argument meaning and error behaviour as picograd's C API
(backend/backend.h:103-136, ops/matmul.h:6-11); device memory is held in torch
CUDA tensors, whose pointers go straight into the C-ABI of libpg_b200.so.
16-bit operands are torch.float16 / torch.bfloat16 tensors (or uint16 bit
patterns with an explicit dtype code); results are always float32.
"""
import ctypes as C

import torch

from ._lib import lib

PG_DTYPE_F32, PG_DTYPE_F16, PG_DTYPE_BF16 = 0, 1, 2          # core/dtype.h:11-16
PG_OK, PG_ERR_UNSUPPORTED, PG_ERR_ALLOC, PG_ERR_COPY, PG_ERR_SYNC, PG_ERR_GEMM = 0, -1, -2, -3, -4, -5

_TORCH2PG = {torch.float32: PG_DTYPE_F32, torch.float16: PG_DTYPE_F16, torch.bfloat16: PG_DTYPE_BF16}


class PgError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        msg = lib.pg_b200_last_error().decode(errors="replace")
        super().__init__(f"{what}: pg_status {status}: {msg}")


def _check(st, what):
    if st != PG_OK:
        raise PgError(st, what)


_initialised = False


def pg_set_device(ordinal=None):
    """pg_set_device(PG_DEV_CUDA) (backend/backend.c:76-90): init the device seat.
    The ordinal defaults to torch's current CUDA device."""
    global _initialised
    if ordinal is None:
        ordinal = torch.cuda.current_device()
    _check(lib.pg_b200_set_device(int(ordinal)), "pg_b200_set_device")
    _check(lib.pg_b200_init(), "pg_b200_init")
    _initialised = True


def _ready():
    if not _initialised:
        pg_set_device()
    # kernels are queued on torch's current stream so that torch events time them.  The library's scratch, counters
    # and status word exist once per process: callers that change torch's current stream must synchronise the old
    # stream first (calls in flight on two streams would share that scratch).
    lib.pg_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))


def pg_dev_sync():
    """pg_dev_sync (backend/backend.c:125-132); raises if a kernel reported a failed wait."""
    _ready()
    _check(lib.pg_b200_sync(), "pg_dev_sync")


def set_option(name, value):
    _check(lib.pg_b200_set_option(name.encode(), int(value)), f"set_option({name})")


def last_path():
    return lib.pg_b200_last_path().decode()


def launch_count():
    return int(lib.pg_b200_launch_count())


def _code(t, dtype):
    if dtype is not None:
        return dtype
    if t.dtype not in _TORCH2PG:
        raise TypeError(f"unsupported tensor dtype {t.dtype}")
    return _TORCH2PG[t.dtype]


def pg_gemm_ex(dtype, m, n, k, a, lda, b, ldb, c, ldc):
    """pg_gemm_ex (backend/backend.c:150-177) on device tensors: C[m,n] f32 = A[m,k] * B[k,n],
    row-major, ld* in elements, C overwritten.  a/b/c are CUDA tensors (any shape; only their
    pointers are used)."""
    _ready()
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise ValueError("pg_gemm_ex takes device tensors; use pg_gemm_ex_host for host buffers")
    if c.dtype != torch.float32:
        raise TypeError("C must be float32")
    _check(lib.pg_b200_gemm_ex(dtype, m, n, k, a.data_ptr(), lda, b.data_ptr(), ldb, c.data_ptr(), ldc),
           "pg_gemm_ex")


def pg_gemm(m, n, k, a, lda, b, ldb, c, ldc):
    """pg_gemm (backend/backend.c:134-148): f32."""
    pg_gemm_ex(PG_DTYPE_F32, m, n, k, a, lda, b, ldb, c, ldc)


def pg_hgemm(m, n, k, a, lda, b, ldb, c, ldc):
    """pg_hgemm (backend/backend.c:179-185)."""
    pg_gemm_ex(PG_DTYPE_F16, m, n, k, a, lda, b, ldb, c, ldc)


def pg_bgemm(m, n, k, a, lda, b, ldb, c, ldc):
    """pg_bgemm (backend/backend.c:186-192)."""
    pg_gemm_ex(PG_DTYPE_BF16, m, n, k, a, lda, b, ldb, c, ldc)


PG_ACT_NONE, PG_ACT_RELU, PG_ACT_GELU = 0, 1, 2   # backend/cpu/gemm.h:37-39


PG_ACT_COPY_ONLY = 0x100   # with c16: the activation goes into the 16-bit copy only, C keeps bias + A*B


def pg_gemm_fused_ex(dtype, m, n, k, a, lda, b, ldb, c, ldc, bias=None, act=PG_ACT_NONE, c16=None, ldc16=0):
    """pg_cpu_gemm_fused_ex (backend/cpu/gemm.c:806-817): C = act(bias[j] + A*B), bias an f32
    tensor of n elements or None, applied in the GEMM kernel's epilogue.  Device tensors, or host
    tensors / numpy arrays throughout (staged inside the call).  c16 (device only, optional): an
    f16/bf16 tensor that receives C rounded to its dtype in the same pass."""
    _ready()

    def ptr(x):
        if x is None:
            return None
        return x.data_ptr() if isinstance(x, torch.Tensor) else x.ctypes.data

    if c16 is None:
        _check(lib.pg_b200_gemm_fused_ex(dtype, m, n, k, ptr(a), lda, ptr(b), ldb, ptr(c), ldc, ptr(bias), act),
               "pg_gemm_fused_ex")
        return
    dt16 = {torch.float16: PG_DTYPE_F16, torch.bfloat16: PG_DTYPE_BF16}.get(c16.dtype)
    if dt16 is None:
        raise TypeError("c16 must be float16 or bfloat16")
    _check(lib.pg_b200_gemm_fused_out16(dtype, m, n, k, ptr(a), lda, ptr(b), ldb, ptr(c), ldc, ptr(bias), act,
                                        ptr(c16), ldc16 or n, dt16), "pg_gemm_fused_ex(out16)")


def pg_gemm_fused(m, n, k, a, lda, b, ldb, c, ldc, bias=None, act=PG_ACT_NONE):
    """pg_cpu_gemm_fused (backend/cpu/gemm.c:685-716), the f32 entry nn/nn.c:60,85 calls."""
    pg_gemm_fused_ex(PG_DTYPE_F32, m, n, k, a, lda, b, ldb, c, ldc, bias, act)


def pg_linear_forward(x, weight, bias=None, relu=False, out16=None):
    """pg_linear_forward / pg_linear_forward_relu (nn/nn.c:46-96) on device tensors:
    x [m, in] times weight [in, out] plus bias [out], optionally through ReLU, one kernel."""
    m, k = x.shape
    k2, n = weight.shape
    if k != k2 or x.dtype != weight.dtype:
        raise ValueError("pg_linear_forward: x [m,in] and weight [in,out] of one dtype")
    dt = {torch.float32: PG_DTYPE_F32, torch.float16: PG_DTYPE_F16, torch.bfloat16: PG_DTYPE_BF16}[x.dtype]
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    pg_gemm_fused_ex(dt, m, n, k, x.contiguous(), k, weight.contiguous(), n, out, n, bias,
                     PG_ACT_RELU if relu else PG_ACT_NONE, out16, n if out16 is not None else 0)
    return out


def pg_conv2d(x, w, b=None, stride=1, padding=0):
    """pg_conv2d (ops/conv.c:10-146): x [N,Cin,H,W], w [Cout,Cin,kh,kw], b [Cout] or None, f32 device tensors;
    returns [N,Cout,OH,OW].  Raises where picograd returns NULL."""
    _ready()
    if x.dim() != 4 or w.dim() != 4 or x.shape[1] != w.shape[1]:
        raise ValueError("pg_conv2d: x [N,Cin,H,W] and w [Cout,Cin,kh,kw]")
    if b is not None and (b.dim() != 1 or b.shape[0] != w.shape[0]):
        raise ValueError("pg_conv2d: bias [Cout]")
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise TypeError("pg_conv2d: float32")
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    if stride <= 0 or h + 2 * padding < kh or wd + 2 * padding < kw:
        raise ValueError("pg_conv2d: empty output")
    oh, ow = (h + 2 * padding - kh) // stride + 1, (wd + 2 * padding - kw) // stride + 1
    x, w = x.contiguous(), w.contiguous()
    out = torch.empty((n, cout, oh, ow), dtype=torch.float32, device=x.device)
    _check(lib.pg_b200_conv2d(n, cin, h, wd, cout, kh, kw, stride, padding, x.data_ptr(), w.data_ptr(),
                              b.contiguous().data_ptr() if b is not None else None, out.data_ptr()), "pg_conv2d")
    return out


def pg_attention_bmm(q, kt, v):
    """softmax-weighted product as picograd's callers chain it: pg_bmm(q, kt) -> pg_softmax(axis -1) ->
    cast to the operand dtype -> pg_bmm(., v) (ops/matmul.c:340-369, ops/activations.c:22-45), in one call.
    q [B,Sq,D], kt [B,D,Sk], v [B,Sk,D] f16/bf16 device tensors; returns f32 [B,Sq,D]."""
    _ready()
    if q.dim() != 3 or kt.dim() != 3 or v.dim() != 3:
        raise ValueError("pg_attention_bmm: 3-D operands")
    bt, sq, d = q.shape
    if kt.shape[0] != bt or kt.shape[1] != d or v.shape != (bt, kt.shape[2], d) or not (q.dtype == kt.dtype == v.dtype):
        raise ValueError("pg_attention_bmm: q [B,Sq,D], kt [B,D,Sk], v [B,Sk,D] of one dtype")
    dt = {torch.float16: PG_DTYPE_F16, torch.bfloat16: PG_DTYPE_BF16}.get(q.dtype)
    if dt is None:
        raise TypeError("pg_attention_bmm: float16 or bfloat16")
    q, kt, v = q.contiguous(), kt.contiguous(), v.contiguous()
    o = torch.empty((bt, sq, d), dtype=torch.float32, device=q.device)
    _check(lib.pg_b200_attention_bmm(dt, bt, sq, kt.shape[2], d, q.data_ptr(), kt.data_ptr(), v.data_ptr(), o.data_ptr()),
           "pg_attention_bmm")
    return o


def pg_gemm_ex_host(dtype, m, n, k, a, lda, b, ldb, c, ldc):
    """pg_gemm_ex with HOST buffers, the way ops/matmul.c:264-271 calls it: a, b, c are CPU
    tensors (pinned or pageable) or numpy arrays; staging copies happen inside the call."""
    _ready()

    def ptr(x):
        return x.data_ptr() if isinstance(x, torch.Tensor) else x.ctypes.data

    _check(lib.pg_b200_gemm_ex(dtype, m, n, k, ptr(a), lda, ptr(b), ldb, ptr(c), ldc), "pg_gemm_ex(host)")


def _gemm_batched(dta, dtb, ta, tb, batch, m, n, k, a, lda, sa, b, ldb, sb, c, ldc, sc, accumulate=False):
    _ready()
    _check(lib.pg_b200_gemm_batched(dta, dtb, int(ta), int(tb), batch, m, n, k, a.data_ptr(), lda, sa,
                                    b.data_ptr(), ldb, sb, c.data_ptr(), ldc, sc, int(accumulate)),
           "pg_b200_gemm_batched")


class _Tensor(C.Structure):
    """pg_b200_tensor (include/pg_b200.h): what picograd's callers read of a pg_tensor, with a device pointer."""
    _fields_ = [("dtype", C.c_int), ("ndim", C.c_size_t), ("shape", C.c_size_t * 8), ("stride", C.c_size_t * 8),
                ("data", C.c_void_p)]


def _desc(t, dtype=None):
    d = _Tensor()
    d.dtype = _code(t, dtype)
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    d.data = t.data_ptr()
    return d


def _result(shape_call, run_call, device):
    """Two steps through the C entries: the shape rules fill the result's shape (or refuse: None, as picograd
    returns NULL), the result is allocated as a torch tensor, then the call proper runs into it."""
    out = _Tensor()
    st = shape_call(C.byref(out))
    if st == PG_ERR_UNSUPPORTED:
        return None
    _check(st, "result shape")
    res = torch.empty([out.shape[i] for i in range(out.ndim)], dtype=torch.float32, device=device)
    out.data = res.data_ptr()
    if res.numel():
        _check(run_call(C.byref(out)), "matmul")
    return res


def _usable(*ts):
    return all(t is not None and isinstance(t, torch.Tensor) and 1 <= t.dim() <= 8 and t.is_cuda for t in ts)


def pg_matmul(a, b, dtype=None):
    """pg_matmul (ops/matmul.c:186-284): NumPy-style matmul with 1-D promotion; batch dims must be
    equal or one side unbatched; dtypes must match; last-dim stride must be 1; output float32.
    The shape rules run in the C library (pg_b200_matmul).  Returns None where picograd returns NULL."""
    if not _usable(a, b) or a.dtype != b.dtype:
        return None
    _ready()
    da, db = _desc(a, dtype), _desc(b, dtype)
    return _result(lambda o: lib.pg_b200_matmul_result_shape(C.byref(da), C.byref(db), o),
                   lambda o: lib.pg_b200_matmul(C.byref(da), C.byref(db), o), a.device)


def pg_bmm(a, b, dtype=None):
    """pg_bmm (ops/matmul.c:340-369): strict [B,M,K] x [B,K,N] -> float32 [B,M,N]."""
    if not _usable(a, b) or a.dim() != 3 or b.dim() != 3:
        return None
    if a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1] or a.dtype != b.dtype:
        return None
    _ready()
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty((a.shape[0], a.shape[1], b.shape[2]), dtype=torch.float32, device=a.device)
    da, db, do = _desc(a, dtype), _desc(b, dtype), _desc(out, PG_DTYPE_F32)
    st = lib.pg_b200_bmm(C.byref(da), C.byref(db), C.byref(do))
    if st == PG_ERR_UNSUPPORTED:
        return None
    _check(st, "pg_bmm")
    return out


def pg_addmm(inp, m1, m2, alpha=1.0, beta=1.0):
    """pg_addmm (ops/matmul.c:371-405): beta * inp + alpha * (m1 @ m2); m1 [m,k], m2 [k,n] of one dtype, inp f32
    broadcastable to [m,n].  Returns f32 [m,n], or None where picograd returns NULL."""
    _ready()
    if inp is None or m1 is None or m2 is None or m1.dim() != 2 or m2.dim() != 2:
        return None
    if m1.shape[1] != m2.shape[0] or m1.dtype != m2.dtype:
        return None
    m, k = m1.shape
    n = m2.shape[1]
    shape = [1] * (2 - inp.dim()) + list(inp.shape) if inp.dim() <= 2 else None
    if shape is None or shape[0] not in (1, m) or shape[1] not in (1, n) or inp.dtype != torch.float32:
        return None
    inp, m1, m2 = inp.contiguous(), m1.contiguous(), m2.contiguous()
    rs = 0 if shape[0] == 1 else shape[1]
    cs = 0 if shape[1] == 1 else 1
    out = torch.empty((m, n), dtype=torch.float32, device=m1.device)
    _check(lib.pg_b200_addmm(_TORCH2PG[m1.dtype], m, n, k, m1.data_ptr(), k, m2.data_ptr(), n, out.data_ptr(), n,
                             inp.data_ptr(), rs, cs, float(alpha), float(beta)), "pg_addmm")
    return out


def pg_gather_relayout(staging, full, shards, rows, width, n):
    """The re-layout after an all-gather of N-column shards (no counterpart in picograd, which is single-device):
    staging [shards][rows][width] f32 (shard g a contiguous row-major block) -> full [rows][n] row-major, columns
    [g*width, (g+1)*width) from shard g.  Device tensors."""
    _ready()
    if staging.dtype != torch.float32 or full.dtype != torch.float32:
        raise TypeError("pg_gather_relayout: float32")
    _check(lib.pg_b200_gather_relayout(staging.data_ptr(), full.data_ptr(), shards, rows, width, n, full.stride(0)),
           "pg_b200_gather_relayout")


def pg_gemm_ex_scatter(dtype, m, n, k, a, lda, b, ldb, dst_ptrs, ldc, col0):
    """The column shard C[:, col0:col0+n] = A * B written by the GEMM kernel itself into every full C in `dst_ptrs`
    (device addresses of row-major m x ldc f32 matrices: this device's and, mapped with PeerMatrix, the other
    devices').  No counterpart in picograd.  PgError(UNSUPPORTED) when the shard cannot go through TMA stores."""
    _ready()
    import ctypes
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[int(x) for x in dst_ptrs])
    _check(lib.pg_b200_gemm_ex_scatter(dtype, m, n, k, a.data_ptr(), lda, b.data_ptr(), ldb, arr, len(dst_ptrs), ldc, col0),
           "pg_b200_gemm_ex_scatter")


def _permute_copy(t, perm):
    """permute_copy (ops/matmul.c:21-42) with the library's own kernel: a new contiguous tensor whose dimension d
    is dimension perm[d] of t."""
    _ready()
    import ctypes
    t = t.contiguous()
    if list(perm) == list(range(t.dim())):
        return t
    nd = t.dim()
    out = torch.empty([t.shape[d] for d in perm], dtype=t.dtype, device=t.device)
    arr = ctypes.c_size_t * nd
    _check(lib.pg_b200_permute_copy(_TORCH2PG[t.dtype], nd, arr(*t.shape), arr(*perm), t.data_ptr(), out.data_ptr()),
           "pg_b200_permute_copy")
    return out


def pg_tensordot(a, b, axes_a, axes_b, dtype=None):
    """pg_tensordot (ops/matmul.c:407-490): contract axes_a of a with axes_b of b — permute to
    (free, contracted) x (contracted, free), reshape to 2-D, matmul, reshape back; all inside pg_b200_tensordot."""
    if not _usable(a, b) or a.dtype != b.dtype or len(axes_a) != len(axes_b):
        return None
    _ready()
    nd = len(axes_a)
    arr = C.c_size_t * max(nd, 1)
    try:
        xa, xb = arr(*axes_a), arr(*axes_b)
    except (TypeError, OverflowError):
        return None
    da, db = _desc(a, dtype), _desc(b, dtype)
    return _result(lambda o: lib.pg_b200_tensordot_result_shape(C.byref(da), C.byref(db), nd, xa, xb, o),
                   lambda o: lib.pg_b200_tensordot(C.byref(da), C.byref(db), nd, xa, xb, o), a.device)


def _zeros_f32(shape, device):
    """A zeroed f32 gradient (pg_backward zeroes them, autograd.c:2490-2492), filled by the library's kernel."""
    t = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    _check(lib.pg_b200_fill_f32(t.data_ptr(), 0.0, t.numel()), "pg_b200_fill_f32")
    return t


def pg_matmul_backward_act(a, b, g, act, act_input, need_a=True, need_b=True, want_pre=False, dtype=None):
    """bwd of an activation node (autograd/autograd.c:794-801 GELU, :557 ReLU) followed by bwd_matmul (:561-706) in
    one call: the gradient entering the products is g * act'(act_input).  a [m,k] (or [batch,m,k] with a shared
    b [k,n]), g and act_input float32 of the matmul output's shape.  Returns (ga, gb, g') with g' None unless
    want_pre; fresh gradients are overwritten (pg_backward would have zeroed them)."""
    _ready()
    a, b, g, act_input = a.contiguous(), b.contiguous(), g.contiguous(), act_input.contiguous()
    dt = _code(a, dtype)
    m, k = a.shape[-2], a.shape[-1]
    n = b.shape[-1]
    batch = 1
    for d in a.shape[:-2]:
        batch *= d
    ga = torch.empty(a.shape, dtype=torch.float32, device=a.device) if need_a else None
    gb = torch.empty(b.shape, dtype=torch.float32, device=a.device) if need_b else None
    pre = torch.empty(g.shape, dtype=torch.float32, device=a.device) if want_pre else None
    _check(lib.pg_b200_matmul_backward_act(dt, batch, m, n, k, a.data_ptr(), b.data_ptr(), int(b.dim() > 2), g.data_ptr(),
                                           int(act), act_input.data_ptr(), pre.data_ptr() if want_pre else None,
                                           ga.data_ptr() if need_a else None, gb.data_ptr() if need_b else None, 0),
           "pg_b200_matmul_backward_act")
    return ga, gb, pre


def pg_matmul_backward(a, b, g, need_a=True, need_b=True, ga=None, gb=None, dtype=None):
    """bwd_matmul (autograd/autograd.c:561-706): ga += g * B^T, gb += A^T * g with float32 g and float32
    gradients; a and b as pg_matmul takes them (1-D operands, batches, a batch-shared operand whose gradient sums
    over the batch), of one dtype; g has the shape of pg_matmul(a, b).  Gradient tensors are created when not
    passed in — pg_backward would have zeroed them (:2490-2492), so the products then overwrite instead of adding
    to zeros; gradients passed in are accumulated into, as in picograd.  Shape logic: pg_b200_matmul_backward_nd."""
    _ready()
    a, b, g = a.contiguous(), b.contiguous(), g.contiguous()
    fresh_a, fresh_b = need_a and ga is None, need_b and gb is None
    overwrite = (fresh_a or not need_a) and (fresh_b or not need_b)
    if fresh_a:
        ga = torch.empty(a.shape, dtype=torch.float32, device=a.device) if overwrite else _zeros_f32(a.shape, a.device)
    if fresh_b:
        gb = torch.empty(b.shape, dtype=torch.float32, device=a.device) if overwrite else _zeros_f32(b.shape, a.device)
    da, db = _desc(a, dtype), _desc(b, dtype)
    _check(lib.pg_b200_matmul_backward_nd(C.byref(da), C.byref(db), g.data_ptr(), ga.data_ptr() if need_a else None,
                                          gb.data_ptr() if need_b else None, 0 if overwrite else 1),
           "pg_b200_matmul_backward_nd")
    return ga, gb
