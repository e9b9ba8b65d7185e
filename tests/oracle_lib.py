"""ctypes bindings of the CPU checkers (test infrastructure only).

`oracle()` loads oracle/liboracle.so, our C restatement of picograd's CPU GEMM
path.  `reference()` loads oracle/_ref/libpicograd_ref.so, the unmodified
picograd library compiled from its own sources, when that build exists
(it is git-ignored and built by `make -C oracle ref`).
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32, F16, BF16 = 0, 1, 2
_sz = C.c_size_t
_vp = C.c_void_p


def _ptr(a):
    return a.ctypes.data_as(_vp)


class Oracle:
    def __init__(self, path):
        L = C.CDLL(path)
        self.L = L
        L.pgo_gemm_ex.argtypes = [C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]
        L.pgo_gemm_ex_panel.argtypes = L.pgo_gemm_ex.argtypes + [_sz] * 4
        L.pgo_gemm_fused_ex.argtypes = L.pgo_gemm_ex.argtypes + [_vp, C.c_int]
        L.pgo_bmm.argtypes = [C.c_int, _sz, _sz, _sz, _sz, _vp, _vp, _vp]
        L.pgo_matmul_backward.argtypes = [C.c_int, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp]
        L.pgo_softmax_rows.argtypes = [_vp, _vp, _sz, _sz]
        L.pgo_addmm.argtypes = [C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _sz, C.c_float, C.c_float]
        L.pgo_conv2d.argtypes = [_sz] * 7 + [C.c_int, C.c_int, _vp, _vp, _vp, _vp]
        L.pgo_gelu.argtypes = [_vp, _vp, _sz]
        L.pgo_gelu_grad.argtypes = [_vp, _vp, _vp, _sz]
        for n in ("pgo_f32_to_bf16_n", "pgo_f32_to_f16_n", "pgo_bf16_to_f32_n", "pgo_f16_to_f32_n"):
            getattr(L, n).argtypes = [_vp, _vp, _sz]
        L.pgo_num_threads.restype = C.c_int

    def threads(self):
        return int(self.L.pgo_num_threads())

    def gemm_ex(self, dtype, a, b, m=None, n=None, k=None, lda=None, ldb=None, ldc=None, c=None):
        """a: [m,lda-ish] array (f32 or uint16), b likewise; returns f32 C [m,ldc]."""
        m = a.shape[0] if m is None else m
        k = a.shape[1] if k is None else k
        n = b.shape[1] if n is None else n
        lda = a.strides[0] // a.itemsize if lda is None else lda
        ldb = b.strides[0] // b.itemsize if ldb is None else ldb
        if c is None:
            ldc = n if ldc is None else ldc
            c = np.zeros((m, ldc), np.float32)
        else:
            ldc = c.strides[0] // 4
        self.L.pgo_gemm_ex(dtype, m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), ldc)
        return c

    def gemm_fused_ex(self, dtype, a, b, bias=None, act=0):
        """C = act(bias + a @ b), picograd's pg_cpu_gemm_fused_ex; bias f32 [n] or None."""
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32)
        self.L.pgo_gemm_fused_ex(dtype, m, n, k, _ptr(a), max(a.strides[0] // a.itemsize, 1), _ptr(b),
                                 b.strides[0] // b.itemsize, _ptr(c), n,
                                 _ptr(bias) if bias is not None else None, act)
        return c

    def gemm_ex_panel(self, dtype, a, b, r0, r1, c0, c1):
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32) if m * n <= (1 << 24) else None
        if c is None:
            # compute into a compact panel buffer by offsetting the C pointer
            pan = np.zeros((r1 - r0, c1 - c0), np.float32)
            ldc = c1 - c0
            base = pan.ctypes.data - (r0 * ldc + c0) * 4
            self.L.pgo_gemm_ex_panel(dtype, m, n, k, _ptr(a), a.strides[0] // a.itemsize,
                                     _ptr(b), b.strides[0] // b.itemsize,
                                     _vp(base), ldc, r0, r1, c0, c1)
            return pan
        self.L.pgo_gemm_ex_panel(dtype, m, n, k, _ptr(a), a.strides[0] // a.itemsize,
                                 _ptr(b), b.strides[0] // b.itemsize, _ptr(c), n, r0, r1, c0, c1)
        return c[r0:r1, c0:c1].copy()

    def bmm(self, dtype, a, b):
        bt, m, k = a.shape
        n = b.shape[2]
        c = np.zeros((bt, m, n), np.float32)
        self.L.pgo_bmm(dtype, bt, m, n, k, _ptr(a), _ptr(b), _ptr(c))
        return c

    def matmul_backward(self, dtype, a, b, g, want_a=True, want_b=True):
        m, k = a.shape
        n = b.shape[1]
        ga = np.zeros((m, k), np.float32) if want_a else None
        gb = np.zeros((k, n), np.float32) if want_b else None
        self.L.pgo_matmul_backward(dtype, m, n, k, _ptr(a), _ptr(b), _ptr(g),
                                   _ptr(ga) if want_a else None, _ptr(gb) if want_b else None)
        return ga, gb

    def addmm(self, dtype, inp, a, b, alpha, beta):
        """pg_addmm: beta * inp + alpha * (a @ b); inp f32 of shape [m,n], [1,n], [n], [m,1] or [1,1]."""
        m, k = a.shape
        n = b.shape[1]
        inp2 = np.ascontiguousarray(inp, np.float32).reshape((1,) * (2 - inp.ndim) + inp.shape) if inp.ndim < 2 else np.ascontiguousarray(inp, np.float32)
        rs = 0 if inp2.shape[0] == 1 else inp2.shape[1]
        cs = 0 if inp2.shape[1] == 1 else 1
        c = np.zeros((m, n), np.float32)
        self.L.pgo_addmm(dtype, m, n, k, _ptr(a), a.strides[0] // a.itemsize, _ptr(b), b.strides[0] // b.itemsize, _ptr(c), n,
                         _ptr(inp2), rs, cs, alpha, beta)
        return c

    def conv2d(self, x, w, bias=None, stride=1, padding=0):
        """pg_conv2d: x [N,Cin,H,W], w [Cout,Cin,kh,kw] f32 -> [N,Cout,OH,OW]."""
        n, cin, h, wd = x.shape
        cout, _, kh, kw = w.shape
        oh, ow = (h + 2 * padding - kh) // stride + 1, (wd + 2 * padding - kw) // stride + 1
        out = np.empty((n, cout, oh, ow), np.float32)
        st = self.L.pgo_conv2d(n, cin, h, wd, cout, kh, kw, stride, padding, _ptr(x), _ptr(w),
                               _ptr(bias) if bias is not None else None, _ptr(out))
        assert st == 0
        return out

    def softmax_rows(self, x):
        out = np.empty_like(x)
        self.L.pgo_softmax_rows(_ptr(out), _ptr(x), x.size // x.shape[-1], x.shape[-1])
        return out

    def gelu(self, x):
        out = np.empty_like(x)
        self.L.pgo_gelu(_ptr(out), _ptr(x), x.size)
        return out

    def gelu_grad(self, x, gy):
        out = np.empty_like(x)
        self.L.pgo_gelu_grad(_ptr(out), _ptr(x), _ptr(gy), x.size)
        return out

    def to_bf16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.L.pgo_f32_to_bf16_n(_ptr(out), _ptr(x), x.size)
        return out

    def to_f16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.L.pgo_f32_to_f16_n(_ptr(out), _ptr(x), x.size)
        return out

    def from_bf16(self, x):
        out = np.empty(x.shape, np.float32)
        self.L.pgo_bf16_to_f32_n(_ptr(out), _ptr(x), x.size)
        return out

    def from_f16(self, x):
        out = np.empty(x.shape, np.float32)
        self.L.pgo_f16_to_f32_n(_ptr(out), _ptr(x), x.size)
        return out


class _PgTensor(C.Structure):
    """Head of picograd's pg_tensor (core/tensor.h:21-36), enough to reach the data pointer."""
    _fields_ = [("ndim", _sz), ("shape", _sz * 8), ("stride", _sz * 8), ("numel", _sz), ("data", _vp)]


class _ConvCfg(C.Structure):
    _fields_ = [("stride", C.c_int), ("padding", C.c_int)]       # ops/conv.h:7-10


class Reference:
    """The unmodified picograd CPU library (backend/backend.h:103-136)."""

    def __init__(self, path):
        L = C.CDLL(path)
        self.L = L
        L.pg_gemm.argtypes = [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]
        L.pg_gemm_ex.argtypes = [C.c_int, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]
        L.pg_thread_pool_size.restype = C.c_int
        L.pg_cpu_gemm_fused.argtypes = L.pg_gemm.argtypes + [_vp, C.c_int]
        L.pg_cpu_gemm_fused_ex.argtypes = L.pg_gemm_ex.argtypes + [_vp, C.c_int]

    def threads(self):
        return int(self.L.pg_thread_pool_size())

    def gemm_fused_ex(self, dtype, a, b, bias=None, act=0, plain_f32_entry=False):
        """backend/cpu/gemm.c:685-817; plain_f32_entry calls pg_cpu_gemm_fused (what nn/nn.c:60 uses)."""
        m, k = a.shape
        n = b.shape[1]
        c = np.full((m, n), np.nan, np.float32)
        lda, ldb = max(a.strides[0] // a.itemsize, 1), b.strides[0] // b.itemsize
        bp = _ptr(bias) if bias is not None else None
        if plain_f32_entry:
            assert dtype == F32
            self.L.pg_cpu_gemm_fused(m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), n, bp, act)
        else:
            self.L.pg_cpu_gemm_fused_ex(dtype, m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), n, bp, act)
        return c

    def addmm(self, inp, a, b, alpha, beta):
        """pg_addmm (ops/matmul.c:371-405) on picograd's own f32 tensors."""
        L = self.L
        L.pg_tensor_from_data.restype = C.POINTER(_PgTensor)
        L.pg_tensor_from_data.argtypes = [_sz, C.POINTER(_sz), _vp]
        L.pg_addmm.restype = C.POINTER(_PgTensor)
        L.pg_addmm.argtypes = [C.POINTER(_PgTensor)] * 3 + [C.c_float, C.c_float]
        L.pg_tensor_free.argtypes = [C.POINTER(_PgTensor)]

        def mk(x):
            x = np.ascontiguousarray(x, np.float32)
            return L.pg_tensor_from_data(x.ndim, (_sz * x.ndim)(*x.shape), _ptr(x))

        ti, ta, tb = mk(inp), mk(a), mk(b)
        y = L.pg_addmm(ti, ta, tb, alpha, beta)
        assert y, "pg_addmm returned NULL"
        t = y.contents
        out = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_float)), shape=(t.numel,)).reshape(t.shape[0], t.shape[1]).copy()
        for h in (y, ti, ta, tb):
            L.pg_tensor_free(h)
        return out

    def conv2d(self, x, w, bias=None, stride=1, padding=0):
        """pg_conv2d (ops/conv.c:10-146) on picograd's own tensors."""
        L = self.L
        L.pg_tensor_from_data.restype = C.POINTER(_PgTensor)
        L.pg_tensor_from_data.argtypes = [_sz, C.POINTER(_sz), _vp]
        L.pg_conv2d.restype = C.POINTER(_PgTensor)
        L.pg_conv2d.argtypes = [C.POINTER(_PgTensor)] * 3 + [_ConvCfg]
        L.pg_tensor_free.argtypes = [C.POINTER(_PgTensor)]

        def mk(a):
            a = np.ascontiguousarray(a, np.float32)
            return L.pg_tensor_from_data(a.ndim, (_sz * a.ndim)(*a.shape), _ptr(a))

        tx, tw = mk(x), mk(w)
        tb = mk(bias) if bias is not None else None
        y = L.pg_conv2d(tx, tw, tb, _ConvCfg(stride, padding))
        assert y, "pg_conv2d returned NULL"
        t = y.contents
        shape = tuple(t.shape[i] for i in range(t.ndim))
        out = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_float)), shape=(t.numel,)).reshape(shape).copy()
        for h in (y, tx, tw) + ((tb,) if tb is not None else ()):
            L.pg_tensor_free(h)
        return out

    def gemm_ex(self, dtype, a, b, c=None):
        m, k = a.shape
        n = b.shape[1]
        if c is None:
            c = np.zeros((m, n), np.float32)
        lda, ldb, ldc = a.strides[0] // a.itemsize, b.strides[0] // b.itemsize, c.strides[0] // 4
        if dtype == F32:
            self.L.pg_gemm(m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), ldc)
        else:
            self.L.pg_gemm_ex(dtype, m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), ldc)
        return c


_ORACLE = None
_REF = None


def oracle_path():
    return os.path.join(ROOT, "oracle", "liboracle.so")


def reference_path():
    return os.path.join(ROOT, "oracle", "_ref", "libpicograd_ref.so")


def oracle():
    global _ORACLE
    if _ORACLE is None:
        _ORACLE = Oracle(oracle_path())
    return _ORACLE


def reference():
    """None when oracle/_ref has not been built on this machine."""
    global _REF
    if _REF is None and os.path.exists(reference_path()):
        _REF = Reference(reference_path())
    return _REF
