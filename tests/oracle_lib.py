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

    def matmul_backward_nd(self, dtype, a, b, g):
        """bwd_matmul with picograd's shape modes (autograd/autograd.c:591-706): a 1-D operand is a row / column
        vector, batch dimensions are looped over, and a B shared by the batch sums its gradient over the batch.
        g has the shape of the matmul's output.  Returns gradients with the shapes of a and b."""
        av, bv = a.ndim == 1, b.ndim == 1
        a2 = a.reshape(1, -1) if av else a
        b2 = b.reshape(-1, 1) if bv else b
        m, k = a2.shape[-2:]
        n = b2.shape[-1]
        abat, bbat = a2.ndim > 2, b2.ndim > 2
        nbatch = int(np.prod(a2.shape[:-2])) if abat else (int(np.prod(b2.shape[:-2])) if bbat else 1)
        a3 = a2.reshape(nbatch if abat else 1, m, k)
        b3 = b2.reshape(nbatch if bbat else 1, k, n)
        g3 = np.ascontiguousarray(g, np.float32).reshape(nbatch, m, n)
        ga = np.zeros(a3.shape, np.float32)
        gb = np.zeros(b3.shape, np.float32)
        for s in range(nbatch):
            x, y = self.matmul_backward(dtype, np.ascontiguousarray(a3[s if abat else 0]),
                                        np.ascontiguousarray(b3[s if bbat else 0]), g3[s])
            ga[s if abat else 0] += x
            gb[s if bbat else 0] += y
        return ga.reshape(a.shape), gb.reshape(b.shape)

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


class _PgTensorFull(C.Structure):
    """All of pg_tensor (core/tensor.h:21-36): needed to read the dtype of a value."""
    _fields_ = [("ndim", _sz), ("shape", _sz * 8), ("stride", _sz * 8), ("numel", _sz), ("data", _vp),
                ("data_ref", _vp), ("is_view", C.c_bool), ("view_parent", _vp), ("dtype", C.c_int), ("elem_size", _sz)]


class _PgNode(C.Structure):
    """pg_node (autograd/autograd.h:51-62); public in picograd, so that a 16-bit leaf can be built by hand."""
    _fields_ = [("value", C.POINTER(_PgTensorFull)), ("grad", C.POINTER(_PgTensorFull)), ("nparents", _sz),
                ("parents", _vp), ("ctx", _vp), ("backward", _vp), ("ag_op", C.c_int), ("requires_grad", C.c_bool),
                ("refs", C.c_uint), ("mark", C.c_ubyte)]


def _tensor_to_numpy(tp):
    """f32 pg_tensor* -> numpy copy with the tensor's shape."""
    t = tp.contents
    shape = tuple(t.shape[i] for i in range(t.ndim))
    return np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_float)), shape=(t.numel,)).reshape(shape).copy()


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

    # ---- autograd (autograd/autograd.h:64-66, :113, :117, :155) -------------------------------
    def _ag_bind(self):
        L = self.L
        NP, TP, SP = C.POINTER(_PgNode), C.POINTER(_PgTensorFull), C.POINTER(_sz)
        L.pg_var_from_data.restype = NP
        L.pg_var_from_data.argtypes = [_sz, SP, _vp, C.c_bool]
        L.pg_var_uniform.restype = NP
        L.pg_var_uniform.argtypes = [_sz, SP, C.c_float, C.c_float, C.c_bool]
        for name in ("pg_ag_matmul", "pg_ag_mul", "pg_ag_add"):
            getattr(L, name).restype = NP
            getattr(L, name).argtypes = [NP, NP]
        for name in ("pg_ag_sum_all", "pg_ag_mean_all", "pg_ag_sigmoid"):
            getattr(L, name).restype = NP
            getattr(L, name).argtypes = [NP]
        L.pg_backward.argtypes = [NP]
        L.pg_backward.restype = None
        L.pg_node_free.argtypes = [NP]
        L.pg_node_free.restype = None
        L.pg_tensor_from_data_dtype.restype = TP
        L.pg_tensor_from_data_dtype.argtypes = [C.c_int, _sz, SP, _vp]
        L.pg_tensor_free.argtypes = [_vp]
        L.pg_tensor_free.restype = None
        L.pg_seed.argtypes = [C.c_ulonglong]
        L.pg_autograd_set_jit.argtypes = [C.c_bool]
        return L

    def _leaf(self, dtype, arr, requires_grad=True):
        """A leaf node holding `arr` (f32 values, or uint16 bit patterns of f16/bf16).  A 16-bit leaf is an
        f32 leaf whose value tensor is swapped for one of the 16-bit dtype, as autograd.c:566-590 expects."""
        L = self.L
        arr = np.ascontiguousarray(arr)
        shape = (_sz * arr.ndim)(*arr.shape)
        if dtype == F32:
            arr = np.ascontiguousarray(arr, np.float32)
            node = L.pg_var_from_data(arr.ndim, shape, _ptr(arr), requires_grad)
            assert node
            return node
        zeros = np.zeros(arr.shape, np.float32)
        node = L.pg_var_from_data(arr.ndim, shape, _ptr(zeros), requires_grad)
        assert node and arr.dtype == np.uint16
        t16 = L.pg_tensor_from_data_dtype(dtype, arr.ndim, shape, _ptr(arr))
        assert t16 and t16.contents.dtype == dtype
        L.pg_tensor_free(C.cast(node.contents.value, _vp))
        node.contents.value = t16
        return node

    def matmul_backward(self, dtype, a, b, upstream=None, jit=True):
        """pg_ag_matmul(a, b) followed by pg_backward of loss = sum(y * upstream) (loss = sum(y) when upstream
        is None, the form of picograd's tests/test_autograd.c:281-286).  Returns (y, grad a, grad b)."""
        L = self._ag_bind()
        L.pg_autograd_set_jit(bool(jit))
        A, B = self._leaf(dtype, a), self._leaf(dtype, b)
        y = L.pg_ag_matmul(A, B)
        assert y, "pg_ag_matmul returned NULL"
        nodes = [A, B, y]
        top = y
        if upstream is not None:
            w = self._leaf(F32, np.ascontiguousarray(upstream, np.float32), requires_grad=False)
            top = L.pg_ag_mul(y, w)
            assert top, "pg_ag_mul returned NULL"
            nodes += [w, top]
        loss = L.pg_ag_sum_all(top)
        assert loss
        nodes.append(loss)
        L.pg_backward(loss)
        out = (_tensor_to_numpy(y.contents.value), _tensor_to_numpy(A.contents.grad), _tensor_to_numpy(B.contents.grad))
        for n in reversed(nodes):
            L.pg_node_free(n)
        L.pg_autograd_set_jit(True)
        return out

    def uniform(self, seed, shapes, lo=-1.0, hi=1.0):
        """pg_seed(seed) then one pg_var_uniform per shape, as picograd's tests draw their leaves
        (tests/test_autograd.c:319-330); returns the drawn f32 arrays."""
        L = self._ag_bind()
        L.pg_seed(seed)
        out = []
        for shp in shapes:
            n = L.pg_var_uniform(len(shp), (_sz * len(shp))(*shp), lo, hi, True)
            assert n
            out.append(_tensor_to_numpy(n.contents.value))
            L.pg_node_free(n)
        return out

    def mlp_backward(self, x, w1, b1, w2, b2):
        """The two-layer network of picograd's tests/test_autograd.c:393-421: mean(sigmoid(x w1 + b1) w2 + b2),
        pg_backward.  Returns the values and gradients around both matmul nodes."""
        L = self._ag_bind()
        X, W1, B1, W2, B2 = (self._leaf(F32, t) for t in (x, w1, b1, w2, b2))
        mm1 = L.pg_ag_matmul(X, W1)
        z1 = L.pg_ag_add(mm1, B1)
        h = L.pg_ag_sigmoid(z1)
        mm2 = L.pg_ag_matmul(h, W2)
        y = L.pg_ag_add(mm2, B2)
        loss = L.pg_ag_mean_all(y)
        assert mm1 and z1 and h and mm2 and y and loss
        L.pg_backward(loss)
        val = lambda n: _tensor_to_numpy(n.contents.value)
        grd = lambda n: _tensor_to_numpy(n.contents.grad)
        out = {"h": val(h), "g_mm1": grd(mm1), "g_mm2": grd(mm2), "g_x": grd(X), "g_w1": grd(W1), "g_h": grd(h),
               "g_w2": grd(W2)}
        for n in (loss, y, mm2, h, z1, mm1, B2, W2, B1, W1, X):
            L.pg_node_free(n)
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
