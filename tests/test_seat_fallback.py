"""Host-side failure forms of the CUDA seat (picograd_b200/host/cuda_backend.c), without a GPU fault: the device
library is replaced by small fakes, or is the real one on a machine where its init cannot succeed, and picograd's
own dispatcher — compiled from picograd's sources with our seat in place of its src/backend/cuda/*.c
(oracle/_ref/libpicograd_dropin.so, built where those sources are present) — must behave as picograd's does when
its CUDA backend is unavailable: pg_set_device(PG_DEV_CUDA) returns the failing status and leaves the device on the
CPU (backend/backend.c:76-90), and pg_gemm keeps working there.  Each case is its own process: the seat caches its
first init result, as picograd's does (backend/cuda/cuda.c:32-33)."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "libpicograd_dropin.so")

CHILD = textwrap.dedent("""
    import ctypes, sys
    import numpy as np
    L = ctypes.CDLL(sys.argv[1])
    L.pg_set_device.argtypes = [ctypes.c_int]
    st = L.pg_set_device(1)                      # PG_DEV_CUDA
    dev = L.pg_get_device()
    sz = ctypes.c_size_t
    L.pg_gemm.argtypes = [sz, sz, sz, ctypes.c_void_p, sz, ctypes.c_void_p, sz, ctypes.c_void_p, sz]
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(8, dtype=np.float32).reshape(4, 2)
    c = np.zeros((3, 2), np.float32)
    L.pg_gemm(3, 2, 4, a.ctypes.data, 4, b.ctypes.data, 2, c.ctypes.data, 2)
    print("RESULT", st, dev, int(np.array_equal(c, a @ b)))
""")

FAKE_NO_SYMBOLS = "int pg_b200_init(void) { return 0; }\n"            # lacks every other entry the seat binds
FAKE_INIT_FAILS = textwrap.dedent("""
    #include <stddef.h>
    #include <stdint.h>
    int pg_b200_init(void) { return %d; }
    void *pg_b200_malloc(size_t n) { (void)n; return 0; }
    void pg_b200_free(void *p) { (void)p; }
    int pg_b200_copy_h2d(void *d, const void *s, size_t n) { (void)d; (void)s; (void)n; return -3; }
    int pg_b200_copy_d2h(void *d, const void *s, size_t n) { (void)d; (void)s; (void)n; return -3; }
    int pg_b200_sync(void) { return -4; }
    void pg_b200_gemm(size_t m, size_t n, size_t k, const float *a, size_t lda, const float *b, size_t ldb, float *c, size_t ldc)
    { (void)m; (void)n; (void)k; (void)a; (void)lda; (void)b; (void)ldb; (void)c; (void)ldc; }
    void pg_b200_hgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb, float *c, size_t ldc)
    { (void)m; (void)n; (void)k; (void)a; (void)lda; (void)b; (void)ldb; (void)c; (void)ldc; }
    void pg_b200_bgemm(size_t m, size_t n, size_t k, const uint16_t *a, size_t lda, const uint16_t *b, size_t ldb, float *c, size_t ldc)
    { (void)m; (void)n; (void)k; (void)a; (void)lda; (void)b; (void)ldb; (void)c; (void)ldc; }
    int pg_b200_gemm_ex(int dt, size_t m, size_t n, size_t k, const void *a, size_t lda, const void *b, size_t ldb, float *c, size_t ldc)
    { (void)dt; (void)m; (void)n; (void)k; (void)a; (void)lda; (void)b; (void)ldb; (void)c; (void)ldc; return -1; }
    const char *pg_b200_last_error(void) { return "fake device library: init fails on purpose"; }
""")


def _run(env_lib):
    env = dict(os.environ)
    env["PG_B200_LIB"] = env_lib
    r = subprocess.run([sys.executable, "-c", CHILD, DROPIN], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    st, dev, ok = (int(x) for x in r.stdout.split("RESULT")[1].split())
    return st, dev, ok


def _build(tmp_path, name, source):
    src = tmp_path / (name + ".c")
    src.write_text(source)
    out = tmp_path / (name + ".so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-o", str(out), str(src)])
    return str(out)


@pytest.fixture(autouse=True)
def _needs_the_dropin_build():
    if not os.path.exists(DROPIN):
        pytest.skip("oracle/_ref/libpicograd_dropin.so not built on this machine (needs picograd's sources)")


def test_real_library_without_a_gpu_leaves_the_device_on_cpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the real library's init succeeds")
    st, dev, ok = _run(os.path.join(ROOT, "picograd_b200", "lib", "libpg_b200.so"))
    assert st == -1 and dev == 0 and ok == 1            # PG_ERR_UNSUPPORTED, PG_DEV_CPU, CPU product correct


def test_library_that_lacks_an_entry_is_refused(tmp_path):
    st, dev, ok = _run(_build(tmp_path, "fake_nosym", FAKE_NO_SYMBOLS))
    assert st == -1 and dev == 0 and ok == 1


@pytest.mark.parametrize("status", [-1, -2, -5], ids=["unsupported", "alloc", "gemm"])
def test_failing_init_status_is_passed_on_and_cpu_stays(tmp_path, status):
    st, dev, ok = _run(_build(tmp_path, "fake_init", FAKE_INIT_FAILS % status))
    assert st == status and dev == 0 and ok == 1
