"""pg_b200_gemm_ex_static_scratch — the entry point for callers that must not allocate.

Some users of this library run where cudaMalloc is not an option (their own arena owns the free
HBM, or their loop may not take the allocator's lock).  For them one entry point keeps the split-K
slices in a fixed array inside the library.  This file checks, through the C-ABI, that it returns
what the regular pg_b200_gemm_ex returns and what the CPU oracle computes, twice in a row with
different inputs (the array keeps the previous call's contents, so a stale read would show on the
second call), that it refuses a product whose slices do not fit, and — in a fresh process that never
ran pg_b200_init — that free device memory is the same before and after a call once the first call
has loaded the library's code.  Collected last on purpose: a run that stops at the first failure
has by then run every other test.  It passes alone in a fresh process as well as after the others.
"""
import numpy as np
import pytest
import torch

import workloads as wl
from gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _both(lib, dtype, a_bits, b_bits, k_splits):
    m, k = a_bits.shape
    n = b_bits.shape[1]
    a, b = to_dev(a_bits, dtype), to_dev(b_bits, dtype)
    c_new = torch.full((m, n), 7.0, device="cuda")
    c_old = torch.full((m, n), 9.0, device="cuda")
    lib.pg_b200_set_stream(torch.cuda.current_stream().cuda_stream)
    st = lib.pg_b200_gemm_ex_static_scratch(dtype, m, n, k, a.data_ptr(), k, b.data_ptr(), n, c_new.data_ptr(), n,
                                            k_splits)
    assert st == 0, lib.pg_b200_last_error()
    st = lib.pg_b200_gemm_ex(dtype, m, n, k, a.data_ptr(), k, b.data_ptr(), n, c_old.data_ptr(), n)
    assert st == 0, lib.pg_b200_last_error()
    assert lib.pg_b200_sync() == 0
    return c_new.cpu().numpy(), c_old.cpu().numpy()


def test_static_scratch_matches_regular_entry_twice(oracle):
    from picograd_b200._lib import lib
    torch.cuda.set_device(0)
    # the very first use of the library in a fresh process may be this call: no pg_b200_init before it
    for call, (m, n, k, dtype, splits) in enumerate([(16, 4096, 4096, wl.F16, 0), (200, 328, 1096, wl.BF16, 3)]):
        a, b = (wl.config3(m, n, k) if dtype == wl.F16 else wl.config2(m, n, k))
        got, want = _both(lib, dtype, a, b, splits)
        assert wl.relerr(got, want) <= wl.tolerance(dtype, k), f"call {call}"
        # split-K only reorders the f32 sum over K: far tighter than the path tolerance
        assert wl.relerr(got, want) <= 1e-6, f"call {call}"
        # and against the CPU oracle on the same bytes
        assert wl.relerr(got, oracle.gemm_ex(dtype, a, b)) <= wl.tolerance(dtype, k), f"call {call} vs oracle"
    # same inputs again: identical bits (the slices are fully rewritten, nothing stale is read)
    a, b = wl.config2(200, 328, 1096)
    again, _ = _both(lib, wl.BF16, a, b, 3)
    assert np.array_equal(again, got)


def test_static_scratch_rejects_what_does_not_fit():
    from picograd_b200._lib import lib
    torch.cuda.set_device(0)
    m, n, k = 2048, 2048, 512            # 4 slices x 2048 x 2048 x 4 B = 64 MiB > 16 MiB
    a = torch.zeros(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(k, n, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(m, n, device="cuda")
    st = lib.pg_b200_gemm_ex_static_scratch(wl.BF16, m, n, k, a.data_ptr(), k, b.data_ptr(), n, c.data_ptr(), n, 4)
    assert st == -1
    msg = lib.pg_b200_last_error().decode()
    assert "static array holds" in msg and "67108864" in msg
    # unaligned leading dimension: refused, not silently rerouted
    st = lib.pg_b200_gemm_ex_static_scratch(wl.BF16, 64, 64, 512, a.data_ptr(), 513, b.data_ptr(), 64, c.data_ptr(), 64, 2)
    assert st == -1


_FRESH = r"""
import ctypes, sys
import numpy as np, torch
sys.path[:0] = [{root!r}, {tests!r}]
import workloads as wl
from gpu_util import to_dev
from picograd_b200._lib import lib            # loads the .so; pg_b200_init is never called in this process
torch.cuda.set_device(0)
a_bits, b_bits = wl.config2(200, 328, 1096)
a, b = to_dev(a_bits, wl.BF16), to_dev(b_bits, wl.BF16)
c = torch.zeros(200, 328, device="cuda")
torch.cuda.synchronize()
lib.pg_b200_set_stream(None)
def call():
    st = lib.pg_b200_gemm_ex_static_scratch(wl.BF16, 200, 328, 1096, a.data_ptr(), 1096, b.data_ptr(), 328, c.data_ptr(), 328, 3)
    assert st == 0, lib.pg_b200_last_error()
free0 = torch.cuda.mem_get_info()[0]
call()                                        # first call on the device: the driver loads the kernels and the array
free1 = torch.cuda.mem_get_info()[0]
call()
free2 = torch.cuda.mem_get_info()[0]
call()
free3 = torch.cuda.mem_get_info()[0]
np.save({out!r}, c.cpu().numpy())
print("FREE", free0, free1, free2, free3)
"""


def test_fresh_process_without_init_allocates_nothing_after_the_first_call(oracle, tmp_path):
    """cudaMemGetInfo around calls in a process whose first use of the library is this entry point: the first call
    makes the driver load the library's kernels and the static array (a one-time reservation, reported, not
    asserted); the calls after it leave free memory exactly where it was."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "c.npy")
    code = _FRESH.format(root=root, tests=os.path.join(root, "tests"), out=out)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    free = [int(x) for x in r.stdout.split("FREE")[1].split()]
    print(f"free bytes: before {free[0]}, after first call {free[1]} (one-time load: {free[0] - free[1]}), "
          f"after second {free[2]}, after third {free[3]}")
    assert free[1] == free[2] == free[3]
    a, b = wl.config2(200, 328, 1096)
    assert wl.relerr(np.load(out), oracle.gemm_ex(wl.BF16, a, b)) <= wl.tolerance(wl.BF16, 1096)
