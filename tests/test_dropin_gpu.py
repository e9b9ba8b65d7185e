"""picograd's own binaries, linked against picograd's objects + OUR CUDA seat, on a B200.

oracle/Makefile `dropin` builds them where picograd's sources are present; the binaries travel with
the repository (oracle/_ref is git-ignored).  Where they are absent the tests skip.
  test_backend     picograd's tests/test_backend.c, unmodified
  bench_gemm_cuda  picograd's benchmarks/bench_gemm_cuda.c, unmodified (its correctness line)
  dropin_callers   tests/c/dropin_callers.c: picograd's pg_matmul / pg_bmm / pg_tensordot, CPU vs CUDA device
"""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _run(name, timeout=300):
    exe = os.path.join(REF, name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built on this machine")
    env = dict(os.environ, PG_CUDA_DEBUG="1")
    return subprocess.run([exe], capture_output=True, text=True, timeout=timeout, env=env)


def test_picograd_test_backend_passes_with_our_seat():
    r = _run("test_backend")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout
    assert "cuda not available" not in r.stdout, "the seat did not come up on a GPU box"
    assert "init ok (B200 tensor-core GEMM)" in r.stderr


def test_picograd_bench_gemm_cuda_correctness_line():
    r = _run("bench_gemm_cuda")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "max abs err 0" in r.stdout          # docs/gpu-plan.md:62: exact on dyadic data


def test_picograd_callers_cpu_vs_cuda_device():
    r = _run("dropin_callers")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout
