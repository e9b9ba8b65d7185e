"""The C-ABI entries beyond picograd's vtable called from plain C (tests/c/cabi_extras.c, built by
picograd_b200/host/Makefile): fused bias/activation GEMM with device and with host pointers, pg_conv2d, and the
attention-shaped chain, each against loops written from picograd's definitions."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_caller_of_the_extra_entries():
    exe = os.path.join(ROOT, "picograd_b200", "lib", "cabi_extras")
    lib = os.path.join(ROOT, "picograd_b200", "lib", "libpg_b200.so")
    assert os.path.exists(exe) and os.path.exists(lib), "run __graft_entry__.build() first"
    r = subprocess.run([exe, lib], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout
