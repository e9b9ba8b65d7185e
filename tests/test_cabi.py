"""The C-ABI library loads on a machine without a GPU and exports what include/pg_b200.h declares."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pg_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pg_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_vtable_entries():
    names = declared_symbols()
    for want in ("pg_b200_init", "pg_b200_malloc", "pg_b200_free", "pg_b200_copy_h2d", "pg_b200_copy_d2h",
                 "pg_b200_sync", "pg_b200_gemm", "pg_b200_hgemm", "pg_b200_bgemm", "pg_b200_gemm_ex"):
        assert want in names


def test_library_exports_every_declared_symbol():
    from picograd_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/pg_b200.h but not exported"
    assert set(_lib.SIGNATURES) == set(declared_symbols()), "Python signatures out of step with the header"


def test_no_cpu_fallback_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from picograd_b200 import _lib
    assert _lib.lib.pg_b200_init() == -1           # PG_ERR_UNSUPPORTED, like cuda.c:85-92 without a driver
    assert _lib.lib.pg_b200_malloc(16) is None
    assert _lib.lib.pg_b200_gemm_ex(2, 4, 4, 4, None, 4, None, 4, None, 4) != 0
    assert _lib.lib.pg_b200_last_error() != b""


def test_missing_library_fails_loudly(tmp_path):
    from picograd_b200 import _lib
    with pytest.raises(ImportError):
        _lib.load(str(tmp_path / "libpg_b200.so"))


def test_product_does_not_touch_the_oracle():
    """Nothing under picograd_b200/ or include/ may reference oracle/."""
    bad = []
    for base in ("picograd_b200", "include"):
        for dp, _, files in os.walk(os.path.join(ROOT, base)):
            if "/lib" in dp:
                continue
            for f in files:
                if f.endswith((".py", ".cu", ".h", ".c", ".cuh")):
                    text = open(os.path.join(dp, f), errors="replace").read()
                    if "pg_oracle" in text or "liboracle" in text or "oracle_lib" in text:
                        bad.append(os.path.join(dp, f))
    assert not bad, bad
