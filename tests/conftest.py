import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib
    if not os.path.exists(oracle_lib.oracle_path()):
        import subprocess
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"])
    return oracle_lib.oracle()


@pytest.fixture(scope="session")
def reference():
    """The compiled unmodified picograd library, or None when oracle/_ref was not built here."""
    import oracle_lib
    return oracle_lib.reference()


@pytest.fixture(scope="session")
def pg():
    """The product's Python mirror, bound to cuda:0; fails loudly if the CUDA library is missing."""
    import torch
    assert torch.cuda.is_available(), "a -m gpu test needs a GPU"
    import picograd_b200 as pg
    pg.pg_set_device(0)
    return pg


@pytest.fixture(autouse=True)
def _reset_options(request):
    yield
    if "gpu" in request.keywords:
        import picograd_b200 as pg
        for name, val in (("path", 0), ("tile_config", -1), ("epilogue", -1), ("k_splits", 0),
                          ("f32_parts", 2), ("f32_tensor_cores", 0), ("host_pipeline", 1), ("stages", 0), ("debug", 0), ("fused_splitk", 1), ("swap_skinny", 1), ("stream_k", 0), ("pdl", 1), ("small_f32_pipe", 1), ("big_f32_pipe", 1), ("f32_retranspose", 1), ("big_f32_min_ctas", 140), ("die_aware", 1), ("serpentine", 1), ("k_serpentine", 1), ("f32_chunk", 512), ("fused_attention", 1), ("attn_q_tmem", 1)):
            pg.set_option(name, val)
