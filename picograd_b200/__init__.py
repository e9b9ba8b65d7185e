"""picograd_b200 — a B200 (sm_100a) device path for picograd's dense matrix multiply.

The product is the C-ABI library `lib/libpg_b200.so` (include/pg_b200.h) and the
C11 host seat `host/cuda_backend.c`; this package is the thin Python mirror of
picograd's operator interface for that path, used by the tests and benchmark.
"""
from .backend import (  # noqa: F401
    PG_ACT_COPY_ONLY, PG_ACT_GELU, PG_ACT_NONE, PG_ACT_RELU, PG_DTYPE_BF16, PG_DTYPE_F16, PG_DTYPE_F32, PG_OK, PgError,
    pg_addmm, pg_attention_bmm, pg_conv2d, pg_gemm_fused, pg_gemm_fused_ex, pg_linear_forward,
    pg_bgemm, pg_bmm, pg_dev_sync, pg_gemm, pg_gemm_ex, pg_gemm_ex_host, pg_hgemm, pg_matmul,
    pg_gather_relayout, pg_gemm_ex_scatter, pg_matmul_backward, pg_matmul_backward_act, pg_set_device, pg_tensordot, last_path, launch_count, set_option,
)
