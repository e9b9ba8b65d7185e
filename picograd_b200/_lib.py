"""Loader of libpg_b200.so, the C-ABI declared in include/pg_b200.h.

There is no fallback: if the shared library has not been built (run
`python -c "import __graft_entry__ as g; g.build()"` or `make -C
picograd_b200/csrc`) importing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# $PG_B200_LIBRARY: another build of the same library (e.g. the one with the timing experiments compiled in)
LIB_PATH = os.environ.get("PG_B200_LIBRARY") or os.path.join(_HERE, "lib", "libpg_b200.so")

_sz = C.c_size_t
_vp = C.c_void_p
_i = C.c_int

# name -> (restype, argtypes); one entry per declaration of include/pg_b200.h
SIGNATURES = {
    "pg_b200_init": (_i, []),
    "pg_b200_malloc": (_vp, [_sz]),
    "pg_b200_free": (None, [_vp]),
    "pg_b200_copy_h2d": (_i, [_vp, _vp, _sz]),
    "pg_b200_copy_d2h": (_i, [_vp, _vp, _sz]),
    "pg_b200_sync": (_i, []),
    "pg_b200_gemm": (None, [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]),
    "pg_b200_hgemm": (None, [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]),
    "pg_b200_bgemm": (None, [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]),
    "pg_b200_gemm_ex": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz]),
    "pg_b200_gemm_fused_ex": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _i]),
    "pg_b200_gemm_fused": (None, [_sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _i]),
    "pg_b200_gemm_fused_out16": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _i, _vp, _sz, _i]),
    "pg_b200_gemm_batched": (_i, [_i, _i, _i, _i, _sz, _sz, _sz, _sz, _vp, _sz, _sz, _vp, _sz, _sz,
                                  _vp, _sz, _sz, _i]),
    "pg_b200_matmul_backward": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _vp, _i, _vp, _vp, _vp]),
    "pg_b200_matmul_backward_ex": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _vp, _i, _vp, _vp, _vp, _i]),
    "pg_b200_matmul_backward_act": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i]),
    "pg_b200_addmm": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _sz, C.c_float, C.c_float]),
    "pg_b200_permute_copy": (_i, [_i, _sz, _vp, _vp, _vp, _vp]),
    "pg_b200_conv2d": (_i, [_sz] * 7 + [_i, _i, _vp, _vp, _vp, _vp]),
    "pg_b200_attention_bmm": (_i, [_i, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp]),
    "pg_b200_softmax_rows": (_i, [_vp, _vp, _vp, _i, _sz, _sz]),
    "pg_b200_gelu": (_i, [_vp, _vp, _vp, _i, _sz]),
    "pg_b200_gelu_grad": (_i, [_vp, _vp, _vp, _sz]),
    "pg_b200_cast_f32": (_i, [_vp, _vp, _i, _sz]),
    "pg_b200_fill_f32": (_i, [_vp, C.c_float, _sz]),
    "pg_b200_matmul": (_i, [_vp, _vp, _vp]),
    "pg_b200_bmm": (_i, [_vp, _vp, _vp]),
    "pg_b200_matmul_result_shape": (_i, [_vp, _vp, _vp]),
    "pg_b200_tensordot_result_shape": (_i, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "pg_b200_tensordot": (_i, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "pg_b200_matmul_backward_nd": (_i, [_vp, _vp, _vp, _vp, _vp, _i]),
    "pg_b200_gather_relayout": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _sz]),
    "pg_b200_gemm_ex_static_scratch": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _i]),
    "pg_b200_set_device": (_i, [_i]),
    "pg_b200_set_stream": (_i, [_vp]),
    "pg_b200_last_error": (C.c_char_p, []),
    "pg_b200_set_option": (_i, [C.c_char_p, _i]),
    "pg_b200_num_tile_configs": (_i, []),
    "pg_b200_tile_config_name": (C.c_char_p, [_i]),
    "pg_b200_launch_count": (C.c_uint64, []),
    "pg_b200_last_path": (C.c_char_p, []),
    "pg_b200_die_table": (_i, [_vp, _sz]),
    "pg_b200_debug_counters": (_i, [_vp, _sz]),
    "pg_b200_debug_tail_schedule": (_i, [C.c_uint64, C.c_uint, C.c_uint, C.c_uint, C.c_uint, _vp]),
    "pg_b200_gemm_ex_scatter": (_i, [_i, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _sz, _sz]),
    "pg_b200_ipc_export": (_i, [_vp, _vp]),
    "pg_b200_ipc_open": (_i, [_vp, _vp]),
    "pg_b200_ipc_close": (_i, [_vp]),
    "pg_b200_debug_walk": (_i, [C.c_uint] * 11 + [_vp]),
    "pg_b200_selftest_wait_timeout": (_i, [C.c_uint]),
}


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: the CUDA library of picograd_b200 has not been built "
            "(make -C picograd_b200/csrc). There is no CPU fallback.")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the .so lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()
