"""ctypes binding of libvkgrad_b200.so (the C ABI in include/vkgrad_b200.h).

There is no fallback: if the shared library is missing, or a call fails, the
caller gets an exception.  The library is built in-tree by vkgrad_b200.build.
"""

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvkgrad_b200.so")

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_GELU, ACT_RELU = 0, 1, 2
# keys of vkg_set_tuning (include/vkgrad_b200.h)
TUNE_PDL, TUNE_PDL_FAMILIES, TUNE_TMA_STORE, TUNE_WAIT_TIMEOUT_MS, TUNE_SM_LIMIT = 0, 1, 2, 3, 4
TUNE_PAIR_MIN_WAVES, TUNE_ATTN_ONE_PASS, TUNE_PAIR_192 = 5, 6, 7

vp = C.c_void_p
i32 = C.c_int
i64 = C.c_int64
f32 = C.c_float
sz = C.c_size_t


class GemmArgs(C.Structure):
    """Mirror of struct vkg_gemm_args."""
    _fields_ = [
        ("trans_a", C.c_int32), ("trans_b", C.c_int32),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("nb0", C.c_int32), ("nb1", C.c_int32),
        ("in_dtype", C.c_int32),
        ("A", vp), ("lda", i64), ("sA0", i64), ("sA1", i64),
        ("B", vp), ("ldb", i64), ("sB0", i64), ("sB1", i64),
        ("C", vp), ("ldc", i64), ("sC0", i64), ("sC1", i64), ("c_dtype", C.c_int32),
        ("act", C.c_int32),
        ("C2", vp),
        ("bias", vp),
        ("pre", vp),
        ("dact_z", vp),
        ("dact", C.c_int32),
        ("residual", vp),
        ("tile_n", C.c_int32),
        ("max_ctas", C.c_int32),
        ("alpha", C.c_float),
        ("split_k", C.c_int32),
        ("workspace", vp),
        ("workspace_bytes", i64),
        ("causal", C.c_int32),
        ("cta_pair", C.c_int32),
        ("colsum", vp),
        ("colsum_scratch", vp),
    ]


# name -> (restype, [argtypes]); every int-returning entry is a status code.
_SIGNATURES = {
    "vkg_last_error": (C.c_char_p, []),
    "vkg_version": (C.c_char_p, []),
    "vkg_device_count": (i32, [C.POINTER(i32)]),
    "vkg_device_create": (i32, [i32, C.POINTER(vp)]),
    "vkg_device_destroy": (i32, [vp]),
    "vkg_device_info": (i32, [vp, C.c_char_p, sz, C.POINTER(i32), C.POINTER(sz),
                              C.POINTER(i32), C.POINTER(i32)]),
    "vkg_device_stream": (vp, [vp]),
    "vkg_set_pdl": (i32, [vp, i32]),
    "vkg_set_tuning": (i32, [vp, i32, i64]),
    "vkg_sync": (i32, [vp]),
    "vkg_selftest_wait_deadline": (i32, [i64, i64, C.c_double, C.POINTER(i32)]),
    "vkg_alloc": (i32, [vp, sz, i32, C.POINTER(vp), C.POINTER(vp)]),
    "vkg_free": (i32, [vp, vp, vp, i32]),
    "vkg_upload": (i32, [vp, vp, vp, sz]),
    "vkg_download": (i32, [vp, vp, vp, sz]),
    "vkg_copy": (i32, [vp, vp, vp, sz]),
    "vkg_copy_h2d_async": (i32, [vp, vp, vp, sz]),
    "vkg_copy_d2h_async": (i32, [vp, vp, vp, sz]),
    "vkg_memset0": (i32, [vp, vp, sz]),
    "vkg_timer_begin": (i32, [vp]),
    "vkg_timer_end": (i32, [vp, C.POINTER(C.c_double)]),
    "vkg_graph_begin": (i32, [vp]),
    "vkg_graph_end": (i32, [vp, C.POINTER(vp)]),
    "vkg_graph_launch": (i32, [vp, vp, C.POINTER(C.c_double)]),
    "vkg_graph_launch_async": (i32, [vp, vp]),
    "vkg_graph_destroy": (i32, [vp]),
    "vkg_graph_kernel_count": (i32, [vp, C.POINTER(i32)]),
    "vkg_gemm": (i32, [vp, C.POINTER(GemmArgs)]),
    "vkg_gemm_colsum_scratch_floats": (i64, [i32, i32]),
    "vkg_selftest_wait_timeout": (i32, [vp, i64]),
    "vkg_gemm_group_table_bytes": (i64, [i32]),
    "vkg_gemm_group_prepare": (i32, [vp, C.POINTER(GemmArgs), i32, vp, i32, C.POINTER(i32)]),
    "vkg_gemm_group_launch": (i32, [vp, vp, i32, i32]),
    "vkg_bias_act": (i32, [vp, vp, vp, vp, vp, i64, i32, i32]),
    "vkg_bias_act_bwd": (i32, [vp, vp, vp, vp, vp, i64, i32]),
    "vkg_bias": (i32, [vp, vp, vp, vp, i64, i32]),
    "vkg_col_sum": (i32, [vp, vp, vp, i32, i32]),
    "vkg_softmax_ce": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32]),
    "vkg_adamw": (i32, [vp, vp, vp, vp, vp, vp, vp, i64, f32]),
    "vkg_adamw_table_create": (i32, [vp, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                     C.POINTER(vp), C.POINTER(vp), C.POINTER(i64),
                                     C.POINTER(f32), C.POINTER(vp)]),
    "vkg_adamw_table_destroy": (i32, [vp, vp]),
    "vkg_adamw_multi": (i32, [vp, vp, vp]),
    "vkg_cast16": (i32, [vp, vp, vp, i64]),
    "vkg_layernorm": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32]),
    "vkg_layernorm_bwd": (i32, [vp] + [vp] * 14 + [i32, i32]),
    "vkg_layernorm_bwd_scratch_floats": (i64, [i32, i32]),
    "vkg_finals_defer": (i32, [vp, i32]),
    "vkg_finals_flush": (i32, [vp]),
    "vkg_attn_softmax": (i32, [vp, vp, vp, vp, i64, i32, i32, f32, i32]),
    "vkg_attn_softmax_bwd": (i32, [vp, vp, vp, vp, i64, i32, f32, i32]),
    "vkg_attn_fwd": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, f32]),
    "vkg_attn_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32]),
    "vkg_attn_bwd_dbias_scratch_floats": (i64, [i32, i32, i32, i32]),
    "vkg_split_qkv": (i32, [vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32]),
    "vkg_merge_qkv_grad": (i32, [vp, vp, vp, vp, vp, i64, i32, i32, i32, i32]),
    "vkg_merge_heads": (i32, [vp, vp, vp, i64, i32, i32, i32, i32]),
    "vkg_split_heads": (i32, [vp, vp, vp, i64, i32, i32, i32, i32]),
    "vkg_col_sum_det": (i32, [vp, vp, i32, vp, vp, i32, i32, i32]),
    "vkg_col_sum_scratch_floats": (i64, [i32, i32]),
    "vkg_col_sum_static": (i32, [vp, vp, i32, vp, i32, i32, i32]),
    "vkg_col_sum_static_max_floats": (i64, []),
    "vkg_embed": (i32, [vp, vp, vp, vp, vp, vp, i64, i32, i32]),
    "vkg_embed_bwd": (i32, [vp, vp, vp, vp, vp, vp, i64, i32, i32]),
    "vkg_embed_bwd_det": (i32, [vp, vp, vp, vp, vp, vp, vp, i64, i32, i32]),
    "vkg_embed_bwd_scratch_bytes": (i64, [i64]),
    "vkg_residual": (i32, [vp, vp, vp, vp, vp, i64, i32]),
    "vkg_add": (i32, [vp, vp, vp, vp, vp, i64]),
    "vkg_add_bias": (i32, [vp, vp, vp, i64, i32]),
    "vkg_grad_add": (i32, [vp, vp, vp, i64, i64]),
    "vkg_grad_pull": (i32, [vp, vp, vp, i64, i64, f32]),
    "vkg_bucket_pack16": (i32, [vp, vp, vp, i32, i64, f32]),
    "vkg_bucket_unpack16": (i32, [vp, vp, i32, vp, i64, f32]),
    "vkg_comm_unique_id": (i32, [C.POINTER(C.c_uint8)]),
    "vkg_comm_create": (i32, [vp, i32, i32, C.POINTER(C.c_uint8), C.POINTER(vp)]),
    "vkg_comm_create_limited": (i32, [vp, i32, i32, C.POINTER(C.c_uint8), i32, C.POINTER(vp)]),
    "vkg_comm_destroy": (i32, [vp]),
    "vkg_allreduce_sum": (i32, [vp, vp, i64, i32]),
    "vkg_comm_side_begin": (i32, [vp]),
    "vkg_allreduce_sum_side": (i32, [vp, vp, i64, i32, i32]),
    "vkg_comm_side_wait": (i32, [vp, i32]),
    "vkg_comm_max_double": (i32, [vp, C.POINTER(C.c_double)]),
    "vkg_comm_barrier": (i32, [vp]),
}

# Entries whose int return value is not a status code.
_NOT_STATUS = {"vkg_last_error", "vkg_version", "vkg_device_stream",
               "vkg_layernorm_bwd_scratch_floats", "vkg_col_sum_scratch_floats",
               "vkg_embed_bwd_scratch_bytes",
               "vkg_col_sum_static_max_floats"}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def exported_names():
    return sorted(_SIGNATURES)


def load():
    """Load the shared library once and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is missing: run `python -m vkgrad_b200.build` "
            "(there is no CPU or interpreter fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    return load().vkg_last_error().decode(errors="replace")
