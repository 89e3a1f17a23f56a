"""ctypes binding of the C ABI declared in include/recsdk_b200.h.

The shared library is built in-tree (``python -m recsdk_b200.build``).  There is
no fallback: if the library is missing or a symbol is absent, importing fails.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "librecsdk_b200.so")

c_i64p = C.POINTER(C.c_int64)
c_i32p = C.POINTER(C.c_int32)
c_f32p = C.POINTER(C.c_float)
vp = C.c_void_p

STATUS_WORDS = 4

OK = 0
ERR_INVALID_ARG, ERR_WORKSPACE, ERR_CUDA, ERR_NEGATIVE_KEY, ERR_TABLE_FULL = 1, 2, 3, 4, 5
ERR_CACHE_TOO_SMALL, ERR_INDEX_RANGE, ERR_HASH_FULL, ERR_TOO_LARGE, ERR_STATIC_SCRATCH = 6, 7, 8, 9, 10

POOL_SUM, POOL_MEAN, POOL_NONE = 0, 1, 2
OPT_ADAGRAD, OPT_ADAM, OPT_SGD = 1, 2, 3


MAX_SHARDS = 16


class SampleShards(C.Structure):
    _fields_ = [
        ("num_shards", C.c_int32), ("row_stride", C.c_int32), ("shard_B", C.c_int64), ("col_offsets", vp),
        ("ptrs", vp * MAX_SHARDS),
    ]


class TbeForwardArgs(C.Structure):
    _fields_ = [
        ("dev_weights", vp), ("weights_offsets", vp), ("D_offsets", vp), ("indices", vp), ("offsets", vp),
        ("out", vp), ("T", C.c_int64), ("B", C.c_int64), ("N", C.c_int64), ("total_D", C.c_int32),
        ("max_D", C.c_int32), ("pooling_mode", C.c_int32), ("weights_numel", C.c_int64), ("dev_status", vp),
        ("out_shards", SampleShards), ("flags", C.c_int32),
    ]


class TbeBackwardArgs(C.Structure):
    _fields_ = [
        ("grad_output", vp), ("dev_weights", vp), ("momentum1", vp), ("momentum2", vp), ("weights_offsets", vp),
        ("D_offsets", vp), ("hash_size_cumsum", vp), ("indices", vp), ("offsets", vp), ("unique_ids", vp),
        ("unique_offsets", vp), ("unique_inverse", vp), ("T", C.c_int64), ("B", C.c_int64), ("N", C.c_int64),
        ("num_unique_capacity", C.c_int64), ("total_D", C.c_int32), ("max_D", C.c_int32),
        ("pooling_mode", C.c_int32), ("optimizer", C.c_int32), ("total_hash_size_bits", C.c_int32),
        ("reduce_chunk", C.c_int32), ("learning_rate", C.c_float), ("eps", C.c_float), ("beta1", C.c_float),
        ("beta2", C.c_float), ("iter", C.c_int64), ("gradient_clipping", C.c_int32), ("max_gradient", C.c_float),
        ("weights_numel", C.c_int64), ("dev_status", vp), ("workspace", vp), ("workspace_bytes", C.c_size_t),
        ("ev_update_start", vp), ("ev_update_stop", vp), ("grad_shards", SampleShards), ("flags", C.c_int32),
    ]


class MapperT(C.Structure):
    _fields_ = [
        ("table", vp), ("hash_capacity", C.c_int64), ("slot_key", vp), ("mark", vp), ("counters", vp),
        ("init_max_index", C.c_int64), ("only_device_mem", C.c_int32),
    ]


class SwapT(C.Structure):
    _fields_ = [
        ("table", vp), ("hash_capacity", C.c_int64), ("slot_key", vp), ("slot_version", vp), ("counters", vp),
        ("cache_size", C.c_int64), ("mem_start_offset", C.c_int64),
    ]


class FilterT(C.Structure):
    _fields_ = [
        ("table", vp), ("hash_capacity", C.c_int64), ("counters", vp), ("admit_threshold", C.c_int64),
        ("evict_threshold", C.c_int64), ("evict_step_interval", C.c_int64),
    ]


XCHG_TABLE_WISE, XCHG_ROW_WISE = 0, 1


class XchgT(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("partition", C.c_int32), ("D", C.c_int32), ("F", C.c_int64),
        ("B", C.c_int64), ("max_ids", C.c_int64), ("inbox_cap", C.c_int64), ("key_bits", C.c_int32),
        ("flags", C.c_int32), ("part_base", vp), ("rank_base", vp), ("table_rows", vp), ("local_rows", C.c_int64),
        ("tables", vp * MAX_SHARDS), ("inbox_ids", vp * MAX_SHARDS), ("inbox_counts", vp * MAX_SHARDS),
        ("inbox_grads", vp * MAX_SHARDS), ("workspace", vp), ("workspace_bytes", C.c_size_t), ("dev_status", vp),
    ]


# symbol -> (restype, argtypes); every symbol include/recsdk_b200.h declares
SIGNATURES = {
    "recsdk_status_clear": (C.c_int, [vp, vp]),
    "recsdk_error_string": (C.c_char_p, [C.c_int]),
    "recsdk_version": (C.c_int, []),
    "recsdk_tbe_forward": (C.c_int, [C.POINTER(TbeForwardArgs), vp]),
    "recsdk_unique_sorted_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "recsdk_unique_sorted": (C.c_int, [vp, C.c_int64, C.c_int, vp, vp, vp, vp, C.c_size_t, vp]),
    "recsdk_unique_sorted_static_max_n": (C.c_int64, []),
    "recsdk_unique_sorted_static": (C.c_int, [vp, C.c_int64, C.c_int, vp, vp, vp, vp]),
    "recsdk_tbe_backward_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "recsdk_tbe_backward": (C.c_int, [C.POINTER(TbeBackwardArgs), vp]),
    "recsdk_adam_beta2sqrt": (C.c_float, [C.c_float, C.c_float, C.c_int64]),
    "recsdk_gather_rows": (C.c_int, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int64, vp, vp]),
    "recsdk_gather_rows_wait_limit": (C.c_int, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int64, vp, C.c_int32, vp]),
    "recsdk_scatter_rows": (C.c_int, [vp, vp, C.c_int64, C.c_int32, vp, C.c_int64, vp, vp]),
    "recsdk_lookup_by_address": (C.c_int, [vp, C.c_int64, C.c_int32, vp, vp]),
    "recsdk_update_by_address": (C.c_int, [vp, C.c_int64, C.c_int32, vp, C.c_int32, vp]),
    "recsdk_lazy_adam": (C.c_int, [vp, vp, C.c_int64, C.c_int32, vp, vp, vp, C.c_float, C.c_float, C.c_float,
                                   C.c_float, vp]),
    "recsdk_sgd": (C.c_int, [vp, vp, C.c_int64, C.c_int32, vp, C.c_float, C.c_float, C.c_int32, vp, C.c_size_t,
                             vp]),
    "recsdk_restore": (C.c_int, [vp, vp, vp, vp, C.c_int64, C.c_int64, vp, vp]),
    "recsdk_complete_cumsum_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "recsdk_complete_cumsum": (C.c_int, [vp, C.c_int64, vp, vp, C.c_size_t, vp]),
    "recsdk_permute_sparse_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "recsdk_permute_2d_sparse_data": (C.c_int, [vp, C.c_int64, vp, C.c_int64, C.c_int64, vp, C.c_int32, vp, vp, vp, vp,
                                                C.c_int64, vp, vp, vp, C.c_size_t, vp]),
    "recsdk_jagged_to_padded_dense": (C.c_int, [vp, vp, C.c_int64, C.c_int32, C.c_int64, C.c_float, vp, vp]),
    "recsdk_dense_to_jagged": (C.c_int, [vp, vp, C.c_int64, C.c_int32, C.c_int64, vp, vp]),
    "recsdk_peer_export": (C.c_int, [vp, vp, C.POINTER(C.c_int64)]),
    "recsdk_peer_import": (C.c_int, [vp, C.c_int64, C.POINTER(vp)]),
    "recsdk_peer_release": (C.c_int, [vp, C.c_int64]),
    "recsdk_peer_copy": (C.c_int, [vp, vp, C.c_size_t, vp]),
    "recsdk_xchg_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int64]),
    "recsdk_xchg_forward": (C.c_int, [C.POINTER(XchgT), vp, vp, C.c_int64, C.c_int32, vp, C.c_int32, vp]),
    "recsdk_xchg_backward_local": (C.c_int, [C.POINTER(XchgT), vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_float, vp]),
    "recsdk_xchg_backward_owner": (C.c_int, [C.POINTER(XchgT), vp, vp, vp, C.c_int32, C.c_float, C.c_float, C.c_float,
                                             C.c_float, C.c_int64, vp, vp, C.c_int32, vp]),
    "recsdk_xchg_counters": (C.c_int, [C.POINTER(XchgT), C.POINTER(C.c_int64), vp]),
    "recsdk_host_table_create": (vp, [C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_float, C.c_float, C.c_float,
                                      C.c_int64, C.c_int64]),
    "recsdk_host_table_destroy": (None, [vp]),
    "recsdk_host_table_size": (C.c_int64, [vp]),
    "recsdk_host_table_find_or_insert": (C.c_int, [vp, vp, C.c_int64, vp, vp, vp]),
    "recsdk_host_table_insert_or_assign": (C.c_int, [vp, vp, C.c_int64, vp, vp, vp]),
    "recsdk_host_table_remove": (C.c_int, [vp, vp, C.c_int64]),
    "recsdk_host_table_export": (C.c_int64, [vp, vp, vp, vp, vp, C.c_int64]),
    "recsdk_mapper_table_bytes": (C.c_size_t, [C.c_int64]),
    "recsdk_mapper_init": (C.c_int, [C.POINTER(MapperT), vp]),
    "recsdk_mapper_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "recsdk_mapper_unique_out": (C.c_int, [C.POINTER(MapperT), vp, vp, C.c_int64, C.c_int64, vp, vp, vp, vp,
                                           C.c_int64, vp, vp, C.c_size_t, vp]),
    "recsdk_mapper_ids2indices_unique": (C.c_int, [C.POINTER(MapperT), vp, C.c_int64, vp, vp, vp, vp, vp, vp,
                                                   C.c_size_t, vp]),
    "recsdk_swap_init": (C.c_int, [C.POINTER(SwapT), vp]),
    "recsdk_swap_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "recsdk_swap_compute": (C.c_int, [C.POINTER(SwapT), vp, C.c_int64, vp, vp, vp, vp, vp, vp, vp, vp, C.c_size_t,
                                      vp]),
    "recsdk_swap_remove": (C.c_int, [C.POINTER(SwapT), vp, C.c_int64, vp, vp]),
    "recsdk_filter_init": (C.c_int, [C.POINTER(FilterT), vp]),
    "recsdk_filter_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "recsdk_filter_statistics": (C.c_int, [C.POINTER(FilterT), vp, vp, C.c_int64, vp, vp]),
    "recsdk_filter_count_filter": (C.c_int, [C.POINTER(FilterT), vp, C.c_int64, vp]),
    "recsdk_filter_record_timestamp": (C.c_int, [C.POINTER(FilterT), vp, vp, C.c_int64, vp, C.c_int64, vp, vp,
                                                 C.c_size_t, vp]),
    "recsdk_filter_clear_evict": (C.c_int, [C.POINTER(FilterT), vp]),
    "recsdk_filter_count_of": (C.c_int, [C.POINTER(FilterT), vp, C.c_int64, vp, vp]),
    "recsdk_key_table_stats": (C.c_int, [vp, C.c_int64, C.c_int32, vp, vp]),
    "recsdk_key_table_rebuild_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "recsdk_key_table_rebuild": (C.c_int, [vp, C.c_int64, C.c_int32, C.c_int64, vp, vp, C.c_size_t, vp]),
    "recsdk_bucketize_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "recsdk_bucketize": (C.c_int, [vp, C.c_int64, vp, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, vp,
                                   vp, vp, vp, vp, vp, C.c_size_t, vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads librecsdk_b200.so and binds every declared symbol.  Raises if the
    library was not built or lacks a symbol: there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m recsdk_b200.build` (needs nvcc); "
            "recsdk_b200 has no CPU or pure-PyTorch fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def error_string(code: int) -> str:
    return load().recsdk_error_string(code).decode()


class RecsdkError(RuntimeError):
    def __init__(self, code: int, where: str = "", detail: str = ""):
        self.code = code
        msg = error_string(code)
        super().__init__(f"{where}: {msg}{(' ' + detail) if detail else ''}" if where else msg)


def check(code: int, where: str = "") -> None:
    if code != OK:
        raise RecsdkError(code, where)
