"""ctypes binding of ``libpat_b200.so`` (the C ABI declared in ``include/pat_b200.h``).

The library is built in-tree by ``python -m pat_b200.build`` and is the only
implementation of the device path: if it is missing, every call raises
``RuntimeError`` - there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpat_b200.so")

i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)


class BucketView(C.Structure):
    _fields_ = [("mnw", C.c_int32 * 3), ("ctas", C.c_int32), ("max_seqs", C.c_int32),
                ("max_blocks", C.c_int32), ("q_table", i32p), ("block_table", i32p),
                ("num_seqs", i32p), ("cta_ranks", i32p), ("kv_in_cta", i32p)]


class PlanBucket(C.Structure):
    _fields_ = [("ctas", C.c_int32), ("q_stride", C.c_int32), ("block_stride", C.c_int32),
                ("reserved", C.c_int32), ("q_table", C.c_void_p), ("block_table", C.c_void_p),
                ("num_seqs", C.c_void_p), ("kv_in_cta", C.c_void_p)]


class WorkOptions(C.Structure):
    _fields_ = [("num_sms", C.c_int32), ("dense_min_rows", C.c_int32), ("chunk_tokens_min", C.c_int32),
                ("chunk_tokens_max", C.c_int32), ("dense_piece_tokens_min", C.c_int32),
                ("items_per_sm", C.c_int32), ("disable_dense", C.c_int32), ("dense_tile_ns", C.c_int32),
                ("grow_slack_pages", C.c_int32), ("reserved", C.c_int32)]


class WorkHeader(C.Structure):
    _fields_ = [("batch", C.c_int32), ("hratio", C.c_int32), ("page_size", C.c_int32), ("kv_heads", C.c_int32),
                ("num_stream_items", C.c_int32), ("num_dense_items", C.c_int32), ("num_dense_ctas", C.c_int32),
                ("num_entries", C.c_int32), ("max_entries_per_list", C.c_int32),
                ("items_off", C.c_int32), ("queries_off", C.c_int32), ("pages_off", C.c_int32),
                ("dense_cta_off", C.c_int32), ("merge_indptr_off", C.c_int32), ("merge_entries_off", C.c_int32),
                ("blob_words", C.c_int32), ("num_segments", C.c_int32), ("max_page_id", C.c_int32),
                ("unique_tokens", C.c_int64), ("stream_tokens", C.c_int64), ("dense_tokens", C.c_int64),
                ("stream_unique_tokens", C.c_int64), ("dense_unique_tokens", C.c_int64),
                ("q_per_req", C.c_int32), ("limits_off", C.c_int32),
                ("dense_q_off", C.c_int32), ("dense_q_width", C.c_int32)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("out", C.c_void_p),
                ("lse_out", C.c_void_p),
                ("q_batch_stride", C.c_int64), ("q_head_stride", C.c_int64),
                ("k_page_stride", C.c_int64), ("k_row_stride", C.c_int64), ("k_head_stride", C.c_int64),
                ("v_page_stride", C.c_int64), ("v_row_stride", C.c_int64), ("v_head_stride", C.c_int64),
                ("out_batch_stride", C.c_int64), ("out_head_stride", C.c_int64),
                ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("page_size", C.c_int32), ("dtype", C.c_int32),
                ("num_pages", C.c_int64), ("softmax_scale", C.c_float), ("flags", C.c_int32),
                ("work_blob", C.c_void_p), ("work", WorkHeader),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("status_word", C.c_void_p), ("wait_limit_us", C.c_int32), ("q_per_req", C.c_int32),
                ("q_pos_stride", C.c_int64), ("out_pos_stride", C.c_int64)]


class AppendArgs(C.Structure):
    _fields_ = [("key", C.c_void_p), ("value", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("slot_mapping", C.c_void_p),
                ("key_token_stride", C.c_int64), ("key_head_stride", C.c_int64),
                ("value_token_stride", C.c_int64), ("value_head_stride", C.c_int64),
                ("k_page_stride", C.c_int64), ("k_row_stride", C.c_int64), ("k_head_stride", C.c_int64),
                ("v_page_stride", C.c_int64), ("v_row_stride", C.c_int64), ("v_head_stride", C.c_int64),
                ("num_pages", C.c_int64),
                ("num_tokens", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("page_size", C.c_int32), ("dtype", C.c_int32), ("reserved", C.c_int32)]


# name -> (restype, argtypes); also the list of symbols the header declares.
SIGNATURES = {
    "pat_b200_strerror": (C.c_char_p, [C.c_int]),
    "pat_b200_abi_version": (C.c_int, []),
    "pat_tree_create": (C.c_void_p, [C.c_int, C.c_int]),
    "pat_tree_destroy": (None, [C.c_void_p]),
    "pat_tree_build": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "pat_tree_build_ragged": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "pat_tree_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "pat_tree_num_buckets": (C.c_int, [C.c_void_p]),
    "pat_tree_bucket": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(BucketView)]),
    "pat_tree_split_per_seq": (i32p, [C.c_void_p, C.POINTER(C.c_int)]),
    "pat_tree_maxima": (C.c_int, [C.c_void_p, i32p]),
    "pat_tree_num_nodes": (C.c_int, [C.c_void_p]),
    "pat_tree_node": (C.c_int, [C.c_void_p, C.c_int, i32p]),
    "pat_tree_node_seqs": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(i32p), C.POINTER(C.c_int)]),
    "pat_tree_node_pages": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(i32p), C.POINTER(C.c_int)]),
    "pat_tree_node_children": (C.c_int, [C.c_void_p, C.c_int, i32p, C.c_int]),
    "pat_work_create": (C.c_void_p, [C.POINTER(PlanBucket), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_int64, C.POINTER(WorkOptions), C.POINTER(C.c_int)]),
    "pat_work_from_tree": (C.c_void_p, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.POINTER(WorkOptions),
                                        C.POINTER(C.c_int)]),
    "pat_work_from_tree_multi": (C.c_void_p, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64,
                                              C.POINTER(WorkOptions), C.POINTER(C.c_int)]),
    "pat_work_advance": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "pat_tree_advance": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "pat_work_destroy": (None, [C.c_void_p]),
    "pat_work_get_header": (C.c_int, [C.c_void_p, C.POINTER(WorkHeader)]),
    "pat_work_blob": (i32p, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "pat_b200_workspace_bytes": (C.c_size_t, [C.POINTER(WorkHeader), C.c_int, C.c_int]),
    "pat_b200_decode": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "pat_b200_last_launch_count": (C.c_int, []),
    "pat_b200_decode_static_scratch": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "pat_b200_selftest_wait": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p]),
    "pat_b200_reorder_heads": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "pat_b200_append_kv": (C.c_int, [C.POINTER(AppendArgs), C.c_void_p]),
}
STATIC_SCRATCH_BYTES = 32 << 20

_lib = None
_lock = threading.Lock()


def load():
    """The loaded library (cached).  Raises ``RuntimeError`` if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m pat_b200.build` "
                "(the CUDA path has no fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def strerror(code: int) -> str:
    return load().pat_b200_strerror(code).decode()
