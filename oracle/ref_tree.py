"""TEST INFRASTRUCTURE ONLY - runs the compiled reference C++ scheduler
(``oracle/_ref/libpat_ref_tree.so``, see ``oracle/build_ref.py``) and returns its
plan as plain lists."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import numpy as np

_LIB = None
_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libpat_ref_tree.so")


def available() -> bool:
    return os.path.isfile(_PATH)


def _lib():
    global _LIB
    if _LIB is None:
        import torch  # noqa: F401  (loads libtorch, which the shim links against)
        lib = C.CDLL(_PATH)
        lib.ref_tree_create.restype = C.c_void_p
        lib.ref_tree_create.argtypes = [C.c_int]
        lib.ref_tree_destroy.argtypes = [C.c_void_p]
        lib.ref_tree_build.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        lib.ref_tree_pack.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.ref_tree_num_buckets.argtypes = [C.c_void_p]
        lib.ref_tree_bucket_shape.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        for name in ("ref_tree_q", "ref_tree_blocks", "ref_tree_num_seqs", "ref_tree_ranks", "ref_tree_kv"):
            fn = getattr(lib, name)
            fn.restype = C.POINTER(C.c_int)
            fn.argtypes = [C.c_void_p, C.c_int]
        lib.ref_tree_split.restype = C.POINTER(C.c_int)
        lib.ref_tree_split.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        lib.ref_tree_maxima.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        lib.ref_tree_num_nodes.argtypes = [C.c_void_p]
        lib.ref_tree_node.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        _LIB = lib
    return _LIB


def _arr(ptr, n):
    return np.ctypeslib.as_array(ptr, shape=(n,)).copy() if n else np.zeros(0, dtype=np.int32)


def run(block_size: int, seq_lens: Sequence[int], padded_table: np.ndarray,
        MNWs: Optional[List[List[int]]], hratio: int, kv_heads: int, packs: int = 1) -> dict:
    """Build + pack (``packs`` times) and return the accumulated plan."""
    lib = _lib()
    lens = np.asarray(seq_lens, dtype=np.int32)
    table = np.ascontiguousarray(padded_table, dtype=np.int32)
    t = lib.ref_tree_create(block_size)
    try:
        lib.ref_tree_build(t, lens.ctypes.data, table.ctypes.data, table.shape[0], table.shape[1])
        if MNWs:
            m = np.asarray(MNWs, dtype=np.int32).reshape(-1, 3)
            mp, mn = m.ctypes.data, m.shape[0]
        else:
            mp, mn = None, 0
        for _ in range(packs):
            lib.ref_tree_pack(t, mp, mn, hratio, kv_heads)
        out = dict(MNWs=[], q_tables=[], block_tables=[], num_seqs_per_CTAs=[], CTA_ranks=[], kv_in_CTAs=[])
        shape = (C.c_int * 6)()
        for i in range(lib.ref_tree_num_buckets(t)):
            lib.ref_tree_bucket_shape(t, i, shape)
            ctas, qw, bw = shape[3], shape[4], shape[5]
            out["MNWs"].append([shape[0], shape[1], shape[2]])
            out["q_tables"].append(_arr(lib.ref_tree_q(t, i), ctas * qw).reshape(ctas, qw).tolist())
            out["block_tables"].append(_arr(lib.ref_tree_blocks(t, i), ctas * bw).reshape(ctas, bw).tolist())
            out["num_seqs_per_CTAs"].append(_arr(lib.ref_tree_num_seqs(t, i), ctas).tolist())
            out["CTA_ranks"].append(_arr(lib.ref_tree_ranks(t, i), ctas).tolist())
            out["kv_in_CTAs"].append(_arr(lib.ref_tree_kv(t, i), ctas).tolist())
        n = C.c_int(0)
        ptr = lib.ref_tree_split(t, C.byref(n))
        out["num_split_per_seq"] = _arr(ptr, n.value).tolist()
        mx = (C.c_int * 3)()
        lib.ref_tree_maxima(t, mx)
        out["max_split_per_seq"], out["max_seqs_in_CTA"], out["max_blocks_in_CTA"] = mx[0], mx[1], mx[2]
        node = (C.c_int * 3)()
        nodes = []
        for i in range(lib.ref_tree_num_nodes(t)):
            lib.ref_tree_node(t, i, node)
            nodes.append([node[0], node[1], node[2]])
        out["nodes"] = nodes
        return out
    finally:
        lib.ref_tree_destroy(t)


def time_pack(seq_lens: np.ndarray, padded_table: np.ndarray, block_size: int, hratio: int, kv_heads: int) -> None:
    """One build + pack of the reference scheduler with the result left unread (for timing it)."""
    lib = _lib()
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    table = np.ascontiguousarray(padded_table, dtype=np.int32)
    t = lib.ref_tree_create(block_size)
    try:
        lib.ref_tree_build(t, lens.ctypes.data, table.ctypes.data, table.shape[0], table.shape[1])
        lib.ref_tree_pack(t, None, 0, hratio, kv_heads)
    finally:
        lib.ref_tree_destroy(t)
