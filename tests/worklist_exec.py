"""CPU execution of a device work list (test helper).

Runs every work item with the fp32 oracle (``oracle/attention_oracle.py``) and
merges the per-entry partials through the list's own merge tables - the same
data flow as the CUDA kernels, so that the host-side packer can be validated
without a GPU."""
import ctypes as C

import numpy as np
import torch

from oracle import attention_oracle as O
from pat_b200 import _native as N
from pat_b200._plan_cache import host_plan_from_lists


def build_work(plan_lists, batch, hratio, kv_heads, page, **opts):
    """``plan_lists`` = (q_tables, block_tables, num_seqs, kv_lens) as nested lists.
    Returns (header, blob ndarray)."""
    lib = N.load()
    hp = host_plan_from_lists(*plan_lists, batch)
    n = len(hp.q_tables)
    buckets = (N.PlanBucket * max(n, 1))()
    for i in range(n):
        buckets[i].ctas = int(hp.num_seqs[i].shape[0])
        buckets[i].q_stride = int(hp.q_tables[i].shape[1])
        buckets[i].block_stride = int(hp.block_tables[i].shape[1])
        buckets[i].q_table = hp.q_tables[i].ctypes.data
        buckets[i].block_table = hp.block_tables[i].ctypes.data
        buckets[i].num_seqs = hp.num_seqs[i].ctypes.data
        buckets[i].kv_in_cta = hp.kv_lens[i].ctypes.data
    o = N.WorkOptions()
    for k, v in opts.items():
        setattr(o, k, v)
    status = C.c_int(0)
    h = lib.pat_work_create(buckets, n, batch, hratio, kv_heads, page, 0, C.byref(o), C.byref(status))
    assert h, N.strerror(status.value)
    header = N.WorkHeader()
    lib.pat_work_get_header(h, C.byref(header))
    words = C.c_size_t()
    ptr = lib.pat_work_blob(h, C.byref(words))
    blob = np.ctypeslib.as_array(ptr, shape=(words.value,)).copy()
    lib.pat_work_destroy(h)
    return header, blob


def items_of(header, blob):
    n = header.num_stream_items + header.num_dense_items
    return blob[header.items_off: header.items_off + 8 * n].reshape(n, 8)


def execute(header, blob, q, k_cache, v_cache, scale):
    """Returns (out [B,H,D] fp32, lse [B,H] fp32)."""
    B, _, H, D = q.shape
    page = header.page_size
    part_o = torch.zeros(header.num_entries, H, D)
    part_l = torch.full((header.num_entries, H), float("nan"))
    written = np.zeros(header.num_entries, dtype=np.int32)
    for it in items_of(header, blob):
        q_off, nq, page_off, kv_len, entry_base = (int(x) for x in it[:5])
        qs = blob[header.queries_off + q_off: header.queries_off + q_off + nq].tolist()
        n_pages = -(-kv_len // page)
        pages = blob[header.pages_off + page_off: header.pages_off + page_off + n_pages].tolist()
        kk = O.gather_request_kv(k_cache, pages, kv_len)
        vv = O.gather_request_kv(v_cache, pages, kv_len)
        o, l = O.segment_attention(q[qs, 0], kk, vv, scale)
        part_o[entry_base: entry_base + nq] = o
        part_l[entry_base: entry_base + nq] = l
        written[entry_base: entry_base + nq] += 1
    assert (written == 1).all(), "every entry must be written exactly once"
    indptr = blob[header.merge_indptr_off: header.merge_indptr_off + B + 1]
    entries = blob[header.merge_entries_off: header.merge_entries_off + header.num_entries]
    out = torch.zeros(B, H, D)
    lse = torch.full((B, H), float("-inf"))
    for b in range(B):
        e = torch.as_tensor(entries[indptr[b]: indptr[b + 1]], dtype=torch.long)
        if len(e):
            out[b], lse[b] = O.merge_partials(part_o[e], part_l[e])
    return out, lse
