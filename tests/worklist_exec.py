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
    B, T, H, D = q.shape
    page, hk, hr = header.page_size, header.kv_heads, header.hratio
    assert H == hk * hr and T == max(1, header.q_per_req) and header.batch == B * T
    qv = q.reshape(B * T, 1, H, D)              # a query of the list is a (request, position) pair
    part_o = torch.zeros(header.num_entries, hr, D)
    part_l = torch.full((header.num_entries, hr), float("nan"))
    written = np.zeros(header.num_entries, dtype=np.int32)
    for idx, it in enumerate(items_of(header, blob)):
        q_off, nq, page_off, kv_len, entry_base, kv_head = (int(x) for x in it[:6])
        tok_lo = int(it[7])
        streaming = idx < header.num_stream_items
        assert (kv_head == -1) == streaming
        qs = blob[header.queries_off + q_off: header.queries_off + q_off + nq].tolist()
        if header.limits_off >= 0:      # tokens of the item each query may see
            lim = blob[header.limits_off + q_off: header.limits_off + q_off + nq].tolist()
            sees = [max(0, min(kv_len, l - tok_lo)) for l in lim]
        else:
            sees = [kv_len] * nq
        n_pages = -(-kv_len // page)
        pages = blob[header.pages_off + page_off: header.pages_off + page_off + n_pages].tolist()
        kk = O.gather_request_kv(k_cache, pages, kv_len)
        vv = O.gather_request_kv(v_cache, pages, kv_len)
        for kvh in (range(hk) if streaming else [kv_head]):
            heads = slice(kvh * hr, (kvh + 1) * hr)
            for i in range(nq):
                e = entry_base + (i * hk + kvh if streaming else i)
                if sees[i] > 0:
                    o, l = O.segment_attention(qv[qs[i]:qs[i] + 1, 0][:, heads], kk[:sees[i], kvh:kvh + 1],
                                               vv[:sees[i], kvh:kvh + 1], scale)
                    part_o[e], part_l[e] = o[0], l[0]
                else:                   # sees nothing of this item: weight zero in the merge
                    part_o[e], part_l[e] = 0.0, float("-inf")
                written[e] += 1
    assert (written == 1).all(), "every entry must be written exactly once"
    n_lists = B * T * hk
    indptr = blob[header.merge_indptr_off: header.merge_indptr_off + n_lists + 1]
    entries = blob[header.merge_entries_off: header.merge_entries_off + int(indptr[-1])]
    assert sorted(entries.tolist()) == list(range(header.num_entries)), "every entry is merged exactly once"
    out = torch.zeros(B * T, H, D)
    lse = torch.full((B * T, H), float("-inf"))
    for b in range(B * T):
        for kvh in range(hk):
            lst = b * hk + kvh
            e = torch.as_tensor(entries[indptr[lst]: indptr[lst + 1]], dtype=torch.long)
            if len(e):
                heads = slice(kvh * hr, (kvh + 1) * hr)
                out[b, heads], lse[b, heads] = O.merge_partials(part_o[e], part_l[e])
    if T > 1:
        return out.reshape(B, T, H, D), lse.reshape(B, T, H)
    return out, lse


def dense_ctas(header, blob):
    """[(first, last)] dense item ranges (indices into the dense section) per persistent CTA."""
    b = blob[header.dense_cta_off: header.dense_cta_off + header.num_dense_ctas + 1].tolist()
    return list(zip(b[:-1], b[1:]))
