"""Helpers for tests that call the C ABI (``pat_b200_decode`` ...) directly through ctypes."""
import ctypes as C

import torch

from pat_b200 import PrefixTreeCPP
from pat_b200 import _native as N


def decode_args(q, k, v, out, work, scale, workspace=None, lse=None, status=None, flags=0, wait_limit_us=0):
    """A filled ``pat_decode_args`` for torch tensors (any strides the op accepts)."""
    a = N.DecodeArgs()
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse_out = lse.data_ptr() if lse is not None else None
    a.q_batch_stride, a.q_head_stride = q.stride(0), q.stride(2)
    a.k_page_stride, a.k_row_stride, a.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
    a.v_page_stride, a.v_row_stride, a.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
    a.out_batch_stride, a.out_head_stride = out.stride(0), out.stride(2)
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = q.shape[0], q.shape[2], k.shape[2], q.shape[3]
    a.page_size, a.num_pages = k.shape[1], k.shape[0]
    a.dtype = 1 if q.dtype == torch.bfloat16 else 0
    a.softmax_scale = scale
    a.flags = flags
    a.work_blob, a.work = work.blob.data_ptr(), work.header
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.status_word = status.data_ptr() if status is not None else None
    a.wait_limit_us = wait_limit_us
    return a


def packed_tree(w, device, kv_heads=None, semantics="cpp"):
    """The workload's plan, packed for ``kv_heads`` KV heads (default: all) and moved to the GPU."""
    tree = PrefixTreeCPP(w.page_size, semantics)
    tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
    tree.pack_schedule(None, w.group, w.num_kv_heads if kv_heads is None else kv_heads)
    tree.kernel_info.to_gpu(device)
    return tree


def workspace_bytes(lib, work, num_q_heads, head_dim):
    return lib.pat_b200_workspace_bytes(C.byref(work.header), num_q_heads, head_dim)
