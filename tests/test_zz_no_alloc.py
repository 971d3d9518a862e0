"""The allocation-free entry point ``pat_b200_decode_static_scratch``.

Some callers cannot allocate device memory when they call the op: an inference server that gave
the whole GPU to its own pool at start-up, or a decode loop in which an allocation may block or
fail.  For them the library keeps the partial results in a fixed 32 MiB device array instead of
a caller-provided workspace.  This test drives both entry points through the C ABI on the same
inputs, twice in a row with different queries (the array keeps the first call's contents), and
expects the same output; it also checks that an oversized work list is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C
import math

import pytest
import torch

from pat_b200 import PrefixTreeCPP
from pat_b200 import _native as N
from pat_b200.workloads import make_values, scaled_down

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(q, k, v, out, work, scale, workspace=None):
    a = N.DecodeArgs()
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.q_batch_stride, a.q_head_stride = q.stride(0), q.stride(2)
    a.k_page_stride, a.k_row_stride, a.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
    a.v_page_stride, a.v_row_stride, a.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
    a.out_batch_stride, a.out_head_stride = out.stride(0), out.stride(2)
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = q.shape[0], q.shape[2], k.shape[2], q.shape[3]
    a.page_size, a.num_pages = k.shape[1], k.shape[0]
    a.dtype = 1 if q.dtype == torch.bfloat16 else 0
    a.softmax_scale = scale
    a.work_blob, a.work = work.blob.data_ptr(), work.header
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


def test_static_scratch_entry_point_matches_the_allocating_one(native_lib):
    lib = native_lib
    w = scaled_down(1, 4)                      # 64 requests, shared 1024-token prefix, bf16
    q, k, v = make_values(w, device=DEV)
    scale = 1.0 / math.sqrt(w.head_dim)
    tree = PrefixTreeCPP(w.page_size)
    tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
    tree.pack_schedule(None, w.group, w.num_kv_heads)
    tree.kernel_info.to_gpu(DEV)
    work = tree.kernel_info.device_work(torch.device(DEV))
    need = lib.pat_b200_workspace_bytes(C.byref(work.header), w.num_q_heads, w.head_dim)
    assert 0 < need <= N.STATIC_SCRATCH_BYTES
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    with torch.cuda.device(DEV):
        for round_ in range(2):                # two calls in a row; the second with other queries
            qr = q if round_ == 0 else (q.float() * -0.7 + 0.05).to(q.dtype)
            ws = torch.empty(need, dtype=torch.uint8, device=DEV)
            want = torch.full_like(qr, float("nan"))
            rc = lib.pat_b200_decode(C.byref(_args(qr, k, v, want, work, scale, ws)), stream)
            assert rc == 0, N.strerror(rc)
            got = torch.full_like(qr, float("nan"))
            rc = lib.pat_b200_decode_static_scratch(C.byref(_args(qr, k, v, got, work, scale)), stream)
            assert rc == 0, N.strerror(rc)
            torch.cuda.synchronize()
            assert torch.isfinite(got.float()).all()
            torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)

        # a work list whose partials do not fit the fixed array is refused, nothing is launched
        big = N.WorkHeader.from_buffer_copy(work.header)
        big.num_entries = N.STATIC_SCRATCH_BYTES // (w.group * (w.head_dim + 1) * 4) + 1
        out = torch.zeros_like(q)
        a = _args(q, k, v, out, work, scale)
        a.work = big
        assert lib.pat_b200_decode_static_scratch(C.byref(a), stream) == -15
        assert "limit" in N.strerror(-15)
        torch.cuda.synchronize()
        assert float(out.float().abs().sum()) == 0.0
