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

from abi_util import decode_args as _args, packed_tree
from pat_b200 import _native as N
from pat_b200.workloads import make_values, scaled_down

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_static_scratch_entry_point_matches_the_allocating_one(native_lib):
    lib = native_lib
    w = scaled_down(1, 4)                      # 64 requests, shared 1024-token prefix, bf16
    q, k, v = make_values(w, device=DEV)
    scale = 1.0 / math.sqrt(w.head_dim)
    tree = packed_tree(w, DEV)
    work = tree.kernel_info.device_work(torch.device(DEV))
    need = lib.pat_b200_workspace_bytes(C.byref(work.header), w.num_q_heads, w.head_dim)
    assert 0 < need <= N.STATIC_SCRATCH_BYTES
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    with torch.cuda.device(DEV):
        for round_ in range(2):                # two calls in a row; the second with other queries
            qr = q if round_ == 0 else (q.float() * -0.7 + 0.05).to(q.dtype)
            ws = torch.empty(need, dtype=torch.uint8, device=DEV)
            ws[:256].zero_()                   # control words of a fresh workspace start at zero
            want = torch.full_like(qr, float("nan"))
            rc = lib.pat_b200_decode(C.byref(_args(qr, k, v, want, work, scale, ws)), stream)
            assert rc == 0, N.strerror(rc)
            got = torch.full_like(qr, float("nan"))
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc = lib.pat_b200_decode_static_scratch(C.byref(_args(qr, k, v, got, work, scale)), stream)
            assert rc == 0, N.strerror(rc)
            torch.cuda.synchronize()
            # the call took no device memory (on its first use too: the array is part of the
            # library image that was loaded long before)
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.isfinite(got.float()).all()
            # same work list, same kernels, same arithmetic: only the address of the partial
            # results differs, so the two outputs are the same bits
            assert torch.equal(got, want)

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
