"""KV-head sharding (host logic) with two gloo ranks on the CPU: each rank takes its head range,
plans with kvHead = Hkv/2, computes its shard (here with the fp32 oracle standing in for the
kernels - this is a test of the partitioning, not of the device code) and the optional
all-gather reassembles the full output."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as O
from pat_b200 import PrefixTreeCPP
from pat_b200.sharding import HeadGather, all_gather_heads, kv_head_range, shard_views
from pat_b200.workloads import make_values, scaled_down


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = scaled_down(2, 8)                     # fp16, 32/4 heads
        q, k, v = make_values(w)
        q, k, v = q.float(), k.float(), v.float()
        scale = w.head_dim ** -0.5
        qs, ks, vs = shard_views(q, k, v, world, rank)
        lo, hi = kv_head_range(w.num_kv_heads, world, rank)
        assert qs.shape[2] == (hi - lo) * w.group and ks.shape[2] == hi - lo
        assert qs.data_ptr() == q[:, :, lo * w.group:].data_ptr()        # views, not copies
        # replicated host work: the plan for this rank's head count
        tree = PrefixTreeCPP(w.page_size)
        tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
        tree.pack_schedule(None, w.group, hi - lo)
        assert tree.kernel_info.num_split_per_seq.shape[0] == w.batch
        out_shard, _ = O.paged_decode_attention(qs, ks, vs, w.seq_lens, w.block_tables, scale)
        full = all_gather_heads(out_shard.contiguous(), world)
        ref, _ = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
        ok = torch.allclose(full, ref, atol=1e-6)
        # the 16-bit form with buffers allocated once (on the GPU the reorder is a kernel of the library)
        hg = HeadGather(out_shard.to(torch.bfloat16), world)
        for _ in range(2):
            full16 = hg(out_shard.to(torch.bfloat16))
            ok = ok and torch.equal(full16, ref.to(torch.bfloat16)) and full16.data_ptr() == hg.full.data_ptr()
        # timing reduction used by the benchmark: max over ranks
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ret[rank] = bool(ok) and t.item() == float(world)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_kv_head_sharding_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def test_head_ranges():
    assert [kv_head_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert kv_head_range(8, 1, 0) == (0, 8)
    with pytest.raises(ValueError):
        kv_head_range(4, 8, 0)
    with pytest.raises(ValueError):
        kv_head_range(8, 2, 2)
