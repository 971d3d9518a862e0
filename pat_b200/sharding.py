"""KV-head sharding across the GPUs of one node.

Every KV head (with its group of query heads) is an independent slice of the decode-attention
problem: the reference's own grid puts the KV head on ``blockIdx.y``
(``csrc/pat_fwd_launch_template.h:37``) and a tensor-parallel vLLM hands the backend per-rank
head counts (``plugin/vllm/attention/backends/prefix_attn.py:617-618``).  Rank ``r`` of ``n``
owns KV heads ``[r*Hkv/n, (r+1)*Hkv/n)`` and the matching query heads; block tables and plans
are replicated host work (packed with ``kvHead = Hkv/n``).  No kernel reads another GPU's
memory and no collective sits on the data path; ``all_gather_heads`` is the one optional
collective, for callers that want the full ``[batch, 1, H, D]`` output on every rank (in a
tensor-parallel model the row-parallel output projection consumes the shard locally instead).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def kv_head_range(num_kv_heads: int, world: int, rank: int) -> Tuple[int, int]:
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split evenly over {world} ranks")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def shard_views(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, world: int, rank: int):
    """Views (no copies) of this rank's heads: ``q [B,1,H/n,D]``, caches ``[pages, page, Hkv/n, D]``.
    The op honours the strides, so the views can be passed as they are."""
    hk = k_cache.shape[2]
    group = q.shape[2] // hk
    lo, hi = kv_head_range(hk, world, rank)
    return q[:, :, lo * group: hi * group], k_cache[:, :, lo:hi], v_cache[:, :, lo:hi]


class HeadGather:
    """The one optional collective of a sharded step: every rank gets all heads.

    Buffers are allocated once: an NCCL all-gather writes the ranks' ``[B, 1, H/n, D]`` outputs
    rank by rank into a staging buffer and one small kernel of this library puts the heads in
    order in ``[B, 1, H, D]``.  Nothing here synchronises with the host.  The result tensor is
    reused by every call.  A caller that captures the gather in a CUDA graph must destroy that
    graph before the process group: tearing down an NCCL communicator waits for every graph that
    holds one of its collectives (a 2-GPU run that kept such graphs alive sat in
    ``destroy_process_group`` until it was killed)."""

    def __init__(self, out_shard: torch.Tensor, world: int, group=None):
        b, one, h, d = out_shard.shape
        if one != 1 or out_shard.element_size() != 2:
            raise ValueError("expected a 16-bit [batch, 1, heads, head_dim] shard")
        self.world, self.group = world, group
        self.staged = torch.empty((world, b, h, d), dtype=out_shard.dtype, device=out_shard.device)
        self.full = torch.empty((b, 1, world * h, d), dtype=out_shard.dtype, device=out_shard.device)

    def __call__(self, out_shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return out_shard
        import ctypes as C
        import torch.distributed as dist
        from . import _native as N
        shard = out_shard if out_shard.is_contiguous() else out_shard.contiguous()
        b, _, h, d = shard.shape
        dist.all_gather_into_tensor(self.staged.view(self.world * b, h, d), shard.view(b, h, d), group=self.group)
        if shard.is_cuda:
            stream = torch.cuda.current_stream(shard.device).cuda_stream
            rc = N.load().pat_b200_reorder_heads(self.staged.data_ptr(), self.full.data_ptr(), self.world, b, h, d,
                                                 C.c_void_p(stream))
            if rc != 0:
                raise RuntimeError(f"head reorder failed: {N.strerror(rc)}")
        else:       # host tensors (multi-process tests of the partitioning on the CPU)
            self.full.copy_(self.staged.permute(1, 0, 2, 3).reshape(b, 1, self.world * h, d))
        return self.full


def all_gather_heads(out_shard: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Concatenate the ranks' ``[B, 1, H/n, D]`` outputs along the head axis (rank order); one-off
    form that allocates its buffers (``HeadGather`` keeps them)."""
    if world == 1:
        return out_shard
    if out_shard.element_size() == 2:
        return HeadGather(out_shard, world, group)(out_shard)
    import torch.distributed as dist
    shard = out_shard.contiguous()
    buf = torch.empty((world,) + tuple(shard.shape), dtype=shard.dtype, device=shard.device)
    dist.all_gather_into_tensor(buf.view(world * shard.shape[0], *shard.shape[1:]), shard, group=group)
    b, one, h, d = shard.shape
    return buf.permute(1, 2, 0, 3, 4).reshape(b, one, world * h, d)      # rank-major head order


class ShardedDecode:
    """One rank's share of a decode step: a plan packed for ``Hkv/n`` KV heads plus the op call."""

    def __init__(self, block_size: int, seq_lens, block_table: torch.Tensor, num_q_heads: int,
                 num_kv_heads: int, world: int, rank: int, device, semantics: str = "cpp"):
        from ._prefix_attn import PrefixTreeCPP
        self.world, self.rank = world, rank
        self.lo, self.hi = kv_head_range(num_kv_heads, world, rank)
        self.group = num_q_heads // num_kv_heads
        self.tree = PrefixTreeCPP(block_size, semantics)
        self.tree.build_radix_tree(seq_lens, block_table)
        self.tree.pack_schedule(None, self.group, self.hi - self.lo)
        self.tree.kernel_info.to_gpu(device)

    def __call__(self, q_shard, k_shard, v_shard, softmax_scale: float, out_shard: Optional[torch.Tensor] = None,
                 lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ._prefix_attn import prefix_attn_with_kvcache
        if out_shard is None:
            out_shard = torch.empty_like(q_shard)
        prefix_attn_with_kvcache(q_shard, k_shard, v_shard, self.tree, softmax_scale, out_shard, lse_out=lse_out)
        return out_shard
