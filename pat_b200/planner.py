"""Plan of a decode batch kept alive across steps.

The reference rebuilds everything in every decode step: radix tree, tile plan, the per-bucket
tables and their host-to-device copies (``prefix_attn/async_tree.py:23-30``, cached once per
forward pass at ``plugin/vllm/attention/backends/prefix_attn.py:318-340`` and left stale by
``advance_step`` at ``:430-438``).  Between two steps of a running batch almost nothing changes:
every request is one token longer and now and then one page longer.  ``DecodePlanner.step`` first
tries to grow the previous step's tree and device work list in place (``PrefixTreeCPP.advance``:
item lengths and appended page ids are patched and the list is copied into the same device buffer)
and only falls back to a rebuild when the batch really changed.  Either way it returns a
``PrefixTreeCPP`` for ``prefix_attn_with_kvcache(q, k_cache, v_cache, tree, scale, out)``.
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from ._prefix_attn import PrefixTreeCPP


class DecodePlanner:
    def __init__(self, block_size: int, HRatio: int, kvHead: int, device: Union[torch.device, str],
                 MNWs: Optional[List[List[int]]] = None, semantics: str = "cpp"):
        self.block_size, self.hratio, self.kv_heads = int(block_size), int(HRatio), int(kvHead)
        self.device = torch.device(device)
        self.mnws, self.semantics = MNWs, semantics
        self.tree: Optional[PrefixTreeCPP] = None
        self.rebuilds = 0           # steps that built tree and work list from scratch
        self.advances = 0           # steps that grew them in place

    def step(self, seq_lens, block_table: torch.Tensor) -> PrefixTreeCPP:
        """``seq_lens``: list of ints or CPU int32 tensor; ``block_table``: padded CPU int32 tensor
        ``[num_seqs, max_blocks]`` (the arguments of ``build_radix_tree``).  Call it on the stream
        the attention runs on: an in-place update is copied to the device on the current stream."""
        if self.tree is not None and self.tree.advance(seq_lens, block_table):
            self.advances += 1
            return self.tree
        tree = PrefixTreeCPP(self.block_size, self.semantics)
        tree.build_radix_tree(seq_lens, block_table)
        tree.pack_schedule(self.mnws, self.hratio, self.kv_heads)
        tree.kernel_info.to_gpu(self.device)
        self.tree = tree
        self.rebuilds += 1
        return tree
