"""Plan building off the critical path.

Mirror of the reference's ``prefix_attn/async_tree.py:8-37``: an ``AsyncTree``
starts building the radix tree, packing the plan and uploading it (tables and
device work list) on a one-worker thread pool as soon as it is constructed;
``.tree`` joins the worker and returns the finished ``PrefixTreeCPP``.  The
native calls release the GIL, so the build overlaps with Python-side work of
the caller.
"""
from __future__ import annotations

import time
from concurrent.futures import Future, ThreadPoolExecutor
from typing import List, Optional, Union

import torch

from ._prefix_attn import PrefixTreeCPP


class AsyncTree(PrefixTreeCPP):
    def __init__(self, block_size: int, seq_lens: Union[List[int], torch.Tensor], table: torch.Tensor,
                 MNWs: Union[None, List[List[int]]], HRatio: int, kvHead: int, device: torch.device):
        super().__init__(block_size)
        self._tree: Optional[PrefixTreeCPP] = None
        self._init_time = time.time()

        def job() -> PrefixTreeCPP:
            built = PrefixTreeCPP(block_size)
            built.build_radix_tree(seq_lens, table)
            built.pack_schedule(MNWs=MNWs, HRatio=HRatio, kvHead=kvHead)
            built.kernel_info.to_gpu(device)
            return built

        self._pool = ThreadPoolExecutor(max_workers=1)
        self._future: Optional[Future] = self._pool.submit(job)
        self._pool.shutdown(wait=False)

    @property
    def tree(self) -> Optional[PrefixTreeCPP]:
        """The built tree; blocks until the worker is done (errors re-raise here)."""
        if self._tree is None:
            self._tree = self._future.result()
        return self._tree
