"""Synthetic request generators and padding helpers.

Mirror of the reference's ``prefix_attn/utils.py``:
``generate_random_kv_cache`` (``:10-46``), ``generate_tree_seqs``
(``:49-100``), ``generate_random_prefix_seqs`` (``:105-164``) and the
``make_ndarray_with_pad`` / ``make_tensor_with_pad`` helpers (``:180-218``).
They consume Python's and torch's global generators in the same order as the
reference so that seeded runs give the same batches.
"""
from __future__ import annotations

import math
import random
from typing import Optional, Tuple, TypeVar, Union

import numpy as np
import torch

from .data_class import SeqGroup

T = TypeVar("T")

TORCH_DTYPE_TO_NUMPY_DTYPE = {
    torch.float16: np.float16,
    torch.float32: np.float32,
    torch.float64: np.float64,
    torch.uint8: np.uint8,
    torch.int32: np.int32,
    torch.int64: np.int64,
}


def generate_random_kv_cache(seq_group: SeqGroup, num_blocks: int, block_size: int, nheads_kv: int,
                             head_dim: int, dtype: torch.dtype = torch.float16, device: str = "cuda",
                             seed: int = 0):
    """Random paged K/V plus the dense per-request view of it.

    Returns ``(seqlens [B] i32, k_cache [B, S, Hkv, D], v_cache, kv_padding_mask
    [B, S] bool, block_table [B, max_blocks] i32 (0-padded), k_cache_paged
    [num_blocks, block_size, Hkv, D], v_cache_paged)`` with
    ``S = max_blocks * block_size``.
    """
    torch.random.manual_seed(seed)
    shape = (num_blocks, block_size, nheads_kv, head_dim)
    k_paged = torch.randn(*shape, dtype=dtype, device=device)
    v_paged = torch.randn(*shape, dtype=dtype, device=device)
    table = torch.tensor(seq_group.get_padded_block_ids(padding_value=0), dtype=torch.int32, device=device)
    batch = table.shape[0]
    k_dense = k_paged[table].reshape(batch, -1, nheads_kv, head_dim)
    v_dense = v_paged[table].reshape(batch, -1, nheads_kv, head_dim)
    seqlens = torch.tensor(seq_group.seqlens, dtype=torch.int32, device=device)
    span = seq_group.max_num_blocks * block_size
    mask = torch.arange(span, device=device)[None, :] < seqlens[:, None]
    return seqlens, k_dense, v_dense, mask, table, k_paged, v_paged


def generate_tree_seqs(tree: str, block_size: int) -> Tuple[SeqGroup, int]:
    """Requests laid out as a level tree, e.g. ``"1,2,4,8_64,256,512,32"``:
    left = nodes per level (the last is the batch size), right = tokens per
    node of that level (multiples of the page size).  Request ``i`` (before
    the random shuffle of positions) takes node ``i // (batch // nodes)`` on
    each level.  Returns ``(SeqGroup, total_pages)``."""
    left, right = tree.split("_")
    nodes = [int(x) for x in left.split(",")]
    tokens = [int(x) for x in right.split(",")]
    assert min(tokens) >= block_size, "every level must span at least one page"
    assert all(t % block_size == 0 for t in tokens), "level sizes must be whole pages"

    batch = nodes[-1]
    context = sum(tokens)
    group = SeqGroup(block_size, min_seqlen=context, max_seqlen=context, num_seqs=batch)

    next_page = 0
    level_pages = []
    for level, count in enumerate(nodes):
        per_node = tokens[level] // block_size
        pages = []
        for _ in range(count):
            pages.append(list(range(next_page, next_page + per_node)))
            next_page += per_node
        level_pages.append(pages)

    slots = list(range(batch))
    random.shuffle(slots)
    for i in range(batch):
        row = []
        for level, count in enumerate(nodes):
            row.extend(level_pages[level][i // (batch // count)])
        group.sequences[slots[i]].append_blocks(row, 0)
    return group, next_page


def generate_random_prefix_seqs(min_seqlen: int, max_seqlen: int, batch_size: int, num_prefix: int,
                                prefix_ratio: float, block_size: int, seed: int = 0) -> Tuple[SeqGroup, int]:
    """Requests that share one common prefix of ``ceil(max_blocks *
    prefix_ratio)`` pages (requests shorter than the prefix get none) followed
    by private pages.  Returns ``(SeqGroup, total_pages)``."""
    assert num_prefix <= batch_size
    random.seed(seed)
    max_blocks = math.ceil(max_seqlen / block_size)
    prefix_pages = math.ceil(max_blocks * prefix_ratio)

    group = SeqGroup(block_size, min_seqlen, max_seqlen, batch_size)
    common = random.sample(range(0, prefix_pages), prefix_pages)
    group.set_common_prefix_blocks(common)
    total = len(common)

    for seq in group.sequences:
        if seq.seqlen < block_size * prefix_pages:
            private_tokens = seq.seqlen
        else:
            private_tokens = seq.seqlen - prefix_pages * block_size
        if private_tokens > 0:
            count = math.ceil(private_tokens / block_size)
            pages = random.sample(range(total, total + count), count)
            seq.append_blocks(pages, 0)
            total += count
    return group, total


def make_ndarray_with_pad(x, pad, dtype, max_len: Optional[int] = None) -> np.ndarray:
    """Ragged rows -> one ``[len(x), max_len]`` array filled with ``pad``."""
    if max_len is None:
        max_len = max(map(len, x), default=0)
    out = np.full((len(x), max_len), pad, dtype=dtype)
    for i, row in enumerate(x):
        assert len(row) <= max_len
        out[i, :len(row)] = row
    return out


def make_tensor_with_pad(x, pad, dtype: torch.dtype, max_len: Optional[int] = None,
                         device: Optional[Union[str, torch.device]] = None,
                         pin_memory: bool = False) -> torch.Tensor:
    """Tensor version of ``make_ndarray_with_pad``."""
    arr = make_ndarray_with_pad(x, pad, TORCH_DTYPE_TO_NUMPY_DTYPE[dtype], max_len=max_len)
    tensor = torch.from_numpy(arr).to(device)
    return tensor.pin_memory() if pin_memory else tensor
