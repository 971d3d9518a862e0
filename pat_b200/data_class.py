"""Host-side metadata objects of the prefix-aware decode-attention path.

These mirror the reference's ``prefix_attn/data_class.py`` (``Sequence`` /
``SeqGroup`` ``:22-98``, ``PackedBox`` ``:101-171``, ``KernelInfo``
``:173-254``, ``create_seq_group`` ``:257-264``): same names, fields and
behaviour, so that schedulers, tests and the serving plugin written against
the reference keep working.  ``KernelInfo.to_tensor`` additionally remembers
the host copy of the plan so that the CUDA path can build its device work
list without reading the tables back from the GPU.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Iterator, List, Optional, Sequence as _Seq, Union

import torch


def make_tensor_merge_split(x, device, dtype: torch.dtype = torch.int32, pad=0,
                            pin_memory: bool = True) -> Iterator[torch.Tensor]:
    """Pad ragged rows to one 2-D tensor, build it once and hand back one view
    per row trimmed to its own length (reference ``data_class.py:8-19``)."""
    sizes = [len(row) for row in x]
    width = max(sizes)
    padded = [list(row) + [pad] * (width - len(row)) for row in x]
    merged = torch.tensor(padded, device=device, dtype=dtype, pin_memory=pin_memory)
    return (merged[i][: sizes[i]] for i in range(len(sizes)))


class Sequence:
    """One request: its physical page ids and its context length in tokens."""

    def __init__(self, block_size, seqlen=0):
        self.block_ids = []
        self.block_size = block_size
        self.seqlen = seqlen

    def append_blocks(self, blocks: List[int], tokens=None):
        """Append pages; the length grows by whole pages unless ``tokens``
        says how many tokens they add (0 = pages of an already counted span)."""
        self.block_ids.extend(blocks)
        self.seqlen += len(blocks) * self.block_size if tokens is None else tokens


class SeqGroup:
    """A batch of ``Sequence`` objects (reference ``data_class.py:39-98``).

    ``num_seqs`` sequences are created with lengths drawn by
    ``random.randint(min_seqlen, max_seqlen)`` from Python's global generator,
    one draw per sequence in order.
    """

    def __init__(self, block_size, min_seqlen=0, max_seqlen=0, num_seqs=0):
        self.sequences = [Sequence(block_size, random.randint(min_seqlen, max_seqlen))
                          for _ in range(num_seqs)]
        self.is_sorted = False

    def __len__(self):
        return len(self.sequences)

    def __str__(self):
        rows = [f"\n[{', '.join(map(str, s.block_ids))}], seqlen={s.seqlen}" for s in self.sequences]
        return f"SeqGroup: {', '.join(rows)}"

    @property
    def seqlens(self):
        return [s.seqlen for s in self.sequences]

    @property
    def max_seqlen(self):
        return max(s.seqlen for s in self.sequences)

    @property
    def max_num_blocks(self):
        return max(len(s.block_ids) for s in self.sequences)

    def set_common_prefix_blocks(self, prefix_blocks: List[int]):
        """Give every sequence that is at least as long as the prefix the same
        leading pages (shorter ones are skipped); lengths are unchanged."""
        span = len(prefix_blocks)
        for s in self.sequences:
            if s.seqlen >= s.block_size * span:
                s.append_blocks(prefix_blocks, 0)

    def add_random_prefix_blocks(self, random_blocks: List[List[int]]):
        for s in self.sequences:
            s.append_blocks(random_blocks[random.randint(0, len(random_blocks) - 1)])
        self.is_sorted = False

    def get_padded_block_ids(self, padding_value=-1) -> List[List[int]]:
        width = self.max_num_blocks
        return [s.block_ids + [padding_value] * (width - len(s.block_ids)) for s in self.sequences]

    def get_block_ids(self) -> List[List[int]]:
        return [list(s.block_ids) for s in self.sequences]

    def sort(self, reverse: bool = False) -> None:
        self.sequences.sort(key=lambda s: s.block_ids, reverse=reverse)
        self.is_sorted = True


def _pad_rows(rows, pad=0):
    width = max(len(r) for r in rows)
    return [list(r) + [pad] * (width - len(r)) for r in rows]


@dataclass
class PackedBox:
    """One unit of work of the reference plan: the queries ``q_table`` (times
    all their heads) attend to the first ``kv_in_CTA`` tokens of the pages in
    ``block_table``; ``CTA_rank`` is the partial slot the reference kernel
    writes (reference ``data_class.py:101-171``).  The legacy v0 planners use
    the same class with list-valued fields (one entry per box)."""

    q_table: Union[list, torch.Tensor] = field(default_factory=list)
    block_table: Union[list, torch.Tensor] = field(default_factory=list)
    num_seqs_per_CTA: Union[list, int, torch.Tensor] = field(default_factory=list)
    CTA_rank: Union[list, int, torch.Tensor] = field(default_factory=list)
    kv_in_CTA: Union[list, int, torch.Tensor] = field(default_factory=list)

    def __str__(self):
        return ("PackedBox("
                f"\n\tq_table={self.q_table},"
                f"\n\tblock_table={self.block_table},"
                f"\n\tnum_seqs_per_CTA={self.num_seqs_per_CTA},"
                f"\n\tCTA_rank={self.CTA_rank},"
                f"\n\tkv_in_CTA={self.kv_in_CTA},"
                ")")

    def __lt__(self, other):
        # "smaller" means more KV, so that a min-heap pops the longest box.
        return self.kv_in_CTA > other.kv_in_CTA

    def sort_by_kv_desc(self):
        """Reorder the (list-valued) fields so that boxes with more KV come
        first; stable for ties."""
        order = sorted(range(len(self.kv_in_CTA)), key=self.kv_in_CTA.__getitem__, reverse=True)
        for name in ("q_table", "block_table", "num_seqs_per_CTA", "CTA_rank", "kv_in_CTA"):
            values = getattr(self, name)
            setattr(self, name, [values[i] for i in order])

    def to_tensor(self, device):
        def as_i32(x):
            return torch.tensor(x, device=device, dtype=torch.int32)

        if not isinstance(self.num_seqs_per_CTA, torch.Tensor):
            self.num_seqs_per_CTA = as_i32(self.num_seqs_per_CTA)
            self.CTA_rank = as_i32(self.CTA_rank)
            self.kv_in_CTA = as_i32(self.kv_in_CTA)
        if not isinstance(self.q_table, torch.Tensor):
            self.q_table = as_i32(_pad_rows(self.q_table))
        if not isinstance(self.block_table, torch.Tensor):
            self.block_table = as_i32(_pad_rows(self.block_table))


@dataclass
class KernelInfo:
    """The whole plan of one decode step, bucketed by tile shape ``[M, N, W]``
    (reference ``data_class.py:173-254``).

    Per bucket ``i``: ``q_tables[i]`` ``[CTAs, max_seqs]``, ``block_tables[i]``
    ``[CTAs, max_blocks]`` (ragged lists, zero-padded once on the device),
    ``num_seqs_per_CTAs[i]``, ``CTA_ranks[i]``, ``kv_in_CTAs[i]`` ``[CTAs]``,
    ``MNWs[i]``.  Shared: ``num_split_per_seq`` ``[batch]`` and the three
    maxima.  ``sort_index`` / ``reverse_index`` are only set by the legacy
    sorting planner.
    """

    q_tables: list = field(default_factory=list)
    block_tables: list = field(default_factory=list)
    num_seqs_per_CTAs: list = field(default_factory=list)
    CTA_ranks: list = field(default_factory=list)
    kv_in_CTAs: list = field(default_factory=list)
    MNWs: List[List[int]] = field(default_factory=list)

    num_split_per_seq: Union[list, torch.Tensor] = field(default_factory=list)
    max_split_per_seq: int = 0
    max_seqs_in_CTA: int = 0
    max_blocks_in_CTA: int = 0
    reverse_index: Optional[Union[list, torch.Tensor]] = None
    sort_index: Optional[Union[list, torch.Tensor]] = None

    def host_plan(self):
        """The plan as plain Python lists (``None`` once only tensors remain
        and no host copy was kept)."""
        return getattr(self, "_host_plan", None)

    def to_tensor(self, device):
        """Turn every list field into an int32 tensor on ``device``; ragged
        tables are padded with 0.  Idempotent."""
        from . import _plan_cache

        was_lists = (not isinstance(self.num_split_per_seq, torch.Tensor)
                     and all(not isinstance(t, torch.Tensor) for t in self.block_tables))
        if was_lists:
            _plan_cache.remember_host_plan(self)

        def as_i32(x):
            return torch.tensor(x, device=device, dtype=torch.int32)

        if not isinstance(self.num_split_per_seq, torch.Tensor):
            self.num_split_per_seq = as_i32(self.num_split_per_seq)
        if self.reverse_index is not None and not isinstance(self.reverse_index, torch.Tensor):
            self.reverse_index = as_i32(self.reverse_index)
        if self.sort_index is not None and not isinstance(self.sort_index, torch.Tensor):
            self.sort_index = as_i32(self.sort_index)

        def listed(seq):   # a list that still holds Python lists (not yet converted)
            return not isinstance(seq, torch.Tensor) and not all(isinstance(t, torch.Tensor) for t in seq)

        if listed(self.num_seqs_per_CTAs):
            self.num_seqs_per_CTAs = [as_i32(x) for x in self.num_seqs_per_CTAs]
        if not all(isinstance(t, torch.Tensor) for t in self.q_tables):
            self.q_tables = [as_i32(_pad_rows(t)) for t in self.q_tables]
        if listed(self.CTA_ranks):
            self.CTA_ranks = [as_i32(x) for x in self.CTA_ranks]
        if listed(self.kv_in_CTAs):
            self.kv_in_CTAs = [as_i32(x) for x in self.kv_in_CTAs]
        if not all(isinstance(t, torch.Tensor) for t in self.block_tables):
            self.block_tables = [as_i32(_pad_rows(t)) for t in self.block_tables]

        if was_lists:
            _plan_cache.attach_to_tensors(self)


def create_seq_group(block_tables: List[List[int]], seq_lens: List[int], block_size: int):
    """A ``SeqGroup`` holding exactly the given tables and lengths."""
    group = SeqGroup(block_size=block_size, num_seqs=len(block_tables))
    for seq, table, length in zip(group.sequences, block_tables, seq_lens):
        seq.block_ids = table
        seq.seqlen = length
    return group
