"""Legacy ("v0") planners kept for API compatibility.

Mirror of the reference's ``prefix_attn/block_scheduler.py``:

* ``schedule`` (``:348-505``) - sort the padded block table lexicographically,
  then sweep one page pointer per request, grouping runs of adjacent requests
  that sit on the same page into boxes of at most ``k`` queries.  The plan
  refers to requests in *sorted* order; ``sort_index`` / ``reverse_index`` tell
  the caller how to permute queries and outputs.
* ``schedule_naive`` (``:508-553``) - one box per request, no sharing.
* ``distribute_naive`` / ``distribute_multi_stream`` (``:205-328``) - spread
  the boxes of a flat plan over tile-shape buckets.
* ``pack_prefix_blocks`` / ``pack_without_prefix`` / ``pack_schedule``
  (``:9-202``, ``:331-345``) - older entry points.  As shipped in the reference
  they fail at the first statement that touches ``PackedBox`` / ``PrefixTree``
  with fields those classes no longer have; here they run and return what
  their docstrings describe (a flat plan with the shared fields attached).
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from .data_class import KernelInfo, PackedBox, SeqGroup
from .prefix_tree import PrefixTree
from .utils import make_ndarray_with_pad


class _FlatPlan(PackedBox):
    """``PackedBox`` with list-valued fields plus the shared per-batch fields
    the oldest entry points return on the same object."""

    def __init__(self, **kw):
        shared = {k: kw.pop(k) for k in ("num_split_per_seq", "max_split_per_seq", "max_seqs_in_CTA",
                                         "max_blocks_in_CTA", "sort_index", "reverse_index") if k in kw}
        super().__init__(**kw)
        self.num_split_per_seq = shared.get("num_split_per_seq", [])
        self.max_split_per_seq = shared.get("max_split_per_seq", 0)
        self.max_seqs_in_CTA = shared.get("max_seqs_in_CTA", 0)
        self.max_blocks_in_CTA = shared.get("max_blocks_in_CTA", 0)
        self.sort_index = shared.get("sort_index")
        self.reverse_index = shared.get("reverse_index")


def _sweep(tables: List[List[int]], seq_lens: List[int], block_size: int, k: int, wrap_single: bool):
    """The pointer sweep shared by ``schedule`` and ``pack_prefix_blocks``.

    Returns ``(plan, split_per_seq, max_seqs_in_CTA, max_blocks_in_CTA)``.
    ``wrap_single`` selects whether ``q_table`` entries are query lists
    (``schedule``) or the first query id only (``pack_prefix_blocks``).
    """
    n = len(tables)
    cursor = [0] * n
    splits = [0] * n
    plan = _FlatPlan()
    max_seqs, max_blocks = 1, 0

    def pending(i):
        return cursor[i] < len(tables[i])

    while any(pending(i) for i in range(n)):
        # runs of consecutive request ids sitting on the same page
        runs_by_page: Dict[int, List[List[int]]] = {}
        for i in range(n):
            if not pending(i):
                continue
            runs = runs_by_page.setdefault(tables[i][cursor[i]], [[]])
            if not runs[-1] or i == runs[-1][-1] + 1:
                runs[-1].append(i)
            else:
                runs.append([i])

        for runs in runs_by_page.values():
            for members in runs:
                if len(members) == 1:
                    # alone on its page: everything that is left goes in one box
                    s = members[0]
                    rest = tables[s][cursor[s]:]
                    plan.q_table.append([s] if wrap_single else s)
                    plan.CTA_rank.append(splits[s])
                    plan.kv_in_CTA.append(seq_lens[s] - cursor[s] * block_size)
                    plan.block_table.append(rest)
                    plan.num_seqs_per_CTA.append(1)
                    max_blocks = max(max_blocks, len(rest))
                    cursor[s] = len(tables[s])
                    splits[s] += 1
                    continue
                for lo in range(0, len(members), k):
                    chosen = members[lo:lo + k]
                    shared: List[int] = []
                    hit_end = False
                    while True:
                        if any(not pending(p) for p in chosen):
                            hit_end = True
                            break
                        page = tables[chosen[0]][cursor[chosen[0]]]
                        if not all(pending(p) and tables[p][cursor[p]] == page for p in chosen):
                            break
                        shared.append(page)
                        for p in chosen:
                            cursor[p] += 1
                    if not shared:
                        continue
                    max_seqs = max(max_seqs, len(chosen))
                    first = chosen[0]
                    plan.q_table.append(chosen if wrap_single else first)
                    plan.block_table.append(list(shared))
                    plan.num_seqs_per_CTA.append(len(chosen))
                    plan.CTA_rank.append(splits[first])
                    if hit_end:
                        pages_total = len(tables[first])
                        kv = block_size * (len(shared) - 1) + seq_lens[first] - (pages_total - 1) * block_size
                    else:
                        kv = block_size * len(shared)
                    plan.kv_in_CTA.append(kv)
                    max_blocks = max(max_blocks, len(shared))
                    for p in chosen:
                        splits[p] += 1
    return plan, splits, max_seqs, max_blocks


def pack_prefix_blocks(seq_group: SeqGroup, block_size: int, k: int = 64) -> PackedBox:
    """Flat plan of a *sorted* ``SeqGroup``: boxes over multi-level shared
    prefixes, at most ``k`` (<= 64) queries each.  ``q_table`` holds the first
    query of each box (queries of a box are consecutive)."""
    assert seq_group.is_sorted, "SeqGroup must be sorted"
    assert k <= 64, "max number of sequences in a CTA should be less than 64"
    tables = [s.block_ids for s in seq_group.sequences]
    lens = [s.seqlen for s in seq_group.sequences]
    plan, splits, max_seqs, max_blocks = _sweep(tables, lens, block_size, k, wrap_single=False)
    n = len(tables)
    plan.num_split_per_seq = list(splits)
    plan.max_split_per_seq = max(splits)
    plan.max_seqs_in_CTA = max_seqs
    plan.max_blocks_in_CTA = max_blocks
    plan.sort_index = np.arange(n)
    plan.reverse_index = np.arange(n)
    return plan


def pack_without_prefix(seq_group: SeqGroup, block_size: int) -> PackedBox:
    """Flat plan with one box per request and no sharing."""
    n = len(seq_group)
    return _FlatPlan(
        q_table=list(range(n)),
        block_table=seq_group.get_block_ids(),
        num_seqs_per_CTA=[1] * n,
        num_split_per_seq=[1] * n,
        CTA_rank=[0] * n,
        kv_in_CTA=[s.seqlen for s in seq_group.sequences],
        max_split_per_seq=1,
        max_seqs_in_CTA=1,
        max_blocks_in_CTA=seq_group.max_num_blocks,
    )


def _empty_lanes(n):
    return ([[] for _ in range(n)] for _ in range(5))


def _flush(info: KernelInfo, lanes, tile_types):
    q, blk, ns, rank, kv = lanes
    for i, mnw in enumerate(tile_types):
        if not q[i]:
            continue
        info.q_tables.append(q[i])
        info.block_tables.append(blk[i])
        info.num_seqs_per_CTAs.append(ns[i])
        info.CTA_ranks.append(rank[i])
        info.kv_in_CTAs.append(kv[i])
        info.MNWs.append(mnw)


def distribute_naive(kernel_information: KernelInfo, Box: PackedBox, h_q_kv_ratio: int = 1,
                     qkv_tile_types: List[List[int]] = None, d: int = 128):
    """Put each box of the flat plan into the first tile type (listed large to
    small) whose M holds its rows; boxes that fit nowhere are dropped."""
    if qkv_tile_types is None:
        qkv_tile_types = [[64, 128, 4]] if d == 128 else [[64, 256, 4]]
    lanes = tuple(_empty_lanes(len(qkv_tile_types)))
    for i in range(len(Box.q_table)):
        rows = Box.num_seqs_per_CTA[i] * h_q_kv_ratio
        for lane, (tile_q, _tile_kv, _warps) in enumerate(qkv_tile_types):
            if rows <= tile_q:
                for dst, src in zip(lanes, (Box.q_table, Box.block_table, Box.num_seqs_per_CTA,
                                            Box.CTA_rank, Box.kv_in_CTA)):
                    dst[lane].append(src[i])
                break
    _flush(kernel_information, lanes, qkv_tile_types)


def distribute_multi_stream(kernel_information: KernelInfo, Box: PackedBox, h_q_kv_ratio: int = 1,
                            qkv_tile_types: List[List[int]] = None, d: int = 128):
    """Bucket by rows and KV length for the fixed 8-entry tile list
    ``[[128,16,4],[64,128,4],[64,64,4],[64,32,4],[64,16,4],[32,32,2],[32,16,2],[16,16,1]]``;
    boxes of 65..128 rows with more than 16 tokens are cut in two and
    bucketed in a second pass."""
    if qkv_tile_types is None:
        qkv_tile_types = [[64, 128, 4]] if d == 128 else [[64, 256, 4]]
    lanes = tuple(_empty_lanes(len(qkv_tile_types)))
    fields = (Box.q_table, Box.block_table, Box.num_seqs_per_CTA, Box.CTA_rank, Box.kv_in_CTA)

    def put(lane, i):
        for dst, src in zip(lanes, fields):
            dst[lane].append(src[i])

    def bucket(lo, hi):
        for i in range(lo, hi):
            kv = Box.kv_in_CTA[i]
            rows = Box.num_seqs_per_CTA[i] * h_q_kv_ratio
            if rows <= 16:
                put(7, i)
            elif rows <= 32:
                put(6 if kv <= 16 else 5, i)
            elif rows <= 64:
                put(4 if kv <= 16 else 3 if kv <= 32 else 2 if kv <= 64 else 1, i)
            elif rows <= 128:
                if kv <= 16:
                    put(0, i)
                    continue
                per_half = 64 // h_q_kv_ratio
                Box.q_table.append(Box.q_table[i])
                Box.block_table.append(Box.block_table[i])
                Box.num_seqs_per_CTA.append(per_half)
                Box.CTA_rank.append(Box.CTA_rank[i])
                Box.kv_in_CTA.append(kv)
                Box.q_table.append(Box.q_table[i] + per_half)
                Box.block_table.append(Box.block_table[i])
                Box.num_seqs_per_CTA.append((rows - 64) // h_q_kv_ratio)
                Box.CTA_rank.append(Box.CTA_rank[i])
                Box.kv_in_CTA.append(kv)

    first_pass = len(Box.q_table)
    bucket(0, first_pass)
    bucket(first_pass, len(Box.q_table))
    _flush(kernel_information, lanes, qkv_tile_types)


def pack_schedule(seq_lens, block_table: torch.Tensor, block_size: int, MNWs: List[List[int]] = None,
                  h_q_kv_ratio: int = 1) -> KernelInfo:
    """Tree plan from a padded block-table tensor: rows are cut to
    ``ceil(len / block_size)`` pages, then the radix-tree packer runs."""
    table = block_table.cpu().numpy()
    rows = [table[i][:(seq_lens[i] + block_size - 1) // block_size].tolist() for i in range(len(seq_lens))]
    tree = PrefixTree(block_size)
    tree.build_radix_tree(list(seq_lens), rows)
    return tree.pack_schedule(MNWs, h_q_kv_ratio)


def schedule(seq_lens: List[int], block_table: List[List[int]], block_size: int, k: int,
             qkv_tile_types: List[List[int]], h_q_kv_ratio: int = 1) -> KernelInfo:
    """Sort-then-sweep planner; needs no pre-sorted input.  Query ids in the
    plan index the *sorted* batch (``sort_index``)."""
    if qkv_tile_types is None:
        qkv_tile_types = [[64, 128, 4]]
    padded = make_ndarray_with_pad(block_table, 0, np.int32)
    order = np.lexsort(padded[:, ::-1].T)
    lens = [seq_lens[i] for i in order]
    padded = padded[order]
    tables = [padded[i][:(lens[i] + block_size - 1) // block_size].tolist() for i in range(len(lens))]

    plan, splits, max_seqs, max_blocks = _sweep(tables, lens, block_size, k, wrap_single=True)
    info = KernelInfo(max_split_per_seq=max(splits), max_seqs_in_CTA=max_seqs,
                      max_blocks_in_CTA=max_blocks, num_split_per_seq=list(splits),
                      reverse_index=np.argsort(order).tolist(), sort_index=order.tolist())
    distribute_naive(info, plan, h_q_kv_ratio, qkv_tile_types)
    return info


def schedule_naive(seq_lens: List[int], block_table: List[List[int]], device: torch.device) -> KernelInfo:
    """One box per request over its whole context, already as device tensors,
    in batch order (identity ``sort_index``)."""
    assert isinstance(seq_lens, list)
    assert isinstance(block_table, list)
    padded = make_ndarray_with_pad(block_table, 0, np.int32)
    n = len(seq_lens)
    order = torch.from_numpy(np.arange(padded.shape[0])).to(device)
    i32 = dict(dtype=torch.int32, device=device)
    return KernelInfo(
        q_tables=[torch.arange(n, **i32)[order]],
        block_tables=[torch.from_numpy(padded).to(device)[order]],
        num_seqs_per_CTAs=[torch.ones(n, **i32)[order]],
        num_split_per_seq=torch.ones(n, **i32)[order],
        CTA_ranks=[torch.zeros(n, **i32)[order]],
        kv_in_CTAs=[torch.tensor(seq_lens, **i32)[order]],
        MNWs=[[64, 128, 4]],
        max_split_per_seq=1,
        max_seqs_in_CTA=1,
        max_blocks_in_CTA=max(len(row) for row in padded),
        reverse_index=torch.from_numpy(np.argsort(np.arange(padded.shape[0]))).to(device),
        sort_index=order,
    )
