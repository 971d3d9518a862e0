"""Pure-Python radix tree over physical page ids and the tile-plan packer.

Host-side mirror of the reference scheduler ``prefix_attn/prefix_tree.py``
(class ``PrefixTree``): the same public attributes and methods, producing
bit-identical trees and plans.  The native scheduler behind ``PrefixTreeCPP``
implements the same algorithm in C++; this module is the readable
specification of it and the one the reference's kernel benchmark uses
(``benchmark/benchmark_kernel.py:234-243``).

Algorithm (reference line numbers in brackets):

* ``insert`` / ``build_radix_tree`` [``:95-149``] - radix tree whose edges are
  runs of page ids, children keyed by the first page id of the edge; an edge
  is split at the longest common page prefix.
* ``_tree_heuristics`` [``:269-323``] - DFS deciding per child whether the
  node's KV is folded into the child ("merge") or computed once for the
  remaining queries and combined later ("split"); boxes of at most
  ``mm = max_M // HRatio`` queries.
* ``_compute_model_tree_heuristics`` [``:16-45``, ``:325-381``] - the same walk
  with a padded-matmul cost model deciding instead.
* ``balancePack`` [``:383-460``] - crop boxes far longer than average, then
  halve the longest box until there are enough boxes to fill the GPU.
* ``getMNW`` / ``pack_schedule`` [``:462-482``, ``:548-616``] - bucket boxes by
  tile shape and emit a ``KernelInfo``.
"""
from __future__ import annotations

from collections import defaultdict
from concurrent.futures import Future
from math import ceil
from threading import Thread
from typing import Callable, DefaultDict, Dict, List, Optional

import torch

from .data_class import KernelInfo, PackedBox

DEFAULT_MNWS = (
    (64, 128, 4), (64, 64, 4), (64, 32, 4),
    (32, 128, 2), (32, 64, 2), (32, 32, 2), (32, 16, 2),
    (16, 128, 1), (16, 64, 1), (16, 32, 1), (16, 16, 1),
)


def _default_buckets() -> List[List[int]]:
    return [list(b) for b in DEFAULT_MNWS]


# --- cost model of the alternative heuristic (reference :16-45) -------------

def _CpadQ(TS, N):
    """Rows of padding when ``N`` rows are tiled by ``TS``."""
    return TS - ((N - 1) % TS + 1)


def _Cmm(nQ, nK, HRatio):
    tile = 64 if nQ * HRatio >= 64 else 16
    return _CpadQ(tile, nQ) * nK * HRatio


def _Cred(nQl, HRatio):
    return 0.1 * nQl * HRatio


def _SplitQCost(nQcurr, nQl, lenv, lenl, HRatio):
    return _Cmm(nQcurr - nQl, lenv, HRatio) + _Cmm(nQl, lenv + lenl, HRatio)


def _SplitKCost(nQcurr, nQl, lenl, lenv, HRatio):
    return _Cmm(nQcurr, lenv, HRatio) + _Cmm(nQl, lenl, HRatio) + _Cred(nQl, HRatio)


class PrefixTree:
    """Radix tree of a decode batch plus the packer that turns it into a plan.

    Nodes live in parallel lists indexed by node id (``parents``, ``s_values``
    = number of requests through the node, ``lens`` = valid tokens on the edge,
    ``seq_indices``, ``block_ids``); ``tree[node]`` maps the first page id of a
    child edge to the child's id, in insertion order.
    """

    def __init__(self, block_size):
        self.block_size = block_size
        self.parents: List[int] = []
        self.s_values: List[int] = []
        self.lens: List[int] = []
        self.seq_indices: List[List[int]] = []
        self.block_ids: List[List[int]] = []
        self.tree: DefaultDict[int, Dict[int, int]] = defaultdict(dict)
        self.num_nodes = 0
        self.root = self.add_node(-1)
        self.split_per_seq: List[int] = []

    # ------------------------------------------------------------------ tree
    def add_node(self, parent: int = -1, s_value: int = 1, length: int = 0,
                 seq_indices: Optional[List[int]] = None,
                 block_ids: Optional[List[int]] = None) -> int:
        nid = self.num_nodes
        self.num_nodes = nid + 1
        self.parents.append(parent)
        self.s_values.append(s_value)
        self.lens.append(length)
        self.seq_indices.append([] if seq_indices is None else seq_indices)
        self.block_ids.append([] if block_ids is None else block_ids)
        return nid

    def get_common_block_length(self, blocks1, blocks2):
        """Index of the last position at which the two page lists still agree
        (-1 if they differ at once), found by bisection: like the reference it
        assumes that agreement at ``i`` implies agreement before ``i``."""
        lo, hi = -1, min(len(blocks1), len(blocks2))
        while hi - lo > 1:
            mid = (lo + hi) >> 1
            if blocks1[mid] == blocks2[mid]:
                lo = mid
            else:
                hi = mid
        return lo

    def insert(self, sId, seq_len, blocks):
        bs = self.block_size
        at = self.root
        left = len(blocks)
        while left:
            kids = self.tree[at]
            head = blocks[0]
            if head not in kids:
                kids[head] = self.add_node(at, 1, seq_len, [sId], blocks)
                return
            child = kids[head]
            edge = self.block_ids[child]
            shared = self.get_common_block_length(blocks, edge) + 1
            if shared == len(edge):
                # the whole edge matches: walk down
                self.s_values[child] += 1
                self.seq_indices[child].append(sId)
                at = child
                left -= shared
                seq_len -= shared * bs
                blocks = blocks[shared:]
                continue
            # split the edge after `shared` pages
            mid = self.add_node(at, self.s_values[child] + 1, shared * bs,
                                self.seq_indices[child].copy(), edge[:shared])
            self.tree[mid][edge[shared]] = child
            kids[edge[0]] = mid
            self.parents[child] = mid
            self.block_ids[child] = edge[shared:]
            self.lens[child] -= shared * bs
            self.seq_indices[mid].append(sId)
            if shared != left:
                rest = blocks[shared:]
                leaf = self.add_node(mid, 1, min(left * bs, seq_len) - shared * bs, [sId], rest)
                self.tree[mid][rest[0]] = leaf
            return

    def build_radix_tree(self, seq_lens: List[int], block_table: List[List[int]]):
        """Insert every request (unpadded page lists) in batch order."""
        for i, blocks in enumerate(block_table):
            self.insert(i, seq_lens[i], blocks)
        self.split_per_seq = [0] * len(block_table)

    def build_from_batch(self, seq_lens: List[int], block_table: List[List[int]]):
        """Build the tree from the lexicographically sorted batch, extending
        the path of the previous request (reference ``:151-257``)."""
        if not block_table:
            return
        bs = self.block_size
        order = sorted(zip(range(len(block_table)), seq_lens, block_table), key=lambda t: t[2])
        last = -1
        prev: List[int] = []
        for sId, seq_len, cur in order:
            if last == -1:
                if cur:
                    last = self.add_node(parent=self.root, length=seq_len, seq_indices=[sId], block_ids=cur)
                    self.tree[self.root][cur[0]] = last
                else:
                    self.s_values[self.root] += 1
                    self.seq_indices[self.root].append(sId)
                    last = self.root
                prev = cur
                continue

            lcp = 0
            if prev and cur and prev[0] == cur[0]:
                lcp = self.get_common_block_length(prev, cur) + 1

            # climb from the previous leaf until the path is no longer than lcp
            depth = len(prev)
            node = last
            while depth > lcp:
                edge = len(self.block_ids[node])
                if depth - edge < lcp:
                    break
                depth -= edge
                node = self.parents[node]
            above = self.parents[node]

            if depth > lcp:
                cut = len(self.block_ids[node]) - (depth - lcp)
                head = self.block_ids[node][:cut]
                tail = self.block_ids[node][cut:]
                mid = self.add_node(parent=above, s_value=self.s_values[node] + 1, length=cut * bs,
                                    seq_indices=self.seq_indices[node].copy(), block_ids=head)
                self.tree[mid][tail[0]] = node
                self.tree[above][self.block_ids[node][0]] = mid
                self.parents[node] = mid
                self.block_ids[node] = tail
                self.lens[node] -= cut * bs
                rest = cur[lcp:]
                leaf = self.add_node(parent=mid, length=seq_len - lcp * bs, seq_indices=[sId], block_ids=rest)
                self.tree[mid][rest[0]] = leaf
                self.seq_indices[mid].append(sId)
                last = leaf
                fork = mid
            else:
                fork = node
                rest = cur[lcp:]
                if rest:
                    leaf = self.add_node(parent=fork, length=seq_len - lcp * bs, seq_indices=[sId], block_ids=rest)
                    self.tree[fork][rest[0]] = leaf
                    last = leaf
                else:
                    last = fork

            up = fork
            while up != -1:
                if sId not in self.seq_indices[up]:
                    self.s_values[up] += 1
                    self.seq_indices[up].append(sId)
                if up == self.root:
                    break
                up = self.parents[up]
            prev = cur
        self.split_per_seq = [0] * len(block_table)

    def print_tree(self):
        def show(node, indent):
            print(" " * indent + f"Node {node}: S={self.s_values[node]}, len={self.lens[node]}, "
                  f"seqs={self.seq_indices[node]}, blocks={self.block_ids[node]}")
            for child in self.tree[node]:
                show(child, indent + 2)
        show(self.root, 0)

    # --------------------------------------------------------------- packing
    def _emit_boxes(self, queries: List[int], count: int, mm: int, pages: List[int], kv_len: int,
                    out: List[PackedBox]) -> None:
        """Boxes of at most ``mm`` queries over one page list.  ``count`` (not
        ``len(queries)``) drives the chunking, exactly as the reference does;
        the rank of a box is the current split count of its first query."""
        for s in range(0, count, mm):
            box = PackedBox()
            box.q_table = queries[s:min(s + mm, count)]
            box.block_table = pages
            box.num_seqs_per_CTA = min(mm, count - s)
            box.kv_in_CTA = kv_len
            box.CTA_rank = self.split_per_seq[box.q_table[0]]
            for q in box.q_table:
                self.split_per_seq[q] += 1
            out.append(box)

    def _walk(self, node: int, mm: int, inherited: List[int],
              fold: Callable[[int, int, int, int], bool]) -> List[PackedBox]:
        """Shared DFS of both heuristics; ``fold(S_now, child, kv_len, node)``
        says whether the child absorbs this node's KV."""
        boxes: List[PackedBox] = []
        kids = self.tree[node]
        if len(kids) == 0:
            kv_len = self.block_size * len(inherited) + self.lens[node]
            self._emit_boxes(self.seq_indices[node], self.s_values[node], mm,
                             inherited + self.block_ids[node], kv_len, boxes)
            return boxes
        children = list(kids.values())
        remaining = self.s_values[node]
        kv_len = self.block_size * len(inherited) + self.lens[node]
        folded, separate = [], []
        for child in children:
            if fold(remaining, child, kv_len, node):
                remaining -= self.s_values[child]
                folded.append(child)
            else:
                separate.append(child)
        if remaining != 0:
            queries: List[int] = []
            for child in separate:
                queries.extend(self.seq_indices[child])
            for s in range(0, remaining, mm):
                self._emit_boxes(queries[s:min(s + mm, remaining)], min(mm, remaining - s), mm,
                                 inherited + self.block_ids[node], kv_len, boxes)
        for child in separate:
            boxes.extend(self._walk(child, mm, [], fold))
        for child in folded:
            boxes.extend(self._walk(child, mm, inherited + self.block_ids[node], fold))
        return boxes

    def _tree_heuristics(self, node, mm, inherited_block_id: List[int]) -> List[PackedBox]:
        def fold(S, child, kv_len, _node):
            sc = self.s_values[child]
            if S == sc:
                return True
            saved_tiles = ceil(S / mm) - ceil((S - sc) / mm) - ceil(sc / mm)
            return saved_tiles * kv_len + 4 * sc >= 0
        return self._walk(node, mm, inherited_block_id, fold)

    def _compute_model_tree_heuristics(self, node, mm, HRatio, inherited_block_id: List[int]) -> List[PackedBox]:
        def fold(S, child, kv_len, _node):
            sc, lc = self.s_values[child], self.lens[child]
            return _SplitKCost(S, sc, kv_len, lc, HRatio) > _SplitQCost(S, sc, kv_len, lc, HRatio)
        return self._walk(node, mm, inherited_block_id, fold)

    def balancePack(self, PackedBoxs: List[PackedBox], kvHead) -> List[PackedBox]:
        if len(PackedBoxs) == 0:
            return []
        bs = self.block_size
        counts = self.split_per_seq

        def piece(src: PackedBox, pages, kv_len, rank) -> PackedBox:
            b = PackedBox()
            b.q_table = src.q_table
            b.block_table = pages
            b.num_seqs_per_CTA = src.num_seqs_per_CTA
            b.kv_in_CTA = kv_len
            b.CTA_rank = rank
            return b

        # phase 1: crop boxes that are much longer than the average long box
        long_pages = [len(b.block_table) for b in PackedBoxs if b.kv_in_CTA > 256]
        if long_pages:
            average = sum(long_pages) / len(long_pages)
            limit = average * 5
            cropped: List[PackedBox] = []
            for box in PackedBoxs:
                n = len(box.block_table)
                if n <= limit:
                    cropped.append(box)
                    continue
                parts = ceil(n / average)
                step = ceil(n / parts)
                for i in range(parts):
                    lo, hi = i * step, min((i + 1) * step, n)
                    kv = min(box.kv_in_CTA - i * step * bs, step * bs)
                    rank = box.CTA_rank if i == 0 else counts[box.q_table[0]]
                    cropped.append(piece(box, box.block_table[lo:hi], kv, rank))
                    if i != 0:
                        for q in box.q_table:
                            counts[q] += 1
        else:
            cropped = PackedBoxs

        # phase 2: halve the longest box until the GPU has enough boxes
        if kvHead <= 4:
            want = 54
        elif kvHead <= 8:
            want = 27
        elif kvHead <= 16:
            want = 13
        elif kvHead <= 32:
            want = 6
        else:
            want = 4
        if len(cropped) >= want:
            return cropped
        while len(cropped) < want and max(counts) < 32:
            pick = max(range(len(cropped)), key=lambda i: len(cropped[i].block_table))
            box = cropped.pop(pick)
            n = len(box.block_table)
            if n <= 8:
                cropped.append(box)
                break
            half = ceil(n / 2)
            first = piece(box, box.block_table[:half], min(box.kv_in_CTA, half * bs), box.CTA_rank)
            second = piece(box, box.block_table[half:],
                           min(box.kv_in_CTA - half * bs, (n - half) * bs), counts[box.q_table[0]])
            for q in first.q_table:
                counts[q] += 1
            cropped.extend([first, second])
        return cropped

    def getMNW(self, m_val: int, kv_in_CTA: int):
        """Tile shape of a box with ``m_val`` query rows and ``kv_in_CTA``
        tokens (note: exactly 128 tokens still maps to N = 64 here)."""
        if m_val > 32:
            m, w = 64, 4
        elif m_val > 16:
            m, w = 32, 2
        else:
            m, w = 16, 1
        if kv_in_CTA < 32:
            n = 16
        elif kv_in_CTA < 64:
            n = 32
        elif kv_in_CTA <= 128:
            n = 64
        else:
            n = 128
        if m == 64:
            n = max(32, n)
        return (m, n, w)

    def _fill_kernel_info(self, boxes: List[PackedBox], buckets, grouped) -> KernelInfo:
        ki = KernelInfo()
        for mnw in buckets:
            group = grouped.get(tuple(mnw), [])
            if not group:
                continue
            ki.MNWs.append(mnw)
            ki.q_tables.append([b.q_table for b in group])
            ki.block_tables.append([b.block_table for b in group])
            ki.num_seqs_per_CTAs.append([b.num_seqs_per_CTA for b in group])
            ki.CTA_ranks.append([b.CTA_rank for b in group])
            ki.kv_in_CTAs.append([b.kv_in_CTA for b in group])
        ki.num_split_per_seq = self.split_per_seq
        ki.max_split_per_seq = max(ki.num_split_per_seq)
        ki.max_seqs_in_CTA = max((len(b.q_table) for b in boxes), default=0)
        ki.max_blocks_in_CTA = max((len(b.block_table) for b in boxes), default=0)
        return ki

    def naive_tree(self, node, mm, HRatio):
        """One set of boxes per tree node, no folding (reference ``:484-503``)."""
        boxes: List[PackedBox] = []
        S = self.s_values[node]
        for s in range(0, S, mm):
            self._emit_boxes(self.seq_indices[node][s:min(s + mm, S)], min(mm, S - s), mm,
                             self.block_ids[node], self.lens[node], boxes)
        for child in self.tree[node].values():
            boxes.extend(self.naive_tree(child, mm, HRatio))
        return boxes

    def naive_schedule(self, HRatio: int = 1):
        buckets = _default_buckets()
        mm = 64 // HRatio
        boxes: List[PackedBox] = []
        for node in self.tree[self.root].values():
            boxes.extend(self.naive_tree(node, mm, HRatio))
        grouped = {tuple(b): [] for b in buckets}
        for box in boxes:
            grouped[self.getMNW(len(box.q_table) * HRatio, box.kv_in_CTA)].append(box)
        return self._fill_kernel_info(boxes, buckets, grouped)

    def pack_schedule(self, MNWs: Optional[List[List[int]]] = None, HRatio: int = 1,
                      kvHead: int = 8, use_compute_model: bool = False):
        """Plan of the current tree: heuristic walk from every child of the
        root, ``balancePack``, bucket by tile shape, emit ``KernelInfo``."""
        buckets = MNWs if MNWs is not None else _default_buckets()
        mm = max(b[0] for b in buckets) // HRatio
        boxes: List[PackedBox] = []
        for node in self.tree[self.root].values():
            if use_compute_model:
                boxes.extend(self._compute_model_tree_heuristics(node, mm, HRatio, []))
            else:
                boxes.extend(self._tree_heuristics(node, mm, []))
        boxes = self.balancePack(boxes, kvHead)
        grouped = {tuple(b): [] for b in buckets}
        if len(buckets) == 1:
            grouped[tuple(buckets[0])].extend(boxes)
        else:
            for box in boxes:
                grouped[self.getMNW(len(box.q_table) * HRatio, box.kv_in_CTA)].append(box)
        return self._fill_kernel_info(boxes, buckets, grouped)


def unpad(lst):
    """Strip trailing zeros, keeping at least one element."""
    end = len(lst) - 1
    while end > 0 and lst[end] == 0:
        end -= 1
    return lst[:end + 1]


def unpad_2d(table):
    return [unpad(row) for row in table]


class AsyncPrefixTreeScheduler(Thread):
    """Runs tree build + packing + upload on a thread and resolves ``future``
    with the ``KernelInfo`` (reference ``prefix_tree.py:632-673``)."""

    def __init__(self, future: Future, block_tables, seq_lens: List[int], num_decode_tokens: int,
                 block_size: int, nheads: int, nheads_kv: int, MNWs: List[List[int]], device):
        super().__init__()
        self.future = future
        self.block_tables = block_tables
        self.seq_lens = seq_lens
        self.num_decode_tokens = num_decode_tokens
        self.block_size = block_size
        self.nheads = nheads
        self.nheads_kv = nheads_kv
        self.MNWs = MNWs
        self.device = device

    def run(self):
        try:
            if isinstance(self.block_tables, torch.Tensor):
                self.block_tables = self.block_tables.cpu().tolist()
            tree = PrefixTree(self.block_size)
            tree.build_radix_tree(self.seq_lens, self.block_tables)
            ratio = self.nheads // self.nheads_kv if self.nheads_kv is not None else 64
            plan: KernelInfo = tree.pack_schedule(self.MNWs, ratio)
            plan.to_tensor(device=self.device)
            self.future.set_result(plan)
        except Exception as exc:  # delivered to whoever waits on the future
            self.future.set_exception(exc)
