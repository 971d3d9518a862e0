"""Work lists built straight from the radix tree, and tree + work list grown in place between
decode steps.  All on the CPU: trees and plans are compared with fresh builds (bit for bit, both
scheduler semantics) and work lists are executed item by item with the fp32 oracle."""
import ctypes as C
import sys

import numpy as np
import pytest
import torch

import cases as CS
import worklist_exec as W
from oracle import attention_oracle as O
from pat_b200 import PrefixTreeCPP
from pat_b200 import _native as N
from pat_b200 import _prefix_attn as P
from pat_b200.planner import DecodePlanner
from pat_b200.workloads import scaled_down

CPU = torch.device("cpu")


def _padded(tables, width=None):
    width = width or max(len(r) for r in tables)
    t = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, r in enumerate(tables):
        t[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
    return t


def _work_arrays(work):
    return work.header, work._host.numpy().copy()


def _values(n_pages, page, hq, hk, d, batch, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(batch, 1, hq, d, generator=g) * 0.5).bfloat16().float()
    k = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).bfloat16().float()
    v = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).bfloat16().float()
    return q, k, v


def _check_attention(tree, lens, tables, page, hratio, hk, n_pages, seed, cfg=None):
    work = tree.kernel_info.device_work(CPU, cfg)
    header, blob = _work_arrays(work)
    q, k, v = _values(n_pages, page, hratio * hk, hk, 32, len(lens), seed)
    out, lse = W.execute(header, blob, q, k, v, 0.2)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, lens, tables, 0.2)
    assert torch.allclose(out, ref_o[:, 0], atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, ref_l, atol=2e-6, rtol=1e-6)
    return header


class _Trace:
    """A running decode batch: shared prompt pages, then every request grows by a few tokens per
    step and gets a fresh page whenever it crosses a page boundary."""

    def __init__(self, seed, page=16):
        rng = np.random.default_rng(seed)
        self.rng, self.page = rng, page
        self.next_page = 0
        groups = int(rng.integers(1, 4))
        self.lens, self.tables = [], []
        for _ in range(groups):
            shared = self._alloc(int(rng.integers(1, 6)))
            for _ in range(int(rng.integers(1, 5))):
                mid = shared + (self._alloc(int(rng.integers(0, 3))) if rng.random() < 0.5 else [])
                for _ in range(int(rng.integers(1, 4))):
                    tail = int(rng.integers(1, 3 * page))
                    self.tables.append(mid + self._alloc(-(-tail // page)))
                    self.lens.append(len(mid) * page + tail)

    def _alloc(self, n):
        first = self.next_page
        self.next_page += n
        return list(range(first, first + n))

    def grow(self, max_tokens=3):
        for i in range(len(self.lens)):
            add = int(self.rng.integers(0, max_tokens + 1))
            self.lens[i] += add
            need = -(-self.lens[i] // self.page)
            if need > len(self.tables[i]):
                self.tables[i] = self.tables[i] + self._alloc(need - len(self.tables[i]))

    def padded(self):
        return _padded(self.tables, width=max(len(t) for t in self.tables) + 2)


def _ends_inside_a_shared_page(lens, tables, page):
    """True for batches a block-id radix tree cannot express (a request ending inside a page that
    another request continues through): both reference schedulers mis-attend those."""
    owners = {}
    for t in tables:
        for p in t:
            owners[p] = owners.get(p, 0) + 1
    return any(l % page and owners[t[-(-l // page) - 1]] > 1 for l, t in zip(lens, tables))


@pytest.mark.parametrize("semantics", ["cpp", "py"])
@pytest.mark.parametrize("seed", [3, 6, 8, 11, 12, 13])
def test_work_list_from_the_tree_attends_exactly(seed, semantics, native_lib):
    case = CS.random_case(seed)
    lens, tables, page = list(case.seq_lens), [list(t[:-(-l // case.block_size)]) for t, l in
                                                zip(case.tables, case.seq_lens)], case.block_size
    if _ends_inside_a_shared_page(lens, tables, page):
        pytest.skip("outside what a radix tree over page ids can express")
    tree = PrefixTreeCPP(page, semantics)
    tree.build_radix_tree(lens, _padded(tables))
    tree._hratio, tree._kv_heads = case.hratio, 2          # no pack needed for the work list
    n_pages = max(max(t) for t in tables) + 1
    header = _check_attention(tree, lens, tables, page, case.hratio, 2, n_pages, seed)
    assert header.unique_tokens == sum(n[2] for n in tree.nodes())


@pytest.mark.parametrize("semantics", ["cpp", "py"])
@pytest.mark.parametrize("seed", range(100, 116))
def test_work_list_from_the_tree_on_random_decode_batches(seed, semantics, native_lib):
    tr = _Trace(seed, page=16 if seed % 2 else 32)
    tree = PrefixTreeCPP(tr.page, semantics)
    tree.build_radix_tree(list(tr.lens), tr.padded())
    hratio = (1, 2, 4, 8)[seed % 4]
    tree._hratio, tree._kv_heads = hratio, 2
    cfg = P.WorkConfig(chunk_tokens_min=16, chunk_tokens_max=48) if seed % 3 == 0 else None
    header = _check_attention(tree, tr.lens, tr.tables, tr.page, hratio, 2, tr.next_page, seed, cfg)
    assert header.unique_tokens == sum(n[2] for n in tree.nodes())


@pytest.mark.parametrize("cfg,factor", [(1, 8), (2, 8), (3, 4), (4, 64)])
def test_work_list_from_the_tree_on_the_benchmark_shapes(cfg, factor, native_lib):
    w = scaled_down(cfg, factor)
    tree = PrefixTreeCPP(w.page_size)
    tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
    tree._hratio, tree._kv_heads = w.group, 2
    header = _check_attention(tree, w.seq_lens, w.block_tables, w.page_size, w.group, 2, w.num_pages, cfg)
    assert header.unique_tokens == w.unique_tokens and header.num_dense_items > 0


def _fresh(trace, semantics, hratio, hk):
    t = PrefixTreeCPP(trace.page, semantics)
    t.build_radix_tree(list(trace.lens), trace.padded())
    t.pack_schedule(None, hratio, hk)
    return t


@pytest.mark.parametrize("semantics", ["cpp", "py"])
def test_two_hundred_decode_traces_grown_in_place_equal_fresh_builds(semantics, native_lib):
    """After k in-place steps the tree, the packed plan and the attention computed from the work
    list equal those of a from-scratch build on the same tables."""
    hratio, hk = 4, 2
    advanced = rebuilt = 0
    for seed in range(200):
        tr = _Trace(seed)
        tree = _fresh(tr, semantics, hratio, hk)
        tree.kernel_info.device_work(CPU)               # the work list exists before the first advance
        for step in range(int(tr.rng.integers(1, 7))):
            tr.grow()
            if tree.advance(list(tr.lens), tr.padded()):
                advanced += 1
            else:                                       # slack used up: rebuild, as a caller would
                rebuilt += 1
                tree = _fresh(tr, semantics, hratio, hk)
                tree.kernel_info.device_work(CPU)
        want = _fresh(tr, semantics, hratio, hk)
        assert tree.nodes() == want.nodes()
        assert CS.native_plan_to_dict(tree.kernel_info) == CS.native_plan_to_dict(want.kernel_info)
        if seed % 10 == 0:
            _check_attention(tree, tr.lens, tr.tables, tr.page, hratio, hk, tr.next_page, seed)
    assert advanced > 500 and rebuilt < advanced // 10


def test_advance_refuses_what_it_cannot_express(native_lib):
    page = 16
    lens = [40, 40, 70]
    tables = [[0, 1, 2], [0, 1, 2], [0, 1, 3, 4, 5]]
    def build():
        t = PrefixTreeCPP(page)
        t.build_radix_tree(lens, _padded(tables, 8))
        t.pack_schedule(None, 4, 2)
        t.kernel_info.device_work(CPU)
        return t
    t = build()
    before = t.nodes()
    # requests 0 and 1 end in the same leaf: growing one of them changes the tree's shape
    assert not t.advance([41, 40, 70], _padded(tables, 8))
    # a request that is not alone in its last segment may still stand still while others grow
    assert t.advance([40, 40, 75], _padded(tables, 8))
    assert t.nodes() != before
    t = build()
    assert not t.advance([40, 40, 69], _padded(tables, 8))                      # shrinks
    assert not t.advance([40, 40], _padded(tables[:2], 8))                      # another batch
    changed = [list(r) for r in tables]
    changed[2][1] = 9
    assert not t.advance([40, 40, 71], _padded(changed, 8))                     # old part of a row changed
    assert t.nodes() == before                                                  # refusals change nothing
    # room for new pages runs out: 8 slots by default
    grown = [list(r) for r in tables]
    grown[2] += list(range(10, 10 + 9))
    assert not t.advance([40, 40, 70 + 9 * 16], _padded(grown, 16))
    grown[2] = grown[2][:-1]
    assert t.advance([40, 40, 70 + 8 * 16], _padded(grown, 16))
    assert not t.advance([40, 40, 70 + 8 * 16 + 11], _padded(grown + [], 16))   # needs a ninth page slot
    with pytest.raises(RuntimeError):
        t.advance([40, 40, 70], torch.zeros(3, 8))                              # not an int32 table


def test_planner_advances_and_rebuilds(native_lib):
    tr = _Trace(7)
    pl = DecodePlanner(tr.page, 4, 2, CPU)
    first = pl.step(list(tr.lens), tr.padded())
    assert pl.rebuilds == 1 and pl.advances == 0
    for _ in range(5):
        tr.grow(1)
        assert pl.step(list(tr.lens), tr.padded()) is first
    assert pl.advances == 5
    _check_attention(first, tr.lens, tr.tables, tr.page, 4, 2, tr.next_page, 1)
    # a new request joins: everything is rebuilt
    tr.lens.append(20)
    tr.tables.append(tr._alloc(2))
    second = pl.step(list(tr.lens), tr.padded())
    assert second is not first and pl.rebuilds == 2
    _check_attention(second, tr.lens, tr.tables, tr.page, 4, 2, tr.next_page, 2)


def test_kernel_info_is_only_materialised_when_read(native_lib):
    w = scaled_down(3, 4)
    tree = PrefixTreeCPP(w.page_size)
    tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
    tree.pack_schedule(None, w.group, w.num_kv_heads)
    info = tree.kernel_info
    info.to_gpu(CPU)
    assert info._vals is None                       # nothing has asked for the plan tensors yet
    assert info.max_split_per_seq >= 1 and len(info.q_tables) == len(info.MNWs) > 0
    assert info._vals is not None and info.num_split_per_seq.shape[0] == w.batch


def test_a_dropped_tree_is_freed_at_once_and_its_plan_stays_readable(native_lib):
    """``PrefixTreeCPP`` and its ``kernel_info`` share the native tree through a holder neither of
    them reaches the other by: no reference cycle, so a decode loop that builds a tree per step
    hands the native memory back with the last reference, not at the next garbage collection."""
    import gc
    import weakref
    w = scaled_down(3, 4)
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        tree = PrefixTreeCPP(w.page_size)
        tree.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
        tree.pack_schedule(None, w.group, w.num_kv_heads)
        info, gone = tree.kernel_info, weakref.ref(tree)
        del tree
        assert gone() is None
        assert len(info.q_tables) == len(info.MNWs) > 0         # the put-off pack still runs
        holder = info._box
        assert holder.handle
        del info
        assert sys.getrefcount(holder) == 2                     # this name and the call's argument
    finally:
        if was_enabled:
            gc.enable()


# ---------------------------------------------------------------------------------------------
# Several query tokens per request
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T", [2, 3, 4, 8])
@pytest.mark.parametrize("seed", [200, 201, 202, 203, 204, 205])
def test_work_list_for_several_query_positions(seed, T, native_lib):
    """Position t of a request sees its first len - T + 1 + t tokens; requests may be shorter than
    a page, shorter than T + 1, and their last tokens may reach back into a shared segment."""
    tr = _Trace(seed)
    hratio, hk, page = (1, 2, 4, 8)[seed % 4], 2, tr.page
    lens = [max(l, T) for l in tr.lens]                     # at least the T new tokens
    tables = [t + tr._alloc(-(-l // page) - len(t)) if -(-l // page) > len(t) else t for t, l in zip(tr.tables, lens)]
    tree = PrefixTreeCPP(page)
    tree.build_radix_tree(lens, _padded(tables))
    tree._hratio, tree._kv_heads = hratio, hk
    cfg = P.WorkConfig(chunk_tokens_min=16, chunk_tokens_max=32) if seed % 2 else None
    work = tree.kernel_info.device_work(CPU, cfg, T)
    header, blob = _work_arrays(work)
    assert header.q_per_req == T and header.batch == len(lens) * T and header.limits_off >= 0
    g = torch.Generator().manual_seed(seed)
    B, H, D = len(lens), hratio * hk, 32
    q = (torch.randn(B, T, H, D, generator=g) * 0.5).bfloat16().float()
    k = (torch.randn(tr.next_page, page, hk, D, generator=g) * 0.5).bfloat16().float()
    v = (torch.randn(tr.next_page, page, hk, D, generator=g) * 0.5).bfloat16().float()
    out, lse = W.execute(header, blob, q, k, v, 0.2)
    ref_o, ref_l = O.paged_multi_position_attention(q, k, v, lens, tables, 0.2)
    assert torch.allclose(out, ref_o, atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, ref_l, atol=2e-6, rtol=1e-6)
    # such a list is rebuilt, not advanced
    tree.kernel_info._work = {k_: v_ for k_, v_ in tree.kernel_info._work.items()}
    assert not tree.advance([l + 1 for l in lens], _padded(tables, max(len(t) for t in tables) + 2))
