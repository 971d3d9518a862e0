"""The host-side work-list builder, validated on the CPU: executing the list
item by item with the fp32 oracle and merging through its own tables must
reproduce plain per-request attention, for every kind of plan (reference plans
with colliding ranks included)."""
import numpy as np
import pytest
import torch

import cases as C
import worklist_exec as W
from oracle import attention_oracle as O
from pat_b200 import PrefixTree
from pat_b200.workloads import make_config, scaled_down


def _values(n_pages, page, hq, hk, d, batch, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(batch, 1, hq, d, generator=g) * 0.5).bfloat16().float()
    k = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).bfloat16().float()
    v = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).bfloat16().float()
    return q, k, v


def _plan_lists(ki):
    return (ki.q_tables, ki.block_tables, ki.num_seqs_per_CTAs, ki.kv_in_CTAs)


class _Lists:
    """Plan of the native scheduler as nested lists (rows cut to their real length)."""

    def __init__(self, info, page):
        self.MNWs = info.MNWs
        self.num_seqs_per_CTAs = [t.tolist() for t in info.num_seqs_per_CTAs]
        self.kv_in_CTAs = [t.tolist() for t in info.kv_in_CTAs]
        self.CTA_ranks = [t.tolist() for t in info.CTA_ranks]
        self.q_tables = [[row[:n] for row, n in zip(t.tolist(), ns)]
                         for t, ns in zip(info.q_tables, self.num_seqs_per_CTAs)]
        self.block_tables = [[row[:-(-kv // page)] for row, kv in zip(t.tolist(), kvs)]
                             for t, kvs in zip(info.block_tables, self.kv_in_CTAs)]


def _consistent(ki):
    return all(n <= len(q) for b in range(len(ki.MNWs))
               for q, n in zip(ki.q_tables[b], ki.num_seqs_per_CTAs[b]))


def _run_case(seq_lens, tables, page, hratio, kv_heads, d=64, seed=0, mnws=None, scheduler="py",
              must_tile=True, **opts):
    if scheduler == "py":
        t = PrefixTree(page)
        t.build_radix_tree(list(seq_lens), [list(r) for r in tables])
        ki = t.pack_schedule(mnws, hratio, kv_heads)
        if not _consistent(ki):
            # prefix_tree.py:303-306 drops a request that ends exactly on an inner node; such
            # a plan claims more queries than it lists and the reference computes garbage
            pytest.skip("the reference Python plan is inconsistent for this batch")
    else:
        from pat_b200 import PrefixTreeCPP
        nt = PrefixTreeCPP(page)
        nt.build_radix_tree(list(seq_lens), [list(r) for r in tables])
        nt.pack_schedule(mnws, hratio, kv_heads)
        ki = _Lists(nt.kernel_info, page)
    B = len(seq_lens)
    n_pages = max(max(r) for r in tables if r) + 1
    q, k, v = _values(n_pages, page, hratio * kv_heads, kv_heads, d, B, seed)
    scale = d ** -0.5
    header, blob = W.build_work(_plan_lists(ki), B, hratio, kv_heads, page, **opts)
    out, lse = W.execute(header, blob, q, k, v, scale)
    # 1. the list must mean exactly what the plan means
    plan_o, plan_l = O.execute_plan(ki, q, k, v, scale)
    assert torch.allclose(out, plan_o, atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, plan_l, atol=2e-6, rtol=1e-6)
    # 2. and, whenever the plan tiles every request exactly once (always, unless a request ends
    #    inside a page it shares - which the block-id radix tree cannot express), plain attention
    seen = [0] * B
    for b in range(len(ki.MNWs)):
        for qs, n, kv in zip(ki.q_tables[b], ki.num_seqs_per_CTAs[b], ki.kv_in_CTAs[b]):
            for s_ in qs[:n]:
                seen[s_] += kv
    if seen == list(seq_lens):
        ref_o, ref_l = O.paged_decode_attention(q, k, v, seq_lens, tables, scale)
        assert torch.allclose(out, ref_o[:, 0], atol=2e-6, rtol=1e-5)
        assert torch.allclose(lse, ref_l, atol=2e-6, rtol=1e-6)
    elif must_tile:
        raise AssertionError("plan does not tile the requests")
    return header, blob, ki


@pytest.mark.parametrize("scheduler", ["py", "cpp"])
@pytest.mark.parametrize("seed", [3, 4, 6, 7, 8, 9, 10, 11, 12, 13, 0, 5, 14])
def test_random_plans_execute_exactly(seed, scheduler, native_lib):
    case = C.random_case(seed)
    try:
        _run_case(case.seq_lens, case.tables, case.block_size, case.hratio, 2, seed=seed, mnws=case.mnws,
                  scheduler=scheduler, must_tile=False)
    except IndexError:
        pytest.skip("the reference scheduler itself rejects this batch")


@pytest.mark.parametrize("opts", [dict(), dict(disable_dense=1), dict(chunk_tokens_min=16, chunk_tokens_max=48),
                                  dict(dense_min_rows=64), dict(items_per_sm=1, num_sms=4)])
def test_cfg0_with_colliding_reference_ranks(opts, native_lib):
    w = make_config(0)
    header, blob, ki = _run_case(w.seq_lens, w.block_tables, w.page_size, w.group, 2, d=64, **opts)
    # the reference's own rank labels collide on this plan (several boxes of one request
    # share a CTA_rank), which is why partial slots are re-derived
    ranks = {}
    collide = False
    for b in range(len(ki.MNWs)):
        for qs, n, r in zip(ki.q_tables[b], ki.num_seqs_per_CTAs[b], ki.CTA_ranks[b]):
            for s in qs[:n]:
                collide |= (s, r) in ranks
                ranks[(s, r)] = 1
    assert collide
    # shared prefix read once: the list's unique tokens equal the workload's
    assert header.unique_tokens == w.unique_tokens


@pytest.mark.parametrize("cfg,factor", [(1, 8), (2, 8), (3, 4), (4, 64)])
def test_scaled_configs(cfg, factor, native_lib):
    w = scaled_down(cfg, factor)
    header, _, _ = _run_case(w.seq_lens, w.block_tables, w.page_size, w.group, 2, d=64, seed=cfg)
    assert header.unique_tokens == w.unique_tokens


@pytest.mark.parametrize("cfg", [1, 2, 3, 4])
def test_full_configs_dedup_every_page(cfg, native_lib):
    """Structure only (no values): at full size every distinct page is read once per
    row tile, entries are private, and the merge lists cover every (request, item)."""
    w = make_config(cfg)
    t = PrefixTree(w.page_size)
    t.build_radix_tree(list(w.seq_lens), [list(r) for r in w.block_tables])
    ki = t.pack_schedule(None, w.group, w.num_kv_heads)
    header, blob = W.build_work(_plan_lists(ki), w.batch, w.group, w.num_kv_heads, w.page_size)
    assert header.unique_tokens == w.unique_tokens
    items = W.items_of(header, blob)
    hk = w.num_kv_heads
    # per (request, KV head): tokens attended == the request's context length
    seen = np.zeros((w.batch, hk), dtype=np.int64)
    for idx, it in enumerate(items):
        qs = blob[header.queries_off + it[0]: header.queries_off + it[0] + it[1]]
        heads = range(hk) if idx < header.num_stream_items else [it[5]]
        for h in heads:
            np.add.at(seen[:, h], qs, it[3])
    assert (seen == np.asarray(w.seq_lens)[:, None]).all()
    # merge lists: a partition of the entries
    indptr = blob[header.merge_indptr_off: header.merge_indptr_off + w.batch * hk + 1]
    entries = blob[header.merge_entries_off: header.merge_entries_off + int(indptr[-1])]
    assert indptr[-1] == header.num_entries
    assert sorted(entries.tolist()) == list(range(header.num_entries))
    # the dense kernel's query-id table repeats the dense items' query lists at a fixed row width
    width = header.dense_q_width
    table = blob[header.dense_q_off: header.dense_q_off + header.num_dense_items * width].reshape(-1, width)
    for d, it in enumerate(items[header.num_stream_items:]):
        want = blob[header.queries_off + it[0]: header.queries_off + it[0] + it[1]].tolist()
        assert table[d, :it[1]].tolist() == want and (table[d, it[1]:] == -1).all()
    # streaming items: longest first
    costs = items[:header.num_stream_items, 6]
    assert (np.diff(costs) <= 0).all()
    assert header.max_page_id < w.num_pages
    # dense items: every CTA gets (nearly) the same number of tokens, cut on 64-token boundaries
    ctas = W.dense_ctas(header, blob)
    assert 0 < len(ctas) <= 148 and ctas[0][0] == 0 and ctas[-1][1] == header.num_dense_items
    dense = items[header.num_stream_items:]
    load = np.array([dense[a:b, 3].sum() for a, b in ctas])
    assert load.sum() == header.dense_tokens * hk
    assert len(ctas) % hk == 0
    busy = load[load > 0]
    assert busy.max() <= 1.15 * busy.mean() + 1024, (busy.max(), busy.mean())
    assert (dense[:, 1] * w.group <= 128).all()
    starts_on_tile = (dense[:, 2] - np.array([0])) >= 0
    assert starts_on_tile.all()


def test_partial_shared_last_page(native_lib):
    # identical requests (parallel sampling): every page is shared, the last one partially filled
    _run_case([40, 40, 40, 40], [[5, 2, 9]] * 4, 16, 4, 2)


def test_same_pages_different_lengths(native_lib):
    # hand-written plan: the same physical pages with different valid lengths.  The full pages
    # are shared, the last page is attended with three different masks.
    class Plan:
        MNWs = [[16, 64, 1]]
        q_tables = [[[0], [1], [2]]]
        block_tables = [[[1, 2, 3]] * 3]
        num_seqs_per_CTAs = [[1, 1, 1]]
        kv_in_CTAs = [[33, 40, 48]]
    q, k, v = _values(4, 16, 4, 2, 64, 3, 1)
    header, blob = W.build_work(_plan_lists(Plan), 3, 2, 2, 16)
    out, lse = W.execute(header, blob, q, k, v, 0.125)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, [33, 40, 48], [[1, 2, 3]] * 3, 0.125)
    assert torch.allclose(out, ref_o[:, 0], atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, ref_l, atol=2e-6, rtol=1e-6)
    assert header.unique_tokens == 32 + 1 + 8 + 16      # pages 1,2 once; page 3 under three masks
    assert header.num_segments == 4


def test_query_attending_a_page_twice_keeps_multiplicity(native_lib):
    class Plan:
        MNWs = [[16, 64, 1]]
        q_tables = [[[0], [0, 1]]]
        block_tables = [[[1, 2], [2, 3]]]
        num_seqs_per_CTAs = [[1, 2]]
        kv_in_CTAs = [[32, 32]]
    q, k, v = _values(4, 16, 4, 2, 64, 2, 2)
    header, blob = W.build_work(_plan_lists(Plan), 2, 2, 2, 16)
    out, lse = W.execute(header, blob, q, k, v, 0.125)
    plan_o, plan_l = O.execute_plan(Plan, q, k, v, 0.125)
    assert torch.allclose(out, plan_o, atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, plan_l, atol=2e-6, rtol=1e-6)


def test_page_size_32(native_lib):
    _run_case([70, 100, 64, 33], [[0, 1, 2], [0, 1, 3, 4], [0, 1], [5, 6]], 32, 4, 2)


def test_bad_plan_is_rejected(native_lib):
    import ctypes as Ct
    from pat_b200 import _native as N
    with pytest.raises(AssertionError):
        W.build_work(([[[7]]], [[[0]]], [[1]], [[16]]), 4, 1, 1, 16)   # query id 7 >= batch 4


def test_dense_share_of_the_sms(native_lib):
    """When a plan has streaming work too, the dense kernel is cut for a share of the SMs
    sized from `dense_tile_ns`; without the estimate (< 0) or without streaming work it is
    cut for all of them.  Whatever the cut, the same tokens are covered."""
    w = make_config(4)
    t = PrefixTree(w.page_size)
    t.build_radix_tree(list(w.seq_lens), [list(r) for r in w.block_tables])
    for hk in (w.num_kv_heads, 1):                       # one GPU, and one rank of eight
        ki = t.pack_schedule(None, w.group, hk)
        lists = _plan_lists(ki)
        counts = {}
        for tile_ns in (-1, 800, 1600, 3200):
            header, blob = W.build_work(lists, w.batch, w.group, hk, w.page_size, dense_tile_ns=tile_ns)
            ctas = W.dense_ctas(header, blob)
            items = W.items_of(header, blob)[header.num_stream_items:]
            assert items[:, 3].sum() == header.dense_tokens * hk
            assert header.num_dense_ctas == len(ctas) <= 148
            assert len(ctas) % hk == 0
            counts[tile_ns] = len(ctas)
        assert counts[800] <= counts[1600] <= counts[3200] <= counts[-1]
        assert counts[1600] < counts[-1]
        assert counts[-1] > 148 - 2 * hk * 2             # all SMs, up to one group of CTAs
    # a short step (one 4096-token prefix, 64 suffixes): the dense kernel keeps clear of the step's
    # critical path with a part of the SMs, and still gets enough CTAs that a CTA has few tiles
    w1 = make_config(1)
    t1 = PrefixTree(w1.page_size)
    t1.build_radix_tree(list(w1.seq_lens), [list(r) for r in w1.block_tables])
    header, blob = W.build_work(_plan_lists(t1.pack_schedule(None, w1.group, w1.num_kv_heads)), w1.batch, w1.group,
                                w1.num_kv_heads, w1.page_size)
    assert 32 <= header.num_dense_ctas <= 96
    header, blob = W.build_work(_plan_lists(t1.pack_schedule(None, w1.group, 1)), w1.batch, w1.group, 1, w1.page_size)
    assert 16 <= header.num_dense_ctas <= 64                 # one rank of eight: pieces of two tiles at least
    # dense work only (every request shares everything): no streaming kernel to run beside
    lens = [4096] * 64
    tables = [list(range(256))] * 64
    t2 = PrefixTree(16)
    t2.build_radix_tree(lens, tables)
    ki = t2.pack_schedule(None, 4, 8)
    header, blob = W.build_work(_plan_lists(ki), 64, 4, 8, 16)
    assert header.num_stream_items == 0 and header.num_dense_ctas > 100
