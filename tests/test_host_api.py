"""Host-side mirror of the reference package: exports, dataclasses, generators, legacy planners,
AsyncTree and the op's argument checks (everything that needs no GPU)."""
import json
import os
import random

import numpy as np
import pytest
import torch

import cases as C
import pat_b200
from pat_b200 import (AsyncTree, KernelInfo, PackedBox, PrefixTree, PrefixTreeCPP, SeqGroup, Sequence,
                      generate_random_kv_cache, generate_random_prefix_seqs, generate_tree_seqs,
                      pack_prefix_blocks, pack_without_prefix, prefix_attn_with_kvcache, schedule, schedule_naive)
from pat_b200.data_class import create_seq_group

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LEGACY = json.load(open(os.path.join(GOLD, "legacy_py.json")))
GENS = json.load(open(os.path.join(GOLD, "generators.json")))
CASES = {c.name: c for c in C.all_cases()}


def test_exports_are_the_reference_list():
    # prefix_attn/__init__.py:10-26
    assert pat_b200.__all__ == [
        "prefix_attn_with_kvcache", "PrefixTree", "PrefixTreeCPP", "AsyncTree", "generate_random_prefix_seqs",
        "generate_random_kv_cache", "generate_tree_seqs", "pack_prefix_blocks", "pack_without_prefix",
        "schedule", "schedule_naive", "PackedBox", "Sequence", "SeqGroup", "KernelInfo"]
    import prefix_attn
    from prefix_attn.prefix_tree import PrefixTree as P2
    from prefix_attn.data_class import create_seq_group as c2
    assert prefix_attn.PrefixTreeCPP is PrefixTreeCPP and P2 is PrefixTree and c2 is create_seq_group


@pytest.mark.parametrize("idx", range(len(C.REFERENCE_TEST_TREES)))
def test_generate_tree_seqs_matches_reference(idx):
    random.seed(100 + idx)
    g, total = generate_tree_seqs(C.REFERENCE_TEST_TREES[idx], 32)
    gold = GENS[f"tree{idx:02d}"]
    assert total == gold["total_blocks"]
    assert C.digest({"lens": g.seqlens, "tables": g.get_block_ids()}) == gold["sha"]


@pytest.mark.parametrize("seed", range(8))
def test_generate_random_prefix_seqs_matches_reference(seed):
    rng = np.random.default_rng(5000 + seed)
    hi = int(rng.integers(200, 1500))
    lo = int(rng.integers(16, hi))
    g, total = generate_random_prefix_seqs(lo, hi, int(rng.integers(2, 48)), 1,
                                           float(rng.choice([0.25, 0.5, 0.75])), 16, seed=seed)
    gold = GENS[f"prefseq{seed:02d}"]
    assert total == gold["total_blocks"]
    assert C.digest({"lens": g.seqlens, "tables": g.get_block_ids()}) == gold["sha"]


def test_generate_random_kv_cache_matches_reference():
    random.seed(7)
    g, total = generate_tree_seqs("1,2,4_64,32,32", 16)
    seqlens, k_dense, v_dense, mask, table, k_paged, v_paged = generate_random_kv_cache(
        g, total, 16, 2, 64, dtype=torch.float32, device="cpu", seed=3)
    gold = GENS["kv_cache"]
    assert seqlens.tolist() == gold["seqlens"] and table.tolist() == gold["table"]
    assert int(mask.sum()) == gold["mask_sum"] and list(k_dense.shape) == gold["k_dense_shape"]
    assert abs(float(k_dense.double().sum()) - gold["k_dense_sum"]) < 1e-6
    assert abs(float(v_paged.double().sum()) - gold["v_paged_sum"]) < 1e-6


@pytest.mark.parametrize("name", sorted(LEGACY))
def test_legacy_planners_match_reference(name):
    case, gold = CASES[name], LEGACY[name]
    t = PrefixTree(case.block_size)
    t.build_radix_tree(list(case.seq_lens), [list(r) for r in case.tables])
    if "raises" in gold["naive_schedule"]:
        with pytest.raises(Exception):
            t.naive_schedule(case.hratio)
    else:
        assert C.plan_to_dict(t.naive_schedule(case.hratio)) == gold["naive_schedule"]
    if "build_from_batch" in gold:
        t2 = PrefixTree(case.block_size)
        if "raises" in gold["build_from_batch"]:
            with pytest.raises(Exception):
                t2.build_from_batch(list(case.seq_lens), [list(r) for r in case.tables])
        else:
            t2.build_from_batch(list(case.seq_lens), [list(r) for r in case.tables])
            assert C.tree_to_dict(t2) == gold["build_from_batch"]
    if "schedule" in gold:
        k = max(1, 64 // case.hratio)
        ki = schedule(list(case.seq_lens), [list(r) for r in case.tables], case.block_size, k, None, case.hratio)
        d = C.plan_to_dict(ki)
        d["sort_index"] = [int(x) for x in ki.sort_index]
        d["reverse_index"] = [int(x) for x in ki.reverse_index]
        assert d == gold["schedule"]
        kn = schedule_naive(list(case.seq_lens), [list(r) for r in case.tables], torch.device("cpu"))
        g = gold["schedule_naive"]
        assert [t_.tolist() for t_ in kn.q_tables] == g["q_tables"]
        assert [t_.tolist() for t_ in kn.block_tables] == g["block_tables"]
        assert [t_.tolist() for t_ in kn.kv_in_CTAs] == g["kv_in_CTAs"]
        assert kn.num_split_per_seq.tolist() == g["num_split_per_seq"]
        assert kn.MNWs == g["MNWs"] and int(kn.max_blocks_in_CTA) == g["max_blocks_in_CTA"]


def test_oldest_entry_points_run_and_cover_every_token():
    # block_scheduler.py:9-202: as shipped in the reference these raise TypeError; here they return
    # the flat plan their docstrings describe
    group = create_seq_group([[0, 1, 2, 3, 4, 5, 10, 11, 12], [0, 1, 2, 3, 4, 5, 13],
                              [0, 1, 2, 6, 7, 8, 14, 15, 16], [0, 1, 2, 6, 7, 8, 17]],
                             [9 * 16, 7 * 16 - 3, 9 * 16, 7 * 16], 16)
    group.sort()
    flat = pack_prefix_blocks(group, 16, k=64)
    assert flat.block_table[0] == [0, 1, 2] and flat.num_seqs_per_CTA[0] == 4 and flat.CTA_rank[0] == 0
    seen = [0] * 4
    for q, n, kv in zip(flat.q_table, flat.num_seqs_per_CTA, flat.kv_in_CTA):
        for s in range(q, q + n):
            seen[s] += kv
    assert seen == group.seqlens
    assert flat.num_split_per_seq == [3, 3, 3, 3] and flat.max_split_per_seq == 3
    solo = pack_without_prefix(group, 16)
    assert solo.num_seqs_per_CTA == [1] * 4 and solo.kv_in_CTA == group.seqlens and solo.max_blocks_in_CTA == 9


def test_dataclasses_behave_like_the_reference():
    s = Sequence(16, 5)
    s.append_blocks([1, 2])
    assert s.seqlen == 37 and s.block_ids == [1, 2]
    s.append_blocks([3], 0)
    assert s.seqlen == 37
    random.seed(0)
    g = SeqGroup(16, 10, 20, 3)
    random.seed(0)
    assert g.seqlens == [random.randint(10, 20) for _ in range(3)]
    g.sequences[0].block_ids = [5, 6]
    g.sequences[1].block_ids = [1]
    g.sequences[2].block_ids = [5, 2, 9]
    assert g.get_padded_block_ids(0) == [[5, 6, 0], [1, 0, 0], [5, 2, 9]] and g.max_num_blocks == 3
    g.sort()
    assert [q.block_ids for q in g.sequences] == [[1], [5, 2, 9], [5, 6]] and g.is_sorted
    box = PackedBox(q_table=[[0], [1]], block_table=[[1], [2, 3]], num_seqs_per_CTA=[1, 1], CTA_rank=[0, 0],
                    kv_in_CTA=[16, 30])
    box.sort_by_kv_desc()
    assert box.kv_in_CTA == [30, 16] and box.block_table == [[2, 3], [1]]
    box.to_tensor("cpu")
    assert box.block_table.tolist() == [[2, 3], [1, 0]] and box.block_table.dtype == torch.int32
    assert PackedBox(kv_in_CTA=5) < PackedBox(kv_in_CTA=3)


def test_kernel_info_to_tensor_pads_and_remembers_the_host_plan():
    t = PrefixTree(16)
    t.build_radix_tree([33, 33, 33], [[0, 1, 5], [0, 2, 6], [3, 4, 7]])
    ki = t.pack_schedule(None, 4, 8)
    ki.to_tensor("cpu")
    assert [x.tolist() for x in ki.q_tables] == [[[2]], [[0, 1], [0, 0], [1, 0]]]
    assert [x.tolist() for x in ki.block_tables] == [[[3, 4, 7]], [[0, 0], [1, 5], [2, 6]]]
    assert ki.num_split_per_seq.dtype == torch.int32
    tag = ki.num_split_per_seq._pat_plan_tag
    assert tag.host_plan.batch == 3 and tag.host_plan.kv_lens[1].tolist() == [16, 17, 17]
    ki.to_tensor("cpu")     # idempotent


def test_async_tree_builds_in_the_background():
    w = C.config_case(0)
    at = AsyncTree(block_size=16, seq_lens=list(w.seq_lens), table=torch.from_numpy(w.padded()), MNWs=None,
                   HRatio=4, kvHead=8, device=torch.device("cpu"))
    tree = at.tree
    assert isinstance(at, PrefixTreeCPP) and isinstance(tree, PrefixTreeCPP)
    assert tree.kernel_info.max_split_per_seq >= 2
    assert sum(int(x.sum()) for x in tree.kernel_info.kv_in_CTAs) > 0
    bad = AsyncTree(16, [5], torch.zeros(2, 2, dtype=torch.int32), None, 1, 8, torch.device("cpu"))
    with pytest.raises(RuntimeError, match="mismatch"):
        bad.tree


def test_native_tree_argument_errors():
    t = PrefixTreeCPP(16)
    with pytest.raises(RuntimeError, match="List\\[int\\] or a CPU Int32 Tensor"):
        t.build_radix_tree(np.array([1]), torch.zeros(1, 1, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        t.build_radix_tree([1], torch.zeros(1, 1, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="before pack_schedule"):
        PrefixTreeCPP(16).pack_schedule()
    with pytest.raises(ValueError):
        PrefixTreeCPP(16, semantics="rust")


def test_op_checks_fire_in_the_reference_order_on_cpu_tensors():
    q = torch.zeros(2, 1, 8, 128, dtype=torch.float16)
    k = torch.zeros(4, 16, 2, 128, dtype=torch.float16)
    tree = PrefixTreeCPP(16)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        prefix_attn_with_kvcache(q.float(), k, k, tree, 1.0, q)
    with pytest.raises(RuntimeError, match="same dtype"):
        prefix_attn_with_kvcache(q, k.bfloat16(), k, tree, 1.0, q)
    with pytest.raises(RuntimeError, match="q must be on CUDA"):
        prefix_attn_with_kvcache(q, k, k, tree, 1.0, q)
    with pytest.raises(TypeError):
        prefix_attn_with_kvcache(q, k)
    with pytest.raises(TypeError):
        prefix_attn_with_kvcache(q, k, k, tree, 1.0, q, None, None)
