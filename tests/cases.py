"""Scheduler test cases shared by the golden generator and the tests.

Every case is fully determined by its name: inputs come from seeded generators
in this repository (never from the reference), so the tests can rebuild them
anywhere and compare plans against the frozen reference outputs in
``tests/golden/``.
"""
from __future__ import annotations

import hashlib
import json
import random
from dataclasses import dataclass, field
from typing import Iterator, List, Optional

import numpy as np

from pat_b200.workloads import make_config

# tree strings the reference's kernel test is parametrised over (test/test.py:171-189)
REFERENCE_TEST_TREES = [
    "1,2,4,16,32,64,128,256,512_3072,1024,32,32,32,32,32,32,32",
    "1,2,4,16,32,64,256_4096,32,128,128,32,256,512",
    "1,2,4,16,32,64,128,256,512_3072,1024,512,256,128,32,256,512,32",
    "1,2,4,16,32,64,128,256,1024_512,32,128,128,32,256,512,32,32",
    "1,2,4,16,32,64,128,512_512,32,128,128,32,256,512,256",
    "1,2,4,16,32,64,128_512,32,128,128,32,256,512",
    "4_4096",
    "4,16_4096,256",
    "1,8_640,32",
    "1,4,16_32,256,32",
    "1,2,4,8,16,32,64_32,512,32,256,32,32,32",
    "1,4,256_32,256,32",
    "1,16,32_2048,1024,256",
    "1,10_4096,416",
]


@dataclass
class PlanCase:
    name: str
    block_size: int
    seq_lens: List[int]
    tables: List[List[int]]          # unpadded
    hratio: int
    kv_heads: int
    mnws: Optional[List[List[int]]] = None
    use_compute_model: bool = False
    big: bool = False                # store digests instead of the full plan
    tags: List[str] = field(default_factory=list)

    def padded(self) -> np.ndarray:
        width = max((len(r) for r in self.tables), default=1)
        out = np.zeros((len(self.tables), max(width, 1)), dtype=np.int32)
        for i, r in enumerate(self.tables):
            out[i, :len(r)] = r
        return out

    def input_digest(self) -> str:
        return digest({"bs": self.block_size, "lens": self.seq_lens, "tables": self.tables})


def digest(obj) -> str:
    return hashlib.sha256(json.dumps(obj, separators=(",", ":"), sort_keys=True).encode()).hexdigest()


def tree_string_case(idx: int, hratio=8, kv_heads=8, block_size=32, name=None) -> PlanCase:
    from pat_b200.utils import generate_tree_seqs
    random.seed(100 + idx)
    group, _ = generate_tree_seqs(REFERENCE_TEST_TREES[idx], block_size)
    return PlanCase(name or f"tree{idx:02d}", block_size, group.seqlens, group.get_block_ids(), hratio, kv_heads,
                    big=True, tags=["tree_string"])


def random_case(seed: int) -> PlanCase:
    """A small random prefix forest with ragged lengths, duplicates and requests
    that end exactly on a shared boundary."""
    rng = np.random.default_rng(seed)
    bs = int(rng.choice([16, 16, 32]))
    n = int(rng.integers(1, 40))
    next_page = [0]

    def fresh(k):
        out = list(range(next_page[0], next_page[0] + k))
        next_page[0] += k
        return out

    roots = [fresh(int(rng.integers(1, 12))) for _ in range(int(rng.integers(1, 4)))]
    mids = {}
    tables, lens = [], []
    for i in range(n):
        kind = rng.integers(0, 10) if seed % 3 == 0 else rng.integers(0, 40)
        if kind == 0 and tables:                      # exact duplicate of an earlier request
            j = int(rng.integers(0, len(tables)))
            tables.append(list(tables[j]))
            lens.append(lens[j])
            continue
        r = int(rng.integers(0, len(roots)))
        row = list(roots[r])
        if rng.random() < 0.6:
            key = (r, int(rng.integers(0, 3)))
            if key not in mids:
                mids[key] = fresh(int(rng.integers(1, 6)))
            row += mids[key]
        if kind == 1:                                  # ends exactly on a shared boundary
            tables.append(row)
            lens.append(len(row) * bs)
            continue
        if kind == 2 and len(row) > 1:                 # ends inside the shared part
            cut = int(rng.integers(1, len(row)))
            row = row[:cut]
            tables.append(row)
            lens.append(len(row) * bs - int(rng.integers(0, bs)))
            continue
        own = int(rng.integers(1, 30))
        row += fresh(own)
        tables.append(row)
        lens.append(len(row) * bs - int(rng.integers(0, bs)))
    hratio = int(rng.choice([1, 2, 4, 8]))
    kv_heads = int(rng.choice([1, 4, 8, 16, 32, 64]))
    pick = rng.integers(0, 6)
    mnws = None
    if pick == 0:
        mnws = [[64, 128, 4]]
    elif pick == 1:
        mnws = [[32, 64, 2]]
    cm = bool(rng.random() < 0.25)
    return PlanCase(f"rand{seed:03d}", bs, lens, tables, hratio, kv_heads, mnws, cm, tags=["random"])


def prefix_seq_case(seed: int) -> PlanCase:
    from pat_b200.utils import generate_random_prefix_seqs
    rng = np.random.default_rng(5000 + seed)
    bs = 16
    hi = int(rng.integers(200, 1500))
    lo = int(rng.integers(16, hi))
    group, _ = generate_random_prefix_seqs(lo, hi, int(rng.integers(2, 48)), 1, float(rng.choice([0.25, 0.5, 0.75])),
                                           bs, seed=seed)
    return PlanCase(f"prefseq{seed:02d}", bs, group.seqlens, group.get_block_ids(),
                    int(rng.choice([1, 4, 8])), 8, tags=["prefix_seqs"])


def config_case(cfg: int, shard: int = 1) -> PlanCase:
    w = make_config(cfg)
    name = f"cfg{cfg}" + (f"_tp{shard}" if shard > 1 else "")
    return PlanCase(name, w.page_size, w.seq_lens, w.block_tables, w.group, w.num_kv_heads // shard,
                    big=cfg >= 1, tags=["config"])


def manual_case() -> PlanCase:
    # inputs of the reference's manual test (test/test.py:233-234)
    return PlanCase("manual", 16, [33, 33, 33], [[0, 1, 5], [0, 2, 6], [3, 4, 7]], 4, 8, tags=["manual"])


def all_cases() -> Iterator[PlanCase]:
    yield manual_case()
    for cfg in range(5):
        yield config_case(cfg)
    for cfg, shards in ((2, (2, 4)), (3, (2, 4, 8)), (4, (2, 4, 8)), (1, (2, 8))):
        for s in shards:
            yield config_case(cfg, s)
    for i in range(len(REFERENCE_TEST_TREES)):
        yield tree_string_case(i)
    yield tree_string_case(8, hratio=1, kv_heads=32, name="tree08_mha")
    for seed in range(60):
        yield random_case(seed)
    for seed in range(8):
        yield prefix_seq_case(seed)


def pad_ragged(rows) -> List[List[int]]:
    width = max((len(r) for r in rows), default=0)
    return [list(r) + [0] * (width - len(r)) for r in rows]


def plan_to_dict(ki) -> dict:
    """A Python-side KernelInfo (list fields, ragged tables) as a plain dict."""
    return {
        "MNWs": [list(m) for m in ki.MNWs],
        "q_tables": [[list(r) for r in t] for t in ki.q_tables],
        "block_tables": [[list(r) for r in t] for t in ki.block_tables],
        "num_seqs_per_CTAs": [list(t) for t in ki.num_seqs_per_CTAs],
        "CTA_ranks": [list(t) for t in ki.CTA_ranks],
        "kv_in_CTAs": [list(t) for t in ki.kv_in_CTAs],
        "num_split_per_seq": list(ki.num_split_per_seq),
        "max_split_per_seq": int(ki.max_split_per_seq),
        "max_seqs_in_CTA": int(ki.max_seqs_in_CTA),
        "max_blocks_in_CTA": int(ki.max_blocks_in_CTA),
    }


def padded_plan(plan: dict) -> dict:
    """Ragged tables zero-padded per bucket (what reaches the device)."""
    out = dict(plan)
    out["q_tables"] = [pad_ragged(t) for t in plan["q_tables"]]
    out["block_tables"] = [pad_ragged(t) for t in plan["block_tables"]]
    return out


def native_plan_to_dict(info) -> dict:
    """``PrefixTreeCPP.kernel_info`` (CPU tensors) as a plain dict of padded tables."""
    return {
        "MNWs": [list(m) for m in info.MNWs],
        "q_tables": [t.tolist() for t in info.q_tables],
        "block_tables": [t.tolist() for t in info.block_tables],
        "num_seqs_per_CTAs": [t.tolist() for t in info.num_seqs_per_CTAs],
        "CTA_ranks": [t.tolist() for t in info.CTA_ranks],
        "kv_in_CTAs": [t.tolist() for t in info.kv_in_CTAs],
        "num_split_per_seq": info.num_split_per_seq.tolist(),
        "max_split_per_seq": int(info.max_split_per_seq),
        "max_seqs_in_CTA": int(info.max_seqs_in_CTA),
        "max_blocks_in_CTA": int(info.max_blocks_in_CTA),
    }


def tree_to_dict(tree) -> dict:
    """Node arrays of a Python-side PrefixTree."""
    return {
        "parents": list(tree.parents), "s_values": list(tree.s_values), "lens": list(tree.lens),
        "seq_indices": [list(s) for s in tree.seq_indices], "block_ids": [list(b) for b in tree.block_ids],
        "children": [list(tree.tree[i].values()) if i in tree.tree else [] for i in range(tree.num_nodes)],
    }


def native_tree_to_dict(tree) -> dict:
    nodes = tree.nodes()
    return {
        "parents": [n[0] for n in nodes], "s_values": [n[1] for n in nodes], "lens": [n[2] for n in nodes],
        "seq_indices": [n[3] for n in nodes], "block_ids": [n[4] for n in nodes],
        "children": [n[5] for n in nodes],
    }
