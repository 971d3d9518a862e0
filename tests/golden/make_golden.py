"""Freezes golden vectors from the reference itself.  Run where the read-only reference
checkout is present (its location: environment variable ``PAT_REFERENCE_ROOT``):

    python tests/golden/make_golden.py

Writes, next to this file:

* ``plans_py.json``   - trees and plans of the reference's Python scheduler
  (``prefix_attn/prefix_tree.py``: ``build_radix_tree`` + ``pack_schedule``) for
  every case of ``tests/cases.py``; small cases in full, big ones as SHA-256
  digests plus a summary;
* ``plans_cpp.json``  - plans of the reference's C++ scheduler
  (``csrc/prefix_tree.h``, compiled by ``oracle/build_ref.py``);
* ``legacy_py.json``  - outputs of ``naive_schedule``, ``build_from_batch`` and the
  v0 planners ``schedule`` / ``schedule_naive``;
* ``generators.json`` - digests of what the reference's own synthetic generators
  produce for seeded calls (checks this repository's mirrors of them);
* ``attention_ref.npz`` - inputs' seeds and outputs of the reference's
  ``attention_ref`` (``test/utils.py``) on small dense problems.
* ``attention_ref_positions.npz`` - the same function called once per query position
  (several query tokens per request, each seeing one more key than the one before).

Nothing here runs in the product; the tests only read the files.
"""
from __future__ import annotations

import json
import os
import random
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import cases as C  # noqa: E402
from oracle import build_ref, ref_loader, ref_tree  # noqa: E402


def summary(plan: dict) -> dict:
    return {
        "MNWs": plan["MNWs"],
        "ctas": [len(x) for x in plan["num_seqs_per_CTAs"]],
        "max_split_per_seq": plan["max_split_per_seq"],
        "max_seqs_in_CTA": plan["max_seqs_in_CTA"],
        "max_blocks_in_CTA": plan["max_blocks_in_CTA"],
        "sum_kv": int(sum(sum(x) for x in plan["kv_in_CTAs"])),
    }


def record(case, plan: dict, tree: dict | None) -> dict:
    out = {"input": case.input_digest(), "hratio": case.hratio, "kv_heads": case.kv_heads,
           "mnws": case.mnws, "use_compute_model": case.use_compute_model, "summary": summary(plan)}
    if case.big:
        out["plan_sha"] = C.digest(plan)
        out["fields_sha"] = {k: C.digest(v) for k, v in plan.items()}
        if tree is not None:
            out["tree_sha"] = C.digest(tree)
    else:
        out["plan"] = plan
        if tree is not None:
            out["tree"] = tree
    return out


def main():
    mods = ref_loader.load_reference_python()
    RefTree = mods["prefix_tree"].PrefixTree
    ref_lib = build_ref.build()
    assert ref_lib, "the reference C++ scheduler did not build"

    plans_py, plans_cpp, legacy = {}, {}, {}
    for case in C.all_cases():
        # ---- Python reference
        try:
            t = RefTree(case.block_size)
            t.build_radix_tree(list(case.seq_lens), [list(r) for r in case.tables])
            tree = C.tree_to_dict(t)
            ki = t.pack_schedule(case.mnws, case.hratio, case.kv_heads, case.use_compute_model)
            plans_py[case.name] = record(case, C.plan_to_dict(ki), tree)
        except Exception as exc:  # the reference itself raises on this input
            plans_py[case.name] = {"input": case.input_digest(), "hratio": case.hratio,
                                   "kv_heads": case.kv_heads, "mnws": case.mnws,
                                   "use_compute_model": case.use_compute_model,
                                   "raises": type(exc).__name__}
        # ---- C++ reference
        plan = ref_tree.run(case.block_size, case.seq_lens, case.padded(), case.mnws, case.hratio, case.kv_heads)
        nodes = plan.pop("nodes")
        rec = record(case, plan, None)
        rec["nodes_sha" if case.big else "nodes"] = C.digest(nodes) if case.big else nodes
        plans_cpp[case.name] = rec
        if case.name in ("manual", "rand003", "cfg0"):
            twice = ref_tree.run(case.block_size, case.seq_lens, case.padded(), case.mnws, case.hratio,
                                 case.kv_heads, packs=2)
            twice.pop("nodes")
            plans_cpp[case.name + "_packed_twice"] = record(case, twice, None)

        # ---- legacy planners (small cases only)
        if not case.big and "raises" not in plans_py[case.name] and len(legacy) < 24:
            leg = {}
            t = RefTree(case.block_size)
            t.build_radix_tree(list(case.seq_lens), [list(r) for r in case.tables])
            try:
                leg["naive_schedule"] = C.plan_to_dict(t.naive_schedule(case.hratio))
            except Exception as exc:
                leg["naive_schedule"] = {"raises": type(exc).__name__}
            if all(len(r) > 0 for r in case.tables):
                t2 = RefTree(case.block_size)
                try:
                    t2.build_from_batch(list(case.seq_lens), [list(r) for r in case.tables])
                    leg["build_from_batch"] = C.tree_to_dict(t2)
                except Exception as exc:
                    leg["build_from_batch"] = {"raises": type(exc).__name__}
                sched = mods["block_scheduler"].schedule
                k = max(1, 64 // case.hratio)
                ki = sched(list(case.seq_lens), [list(r) for r in case.tables], case.block_size, k, None, case.hratio)
                d = C.plan_to_dict(ki)
                d["sort_index"] = [int(x) for x in ki.sort_index]
                d["reverse_index"] = [int(x) for x in ki.reverse_index]
                leg["schedule"] = d
                kn = mods["block_scheduler"].schedule_naive(list(case.seq_lens), [list(r) for r in case.tables],
                                                            torch.device("cpu"))
                leg["schedule_naive"] = {
                    "q_tables": [t_.tolist() for t_ in kn.q_tables],
                    "block_tables": [t_.tolist() for t_ in kn.block_tables],
                    "kv_in_CTAs": [t_.tolist() for t_ in kn.kv_in_CTAs],
                    "num_split_per_seq": kn.num_split_per_seq.tolist(),
                    "MNWs": kn.MNWs, "max_blocks_in_CTA": int(kn.max_blocks_in_CTA),
                }
            legacy[case.name] = leg

    # ---- the reference's generators
    gens = {}
    U = mods["utils"]
    for i, tree in enumerate(C.REFERENCE_TEST_TREES):
        random.seed(100 + i)
        g, total = U.generate_tree_seqs(tree, 32)
        gens[f"tree{i:02d}"] = {"total_blocks": total, "sha": C.digest({"lens": g.seqlens, "tables": g.get_block_ids()})}
    for seed in range(8):
        rng = np.random.default_rng(5000 + seed)
        hi = int(rng.integers(200, 1500))
        lo = int(rng.integers(16, hi))
        g, total = U.generate_random_prefix_seqs(lo, hi, int(rng.integers(2, 48)), 1,
                                                 float(rng.choice([0.25, 0.5, 0.75])), 16, seed=seed)
        gens[f"prefseq{seed:02d}"] = {"total_blocks": total,
                                      "sha": C.digest({"lens": g.seqlens, "tables": g.get_block_ids()})}
    random.seed(7)
    g, total = U.generate_tree_seqs("1,2,4_64,32,32", 16)
    (seqlens, k_dense, v_dense, mask, table, k_paged, v_paged) = U.generate_random_kv_cache(
        g, total, 16, 2, 64, dtype=torch.float32, device="cpu", seed=3)
    gens["kv_cache"] = {"seqlens": seqlens.tolist(), "table": table.tolist(),
                        "mask_sum": int(mask.sum()), "k_dense_sum": float(k_dense.double().sum()),
                        "v_paged_sum": float(v_paged.double().sum()), "k_dense_shape": list(k_dense.shape)}

    # ---- attention_ref outputs
    attention_ref = ref_loader.load_reference_attention()
    att = {}
    specs = [(0, 2, 1, 4, 2, 64, 37, torch.float32), (1, 3, 1, 8, 8, 128, 50, torch.float32),
             (2, 4, 1, 8, 1, 64, 129, torch.bfloat16), (3, 2, 1, 16, 2, 128, 300, torch.float16)]
    for seed, b, t_, h, hk, d, s, dt in specs:
        gen = torch.Generator().manual_seed(seed)
        q = (torch.randn(b, t_, h, d, generator=gen) * 0.5).to(dt)
        k = (torch.randn(b, s, hk, d, generator=gen) * 0.5).to(dt)
        v = (torch.randn(b, s, hk, d, generator=gen) * 0.5).to(dt)
        lens = torch.randint(1, s + 1, (b,), generator=gen)
        mask = torch.arange(s)[None, :] < lens[:, None]
        out, probs = attention_ref(q.float(), k.float(), v.float(), None, mask)
        att[f"out{seed}"] = out.numpy()
        att[f"probs_rowsum{seed}"] = probs.sum(-1).numpy()
        att[f"spec{seed}"] = np.array([seed, b, t_, h, hk, d, s, {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[dt]])
    np.savez_compressed(os.path.join(HERE, "attention_ref.npz"), **att)

    # ---- several query positions per request: the reference's attention_ref has no causal
    # argument, so position t of a request with context L is ONE single-token call whose padding
    # mask keeps the first L - T + 1 + t keys; the outputs are stacked along the position axis
    multi = {}
    for seed, b, t_, h, hk, d, s in [(10, 3, 2, 8, 2, 64, 70), (11, 2, 4, 16, 2, 128, 133), (12, 2, 8, 8, 1, 64, 40)]:
        gen = torch.Generator().manual_seed(seed)
        q = (torch.randn(b, t_, h, d, generator=gen) * 0.5).bfloat16().float()
        k = (torch.randn(b, s, hk, d, generator=gen) * 0.5).bfloat16().float()
        v = (torch.randn(b, s, hk, d, generator=gen) * 0.5).bfloat16().float()
        lens = torch.randint(t_, s + 1, (b,), generator=gen)
        outs = []
        for t in range(t_):
            mask = torch.arange(s)[None, :] < (lens - t_ + 1 + t)[:, None]
            o, _ = attention_ref(q[:, t:t + 1], k, v, None, mask)
            outs.append(o)
        multi[f"out{seed}"] = torch.cat(outs, dim=1).numpy()
        multi[f"spec{seed}"] = np.array([seed, b, t_, h, hk, d, s])
        multi[f"lens{seed}"] = lens.numpy()
    np.savez_compressed(os.path.join(HERE, "attention_ref_positions.npz"), **multi)

    for name, obj in (("plans_py.json", plans_py), ("plans_cpp.json", plans_cpp),
                      ("legacy_py.json", legacy), ("generators.json", gens)):
        with open(os.path.join(HERE, name), "w") as f:
            json.dump(obj, f, separators=(",", ":"), sort_keys=True)
        print(name, os.path.getsize(os.path.join(HERE, name)) // 1024, "KiB", len(obj), "entries")
    raised = [k for k, v in plans_py.items() if "raises" in v]
    print("python reference raised on:", raised)


if __name__ == "__main__":
    main()
