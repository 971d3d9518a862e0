"""Pins the CPU oracle (oracle/attention_oracle.py) to the reference's own attention:
outputs of ``test/utils.py::attention_ref`` frozen in tests/golden/attention_ref.npz, and
the live function when the reference checkout is present."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_ref.npz")
_DT = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}


def _inputs(spec):
    seed, b, t, h, hk, d, s, dt = (int(x) for x in spec)
    gen = torch.Generator().manual_seed(seed)
    dtype = _DT[dt]
    q = (torch.randn(b, t, h, d, generator=gen) * 0.5).to(dtype)
    k = (torch.randn(b, s, hk, d, generator=gen) * 0.5).to(dtype)
    v = (torch.randn(b, s, hk, d, generator=gen) * 0.5).to(dtype)
    lens = torch.randint(1, s + 1, (b,), generator=gen)
    mask = torch.arange(s)[None, :] < lens[:, None]
    return q, k, v, mask


@pytest.mark.parametrize("idx", [0, 1, 2, 3])
def test_dense_attention_matches_frozen_reference_outputs(idx):
    gold = np.load(GOLD)
    q, k, v, mask = _inputs(gold[f"spec{idx}"])
    out, lse = O.dense_attention(q.float(), k.float(), v.float(), mask)
    want = torch.from_numpy(gold[f"out{idx}"])
    assert torch.allclose(out, want, atol=1e-6, rtol=1e-5)
    assert np.allclose(gold[f"probs_rowsum{idx}"], 1.0, atol=1e-5)
    # LSE definition: ln sum exp of the scaled, masked scores
    g = q.shape[2] // k.shape[2]
    scores = torch.einsum("bthd,bshd->bhts", q.float() / q.shape[-1] ** 0.5, k.float().repeat_interleave(g, 2))
    scores = scores.masked_fill(~mask[:, None, None, :], float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(scores, -1), atol=1e-6)


def test_dense_attention_matches_live_reference():
    from oracle import ref_loader
    if not ref_loader.reference_available():
        pytest.skip("reference checkout not present")
    attention_ref = ref_loader.load_reference_attention()
    for spec in ([7, 3, 1, 8, 2, 64, 77, 0], [8, 2, 1, 4, 4, 128, 200, 1]):
        q, k, v, mask = _inputs(spec)
        want, _ = attention_ref(q.float(), k.float(), v.float(), None, mask)
        got, _ = O.dense_attention(q.float(), k.float(), v.float(), mask)
        assert torch.allclose(got, want, atol=1e-6, rtol=1e-5)


def test_paged_and_plan_execution_agree():
    """Gathering pages, running a plan box by box and merging equals dense attention."""
    from pat_b200 import PrefixTree
    from pat_b200.workloads import make_config, make_values
    w = make_config(0)
    q, k, v = make_values(w)
    scale = w.head_dim ** -0.5
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    t = PrefixTree(w.page_size)
    t.build_radix_tree(list(w.seq_lens), [list(r) for r in w.block_tables])
    ki = t.pack_schedule(None, w.group, w.num_kv_heads)
    out, lse = O.execute_plan(ki, q, k, v, scale)
    assert torch.allclose(out, ref_o[:, 0], atol=1e-6, rtol=1e-5)
    assert torch.allclose(lse, ref_l, atol=2e-6)


def test_merge_is_order_independent_and_exact():
    g = torch.Generator().manual_seed(0)
    o = torch.randn(5, 3, 16, generator=g)
    l = torch.randn(5, 3, generator=g) * 3
    a, la = O.merge_partials(o, l)
    perm = torch.tensor([3, 0, 4, 1, 2])
    b, lb = O.merge_partials(o[perm], l[perm])
    assert torch.allclose(a, b, atol=1e-6) and torch.allclose(la, lb, atol=1e-6)
    one, lone = O.merge_partials(o[:1], l[:1])
    assert torch.equal(one, o[0]) and torch.allclose(lone, l[0])


GOLD_POS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_ref_positions.npz")


@pytest.mark.parametrize("seed", [10, 11, 12])
def test_multi_position_attention_matches_frozen_reference_outputs(seed):
    """Several query tokens per request: frozen outputs of one real ``attention_ref`` call per
    position (tests/golden/make_golden.py)."""
    gold = np.load(GOLD_POS)
    _, b, t_, h, hk, d, s = (int(x) for x in gold[f"spec{seed}"])
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(b, t_, h, d, generator=gen) * 0.5).bfloat16().float()
    k = (torch.randn(b, s, hk, d, generator=gen) * 0.5).bfloat16().float()
    v = (torch.randn(b, s, hk, d, generator=gen) * 0.5).bfloat16().float()
    lens = torch.randint(t_, s + 1, (b,), generator=gen)
    assert lens.tolist() == gold[f"lens{seed}"].tolist()
    out, lse = O.multi_position_attention(q, k, v, lens.tolist())
    assert torch.allclose(out, torch.from_numpy(gold[f"out{seed}"]), atol=1e-6, rtol=1e-5)
    # the last position is plain decode attention over the whole context
    mask = torch.arange(s)[None, :] < lens[:, None]
    last, last_lse = O.dense_attention(q[:, -1:], k, v, mask)
    assert torch.equal(out[:, -1:], last) and torch.equal(lse[:, -1], last_lse[:, :, 0])
