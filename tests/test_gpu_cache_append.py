"""KV-cache append on the GPU against the CPU restatement (bit-exact) and, where it loads,
against vLLM's own op - which pins the restatement."""
import math

import numpy as np
import pytest
import torch

from oracle import cache_oracle as CO
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(tokens, heads, dim, pages, page, dtype, seed, pad_every=0):
    g = torch.Generator().manual_seed(seed)
    key = (torch.randn(tokens, heads, dim, generator=g) * 0.5).to(dtype)
    value = (torch.randn(tokens, heads, dim, generator=g) * 0.5).to(dtype)
    kc = (torch.randn(pages, page, heads, dim, generator=g) * 0.5).to(dtype)
    vc = (torch.randn(pages, page, heads, dim, generator=g) * 0.5).to(dtype)
    rng = np.random.default_rng(seed)
    slots = torch.from_numpy(rng.permutation(pages * page)[:tokens].astype(np.int64))
    if pad_every:
        slots[::pad_every] = -1
    return key, value, kc, vc, slots


@pytest.mark.parametrize("tokens,heads,dim,pages,page,dtype,pad", [
    (256, 8, 128, 700, 16, torch.bfloat16, 0),
    (64, 4, 64, 90, 16, torch.float16, 5),
    (1, 1, 128, 3, 32, torch.bfloat16, 0),
    (37, 2, 128, 11, 16, torch.float16, 3),
    (0, 8, 128, 4, 16, torch.bfloat16, 0),
])
def test_append_is_bit_exact(tokens, heads, dim, pages, page, dtype, pad, native_lib):
    from pat_b200.cache_ops import reshape_and_cache_flash
    key, value, kc, vc, slots = _case(tokens, heads, dim, pages, page, dtype, 7 + tokens, pad)
    kd, vd = kc.to(DEV), vc.to(DEV)
    reshape_and_cache_flash(key.to(DEV), value.to(DEV), kd, vd, slots.to(DEV), "auto", None, None)
    torch.cuda.synchronize()
    CO.reshape_and_cache_flash(key, value, kc, vc, slots)
    assert torch.equal(kd.cpu(), kc) and torch.equal(vd.cpu(), vc)


def test_append_into_the_two_halves_of_one_cache_and_strided_keys(native_lib):
    """The serving backend keeps K and V as kv_cache[0] / kv_cache[1] and passes keys that are
    slices of a fused projection output (plugin/vllm/attention/backends/prefix_attn.py:806-837)."""
    from pat_b200.cache_ops import reshape_and_cache_flash
    tokens, heads, dim, pages, page = 48, 8, 128, 40, 16
    key, value, kc, vc, slots = _case(tokens, heads, dim, pages, page, torch.bfloat16, 3, 7)
    kv = torch.stack([kc, vc]).to(DEV)
    qkv = torch.zeros(tokens, 3 * heads * dim, dtype=torch.bfloat16, device=DEV)
    qkv[:, heads * dim:2 * heads * dim] = key.reshape(tokens, -1).to(DEV)
    qkv[:, 2 * heads * dim:] = value.reshape(tokens, -1).to(DEV)
    k_view = qkv[:, heads * dim:2 * heads * dim].view(tokens, heads, dim)
    v_view = qkv[:, 2 * heads * dim:].view(tokens, heads, dim)
    reshape_and_cache_flash(k_view, v_view, kv[0], kv[1], slots.to(DEV).view(-1, 1), "auto")
    torch.cuda.synchronize()
    CO.reshape_and_cache_flash(key, value, kc, vc, slots)
    assert torch.equal(kv[0].cpu(), kc) and torch.equal(kv[1].cpu(), vc)


def test_restatement_against_vllms_own_op(native_lib):
    """Pins oracle/cache_oracle.py: same result as the op the reference calls."""
    try:
        import vllm._custom_ops as ops      # noqa: F401
        fn = torch.ops._C_cache_ops.reshape_and_cache_flash
    except Exception as exc:                # vLLM's extension did not load here
        pytest.skip(f"vLLM's cache ops are not available: {exc}")
    key, value, kc, vc, slots = _case(96, 8, 128, 64, 16, torch.bfloat16, 11, 6)
    kd, vd = kc.to(DEV), vc.to(DEV)
    one = torch.ones(1, dtype=torch.float32, device=DEV)
    try:
        fn(key.to(DEV), value.to(DEV), kd, vd, slots.to(DEV), "auto", one, one)
    except Exception as exc:
        pytest.skip(f"vLLM's op could not be called: {exc}")
    torch.cuda.synchronize()
    CO.reshape_and_cache_flash(key, value, kc, vc, slots)
    assert torch.equal(kd.cpu(), kc) and torch.equal(vd.cpu(), vc)


def test_append_then_attend(native_lib):
    """A decode step as the backend runs it: append the new token of every request, then
    attend over the context that now includes it."""
    from pat_b200 import PrefixTreeCPP, prefix_attn_with_kvcache
    from pat_b200.cache_ops import reshape_and_cache_flash
    from pat_b200.workloads import make_values, scaled_down
    w = scaled_down(1, 8)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    # the last token of every request is the "new" one: blank it in the cache, then append it
    last_page = [t[(L - 1) // w.page_size] for L, t in zip(w.seq_lens, w.block_tables)]
    last_row = [(L - 1) % w.page_size for L in w.seq_lens]
    slots = torch.tensor([p * w.page_size + r for p, r in zip(last_page, last_row)], dtype=torch.int64)
    # requests that share their last page would write the same slot; keep the first writer only
    seen = set()
    for i, s in enumerate(slots.tolist()):
        if s in seen:
            slots[i] = -1
        seen.add(s)
    new_k = torch.stack([k[p, r] for p, r in zip(last_page, last_row)])
    new_v = torch.stack([v[p, r] for p, r in zip(last_page, last_row)])
    kd, vd = k.clone().to(DEV), v.clone().to(DEV)
    for p, r in zip(last_page, last_row):
        kd[p, r] = float("nan")
        vd[p, r] = float("nan")
    reshape_and_cache_flash(new_k.to(DEV), new_v.to(DEV), kd, vd, slots.to(DEV))
    tree = PrefixTreeCPP(w.page_size)
    table = torch.zeros(w.batch, max(len(t) for t in w.block_tables), dtype=torch.int32)
    for i, t in enumerate(w.block_tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    tree.build_radix_tree(list(w.seq_lens), table)
    tree.pack_schedule(None, w.group, w.num_kv_heads)
    tree.kernel_info.to_gpu(torch.device(DEV))
    qd = q.to(DEV)
    out = torch.empty_like(qd)
    prefix_attn_with_kvcache(qd, kd, vd, tree, scale, out)
    torch.cuda.synchronize()
    ref_o, _ = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    err = (out.float().cpu()[:, 0] - ref_o[:, 0]).abs()
    assert bool((err <= 2e-2 + 2e-2 * ref_o[:, 0].abs()).all()), err.max().item()


def test_append_argument_checks(native_lib):
    from pat_b200.cache_ops import reshape_and_cache_flash
    key, value, kc, vc, slots = _case(4, 2, 64, 4, 16, torch.float16, 1)
    args = [t.to(DEV) for t in (key, value, kc, vc, slots)]
    with pytest.raises(RuntimeError):
        reshape_and_cache_flash(*args, "fp8")
    with pytest.raises(RuntimeError):
        reshape_and_cache_flash(args[0], args[1].float(), *args[2:])
    with pytest.raises(RuntimeError):
        reshape_and_cache_flash(args[0].cpu(), *args[1:])
    with pytest.raises(RuntimeError):
        reshape_and_cache_flash(args[0], args[1], args[2], args[3], args[4][:2])
