"""The vLLM V1 attention backend (pat_b200/vllm_v1.py) against the V1 interface classes of the
vLLM installed in this environment; skipped where vLLM does not import.  The CPU tests drive the
metadata builder (plan building and in-place growth across steps); the GPU test runs decode and
speculative-decode steps through ``PrefixAttnImpl.forward`` and checks them against the oracle."""
import math
from types import SimpleNamespace

import pytest
import torch

from oracle import attention_oracle as O
from pat_b200 import PrefixTreeCPP
from pat_b200.workloads import make_values, scaled_down, torch_dtype

import cases as CS

try:
    from vllm.v1.attention.backend import (AttentionBackend, AttentionImpl, AttentionMetadataBuilder,
                                           CommonAttentionMetadata)
    from pat_b200 import vllm_v1 as V
    _SKIP = None
except Exception as exc:    # vLLM absent or not importable here
    _SKIP = f"vLLM's V1 attention interface does not import: {exc}"

pytestmark = pytest.mark.skipif(_SKIP is not None, reason=_SKIP or "")


def _config(hq, hk, d):
    model = SimpleNamespace(get_num_attention_heads=lambda pc: hq, get_num_kv_heads=lambda pc: hk,
                            get_head_size=lambda: d)
    return SimpleNamespace(model_config=model, parallel_config=SimpleNamespace())


def _common(w, query_len, device, lens=None, table=None):
    lens = list(w.seq_lens) if lens is None else lens
    B = len(lens)
    qsl = torch.arange(0, (B + 1) * query_len, query_len, dtype=torch.int32)
    tab = torch.from_numpy(w.padded_table()) if table is None else table
    seq = torch.tensor(lens, dtype=torch.int32)
    slots = []
    for b, L in enumerate(lens):
        for pos in range(L - query_len, L):
            slots.append(int(tab[b, pos // w.page_size]) * w.page_size + pos % w.page_size)
    return CommonAttentionMetadata(
        query_start_loc=qsl.to(device), query_start_loc_cpu=qsl, seq_lens=seq.to(device), num_reqs=B,
        num_actual_tokens=B * query_len, max_query_len=query_len, max_seq_len=max(lens),
        block_table_tensor=tab.to(device), slot_mapping=torch.tensor(slots, dtype=torch.int64, device=device),
        causal=True, _seq_lens_cpu=seq)


def test_backend_follows_the_v1_interface():
    B = V.PrefixAttnBackend
    assert issubclass(B, AttentionBackend) and issubclass(V.PrefixAttnImpl, AttentionImpl)
    assert issubclass(V.PrefixAttnMetadataBuilder, AttentionMetadataBuilder)
    assert B.get_name() == "PREFIX_ATTN" and B.get_impl_cls() is V.PrefixAttnImpl
    assert B.get_builder_cls() is V.PrefixAttnMetadataBuilder
    assert B.get_kv_cache_shape(10, 16, 8, 128) == (2, 10, 16, 8, 128)
    with pytest.raises(ValueError):
        B.get_kv_cache_shape(10, 24, 8, 128)
    assert B.supports_head_size(128) and B.supports_head_size(64) and not B.supports_head_size(96)
    assert B.supports_block_size(16) and B.supports_block_size(32) and not B.supports_block_size(8)
    assert B.forward_includes_kv_cache_update is False
    with pytest.raises(NotImplementedError):
        V.PrefixAttnImpl(8, 128, 0.1, 8, alibi_slopes=[1.0] * 8)
    with pytest.raises(NotImplementedError):
        V.PrefixAttnImpl(8, 128, 0.1, 8, kv_cache_dtype="fp8")


def test_builder_plans_decode_steps_and_grows_them_in_place(native_lib):
    w = scaled_down(1, 4)
    dev = torch.device("cpu")
    builder = V.PrefixAttnMetadataBuilder(SimpleNamespace(block_size=w.page_size, dtype=torch.bfloat16), ["l0"],
                                          _config(w.num_q_heads, w.num_kv_heads, w.head_dim), dev)
    md = builder.build(0, _common(w, 1, dev))
    assert md.query_len == 1 and md.num_reqs == w.batch and md.num_actual_tokens == w.batch
    fresh = PrefixTreeCPP(w.page_size)
    fresh.build_radix_tree(list(w.seq_lens), torch.from_numpy(w.padded_table()))
    fresh.pack_schedule(None, w.group, w.num_kv_heads)
    assert CS.native_plan_to_dict(md.tree.kernel_info) == CS.native_plan_to_dict(fresh.kernel_info)
    # next step: every request one token longer, inside its last page -> same tree object, grown
    lens = [l + 1 if l % w.page_size else l for l in w.seq_lens]      # (requests at a page end stand still here)
    assert lens != list(w.seq_lens)
    md2 = builder.build(0, _common(w, 1, dev, lens=lens))
    assert md2.tree is md.tree and builder._planners[1].advances == 1
    grown = PrefixTreeCPP(w.page_size)
    grown.build_radix_tree(lens, torch.from_numpy(w.padded_table()))
    assert md2.tree.nodes() == grown.nodes()
    # a step with 4 query tokens per request has its own planner; a ragged (prefill) step has no tree
    md4 = builder.build(0, _common(w, 4, dev))
    assert md4.query_len == 4 and md4.tree is not md.tree
    ragged = _common(w, 1, dev)
    ragged.query_start_loc_cpu = ragged.query_start_loc_cpu.clone()
    ragged.query_start_loc_cpu[-1] += 5
    md5 = builder.build(0, ragged)
    assert md5.tree is None and md5.query_len == 0


@pytest.mark.gpu
@pytest.mark.parametrize("query_len", [1, 4])
def test_forward_through_the_v1_interface_against_the_oracle(query_len, native_lib):
    dev = torch.device("cuda:0")
    w = scaled_down(1, 4)
    _, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    B, H, hk, D, T = w.batch, w.num_q_heads, w.num_kv_heads, w.head_dim, query_len
    g = torch.Generator().manual_seed(3)
    q = (torch.randn(B * T, H, D, generator=g) * 0.5).to(dtype)
    new_k = (torch.randn(B * T, hk, D, generator=g) * 0.5).to(dtype)
    new_v = (torch.randn(B * T, hk, D, generator=g) * 0.5).to(dtype)
    builder = V.PrefixAttnMetadataBuilder(SimpleNamespace(block_size=w.page_size, dtype=dtype), ["l0"],
                                          _config(H, hk, D), dev)
    impl = V.PrefixAttnImpl(H, D, 1.0 / math.sqrt(D), hk)
    cam = _common(w, T, dev)
    md = builder.build(0, cam)
    kv_cache = torch.stack([k, v]).to(dev)
    # the step's new tokens are written by the backend's own cache update, then attended
    impl.do_kv_cache_update(None, new_k.to(dev), new_v.to(dev), kv_cache, cam.slot_mapping)
    out = torch.full((B * T + 3, H * D), float("nan"), dtype=dtype, device=dev)     # padded like vLLM's buffers
    qpad = torch.cat([q, torch.zeros(3, H, D, dtype=dtype)]).to(dev)
    impl.forward(None, qpad, None, None, kv_cache, md, out)
    torch.cuda.synchronize()
    # oracle on the updated cache
    slots = cam.slot_mapping.cpu()
    k2, v2 = k.clone(), v.clone()
    k2.view(-1, hk, D)[slots] = new_k
    v2.view(-1, hk, D)[slots] = new_v
    scale = 1.0 / math.sqrt(D)
    ref, _ = O.paged_multi_position_attention(q.view(B, T, H, D), k2, v2, w.seq_lens, w.block_tables, scale)
    got = out[:B * T].float().cpu().view(B, T, H, D)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-2
    assert bool(((got - ref).abs() <= tol + tol * ref.abs()).all())
    assert torch.isnan(out[B * T:].float()).all()
