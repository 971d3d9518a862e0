"""TEST INFRASTRUCTURE ONLY - CPU restatement of the reference attention path.

This file is the checker for the CUDA kernels; it is never the thing that is
shipped or (except for the reported CPU baseline) timed.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import it.

What it restates, in fp32 PyTorch on the host:

* ``dense_attention``  - the reference's oracle ``attention_ref``
  (``test/utils.py:7-58``): scores = (q / sqrt(d)) . k^T with the GQA repeat
  of K/V heads, ``-inf`` on padded keys, softmax, times V.  Additionally returns
  the natural-log LSE of the scaled scores, which is the quantity the
  reference kernel writes to ``softmax_lse`` (``csrc/softmax.h:168-188``,
  ``csrc/pat_fwd_kernel.h:421``) but never hands back to Python.
* ``paged_decode_attention`` - the dense K/V gather from the paged cache that
  the reference's generator performs (``prefix_attn/utils.py:34-44``), done per
  request so that the large workloads fit in memory.
* ``multi_position_attention`` - several query tokens per request, defined through one
  ``attention_ref`` call per position (the reference has no such path of its own).
* ``execute_plan`` - what a reference plan *means*: each box attends
  ``q_table[:num_seqs]`` x all their heads to the first ``kv_in_CTA`` tokens of
  its page list (``csrc/pat_fwd_kernel.h:25-299``, ``csrc/block_info.h:14-39``)
  and the per-query partials are combined by log-sum-exp
  (``csrc/pat_fwd_kernel.h:314-467``), with one slot per (box, query).

Pinning: ``tests/test_oracle.py`` checks ``dense_attention`` and
``multi_position_attention`` against outputs of the real ``attention_ref`` frozen under
``tests/golden/attention_*.npz`` and, when the reference checkout is present, against
``attention_ref`` run live.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    key_padding_mask: Optional[torch.Tensor] = None,
                    softmax_scale: Optional[float] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,T,H,D], k/v [B,S,Hkv,D], mask [B,S] (True = keep).

    Returns ``(out [B,T,H,D] fp32, lse [B,H,T] fp32)``.  Follows
    ``test/utils.py:32-58`` (scale applied to q, K/V heads repeated
    ``h -> (h g)``), all in fp32.
    """
    q32, k32, v32 = q.float(), k.float(), v.float()
    g = q32.shape[2] // k32.shape[2]
    k32 = k32.repeat_interleave(g, dim=2)
    v32 = v32.repeat_interleave(g, dim=2)
    d = q32.shape[-1]
    scale = (1.0 / math.sqrt(d)) if softmax_scale is None else softmax_scale
    if softmax_scale is None:
        scores = torch.einsum("bthd,bshd->bhts", q32 / math.sqrt(d), k32)
    else:
        scores = torch.einsum("bthd,bshd->bhts", q32 * scale, k32)
    if key_padding_mask is not None:
        scores = scores.masked_fill(~key_padding_mask[:, None, None, :], float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("bhts,bshd->bthd", probs, v32)
    return out, lse


def gather_request_kv(cache: torch.Tensor, pages: Sequence[int], length: int) -> torch.Tensor:
    """Dense ``[length, Hkv, D]`` keys (or values) of one request from the paged
    cache ``[num_pages, page, Hkv, D]`` (``prefix_attn/utils.py:34-38``)."""
    idx = torch.as_tensor(list(pages), dtype=torch.long)
    dense = cache[idx].reshape(-1, cache.shape[2], cache.shape[3])
    return dense[:length]


def paged_decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           seq_lens: Sequence[int], block_tables: Sequence[Sequence[int]],
                           softmax_scale: Optional[float] = None,
                           requests: Optional[Sequence[int]] = None
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Decode attention of every request (or the listed ones) over its own pages.

    q [B,1,H,D]; returns ``(out [n,1,H,D] fp32, lse [n,H] fp32)`` in the order
    of ``requests``.
    """
    page = k_cache.shape[1]
    ids = list(range(q.shape[0])) if requests is None else list(requests)
    outs, lses = [], []
    for b in ids:
        n_pages = -(-seq_lens[b] // page)
        kk = gather_request_kv(k_cache, block_tables[b][:n_pages], seq_lens[b])[None]
        vv = gather_request_kv(v_cache, block_tables[b][:n_pages], seq_lens[b])[None]
        o, l = dense_attention(q[b:b + 1], kk, vv, None, softmax_scale)
        outs.append(o[0])
        lses.append(l[0, :, 0])
    return torch.stack(outs), torch.stack(lses)


def multi_position_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lens: Sequence[int],
                             softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Several query tokens per request, the last ``T`` tokens of each context: q [B,T,H,D],
    k/v [B,S,Hkv,D], ``lens[b]`` = context length including those ``T`` tokens.  Position ``t``
    attends to the first ``lens[b] - T + 1 + t`` keys.

    The reference has no such path of its own (its serving backend hands steps with more than
    one query token to another library, ``plugin/vllm/attention/backends/prefix_attn.py:877-904``)
    and ``attention_ref`` has no causal argument (``test/utils.py:7-15``), so the definition is:
    one single-token ``attention_ref`` call per position, with the padding mask cut at that
    position's last visible key.  Returns ``(out [B,T,H,D], lse [B,T,H])``."""
    B, T = q.shape[0], q.shape[1]
    S = k.shape[1]
    lens_t = torch.as_tensor(list(lens))
    outs, lses = [], []
    for t in range(T):
        mask = torch.arange(S)[None, :] < (lens_t - T + 1 + t)[:, None]
        o, l = dense_attention(q[:, t:t + 1], k, v, mask, softmax_scale)
        outs.append(o)
        lses.append(l[:, :, 0])
    return torch.cat(outs, dim=1), torch.stack(lses, dim=1)


def paged_multi_position_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                   seq_lens: Sequence[int], block_tables: Sequence[Sequence[int]],
                                   softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``multi_position_attention`` over a paged cache, request by request.
    q [B,T,H,D]; returns ``(out [B,T,H,D] fp32, lse [B,T,H] fp32)``."""
    page = k_cache.shape[1]
    outs, lses = [], []
    for b in range(q.shape[0]):
        n_pages = -(-seq_lens[b] // page)
        kk = gather_request_kv(k_cache, block_tables[b][:n_pages], seq_lens[b])[None]
        vv = gather_request_kv(v_cache, block_tables[b][:n_pages], seq_lens[b])[None]
        o, l = multi_position_attention(q[b:b + 1], kk, vv, [seq_lens[b]], softmax_scale)
        outs.append(o[0])
        lses.append(l[0])
    return torch.stack(outs), torch.stack(lses)


def segment_attention(q_rows: torch.Tensor, k_seg: torch.Tensor, v_seg: torch.Tensor,
                      scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Partial attention of ``q_rows [n,H,D]`` over one KV segment
    ``[S,Hkv,D]``: returns the segment-normalised output ``[n,H,D]`` and the
    segment LSE ``[n,H]`` - the pair a box writes
    (``csrc/pat_fwd_kernel.h:254-298``)."""
    g = q_rows.shape[1] // k_seg.shape[1]
    kh = k_seg.float().repeat_interleave(g, dim=1)
    vh = v_seg.float().repeat_interleave(g, dim=1)
    s = torch.einsum("nhd,shd->nhs", q_rows.float(), kh) * scale
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("nhs,shd->nhd", torch.softmax(s, dim=-1), vh)
    return o, lse


def merge_partials(outs: torch.Tensor, lses: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """LSE merge of ``outs [n,H,D]`` / ``lses [n,H]`` along n
    (``csrc/pat_fwd_kernel.h:383-466``): ``lse = m + ln sum e^(lse_i - m)``,
    ``out = sum e^(lse_i - lse) out_i``."""
    lse = torch.logsumexp(lses, dim=0)
    w = torch.exp(lses - lse[None])
    return (w[..., None] * outs).sum(dim=0), lse


def iter_boxes(plan):
    """Yield ``(queries, pages, kv_len)`` for every box of a plan given as an
    object with list fields (``q_tables``, ``block_tables``,
    ``num_seqs_per_CTAs``, ``kv_in_CTAs``)."""
    for b in range(len(plan.MNWs)):
        for j, n in enumerate(plan.num_seqs_per_CTAs[b]):
            yield (list(plan.q_tables[b][j][:n]), list(plan.block_tables[b][j]),
                   int(plan.kv_in_CTAs[b][j]))


def execute_plan(plan, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Run a plan box by box in fp32 and merge per query with one slot per
    (box, query).  Returns ``(out [B,H,D], lse [B,H])``."""
    page = k_cache.shape[1]
    B, _, H, D = q.shape
    parts: List[List[Tuple[torch.Tensor, torch.Tensor]]] = [[] for _ in range(B)]
    for queries, pages, kv_len in iter_boxes(plan):
        n_pages = -(-kv_len // page)
        kk = gather_request_kv(k_cache, pages[:n_pages], kv_len)
        vv = gather_request_kv(v_cache, pages[:n_pages], kv_len)
        o, l = segment_attention(q[queries, 0], kk, vv, scale)
        for i, b in enumerate(queries):
            parts[b].append((o[i], l[i]))
    out = torch.zeros(B, H, D)
    lse = torch.full((B, H), float("-inf"))
    for b in range(B):
        if parts[b]:
            o = torch.stack([p[0] for p in parts[b]])
            l = torch.stack([p[1] for p in parts[b]])
            out[b], lse[b] = merge_partials(o, l)
    return out, lse
