"""Seeded synthetic decode batches: the five benchmark trees plus helpers.

Every workload is a set of decode requests over a paged KV cache (16-token
pages by default) whose block tables share physical pages wherever the requests
share a prefix.  The generator is pinned so that sizes reproduce exactly:

* ``rng = numpy.random.default_rng(seed)``;
* all length draws come first, in the order documented per workload;
* ``perm = rng.permutation(total_pages)``; shared segments take consecutive
  slices of ``perm`` in first-use order, then each request's private pages in
  request order (random physical placement);
* values: ``torch.manual_seed(seed)`` on the CPU generator, ``q``, ``k_cache``,
  ``v_cache`` drawn in that order as ``randn * 0.5`` in fp32 and rounded to the
  workload dtype.  ``softmax_scale = 1/sqrt(head_dim)``.

The reference's own kernel benchmark is synthetic in the same way
(``prefix_attn/utils.py:49-100`` builds block tables from a tree string and
``prefix_attn/utils.py:10-46`` fills a random paged cache).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np

PAGE = 16


@dataclass
class Workload:
    """Block tables and geometry of one synthetic decode batch."""

    name: str
    seed: int
    dtype: str                      # "bf16" | "fp16"
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    page_size: int
    seq_lens: List[int]
    block_tables: List[List[int]]   # unpadded physical page ids per request
    num_pages: int
    unique_tokens: int              # valid tokens summed over distinct segments
    description: str = ""
    extra: Dict[str, object] = field(default_factory=dict)

    @property
    def batch(self) -> int:
        return len(self.seq_lens)

    @property
    def group(self) -> int:
        """Query heads per KV head."""
        return self.num_q_heads // self.num_kv_heads

    @property
    def total_tokens(self) -> int:
        return int(sum(self.seq_lens))

    @property
    def elt_bytes(self) -> int:
        return 2

    def dedup_kv_bytes(self, kv_heads: int | None = None, q_heads: int | None = None) -> int:
        """Algorithmic bytes of one decode step: every distinct valid K and V
        token read once, plus Q read and O written."""
        hk = self.num_kv_heads if kv_heads is None else kv_heads
        hq = self.num_q_heads if q_heads is None else q_heads
        kv = 2 * self.unique_tokens * hk * self.head_dim * self.elt_bytes
        qo = 2 * self.batch * hq * self.head_dim * self.elt_bytes
        return kv + qo

    def padded_table(self) -> np.ndarray:
        width = max(len(r) for r in self.block_tables)
        out = np.zeros((self.batch, width), dtype=np.int32)
        for i, row in enumerate(self.block_tables):
            out[i, : len(row)] = row
        return out


# A request is (path of shared segments, private suffix tokens); a shared
# segment is (hashable key, tokens) with tokens a multiple of the page size.
_Req = Tuple[List[Tuple[object, int]], int]


def _place(reqs: Sequence[_Req], rng: np.random.Generator, page: int):
    seg_tokens: Dict[object, int] = {}
    for path, _ in reqs:
        for key, ntok in path:
            if key not in seg_tokens:
                assert ntok % page == 0, "shared segments are whole pages"
                seg_tokens[key] = ntok
    n_pages = sum(n // page for n in seg_tokens.values())
    n_pages += sum(-(-suffix // page) for _, suffix in reqs)
    perm = rng.permutation(n_pages)
    cursor = 0
    seg_pages: Dict[object, List[int]] = {}
    for key, ntok in seg_tokens.items():
        cnt = ntok // page
        seg_pages[key] = perm[cursor: cursor + cnt].tolist()
        cursor += cnt
    tables: List[List[int]] = []
    lens: List[int] = []
    for path, suffix in reqs:
        row: List[int] = []
        total = 0
        for key, ntok in path:
            row.extend(seg_pages[key])
            total += ntok
        cnt = -(-suffix // page)
        row.extend(perm[cursor: cursor + cnt].tolist())
        cursor += cnt
        tables.append(row)
        lens.append(total + suffix)
    unique = sum(seg_tokens.values()) + sum(s for _, s in reqs)
    return tables, lens, n_pages, unique


def make_config(cfg: int, page: int = PAGE) -> Workload:
    """The five benchmark workloads, ``cfg`` in 0..4 (seed == cfg).

    0: 8 requests, one 1024-token prefix, suffix ``integers(128, 513, 8)``;
       32/8 heads, D=128 (bf16 values; used for the CPU check).
    1: 64 requests, one 4096-token prefix, suffix ``integers(64, 1025, 64)``;
       bf16, 32/8 heads, D=128.
    2: 4 roots x 2048 -> 4 children x 512 -> 8 leaves, suffix
       ``integers(32, 513, 128)``; fp16, 32/4 heads, D=64.
    3: complete 4-ary tree, node levels 0..4 (1+4+16+64+256 nodes) of 256
       tokens each, plus a private 64-token tail per leaf (context 1344);
       bf16, 64/8 heads, D=128.
    4: 7 groups x 32 requests sharing 16384 tokens, suffix
       ``clip(round(exp(ln 2048 + 0.8 * standard_normal(224))), 16, 16384)``,
       then 32 unshared requests ``integers(1024, 16385, 32)``; bf16, 64/8
       heads, D=128.
    """
    rng = np.random.default_rng(cfg)
    reqs: List[_Req] = []
    if cfg == 0:
        suffix = rng.integers(128, 513, size=8)
        reqs = [([("prefix", 1024)], int(s)) for s in suffix]
        dtype, hq, hk, d = "bf16", 32, 8, 128
        desc = "8 req, shared 1024 prefix, suffix U[128,512]"
    elif cfg == 1:
        suffix = rng.integers(64, 1025, size=64)
        reqs = [([("prefix", 4096)], int(s)) for s in suffix]
        dtype, hq, hk, d = "bf16", 32, 8, 128
        desc = "64 req, shared 4096 prefix, suffix U[64,1024]"
    elif cfg == 2:
        suffix = rng.integers(32, 513, size=128)
        i = 0
        for root in range(4):
            for child in range(4):
                for _leaf in range(8):
                    path = [(("root", root), 2048), (("child", root, child), 512)]
                    reqs.append((path, int(suffix[i])))
                    i += 1
        dtype, hq, hk, d = "fp16", 32, 4, 64
        desc = "128 req, 4x2048 roots -> 4x512 children -> 8 leaves, suffix U[32,512]"
    elif cfg == 3:
        for leaf in range(256):
            path = [(("node", lvl, leaf // (4 ** (4 - lvl))), 256) for lvl in range(5)]
            reqs.append((path, 64))
        dtype, hq, hk, d = "bf16", 64, 8, 128
        desc = "256 leaves of a complete 4-ary tree (5 node levels x 256 tok) + 64-token tails"
    elif cfg == 4:
        draw = np.exp(math.log(2048) + 0.8 * rng.standard_normal(224))
        suffix = np.clip(np.round(draw), 16, 16384).astype(int)
        for g in range(7):
            for j in range(32):
                reqs.append(([(("group", g), 16384)], int(suffix[g * 32 + j])))
        ctx = rng.integers(1024, 16385, size=32)
        for j in range(32):
            reqs.append(([], int(ctx[j])))
        dtype, hq, hk, d = "bf16", 64, 8, 128
        desc = "224 req in 7 groups sharing 16384 tok + lognormal suffix; 32 unshared U[1024,16384]"
    else:
        raise ValueError(f"unknown config {cfg}")
    tables, lens, n_pages, unique = _place(reqs, rng, page)
    return Workload(
        name=f"cfg{cfg}", seed=cfg, dtype=dtype, num_q_heads=hq, num_kv_heads=hk,
        head_dim=d, page_size=page, seq_lens=lens, block_tables=tables,
        num_pages=n_pages, unique_tokens=unique, description=desc,
    )


def scaled_down(cfg: int, factor: int, page: int = PAGE) -> Workload:
    """A structurally identical but shorter variant of a benchmark workload
    (every segment length divided by ``factor``, rounded to whole pages for
    shared segments).  Used where the CPU oracle must finish in seconds."""
    full = make_config(cfg, page)
    rng = np.random.default_rng(1000 + cfg)

    def shrink_shared(n):
        return max(page, (n // factor) // page * page)

    def shrink_private(n):
        return max(1, n // factor)

    # Re-derive the request list from the full workload's structure.
    reqs: List[_Req] = []
    if cfg in (0, 1):
        plen = 1024 if cfg == 0 else 4096
        for L in full.seq_lens:
            reqs.append(([("prefix", shrink_shared(plen))], shrink_private(L - plen)))
    elif cfg == 2:
        i = 0
        for root in range(4):
            for child in range(4):
                for _ in range(8):
                    s = full.seq_lens[i] - 2560
                    reqs.append(([(("root", root), shrink_shared(2048)),
                                  (("child", root, child), shrink_shared(512))],
                                 shrink_private(s)))
                    i += 1
    elif cfg == 3:
        for leaf in range(256):
            path = [(("node", lvl, leaf // (4 ** (4 - lvl))), shrink_shared(256)) for lvl in range(5)]
            reqs.append((path, shrink_private(64)))
    elif cfg == 4:
        for i, L in enumerate(full.seq_lens):
            if i < 224:
                reqs.append(([(("group", i // 32), shrink_shared(16384))], shrink_private(L - 16384)))
            else:
                reqs.append(([], shrink_private(L)))
    tables, lens, n_pages, unique = _place(reqs, rng, page)
    return Workload(
        name=f"cfg{cfg}/{factor}", seed=1000 + cfg, dtype=full.dtype,
        num_q_heads=full.num_q_heads, num_kv_heads=full.num_kv_heads,
        head_dim=full.head_dim, page_size=page, seq_lens=lens, block_tables=tables,
        num_pages=n_pages, unique_tokens=unique,
        description=f"{full.description} (lengths / {factor})",
    )


def torch_dtype(name: str):
    import torch
    return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[name]


def make_values(w: Workload, device="cpu", kv_heads: slice | None = None):
    """``(q, k_cache, v_cache)`` for a workload, rounded to its dtype.

    Drawn on the CPU generator so that the CUDA path and the CPU oracle see the
    same bits.  ``kv_heads`` selects a KV-head shard (and the matching query
    heads) after the full draw, which keeps shards consistent across ranks.
    """
    import torch
    gen = torch.Generator(device="cpu")
    gen.manual_seed(w.seed)
    dt = torch_dtype(w.dtype)
    q = (torch.randn(w.batch, 1, w.num_q_heads, w.head_dim, generator=gen) * 0.5).to(dt)
    k = (torch.randn(w.num_pages, w.page_size, w.num_kv_heads, w.head_dim, generator=gen) * 0.5).to(dt)
    v = (torch.randn(w.num_pages, w.page_size, w.num_kv_heads, w.head_dim, generator=gen) * 0.5).to(dt)
    if kv_heads is not None:
        g = w.group
        qs = slice(kv_heads.start * g, kv_heads.stop * g)
        q = q[:, :, qs].contiguous()
        k = k[:, :, kv_heads].contiguous()
        v = v[:, :, kv_heads].contiguous()
    if str(device) != "cpu":
        q, k, v = q.to(device), k.to(device), v.to(device)
    return q, k, v


# ---------------------------------------------------------------------------------------------
# Counter-based cache values for the benchmark
# ---------------------------------------------------------------------------------------------
_MASK32 = 0xFFFFFFFF


def _lsr(x, n: int):
    """Logical right shift of an int64 tensor (torch's ``>>`` is arithmetic)."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def _as_i64(c: int) -> int:
    c &= (1 << 64) - 1
    return c - (1 << 64) if c >= (1 << 63) else c


def synthetic_pages(w: Workload, which: int, page_ids, device="cpu", kv_heads: slice | None = None):
    """K (``which`` = 0) or V (1) values of the listed physical pages of workload ``w``:
    ``[len(page_ids), page_size, heads, head_dim]`` in the workload's dtype, ~ N(0, 1) * 0.5.

    Every element is a pure function of (workload seed, K or V, page, row, global KV head, d): a
    64-bit mix of its linear index feeds a Box-Muller transform.  Any process can therefore
    produce any subset of the cache - a GPU rank its head shard, chunk by chunk, on the device; the
    CPU baseline only the pages of the requests it samples - without materialising the rest.
    (The last bit of the transcendental functions may differ between devices; checks that need
    identical bits read the values back from where they were generated.)
    """
    import torch
    ids = torch.as_tensor(page_ids, dtype=torch.int64, device=device).reshape(-1)
    hk = w.num_kv_heads
    heads = range(hk)[kv_heads] if kv_heads is not None else range(hk)
    h = torch.arange(heads.start, heads.stop, dtype=torch.int64, device=device)
    r = torch.arange(w.page_size, dtype=torch.int64, device=device)
    d = torch.arange(w.head_dim, dtype=torch.int64, device=device)
    idx = ((ids[:, None, None, None] * w.page_size + r[None, :, None, None]) * hk + h[None, None, :, None]) \
        * w.head_dim + d[None, None, None, :]
    x = idx + _as_i64((w.seed * 2 + which + 1) * 0x9E3779B97F4A7C15)
    x = (x ^ _lsr(x, 30)) * _as_i64(0xBF58476D1CE4E5B9)
    x = (x ^ _lsr(x, 27)) * _as_i64(0x94D049BB133111EB)
    x = x ^ _lsr(x, 31)
    u1 = (((x >> 8) & 0xFFFFFF) + 1).to(torch.float32) * (1.0 / (1 << 24))          # (0, 1]
    u2 = ((x >> 36) & 0xFFFFFF).to(torch.float32) * (2.0 * math.pi / (1 << 24))
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(u2)
    return (z * 0.5).to(torch_dtype(w.dtype))


def synthetic_queries(w: Workload, device="cpu", kv_heads: slice | None = None):
    """``q [batch, 1, heads, head_dim]`` of the benchmark, drawn on the CPU generator with the
    workload's seed (same bits in every process), optionally cut to a KV-head shard."""
    import torch
    gen = torch.Generator(device="cpu")
    gen.manual_seed(w.seed)
    q = (torch.randn(w.batch, 1, w.num_q_heads, w.head_dim, generator=gen) * 0.5).to(torch_dtype(w.dtype))
    if kv_heads is not None:
        heads = range(w.num_kv_heads)[kv_heads]
        q = q[:, :, heads.start * w.group: heads.stop * w.group].contiguous()
    return q if str(device) == "cpu" else q.to(device)
