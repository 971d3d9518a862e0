"""Parity of the CUDA path with the fp32 oracle (run with ``-m gpu`` on a B200).

Tolerances are the ones the task states: bf16 atol = rtol = 2e-2, fp16 1e-2 against
the fp32 reference, LSE within 1e-3.  Every call goes through the public op and
therefore through the C ABI (``pat_b200_decode``)."""
import ctypes
import math

import numpy as np
import pytest
import torch

import cases as C
from oracle import attention_oracle as O
from pat_b200 import KernelInfo, PrefixTree, PrefixTreeCPP, AsyncTree, prefix_attn_with_kvcache
from abi_util import decode_args, packed_tree, workspace_bytes
from pat_b200 import _native as N
from pat_b200 import _prefix_attn as P
from pat_b200.sharding import ShardedDecode, kv_head_range, shard_views
from pat_b200.workloads import make_config, make_values, scaled_down, torch_dtype

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.bfloat16: 2e-2, torch.float16: 1e-2}


def _padded(tables):
    width = max(len(r) for r in tables)
    t = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, r in enumerate(tables):
        t[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
    return t


def _values(n_pages, page, hq, hk, d, batch, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(batch, 1, hq, d, generator=g) * 0.5).to(dtype)
    k = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(n_pages, page, hk, d, generator=g) * 0.5).to(dtype)
    return q, k, v


def _run_tree(q, k, v, seq_lens, tables, page, hratio, hk, scale, semantics="cpp", cfg=None, mnws=None, flags=0):
    tree = PrefixTreeCPP(page, semantics)
    if semantics == "cpp":
        tree.build_radix_tree(list(seq_lens), _padded(tables))
    else:
        tree.build_radix_tree(list(seq_lens), [list(r) for r in tables])
    tree.pack_schedule(mnws, hratio, hk)
    P.set_default_config(cfg)
    try:
        tree.kernel_info.to_gpu(torch.device(DEV))
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
        out = torch.full_like(qd, float("nan"))
        lse = torch.full((q.shape[0], q.shape[2]), float("nan"), device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        prefix_attn_with_kvcache(qd, kd, vd, tree, scale, out, lse_out=lse, _status=status, _flags=flags)
        torch.cuda.synchronize()
    finally:
        P.set_default_config(None)
    assert status[0].item() == 0, "a bounded wait gave up inside a kernel"
    return out.float().cpu()[:, 0], lse.cpu(), tree


def _assert_close(out, lse, ref_o, ref_l, dtype):
    tol = TOL[dtype]
    err = (out - ref_o).abs()
    bound = tol + tol * ref_o.abs()
    assert bool((err <= bound).all()), f"max |dO| = {err.max().item():.3e}"
    lerr = (lse - ref_l).abs().max().item()
    assert lerr <= 1e-3, f"max |dLSE| = {lerr:.3e}"


CONFIGS = [
    # (dtype, hq, hk, d, page)
    (torch.bfloat16, 32, 8, 128, 16),
    (torch.float16, 32, 4, 64, 16),
    (torch.bfloat16, 8, 8, 128, 16),      # MHA, ratio 1
    (torch.float16, 16, 8, 128, 32),      # ratio 2, 32-token pages
    (torch.bfloat16, 16, 2, 64, 16),      # ratio 8, D = 64
]


@pytest.mark.parametrize("dtype,hq,hk,d,page", CONFIGS)
@pytest.mark.parametrize("seed", [3, 6, 8, 11])
def test_random_batches(dtype, hq, hk, d, page, seed, native_lib):
    case = C.random_case(seed)
    # rebuild the same structure on the requested page size
    lens = [max(1, l * page // case.block_size - (l % 3)) for l in case.seq_lens]
    tables = [r[:max(1, -(-lens[i] // page))] for i, r in enumerate(case.tables)]
    lens = [min(l, len(t) * page) for l, t in zip(lens, tables)]
    # a request must own its last page unless it fills it
    fresh = max(max(r) for r in tables) + 1
    for i, (l, t) in enumerate(zip(lens, tables)):
        if l % page:
            t[-1] = fresh
            fresh += 1
    q, k, v = _values(fresh, page, hq, hk, d, len(lens), dtype, seed)
    scale = 1.0 / math.sqrt(d)
    out, lse, _ = _run_tree(q, k, v, lens, tables, page, hq // hk, hk, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, lens, tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)


def _random_forest(seed, page=16, cap=400):
    """Requests as root-to-leaf paths of random trees whose segments are 1..44 pages long (ragged
    against the kernels' 128-token tiles), tails of 1..299 tokens, random physical placement."""
    rng = np.random.default_rng(1000 + seed)
    next_page = [0]

    def alloc(n):
        first = next_page[0]
        next_page[0] += n
        return list(range(first, first + n))

    reqs = []

    def grow(prefix, depth):
        if depth == 0 or (depth < 3 and rng.random() < 0.15):
            for _ in range(int(rng.integers(1, 5))):
                tail = int(rng.integers(1, 300))
                reqs.append((prefix + alloc(-(-tail // page)), len(prefix) * page + tail))
            return
        for _ in range(int(rng.integers(2, 6))):
            grow(prefix + alloc(int(rng.integers(1, 45))), depth - 1)

    for _ in range(int(rng.integers(1, 4))):
        grow(alloc(int(rng.integers(1, 60))), int(rng.integers(1, 4)))
    reqs = reqs[:cap]
    order = rng.permutation(next_page[0])
    tables = [[int(order[p]) for p in pages] for pages, _ in reqs]
    return [l for _, l in reqs], tables, next_page[0]


@pytest.mark.parametrize("seed", [2, 4, 5, 10])
@pytest.mark.parametrize("dtype,hq,hk,d", [(torch.bfloat16, 32, 4, 128), (torch.float16, 16, 2, 64)])
def test_random_forests_with_ragged_segments(seed, dtype, hq, hk, d, native_lib):
    """Many dense items per persistent CTA, with 1, 2, 3+ tiles and partial last tiles: the tile
    stream of the tcgen05 kernel crosses item boundaries all the time."""
    lens, tables, pages = _random_forest(seed)
    q, k, v = _values(pages, 16, hq, hk, d, len(lens), dtype, seed)
    scale = 1.0 / math.sqrt(d)
    out, lse, tree = _run_tree(q, k, v, lens, tables, 16, hq // hk, hk, scale)
    hdr = tree.kernel_info.device_work(torch.device(DEV)).header
    assert hdr.num_dense_items > 0 and hdr.num_dense_ctas > 0
    ref_o, ref_l = O.paged_decode_attention(q, k, v, lens, tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)


@pytest.mark.parametrize("cfg", [0, 1, 2])
def test_benchmark_configs_full(cfg, native_lib):
    w = make_config(cfg)
    q, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)


@pytest.mark.parametrize("cfg", [3, 4])
def test_benchmark_configs_full_size_every_request(cfg, native_lib):
    """Full-size workloads: the oracle checks all 256 requests (some tens of seconds of dense fp32
    attention on the host), and the result must not depend on how the work was cut."""
    w = make_config(cfg)
    q, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)
    # other cuts of the same work: streaming kernel only, and tiny chunks
    alt1, lse1, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale,
                              cfg=P.WorkConfig(disable_dense=1))
    alt2, lse2, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale,
                              semantics="py", cfg=P.WorkConfig(chunk_tokens_max=512, dense_piece_tokens_min=128))
    tol = TOL[dtype]
    assert (out - alt1).abs().max().item() <= tol
    assert (out - alt2).abs().max().item() <= tol
    assert (lse - lse1).abs().max().item() <= 1e-3
    assert (lse - lse2).abs().max().item() <= 1e-3


def test_dense_kernel_beside_the_streaming_kernel(native_lib):
    """cfg4 at full size is long enough for the work list to give the dense kernel only a share
    of the SMs and run it beside the streaming kernel.  The result must be bit-identical when the
    streaming kernel is an ordinary launch instead (flag PAT_NO_OVERLAP = 16: same work list, same
    arithmetic, only the launch order differs), and agree with the all-SM cut of the dense work."""
    w = make_config(4)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    args = (q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    out, lse, tree = _run_tree(*args)
    hdr = tree.kernel_info.device_work(torch.device(DEV)).header
    assert 0 < hdr.num_dense_ctas < 100 and hdr.num_stream_items > 0
    serial, lse_s, _ = _run_tree(*args, flags=16)
    assert torch.equal(out, serial) and torch.equal(lse, lse_s)
    wide, lse_w, tree_w = _run_tree(*args, cfg=P.WorkConfig(dense_tile_ns=-1))
    assert tree_w.kernel_info.device_work(torch.device(DEV), P.WorkConfig(dense_tile_ns=-1)).header.num_dense_ctas > hdr.num_dense_ctas
    assert (out - wide).abs().max().item() <= TOL[torch.bfloat16]
    assert (lse - lse_w).abs().max().item() <= 1e-3


@pytest.mark.parametrize("cfg,factor", [(3, 4), (4, 32)])
def test_scaled_configs_all_requests(cfg, factor, native_lib):
    w = scaled_down(cfg, factor)
    q, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)


@pytest.mark.parametrize("opts", [dict(disable_dense=1), dict(dense_min_rows=64),
                                  dict(chunk_tokens_min=16, chunk_tokens_max=64, dense_piece_tokens_min=64),
                                  dict(items_per_sm=64)])
def test_work_cuts_agree_with_oracle(opts, native_lib):
    w = scaled_down(1, 4)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale,
                            cfg=P.WorkConfig(**opts))
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, torch.bfloat16)


@pytest.mark.parametrize("cfg,factor", [(1, 2), (2, 2), (3, 2)])
def test_dense_tiles_against_oracle(cfg, factor, native_lib):
    """Shared segments run on tcgen05/TMEM; half-size workloads, every request checked."""
    w = scaled_down(cfg, factor)
    q, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, tree = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    assert tree.kernel_info.device_work(torch.device(DEV)).header.num_dense_items > 0
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, dtype)


def test_sixteen_argument_form_with_python_scheduler(native_lib):
    """The call the reference's kernel benchmark makes (benchmark/benchmark_kernel.py:234-265)."""
    w = make_config(0)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    tree = PrefixTree(w.page_size)
    tree.build_radix_tree(list(w.seq_lens), [list(r) for r in w.block_tables])
    ki: KernelInfo = tree.pack_schedule(MNWs=None, HRatio=w.group, kvHead=w.num_kv_heads, use_compute_model=False)
    ki.to_tensor(device=DEV)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.empty_like(qd)
    lse = torch.empty(w.batch, w.num_q_heads, device=DEV)

    def call(o):
        prefix_attn_with_kvcache(qd, kd, vd, ki.num_split_per_seq, ki.q_tables, ki.block_tables,
                                 ki.num_seqs_per_CTAs, ki.CTA_ranks, ki.kv_in_CTAs, ki.MNWs, ki.max_split_per_seq,
                                 ki.max_seqs_in_CTA, ki.max_blocks_in_CTA, scale, o, None, lse_out=lse)
    call(out)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out.float().cpu()[:, 0], lse.cpu(), ref_o[:, 0], ref_l, torch.bfloat16)
    # bare tensors without the attached host plan (one D2H read-back) give the same result
    bare = [t.clone() for t in (ki.num_split_per_seq,)]
    out2 = torch.empty_like(qd)
    prefix_attn_with_kvcache(qd, kd, vd, bare[0], [t.clone() for t in ki.q_tables],
                             [t.clone() for t in ki.block_tables], [t.clone() for t in ki.num_seqs_per_CTAs],
                             [t.clone() for t in ki.CTA_ranks], [t.clone() for t in ki.kv_in_CTAs], ki.MNWs,
                             ki.max_split_per_seq, ki.max_seqs_in_CTA, ki.max_blocks_in_CTA, scale, out2)
    assert torch.equal(out, out2)


def test_async_tree_and_strided_views_like_the_serving_backend(native_lib):
    """plugin/vllm/attention/backends/prefix_attn.py:330-338, 806-807, 908-915: AsyncTree from a
    padded CPU table, caches as the two halves of one tensor, q / out as unsqueezed views."""
    w = scaled_down(2, 4)
    q, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    kv = torch.stack([k, v]).to(DEV)                      # [2, pages, page, hk, d]
    key_cache, value_cache = kv[0], kv[1]
    decode_query = q[:, 0].to(DEV)                        # [B, H, D]
    decode_output = torch.empty_like(decode_query)
    at = AsyncTree(block_size=w.page_size, seq_lens=list(w.seq_lens), table=_padded(w.block_tables), MNWs=None,
                   HRatio=w.group, kvHead=w.num_kv_heads, device=torch.device(DEV))
    tree = at.tree
    lse = torch.empty(w.batch, w.num_q_heads, device=DEV)
    prefix_attn_with_kvcache(q=decode_query.unsqueeze(1), k_cache_paged=key_cache, v_cache_paged=value_cache,
                             tree=tree, softmax_scale=scale, out=decode_output.unsqueeze(1), lse_out=lse)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(decode_output.float().cpu(), lse.cpu(), ref_o[:, 0], ref_l, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_against_flash_attention_like_the_reference_test(dtype, native_lib):
    """The reference checks itself against flash-attention's paged decode kernel with
    max |PAT - FlashAttention| <= 1e-2 (test/test.py:64, 150-165).  Same check here, on 256-token
    pages (the page size the installed flash-attention accepts); skipped where that library does
    not load or cannot run."""
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:
        pytest.skip(f"flash_attn is not available: {exc}")
    page, hq, hk, d = 256, 32, 8, 128
    rng = np.random.default_rng(0)
    tables, lens, nxt = [], [], 0
    for _ in range(3):                                   # 3 groups of 8 requests sharing 2 pages
        shared = [nxt, nxt + 1]
        nxt += 2
        for _ in range(8):
            n = int(rng.integers(1, 4))
            tables.append(shared + list(range(nxt, nxt + n)))
            nxt += n
            lens.append(len(tables[-1]) * page - int(rng.integers(0, 255)))
    q, k, v = _values(nxt, page, hq, hk, d, len(lens), dtype, 3)
    scale = 1.0 / math.sqrt(d)
    out, _, _ = _run_tree(q, k, v, lens, tables, page, hq // hk, hk, scale)
    try:
        ref = flash_attn_with_kvcache(q.to(DEV), k.to(DEV), v.to(DEV),
                                      cache_seqlens=torch.tensor(lens, dtype=torch.int32, device=DEV),
                                      block_table=_padded(tables).to(DEV), softmax_scale=scale, causal=True)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"flash_attn could not run here: {exc}")
    assert (ref.float().cpu()[:, 0] - out).abs().max().item() <= 1e-2


def test_garbage_beyond_the_valid_tokens_is_ignored(native_lib):
    """Cache rows past a request's length may hold anything (NaN included)."""
    page, hq, hk, d = 16, 16, 2, 128
    lens = [5, 37, 16, 1, 250]
    tables = [[0], [1, 2, 3], [4], [5], list(range(6, 22))]
    q, k, v = _values(22, page, hq, hk, d, len(lens), torch.bfloat16, 5)
    kk, vv = k.clone(), v.clone()
    for L, t in zip(lens, tables):
        if L % page:
            kk[t[-1], L % page:] = float("nan")
            vv[t[-1], L % page:] = float("inf")
    scale = 1.0 / math.sqrt(d)
    out, lse, _ = _run_tree(q, kk, vv, lens, tables, page, hq // hk, hk, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, lens, tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, torch.bfloat16)


def test_identical_requests_share_every_page(native_lib):
    page, hq, hk, d = 16, 32, 4, 128
    lens = [700] * 40
    tables = [list(range(44))] * 40
    q, k, v = _values(44, page, hq, hk, d, 40, torch.float16, 9)
    scale = 1.0 / math.sqrt(d)
    out, lse, tree = _run_tree(q, k, v, lens, tables, page, hq // hk, hk, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, lens, tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, torch.float16)
    work = tree.kernel_info.device_work(torch.device(DEV))
    assert work.header.unique_tokens == 700 and work.header.num_dense_items > 0


def test_reference_error_behaviour_on_device(native_lib):
    w = scaled_down(0, 8)
    q, k, v = make_values(w, device=DEV)
    tree = PrefixTreeCPP(w.page_size)
    tree.build_radix_tree(list(w.seq_lens), _padded(w.block_tables))
    tree.pack_schedule(None, w.group, w.num_kv_heads)
    out = torch.empty_like(q)
    with pytest.raises(RuntimeError, match="must be on CUDA"):        # plan not moved to the GPU
        prefix_attn_with_kvcache(q, k, v, tree, 0.1, out)
    tree.kernel_info.to_gpu(DEV)
    with pytest.raises(RuntimeError, match="same dtype"):
        prefix_attn_with_kvcache(q, k.half(), v, tree, 0.1, out)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        prefix_attn_with_kvcache(q.float(), k.float(), v.float(), tree, 0.1, out.float())
    with pytest.raises(RuntimeError, match="head_size"):
        prefix_attn_with_kvcache(q[..., :32].contiguous(), k[..., :32].contiguous(), v[..., :32].contiguous(),
                                 tree, 0.1, out[..., :32].contiguous())
    prefix_attn_with_kvcache(q, k, v, tree, 0.1, out)                  # and the good call still works
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert P.last_launch_count() >= 2


# ---------------------------------------------------------------------------------------------
# The shapes one rank of a KV-head-sharded run sees: 8 query heads per KV head, 1 / 2 / 4 KV heads
# ---------------------------------------------------------------------------------------------
def _shard_case(cfg, factor, world, rank):
    w = scaled_down(cfg, factor)
    q, k, v = make_values(w)
    lo, hi = kv_head_range(w.num_kv_heads, world, rank)
    scale = 1.0 / math.sqrt(w.head_dim)
    ref_o, ref_l = O.paged_decode_attention(q[:, :, lo * w.group: hi * w.group].float(), k[:, :, lo:hi].float(),
                                            v[:, :, lo:hi].float(), w.seq_lens, w.block_tables, scale)
    return w, q, k, v, lo, hi, scale, ref_o, ref_l


@pytest.mark.parametrize("cfg,factor", [(4, 16), (3, 2)])
@pytest.mark.parametrize("world,rank", [(8, 5), (4, 1), (2, 1)])
def test_one_rank_of_a_sharded_run_contiguous_caches(cfg, factor, world, rank, native_lib):
    """What the benchmark does on every rank: its own contiguous [pages, page, Hkv/n, D] caches and a
    plan packed with kvHead = Hkv/n."""
    w, q, k, v, lo, hi, scale, ref_o, ref_l = _shard_case(cfg, factor, world, rank)
    g = w.group
    qs, ks, vs = q[:, :, lo * g: hi * g].contiguous(), k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous()
    assert ks.shape[2] == w.num_kv_heads // world and qs.shape[2] == 8 * ks.shape[2]
    out, lse, _ = _run_tree(qs, ks, vs, w.seq_lens, w.block_tables, w.page_size, g, hi - lo, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, torch_dtype(w.dtype))


@pytest.mark.parametrize("cfg,factor", [(4, 16), (3, 2)])
@pytest.mark.parametrize("world,rank", [(8, 2), (4, 3), (2, 0)])
def test_one_rank_of_a_sharded_run_views_of_the_full_cache(cfg, factor, world, rank, native_lib):
    """The other way to shard: the rank's heads as strided views (head stride = D, row stride =
    Hkv * D) of full caches, through ``shard_views`` and ``ShardedDecode``."""
    w, q, k, v, lo, hi, scale, ref_o, ref_l = _shard_case(cfg, factor, world, rank)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    qs, ks, vs = shard_views(qd, kd, vd, world, rank)
    assert not ks.is_contiguous() and ks.data_ptr() == kd[:, :, lo:].data_ptr()
    dec = ShardedDecode(w.page_size, list(w.seq_lens), _padded(w.block_tables), w.num_q_heads, w.num_kv_heads,
                        world, rank, torch.device(DEV))
    full_out = torch.full_like(qd, float("nan"))
    out_view = full_out[:, :, lo * w.group: hi * w.group]           # written in place, strided
    lse = torch.full((w.batch, (hi - lo) * w.group), float("nan"), device=DEV)
    dec(qs, ks, vs, scale, out_view, lse_out=lse)
    torch.cuda.synchronize()
    P.check_status(DEV)
    _assert_close(out_view.float().cpu()[:, 0], lse.cpu(), ref_o[:, 0], ref_l, torch_dtype(w.dtype))
    untouched = torch.ones(w.num_q_heads, dtype=torch.bool)
    untouched[lo * w.group: hi * w.group] = False
    assert torch.isnan(full_out[:, :, untouched.to(DEV)].float()).all()     # other ranks' heads are not written


# ---------------------------------------------------------------------------------------------
# Ordering of the three kernels, and the bounded waits
# ---------------------------------------------------------------------------------------------
def test_merge_waits_for_a_dense_kernel_that_outlasts_the_streaming_kernel(native_lib):
    """The streaming kernel starts while the dense kernel runs and does not use its results; the
    merge needs both.  Here the dense kernel is the long one (one share: 16 CTAs walk the whole
    4096-token prefix while the short suffixes stream on the other SMs).  Direct launches and
    replays of a captured graph must give the bits of the serial order (flag PAT_NO_OVERLAP),
    with the partial-result scratch poisoned before every run."""
    lib = native_lib
    w = make_config(1)
    q, k, v = make_values(w, device=DEV)
    scale = 1.0 / math.sqrt(w.head_dim)
    P.set_default_config(P.WorkConfig(dense_piece_tokens_min=1 << 20, dense_tile_ns=-1))
    try:
        tree = packed_tree(w, DEV)
        work = tree.kernel_info.device_work(torch.device(DEV))
    finally:
        P.set_default_config(None)
    hdr = work.header
    assert hdr.num_dense_ctas <= 2 * w.num_kv_heads and hdr.num_stream_items > 0
    ws = torch.empty(workspace_bytes(lib, work, w.num_q_heads, w.head_dim), dtype=torch.uint8, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)

    def run(out, lse, flags, stream):
        a = decode_args(q, k, v, out, work, scale, ws, lse=lse, status=status, flags=flags)
        rc = lib.pat_b200_decode(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream))
        assert rc == 0, N.strerror(rc)

    def fresh():
        return torch.full_like(q, float("nan")), torch.full((w.batch, w.num_q_heads), float("nan"), device=DEV)

    with torch.cuda.device(DEV):
        cur = torch.cuda.current_stream()
        def poison():
            ws.fill_(0xFF)                              # every float of the scratch is a NaN
            ws[:256].zero_()                            # (the control words at its head stay zero)
        poison()
        want, want_lse = fresh()
        run(want, want_lse, 16, cur)
        torch.cuda.synchronize()
        assert torch.isfinite(want.float()).all()
        for _ in range(3):
            poison()
            got, got_lse = fresh()
            run(got, got_lse, 0, cur)
            torch.cuda.synchronize()
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
        # the same step as a graph: scratch poisoning + decode, replayed
        got, got_lse = fresh()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            poison()
            run(got, got_lse, 0, torch.cuda.current_stream())
        for _ in range(3):
            got.fill_(float("nan"))
            got_lse.fill_(float("nan"))
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
    assert status[0].item() == 0


def test_a_wait_that_runs_out_reports_and_returns(native_lib):
    """Every wait inside the kernels has a limit, after which the kernel records a code in the
    status word and returns.  The self-test kernel waits on a barrier nobody arrives on (nothing
    asynchronous is in flight) with a 50 us limit; afterwards the GPU still decodes correctly."""
    lib = native_lib
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        rc = lib.pat_b200_selftest_wait(50, ctypes.c_void_p(status.data_ptr()),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, N.strerror(rc)
        torch.cuda.synchronize()
    code, waited_ns = status[0].item(), status[1].item()
    assert code == 99, "the wait should have given up"
    assert 50_000 <= waited_ns < 50_000_000, waited_ns
    assert lib.pat_b200_selftest_wait(0, ctypes.c_void_p(status.data_ptr()), None) == -1
    # an ordinary decode on the same GPU afterwards
    w = scaled_down(1, 8)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, _ = _run_tree(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o[:, 0], ref_l, torch.bfloat16)


def test_default_status_word_and_upload_ordering_on_a_side_stream(native_lib):
    """The public op reports into a per-device status word when the caller passes none, and a plan
    uploaded by a worker thread (default stream) is safe to use at once on a non-blocking side
    stream: the first launch there waits for the upload."""
    w = scaled_down(3, 2)
    q, k, v = make_values(w)
    scale = 1.0 / math.sqrt(w.head_dim)
    ref_o, ref_l = O.paged_decode_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(DEV)
    at = AsyncTree(block_size=w.page_size, seq_lens=list(w.seq_lens), table=_padded(w.block_tables), MNWs=None,
                   HRatio=w.group, kvHead=w.num_kv_heads, device=torch.device(DEV))
    out = torch.full_like(qd, float("nan"))
    lse = torch.full((w.batch, w.num_q_heads), float("nan"), device=DEV)
    with torch.cuda.stream(side):
        prefix_attn_with_kvcache(qd, kd, vd, at.tree, scale, out, lse_out=lse)
    side.synchronize()
    P.check_status(DEV)
    assert P.status_word(DEV)[0].item() == 0
    _assert_close(out.float().cpu()[:, 0], lse.cpu(), ref_o[:, 0], ref_l, torch_dtype(w.dtype))


# ---------------------------------------------------------------------------------------------
# Several query tokens per request (speculative decoding, a prefill chunk on a cached prefix)
# ---------------------------------------------------------------------------------------------
def _run_positions(q, k, v, lens, tables, page, hratio, hk, scale):
    tree = PrefixTreeCPP(page)
    tree.build_radix_tree(list(lens), _padded(tables))
    tree.pack_schedule(None, hratio, hk)
    tree.kernel_info.to_gpu(torch.device(DEV))
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.full_like(qd, float("nan"))
    lse = torch.full(tuple(q.shape[:3]), float("nan"), device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    prefix_attn_with_kvcache(qd, kd, vd, tree, scale, out, lse_out=lse, _status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    return out.float().cpu(), lse.cpu(), tree


@pytest.mark.parametrize("cfg,factor", [(1, 4), (3, 2)])
@pytest.mark.parametrize("T", [2, 4, 8])
def test_several_query_tokens_per_request(cfg, factor, T, native_lib):
    """q [B, T, H, D]: the T query tokens are the last T tokens of every context (already in the
    cache); position t attends to the first len - T + 1 + t tokens.  The oracle is one dense
    attention per (request, position), pinned against the reference's attention_ref."""
    w = scaled_down(cfg, factor)
    _, k, v = make_values(w)
    dtype = torch_dtype(w.dtype)
    g = torch.Generator().manual_seed(100 * cfg + T)
    q = (torch.randn(w.batch, T, w.num_q_heads, w.head_dim, generator=g) * 0.5).to(dtype)
    scale = 1.0 / math.sqrt(w.head_dim)
    out, lse, tree = _run_positions(q, k, v, w.seq_lens, w.block_tables, w.page_size, w.group, w.num_kv_heads, scale)
    hdr = tree.kernel_info.device_work(torch.device(DEV), None, T).header
    assert hdr.q_per_req == T and hdr.batch == w.batch * T and hdr.limits_off >= 0
    ref_o, ref_l = O.paged_multi_position_attention(q, k, v, w.seq_lens, w.block_tables, scale)
    _assert_close(out, lse, ref_o, ref_l, dtype)
    # the last position is ordinary decode attention: the T = 1 call on the same tree agrees
    one, one_lse, _ = _run_tree(q[:, -1:].contiguous(), k, v, w.seq_lens, w.block_tables, w.page_size, w.group,
                                w.num_kv_heads, scale)
    assert (out[:, -1] - one).abs().max().item() <= TOL[dtype]
    assert (lse[:, -1] - one_lse).abs().max().item() <= 1e-3


@pytest.mark.parametrize("seed,T,dtype,hq,hk,d", [(2, 3, torch.float16, 16, 2, 64), (4, 8, torch.bfloat16, 32, 4, 128),
                                                  (5, 2, torch.bfloat16, 8, 8, 128), (10, 5, torch.float16, 32, 4, 64)])
def test_query_positions_that_reach_back_into_shared_segments(seed, T, dtype, hq, hk, d, native_lib):
    """Random forests with tails of 1..299 tokens: with T up to 8 the first positions of a short
    tail see only part (or nothing) of the request's own last segment, in streaming and in dense
    items, and q / out are passed as strided views."""
    lens, tables, pages = _random_forest(seed, cap=120)
    lens = [max(l, T) for l in lens]
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    qfull = (torch.randn(B, T + 1, hq, d, generator=g) * 0.5).to(dtype)
    k = (torch.randn(pages, 16, hk, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(pages, 16, hk, d, generator=g) * 0.5).to(dtype)
    scale = 1.0 / math.sqrt(d)
    tree = PrefixTreeCPP(16)
    tree.build_radix_tree(lens, _padded(tables))
    tree.pack_schedule(None, hq // hk, hk)
    tree.kernel_info.to_gpu(torch.device(DEV))
    qd = qfull.to(DEV)[:, 1:]                           # [B, T, H, D] view with a larger batch stride
    outfull = torch.full((B, T + 2, hq, d), float("nan"), dtype=dtype, device=DEV)
    out = outfull[:, :T]
    lse = torch.full((B, T, hq), float("nan"), device=DEV)
    prefix_attn_with_kvcache(qd, k.to(DEV), v.to(DEV), tree, scale, out, lse_out=lse)
    torch.cuda.synchronize()
    P.check_status(DEV)
    ref_o, ref_l = O.paged_multi_position_attention(qfull[:, 1:], k, v, lens, tables, scale)
    _assert_close(out.float().cpu(), lse.cpu(), ref_o, ref_l, dtype)
    assert torch.isnan(outfull[:, T:].float()).all()
