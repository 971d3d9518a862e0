"""Decode-attention benchmark: microseconds per decode step and fraction of the HBM roofline
on deduplicated KV bytes, for the synthetic prefix-tree workloads of pat_b200/workloads.py.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One process per GPU.  With N > 1 the KV heads (and their query heads) are sharded across the
ranks; there is no data-path collective.  Rank 0 prints one JSON line.

A "step" is one call of the public op ``prefix_attn_with_kvcache`` (all kernels of one decode
step of one layer) on the same resident paged KV cache.  ``value`` times the kernels with CUDA
events; ``e2e`` additionally moves the step's host inputs (queries, plan tables / work list)
to the device and the output back inside the timed region.  The KV cache itself is state that
lives on the GPU across steps (a decode step appends one token per request), so it is not
copied per step.

``--impl reference`` times the reference's own attention path - dense fp32 PyTorch attention
per request on the host cores (the CPU restatement in oracle/attention_oracle.py of
test/utils.py::attention_ref) - on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_us_per_step"
UNIT = "us"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=4, help="workload 0..4 (default: long-context mixed batch)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA graph replays")
    ap.add_argument("--library-baselines", action="store_true",
                    help="also time two library decode kernels that know nothing of shared prefixes: FlashInfer's "
                         "paged batch decode on this workload as is, and flash_attn_with_kvcache on the same requests "
                         "laid out in 256-token pages; one GPU, adds JSON keys")
    ap.add_argument("--emulate-shards", type=int, default=0,
                    help="with one GPU: run the work one rank of an S-GPU run would get (S KV-head shards)")
    ap.add_argument("--flags", type=int, default=0, help="extra launch flags (include/pat_b200.h), e.g. 16 = no overlap")
    ap.add_argument("--scale-down", type=int, default=1,
                    help="divide every segment length by this factor (profiling captures on a small case)")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 7] or \
               [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(float(r[0]) for r in rows if r[0].replace(".", "", 1).isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "", 1).isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def flashinfer_baseline(w, q, k_cache, v_cache, out, scale):
    """Context number, not the reference: FlashInfer's paged batch decode (tensor-core path) on the
    bench's own tensors.  It attends every request's whole context; shared pages are re-read per
    request (mostly from L2).  `out` holds this engine's result for the same inputs."""
    import torch
    try:
        import flashinfer
    except Exception as exc:
        return {"unavailable": f"flashinfer does not load: {exc}"}
    dev = q.device
    page, hk, hq, D = k_cache.shape[1], k_cache.shape[2], q.shape[2], q.shape[3]
    indptr, indices, last = [0], [], []
    for L, t in zip(w.seq_lens, w.block_tables):
        npg = -(-L // page)
        indices += t[:npg]
        indptr.append(indptr[-1] + npg)
        last.append(L - (npg - 1) * page)
    try:
        ws = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        wrap = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_tensor_cores=True)
        wrap.plan(torch.tensor(indptr, dtype=torch.int32, device=dev), torch.tensor(indices, dtype=torch.int32, device=dev),
                  torch.tensor(last, dtype=torch.int32, device=dev), hq, hk, D, page, q_data_type=q.dtype, sm_scale=scale)
        q3 = q[:, 0]
        res = wrap.run(q3, (k_cache, v_cache))
        for _ in range(3):
            wrap.run(q3, (k_cache, v_cache))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            wrap.run(q3, (k_cache, v_cache))
        e1.record()
        torch.cuda.synchronize()
        line = {"version": getattr(flashinfer, "__version__", "?"), "us_batch_decode_tensor_cores": e0.elapsed_time(e1) / 10 * 1e3,
                "max_abs_diff": (res.float() - out[:, 0].float()).abs().max().item(),
                "timing": "direct launches, CUDA events, 10 steps; plan() outside the timed region"}
    except Exception as exc:
        return {"unavailable": f"flashinfer could not run: {exc}"}
    # The library's own prefix-aware path: two-level cascade attention (level 0 = the pages a group
    # of requests shares, attended once for the whole group; level 1 = every request's own pages).
    try:
        groups = {}
        for b, t in enumerate(w.block_tables):
            groups.setdefault(t[0], []).append(b)
        groups = sorted(groups.values(), key=lambda m: m[0])
        order = [b for m in groups for b in m]              # the queries of a group must be contiguous
        owners = {}
        for t in w.block_tables:
            for pid in t:
                owners[pid] = owners.get(pid, 0) + 1
        lv = [dict(qo=[0], ptr=[0], idx=[], last=[]) for _ in range(2)]
        for m in groups:
            t = w.block_tables[m[0]]
            ns = 1                                          # an unshared request: its first page is "level 0"
            if len(m) > 1:                                  # the pages common to every request of the group
                ns = min(len(w.block_tables[b]) for b in m)
                for b in m[1:]:
                    tb = w.block_tables[b]
                    i = 0
                    while i < ns and tb[i] == t[i]:
                        i += 1
                    ns = i
                # every request keeps at least one page of its own for level 1
                ns = min(ns, min(-(-w.seq_lens[b] // page) for b in m) - 1)
            lv[0]["idx"] += t[:ns]
            lv[0]["ptr"].append(lv[0]["ptr"][-1] + ns)
            lv[0]["last"].append(page)
            lv[0]["qo"].append(lv[0]["qo"][-1] + len(m))
            for b in m:
                L = w.seq_lens[b]
                npg = -(-L // page)
                own = w.block_tables[b][ns:npg]
                if not own:
                    raise ValueError("a request without pages of its own")
                lv[1]["idx"] += own
                lv[1]["ptr"].append(lv[1]["ptr"][-1] + len(own))
                lv[1]["last"].append(L - (npg - 1) * page)
                lv[1]["qo"].append(lv[1]["qo"][-1] + 1)
        ti = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        ws2 = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
        casc = flashinfer.MultiLevelCascadeAttentionWrapper(2, ws2, "NHD")
        casc.plan([ti(l["qo"]) for l in lv], [ti(l["ptr"]) for l in lv], [ti(l["idx"]) for l in lv],
                  [ti(l["last"]) for l in lv], hq, hk, D, page, causal=False, sm_scale=scale, q_data_type=q.dtype)
        perm = torch.tensor(order, device=dev)
        qs = q[:, 0][perm].contiguous()
        res = casc.run(qs, (k_cache, v_cache))
        for _ in range(3):
            casc.run(qs, (k_cache, v_cache))
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            casc.run(qs, (k_cache, v_cache))
        e1.record()
        torch.cuda.synchronize()
        line["us_cascade_two_levels"] = e0.elapsed_time(e1) / 10 * 1e3
        line["cascade_max_abs_diff"] = (res.float() - out[:, 0][perm].float()).abs().max().item()
    except Exception as exc:
        line["cascade_unavailable"] = str(exc)[:200]
    return line


def flash_attn_baseline(w, hk, hq, D, dt, dev, scale):
    """Context number, not the reference: the flash-attention library's paged decode kernel, which
    reads every request's whole context (no prefix sharing), against this engine on the same
    requests.  That library wants 256-token pages, so both run on a 256-token-page rendition of the
    workload (same lengths, same sharing: a request keeps its group's pages for as long as its
    16-token pages were shared)."""
    import torch
    from pat_b200 import PrefixTreeCPP, prefix_attn_with_kvcache
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:
        return {"unavailable": f"flash_attn does not load: {exc}"}
    page, old = 256, w.page_size
    owners = {}
    for t in w.block_tables:
        for pid in t:
            owners[pid] = owners.get(pid, 0) + 1
    tables, shared, nxt = [], {}, 0
    for b, L in enumerate(w.seq_lens):
        t16 = w.block_tables[b]
        n_shared16 = 0
        while n_shared16 < len(t16) and owners[t16[n_shared16]] > 1:
            n_shared16 += 1
        n_shared = (n_shared16 * old) // page               # whole 256-token pages inside the shared run
        key = t16[0]
        row = []
        if n_shared:
            if key not in shared:
                shared[key] = list(range(nxt, nxt + n_shared))
                nxt += n_shared
            row = list(shared[key][:n_shared])
        own = -(-L // page) - len(row)
        row += list(range(nxt, nxt + own))
        nxt += own
        tables.append(row)
    B = len(tables)
    gen = torch.Generator(device=dev).manual_seed(7)
    q = (torch.randn(B, 1, hq, D, generator=gen, device=dev) * 0.5).to(dt)
    k = torch.empty(nxt, page, hk, D, dtype=dt, device=dev)
    v = torch.empty_like(k)
    for lo in range(0, nxt, 256):
        hi = min(nxt, lo + 256)
        k[lo:hi] = (torch.randn(hi - lo, page, hk, D, generator=gen, device=dev) * 0.5).to(dt)
        v[lo:hi] = (torch.randn(hi - lo, page, hk, D, generator=gen, device=dev) * 0.5).to(dt)
    table = torch.zeros(B, max(len(t) for t in tables), dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    tree = PrefixTreeCPP(page)
    tree.build_radix_tree(list(w.seq_lens), table)
    tree.pack_schedule(None, hq // hk, hk)
    tree.kernel_info.to_gpu(dev)
    out = torch.empty_like(q)
    td, ld = table.to(dev), torch.tensor(list(w.seq_lens), dtype=torch.int32, device=dev)

    def ours():
        prefix_attn_with_kvcache(q, k, v, tree, scale, out)

    def lib():
        return flash_attn_with_kvcache(q, k, v, cache_seqlens=ld, block_table=td, softmax_scale=scale, causal=True)

    def timed(fn, iters=20):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    try:
        ref = lib()
        ours()
        torch.cuda.synchronize()
        diff = (ref.float() - out.float()).abs().max().item()
        return {"page_size": page, "pages": nxt, "us_this_engine": timed(ours), "us_flash_attn_with_kvcache": timed(lib),
                "max_abs_diff": diff, "timing": "direct launches, CUDA events, 20 steps"}
    except Exception as exc:
        return {"unavailable": f"flash_attn could not run: {exc}"}


def cpu_attention_sample(w, q_cpu, k_rows, budget_s, order):
    """Dense fp32 attention per request on the host cores for as many requests (in ``order``)
    as fit in ``budget_s``.  ``k_rows(b)`` returns the request's dense (K, V) fp32 on the CPU.
    Returns (seconds, tokens, requests)."""
    import torch
    from oracle import attention_oracle as O
    spent, tokens, done = 0.0, 0, 0
    for b in order:
        kk, vv = k_rows(b)
        t0 = time.perf_counter()
        O.dense_attention(q_cpu[b:b + 1], kk[None], vv[None], None, None)
        spent += time.perf_counter() - t0
        tokens += w.seq_lens[b]
        done += 1
        if spent >= budget_s:
            break
    return spent, tokens, done


def main():
    args = parse()
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run "
                  f"(--nproc-per-node {args.gpus})", file=sys.stderr)
            sys.exit(2)
    n = world

    from pat_b200.workloads import make_config, scaled_down, torch_dtype
    w = make_config(args.config) if args.scale_down <= 1 else scaled_down(args.config, args.scale_down)
    if w.num_kv_heads % n != 0 or (args.emulate_shards > 1 and w.num_kv_heads % args.emulate_shards != 0):
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": f"{w.num_kv_heads} KV heads do not shard over {n} GPUs"}))
        return
    shards = args.emulate_shards if (n == 1 and args.emulate_shards > 1) else n
    hk = w.num_kv_heads // shards
    hq = hk * w.group
    D, page, B = w.head_dim, w.page_size, w.batch
    scale = 1.0 / math.sqrt(D)
    dt = torch_dtype(w.dtype)
    workload_name = f"{w.name}: {w.description}; {w.num_q_heads}/{w.num_kv_heads} heads, D={D}, {w.dtype}, {page}-token pages"
    config = {"workload": workload_name, "batch": B, "unique_tokens": w.unique_tokens,
              "total_tokens": w.total_tokens, "kv_head_shards": shards,
              "l2": "inputs larger than L2 (per-GPU KV bytes >> 126 MB); no flush between steps"}
    bytes_total = w.dedup_kv_bytes()
    bytes_rank = w.dedup_kv_bytes(kv_heads=hk, q_heads=hq)
    if bytes_rank < 4 * 126e6:
        config["l2"] = "per-GPU KV bytes are below 4x L2: between steps a 512 MB buffer is written and a 256 MB buffer read to flush L2"

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return
        gen = torch.Generator().manual_seed(w.seed)
        q_cpu = (torch.randn(B, 1, w.num_q_heads, D, generator=gen) * 0.5).to(dt).float()
        rng = np.random.default_rng(0)
        order = rng.permutation(B).tolist()

        def rows(b):
            g = torch.Generator().manual_seed(1000 + b)
            L = w.seq_lens[b]
            kk = (torch.randn(L, w.num_kv_heads, D, generator=g) * 0.5).to(dt).float()
            vv = (torch.randn(L, w.num_kv_heads, D, generator=g) * 0.5).to(dt).float()
            return kk, vv

        total_budget = 60.0
        per_step = max(1.0, total_budget / max(1, args.steps + args.warmup))
        vals = []
        for step in range(args.warmup + args.steps):
            s, tok, done = cpu_attention_sample(w, q_cpu, rows, per_step, order[step % B:] + order[:step % B])
            if step >= args.warmup:
                vals.append(s * w.total_tokens / tok)
        est = float(np.mean(vals))
        cores = torch.get_num_threads()
        line = {"impl": "reference", "metric": METRIC, "value": est * 1e6, "unit": UNIT, "n_gpus": n,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": est * 1e3,
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": est * 1e6, "unit": UNIT, "cores": cores, "kind": "port",
                                 "sample": f"per step: as many whole requests as fit in {per_step:.1f} s of dense fp32 "
                                           f"attention on the host, scaled to the workload by token count"},
                "e2e": {"value": est * 1e6, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    # ------------------------------------------------------------------ our arm (GPU)
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if n > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from pat_b200 import PrefixTreeCPP, prefix_attn_with_kvcache
    from pat_b200 import _prefix_attn as P

    gen = torch.Generator(device=dev).manual_seed(w.seed * 100 + rank)
    q_host = (torch.randn(B, 1, hq, D, generator=torch.Generator().manual_seed(w.seed)) * 0.5).to(dt).pin_memory()
    k_cache = torch.empty(w.num_pages, page, hk, D, dtype=dt, device=dev)
    v_cache = torch.empty_like(k_cache)
    step_pages = 4096
    for lo in range(0, w.num_pages, step_pages):        # bounded temporaries
        hi = min(w.num_pages, lo + step_pages)
        k_cache[lo:hi] = (torch.randn(hi - lo, page, hk, D, generator=gen, device=dev) * 0.5).to(dt)
        v_cache[lo:hi] = (torch.randn(hi - lo, page, hk, D, generator=gen, device=dev) * 0.5).to(dt)
    q = q_host.to(dev)
    out = torch.empty_like(q)
    out_host = torch.empty(B, 1, hq, D, dtype=dt).pin_memory()

    table = torch.from_numpy(w.padded_table())
    PrefixTreeCPP(page)                 # loads the library once, outside the plan-build timing
    t0 = time.perf_counter()
    tree = PrefixTreeCPP(page)
    tree.build_radix_tree(list(w.seq_lens), table)
    tree.pack_schedule(None, w.group, hk)
    t1 = time.perf_counter()
    tree.kernel_info.to_gpu(dev)
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    work = tree.kernel_info.device_work(dev)
    hdr = work.header

    # L2 flush for the small workloads: write a buffer larger than L2, then read another one, so that
    # the timed step starts with an L2 that holds none of its inputs and no dirty lines of the
    # flush itself (their write-back would otherwise run during the timed step).
    flush = flush_rd = None
    if bytes_rank < 4 * 126e6:
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        flush_rd = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)

    status = torch.zeros(4, dtype=torch.int32, device=dev)     # set by a kernel whose bounded wait gave up

    def step(flags=0):
        prefix_attn_with_kvcache(q, k_cache, v_cache, tree, scale, out, _flags=flags | args.flags, _status=status)

    def barrier():
        torch.cuda.synchronize()
        if n > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, iters):
        """Average device milliseconds of fn over iters launches (flushes excluded)."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in evs:
            if flush is not None:
                flush.fill_(1)
                flush_rd.max()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / iters

    for _ in range(max(3, args.warmup)):
        step()
    barrier()

    # A step is three short kernels; for the small workloads the Python call costs more host time
    # than the kernels take on the device.  The step is therefore captured once in a CUDA graph
    # (the op launches on the capturing stream; nothing in it synchronises) and `value` times
    # replays of that graph.  `e2e` below goes through the plain call.
    def capture(fn):
        if args.no_graph:
            return fn
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            g.replay()
            torch.cuda.synchronize()
            return g.replay
        except Exception as exc:                      # keep measuring with direct launches
            print(f"[bench] CUDA graph capture failed ({exc}); timing direct launches", file=sys.stderr)
            torch.cuda.synchronize()
            return fn

    launches_per_step = 0
    step()
    launches_per_step = P.last_launch_count()
    run_step = capture(step)
    config["timing"] = "cuda graph replay of one step" if run_step is not step else "direct launches"
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    wall0 = time.time()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run_step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = timed(run_step, args.steps)
        barrier()
    launches = launches_per_step * args.steps
    wall1 = time.time()

    # per-kernel durations (each phase alone; same stream, CUDA events)
    reps = max(3, min(10, args.steps))
    k_ms = {}
    if hdr.num_stream_items:
        k_ms["stream_kernel"] = timed(capture(lambda: step(2 | 4)), reps)
    if hdr.num_dense_items:
        k_ms["dense_kernel"] = timed(capture(lambda: step(1 | 4)), reps)
    k_ms["merge_kernel"] = timed(capture(lambda: step(1 | 2)), reps)
    step()   # leave `out` complete

    # the step right before attention in a serving loop: append one new token per request to the
    # paged cache (rewrites every request's last token with the values it already has)
    from pat_b200.cache_ops import reshape_and_cache_flash
    last = torch.tensor([w.block_tables[b][(w.seq_lens[b] - 1) // page] * page + (w.seq_lens[b] - 1) % page
                         for b in range(B)], dtype=torch.int64, device=dev)
    new_k = k_cache.view(-1, hk, D)[last].clone()
    new_v = v_cache.view(-1, hk, D)[last].clone()
    append_ms = timed(capture(lambda: reshape_and_cache_flash(new_k, new_v, k_cache, v_cache, last)), reps)

    # end to end: host queries + work list in, output back, every step
    blob_host = work._host
    def e2e_step():
        q.copy_(q_host, non_blocking=True)
        work.blob.copy_(blob_host, non_blocking=True)
        step()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    tw1 = time.perf_counter()
    e2e_ms = max(e0.elapsed_time(e1), (tw1 - tw0) * 1e3) / args.steps
    # The timed regions are a few tens of milliseconds, shorter than the sampling period of the
    # clock record: keep the GPU on the same steps (untimed) for a little longer so that the
    # record holds several samples taken under this load.
    soak_end = time.time() + 0.6
    while time.time() < soak_end:
        for _ in range(50):
            run_step()
        torch.cuda.synchronize()
    wall2 = time.time()
    sampler.stop()
    if int(status[0].item()) != 0:
        raise RuntimeError(f"a kernel reported a failed wait (status {status.tolist()}); the timings are void")

    # The one optional collective: every rank gets the other ranks' heads (NCCL all-gather).  A
    # tensor-parallel model consumes the shard locally instead, so it is not part of `value`.
    gather_ms = 0.0
    if n > 1:
        from pat_b200.sharding import all_gather_heads
        for _ in range(3):
            full = all_gather_heads(out, n)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            full = all_gather_heads(out, n)
        e1.record()
        torch.cuda.synchronize()
        gather_ms = e0.elapsed_time(e1) / 10
        assert tuple(full.shape) == (B, 1, hq * n, D)

    vals = torch.tensor([ms, e2e_ms, gather_ms], dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_ms, gather_ms = vals.tolist()

    if rank != 0:
        if n > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    library_baseline = flashinfer_line = None
    if args.library_baselines and n == 1:
        flashinfer_line = flashinfer_baseline(w, q, k_cache, v_cache, out, scale)
        library_baseline = flash_attn_baseline(w, hk, hq, D, dt, dev, scale)

    peak, peak_kind = measured_peak()
    elt = 2
    kv_bytes = lambda tokens: 2 * tokens * hk * D * elt
    dominant = max((k for k in k_ms if k != "merge_kernel"), key=lambda k_: k_ms[k_], default="merge_kernel")
    if dominant == "stream_kernel":
        alg = kv_bytes(hdr.stream_unique_tokens)
    elif dominant == "dense_kernel":
        alg = kv_bytes(hdr.dense_unique_tokens)
    else:
        alg = hdr.num_entries * w.group * (D + 1) * 4 + B * hq * D * elt
    achieved = alg / (k_ms[dominant] * 1e-3) / 1e9
    # DRAM traffic per launch: dram__bytes_read + dram__bytes_write of one ncu capture of the same
    # kernels on this workload with all lengths / 4 (profiles/stream_dense_merge_cfg4_div4_full.md),
    # as a ratio to the algorithmic bytes of that launch, scaled to this launch (the traffic of
    # both kernels grows in proportion to the tokens they read).  Other workloads: not captured.
    ncu_traffic_ratio = {"stream_kernel": 939.8 / 917.8, "dense_kernel": 127.8 / 117.4}
    traffic = int(alg * ncu_traffic_ratio[dominant]) if (args.config == 4 and dominant in ncu_traffic_ratio) else None
    step_gbs = bytes_rank / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": ms * 1e3, "unit": UNIT, "n_gpus": n, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic", "config": config,
        "clocks": dict(sampler.summary(wall0, wall2),
                       window="timed steps, per-kernel and end-to-end loops, then 0.6 s of the same steps untimed"),
        "e2e": {"value": e2e_ms * 1e3, "unit": UNIT,
                "h2d_bytes_per_step": int(q_host.numel() * elt + blob_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * elt)},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": traffic,
                     "algorithmic_bytes_per_launch": alg, "kernel_ms": k_ms[dominant]},
        "step_roofline": {"dedup_bytes_per_gpu": bytes_rank, "dedup_bytes_total": bytes_total,
                          "achieved_gbs_per_gpu": step_gbs, "frac_of_measured_copy": step_gbs / peak,
                          "frac_of_8tbs": step_gbs / 8000.0},
        "kernels_ms": k_ms,
        "work": {"stream_items": hdr.num_stream_items, "dense_items": hdr.num_dense_items, "dense_ctas": hdr.num_dense_ctas,
                 "entries": hdr.num_entries, "segments": hdr.num_segments,
                 "stream_tokens_read": hdr.stream_tokens, "dense_tokens_read": hdr.dense_tokens},
        "plan_build_ms": {"tree_and_pack": (t1 - t0) * 1e3, "work_list_and_upload": (t2 - t1) * 1e3},
        **({"all_gather_outputs": {"us": gather_ms * 1e3, "bytes_per_rank": int(out.numel() * elt),
                                   "note": "optional NCCL all-gather of the output heads; not part of value"}}
           if n > 1 else {}),
        **({"flashinfer_baseline": flashinfer_line} if flashinfer_line else {}),
        **({"flash_attn_baseline": library_baseline} if library_baseline else {}),
        "append_kv": {"us": append_ms * 1e3, "tokens": B, "bytes": int(2 * 2 * B * hk * D * elt),
                      "note": "KV-cache append of one token per request (separate launch, not part of value)"},
    }

    if n == 1 and not args.no_cpu_baseline:
        q_cpu = q_host.float()
        rng = np.random.default_rng(0)
        order = rng.permutation(B).tolist()

        def rows(b):
            L = w.seq_lens[b]
            idx = torch.as_tensor(w.block_tables[b][:-(-L // page)], device=dev, dtype=torch.long)
            kk = k_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
            vv = v_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
            return kk, vv

        s, tok, done = cpu_attention_sample(w, q_cpu, rows, args.cpu_seconds, order)
        est = s * w.total_tokens / tok
        line["cpu_baseline"] = {"value": est * 1e6, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"{done} of {B} requests ({tok} of {w.total_tokens} context tokens), "
                                          f"{s:.1f} s of dense fp32 attention, scaled by token count"}
    print(json.dumps(line))
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
