"""Decode-attention benchmark: microseconds per decode step and fraction of the HBM roofline
on deduplicated KV bytes, for the synthetic prefix-tree workloads of pat_b200/workloads.py.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One process per GPU.  With N > 1 the KV heads (and their query heads) are sharded across the
ranks; there is no data-path collective.  Rank 0 prints one JSON line.

A "step" is one call of the public op ``prefix_attn_with_kvcache`` (all kernels of one decode
step of one layer) on the same resident paged KV cache.  ``value`` times the kernels with CUDA
events; ``e2e`` additionally moves the step's host inputs (queries, work list) to the device and
the output back inside the timed region.  The KV cache itself is state that lives on the GPU
across steps (a decode step appends one token per request), so it is not copied per step.

After the timed regions every rank recomputes a seeded sample of requests with the fp32 CPU
oracle from the K/V values it reads back from its own GPU and compares the output and the LSE of
one more (replayed) step with them (``parity_check``); a mismatch makes the run exit non-zero,
like the PASSED/FAILED line of the reference's own kernel benchmark
(``benchmark/benchmark_kernel.py:55-70, 271-279``).

``--impl reference`` times the reference's own attention path - dense fp32 PyTorch attention
per request on the host cores (``test/utils.py::attention_ref`` itself when a reference checkout
is present, else its CPU restatement in oracle/attention_oracle.py) - on a bounded sample of the
same workload, with all host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_us_per_step"
UNIT = "us"
TRAFFIC_FILE = os.path.join("profiles", "dram_traffic.json")
TOL = {"bf16": 2e-2, "fp16": 1e-2}
LSE_TOL = 1e-3


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
    ap.add_argument("--emulate-shards", type=int, default=0,
                    help="with one GPU: run the work one rank of an S-GPU run would get (S KV-head shards)")
    ap.add_argument("--flags", type=int, default=0, help="extra launch flags (include/pat_b200.h), e.g. 16 = no overlap")
    ap.add_argument("--scale-down", type=int, default=1,
                    help="divide every segment length by this factor (profiling captures on a small case)")
    ap.add_argument("--parity-requests", type=int, default=8, help="requests every rank checks against the oracle")
    ap.add_argument("--plan-repeats", type=int, default=20, help="warm repeats of the plan build (median reported)")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def traffic_record(config: int, scale_down: int, kernel: str):
    """DRAM traffic of one launch as a ratio to its algorithmic bytes, from the tracked summary
    of ncu captures; ``None`` when this workload's kernel has not been captured."""
    try:
        with open(os.path.join(ROOT, TRAFFIC_FILE)) as f:
            table = json.load(f)
    except Exception:
        return None
    return table.get("captures", {}).get(f"cfg{config}", {}).get(kernel)


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


# --------------------------------------------------------------------------------------------
# CPU legs (the only places where bench.py runs anything under oracle/)
# --------------------------------------------------------------------------------------------
def host_attention():
    """(callable, kind): the reference's own ``attention_ref`` when its checkout is present
    ("reference"), else the CPU restatement ("port").  Both take (q [1,1,H,D], k, v [1,S,Hkv,D])."""
    from oracle import attention_oracle as O
    try:
        from oracle import ref_loader
        if os.path.isfile(os.path.join(ref_loader.REFERENCE_ROOT, "test", "utils.py")):
            ref = ref_loader.load_reference_attention()
            return (lambda q, k, v: ref(q, k, v)), "reference"
    except Exception:
        pass
    return (lambda q, k, v: O.dense_attention(q, k, v, None, None)), "port"


def pick_sample(w, budget_s: float, attend, q_cpu, rows):
    """Requests (seeded order) whose dense fp32 attention takes about ``budget_s`` on this host:
    the first request calibrates seconds per token.  Returns [(b, K, V)] with K/V fp32 on the CPU."""
    import numpy as np
    order = np.random.default_rng(w.seed).permutation(w.batch).tolist()
    sample, tokens = [], 0
    kk, vv = rows(order[0])
    attend(q_cpu[order[0]:order[0] + 1], kk[None], vv[None])            # warm the thread pool
    t0 = time.perf_counter()
    attend(q_cpu[order[0]:order[0] + 1], kk[None], vv[None])
    per_token = max((time.perf_counter() - t0) / max(1, w.seq_lens[order[0]]), 1e-9)
    want_tokens = budget_s / per_token
    for b in order:
        if sample and tokens + w.seq_lens[b] > want_tokens:
            break
        if b != order[0]:
            kk, vv = rows(b)
        sample.append((b, kk, vv))
        tokens += w.seq_lens[b]
    return sample, tokens


def time_sample(sample, attend, q_cpu):
    t0 = time.perf_counter()
    for b, kk, vv in sample:
        attend(q_cpu[b:b + 1], kk[None], vv[None])
    return time.perf_counter() - t0


def reference_scheduler_ms(w, hratio, kv_heads, repeats):
    """Median milliseconds of the reference's own C++ scheduler (tree + pack) on this workload,
    when the compiled checker is present; else None."""
    try:
        from oracle import ref_tree
        if not ref_tree.available():
            return None
        import numpy as np
        table = w.padded_table()
        lens = np.asarray(w.seq_lens, dtype=np.int32)
        times = []
        for _ in range(max(3, repeats)):
            t0 = time.perf_counter()
            ref_tree.time_pack(lens, table, w.page_size, hratio, kv_heads)
            times.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(times)
    except Exception:
        return None


def own_scheduler_ms(w, hratio, kv_heads, repeats):
    """This library's scheduler timed the way ``reference_scheduler_ms`` times the reference's: the
    same arrays, back to back on a warm cache.  Returns (tree only, tree + packed plan): the
    kernels need only the tree (the work list is built from its edges), the plan is what the
    reference's scheduler also produces."""
    import numpy as np
    import torch
    from pat_b200 import PrefixTreeCPP
    table = torch.from_numpy(np.ascontiguousarray(w.padded_table(), dtype=np.int32))
    lens = torch.from_numpy(np.asarray(w.seq_lens, dtype=np.int32))
    only, packed = [], []
    for _ in range(max(3, repeats)):
        t0 = time.perf_counter()
        tree = PrefixTreeCPP(w.page_size)
        tree.build_radix_tree(lens, table)
        t1 = time.perf_counter()
        tree.pack_schedule(None, hratio, kv_heads)
        tree._ensure_packed()
        t2 = time.perf_counter()
        only.append((t1 - t0) * 1e3)
        packed.append((t2 - t0) * 1e3)
    return statistics.median(only), statistics.median(packed)


def leave_group(n: int, code: int):
    """Last barrier and teardown of the process group; exits with `code` when it is not 0.  The
    teardown runs beside a 30 s timer: a communicator that does not come down (e.g. because a CUDA
    graph still holds one of its collectives) must not keep a finished run from exiting."""
    if n > 1:
        import torch
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()
        t = threading.Thread(target=dist.destroy_process_group, daemon=True)
        t.start()
        t.join(30.0)
        if t.is_alive():
            print("[bench] process group teardown did not finish in 30 s; exiting without it", file=sys.stderr, flush=True)
            sys.stdout.flush()
            os._exit(code)
    if code:
        sys.exit(code)


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

    from pat_b200.workloads import make_config, scaled_down, synthetic_pages, synthetic_queries, torch_dtype
    w = make_config(args.config) if args.scale_down <= 1 else scaled_down(args.config, args.scale_down)
    if w.num_kv_heads % n != 0 or (args.emulate_shards > 1 and w.num_kv_heads % args.emulate_shards != 0):
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": f"{w.num_kv_heads} KV heads do not shard over {n} GPUs",
                              **({"impl": "reference"} if args.impl == "reference" else {})}))
        return
    shards = args.emulate_shards if (n == 1 and args.emulate_shards > 1) else n
    hk = w.num_kv_heads // shards
    hq = hk * w.group
    shard_rank = rank if shards == n else 0
    heads = slice(shard_rank * hk, (shard_rank + 1) * hk)
    D, page, B = w.head_dim, w.page_size, w.batch
    scale = 1.0 / math.sqrt(D)
    dt = torch_dtype(w.dtype)
    workload_name = f"{w.name}: {w.description}; {w.num_q_heads}/{w.num_kv_heads} heads, D={D}, {w.dtype}, {page}-token pages"
    bytes_total = w.dedup_kv_bytes()
    bytes_rank = w.dedup_kv_bytes(kv_heads=hk, q_heads=hq)
    small = bytes_rank < 4 * 126e6
    config = {"workload": workload_name, "batch": B, "unique_tokens": w.unique_tokens,
              "total_tokens": w.total_tokens, "kv_head_shards": shards,
              "l2": ("per-GPU KV bytes are below 4x L2: between steps a 512 MB buffer is written and a 256 MB buffer "
                     "read to flush L2") if small else
                    "inputs larger than L2 (per-GPU KV bytes >> 126 MB); no flush between steps"}

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)      # torchrun starts its workers with one thread
        attend, kind = host_attention()
        q_cpu = synthetic_queries(w).float()

        def rows(b):
            L = w.seq_lens[b]
            ids = w.block_tables[b][:-(-L // page)]
            kk = synthetic_pages(w, 0, ids).reshape(-1, w.num_kv_heads, D)[:L].float()
            vv = synthetic_pages(w, 1, ids).reshape(-1, w.num_kv_heads, D)[:L].float()
            return kk, vv

        total_budget = 40.0
        per_step = max(0.5, total_budget / max(1, args.steps + args.warmup))
        sample, tok = pick_sample(w, per_step, attend, q_cpu, rows)
        vals = []
        for step in range(args.warmup + args.steps):
            s = time_sample(sample, attend, q_cpu)
            if step >= args.warmup:
                vals.append(s * w.total_tokens / tok)
        est = float(np.mean(vals))
        cores = torch.get_num_threads()
        line = {"impl": "reference", "metric": METRIC, "value": est * 1e6, "unit": UNIT, "n_gpus": n,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": est * 1e3,
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": est * 1e6, "unit": UNIT, "cores": cores, "kind": kind,
                                 "extrapolated": tok < w.total_tokens,
                                 "sample": f"every step runs dense fp32 attention (the reference's PyTorch path) over the "
                                           f"same {len(sample)} of {B} requests of this workload ({tok} of {w.total_tokens} "
                                           f"context tokens, its own K/V values, about {per_step:.1f} s), and the time is "
                                           f"scaled to the whole workload by token count"},
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

    q_host = synthetic_queries(w, kv_heads=heads).pin_memory()
    k_cache = torch.empty(w.num_pages, page, hk, D, dtype=dt, device=dev)
    v_cache = torch.empty_like(k_cache)
    step_pages = 4096
    for lo in range(0, w.num_pages, step_pages):        # bounded temporaries
        ids = torch.arange(lo, min(w.num_pages, lo + step_pages), device=dev)
        k_cache[lo:lo + step_pages] = synthetic_pages(w, 0, ids, dev, heads)
        v_cache[lo:lo + step_pages] = synthetic_pages(w, 1, ids, dev, heads)
    q = q_host.to(dev)
    out = torch.empty_like(q)
    lse = torch.empty(B, hq, dtype=torch.float32, device=dev)
    out_host = torch.empty(B, 1, hq, D, dtype=dt).pin_memory()

    # ---- plan build: median of warm repeats (tree + pack on the host; work list + uploads)
    table = torch.from_numpy(w.padded_table())
    lens_list = list(w.seq_lens)
    PrefixTreeCPP(page)                 # loads the library once, outside the plan-build timing
    t_pack, t_work = [], []
    tree = None
    for _ in range(max(1, args.plan_repeats) + 1):
        t0 = time.perf_counter()
        tree = PrefixTreeCPP(page)
        tree.build_radix_tree(lens_list, table)
        tree.pack_schedule(None, w.group, hk)
        t1 = time.perf_counter()
        tree.kernel_info.to_gpu(dev)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        t_pack.append((t1 - t0) * 1e3)
        t_work.append((t2 - t1) * 1e3)
    plan_ms = {"tree_and_pack": statistics.median(t_pack[1:]) if len(t_pack) > 1 else t_pack[0],
               "work_list_and_upload": statistics.median(t_work[1:]) if len(t_work) > 1 else t_work[0],
               "first_call": {"tree_and_pack": t_pack[0], "work_list_and_upload": t_work[0]},
               "repeats": len(t_pack) - 1, "statistic": "median of warm repeats"}
    work = tree.kernel_info.device_work(dev)
    hdr = work.header

    # ---- the same plan carried over decode steps: every request one token longer per step, a new
    # page where it crosses a page boundary; tree and device work list are grown in place and the
    # list is copied to the device again (a separate planner: the timed steps below keep the
    # workload exactly as named)
    from pat_b200.planner import DecodePlanner
    planner = DecodePlanner(page, w.group, hk, dev)
    grow_lens = torch.tensor(lens_list, dtype=torch.int32)
    grow_table = torch.zeros(B, table.shape[1] + 4, dtype=torch.int32)
    grow_table[:, :table.shape[1]] = table
    planner.step(grow_lens, grow_table)
    torch.cuda.synchronize()
    t_adv = []
    spare = 0
    for _ in range(max(1, args.plan_repeats)):
        grow_lens += 1
        crossing = ((grow_lens - 1) % page == 0).nonzero().flatten().tolist()
        for b in crossing:              # (page ids only have to be valid numbers here: nothing is executed)
            grow_table[b, (int(grow_lens[b]) - 1) // page] = spare % w.num_pages
            spare += 1
        t0 = time.perf_counter()
        planner.step(grow_lens, grow_table)
        torch.cuda.synchronize()
        t_adv.append((time.perf_counter() - t0) * 1e3)
    plan_ms["next_step_in_place"] = statistics.median(t_adv)
    plan_ms["next_step_in_place_count"] = planner.advances
    plan_ms["next_step_rebuilds"] = planner.rebuilds - 1
    del planner

    # L2 flush for the small workloads: write a buffer larger than L2, then read another one, so that
    # the timed step starts with an L2 that holds none of its inputs and no dirty lines of the
    # flush itself (their write-back would otherwise run during the timed step).
    flush = flush_rd = None
    if small:
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        flush_rd = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)

    status = torch.zeros(4, dtype=torch.int32, device=dev)     # set by a kernel whose bounded wait gave up

    def step(flags=0):
        prefix_attn_with_kvcache(q, k_cache, v_cache, tree, scale, out, lse_out=lse,
                                 _flags=flags | args.flags, _status=status)

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

    # ---- parity: one more step of the timed kind (a graph replay), checked against the oracle
    out.fill_(float("nan"))
    lse.fill_(float("nan"))
    run_step()
    torch.cuda.synchronize()
    out_checked = out.float().cpu()[:, 0]
    lse_checked = lse.cpu()

    # per-kernel durations (each phase alone; same stream, CUDA events)
    reps = max(3, min(10, args.steps))
    k_ms = {}
    if hdr.num_stream_items:
        k_ms["stream_kernel"] = timed(capture(lambda: step(2 | 4)), reps)
    if hdr.num_dense_items:
        k_ms["dense_tc_kernel"] = timed(capture(lambda: step(1 | 4)), reps)
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
    # host time of the Python call alone (argument checks, ctypes, three launches), kernels not awaited
    torch.cuda.synchronize()
    tc0 = time.perf_counter()
    for _ in range(20):
        step()
    call_us = (time.perf_counter() - tc0) / 20 * 1e6
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

    # The one optional collective: every rank gets the other ranks' heads (NCCL all-gather into a
    # buffer allocated once, then one small kernel of this library that puts the heads in order).
    # A tensor-parallel model consumes the shard locally instead, so it is not part of `value`;
    # `value_with_gather` times the step's graph replay followed by the gather.
    gather_ms = with_gather_ms = 0.0
    if n > 1:
        from pat_b200.sharding import HeadGather
        hg = HeadGather(out, n)
        for _ in range(3):
            full = hg(out)
        barrier()
        assert tuple(full.shape) == (B, 1, hq * n, D)
        # The collective is launched directly, not from a captured graph: a graph that holds an
        # NCCL collective keeps the communicator's teardown waiting until the graph is destroyed.
        gather_ms = timed(lambda: hg(out), 10)
        barrier()
        with_gather_ms = timed(lambda: (run_step(), hg(out)), max(5, min(20, args.steps)))
        barrier()
        # the gathered heads of rank r must be rank r's output: check our own block and one neighbour's checksum
        mine = full[:, :, rank * hq:(rank + 1) * hq]
        if not torch.equal(mine, out):
            raise RuntimeError("all-gather of the output heads returned the wrong block for this rank")

    # ---- parity check of the replayed step (every rank)
    from oracle import attention_oracle as O
    rng = np.random.default_rng(1000 * args.config + shard_rank)
    picks = sorted(set(rng.choice(B, size=min(B, max(1, args.parity_requests)), replace=False).tolist()))
    q_cpu = q_host.float()
    tol = TOL[w.dtype]
    max_err = max_lse = 0.0
    ok = True
    for b in picks:
        L = w.seq_lens[b]
        idx = torch.as_tensor(w.block_tables[b][:-(-L // page)], device=dev, dtype=torch.long)
        kk = k_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
        vv = v_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
        ro, rl = O.dense_attention(q_cpu[b:b + 1], kk[None], vv[None], None, scale)
        err = (out_checked[b] - ro[0, 0]).abs()
        ok = ok and bool((err <= tol + tol * ro[0, 0].abs()).all())
        lerr = (lse_checked[b] - rl[0, :, 0]).abs().max().item()
        ok = ok and lerr <= LSE_TOL and bool(torch.isfinite(out_checked[b]).all())
        max_err, max_lse = max(max_err, err.max().item()), max(max_lse, lerr)

    vals = torch.tensor([ms, e2e_ms, gather_ms, with_gather_ms, max_err, max_lse, 0.0 if ok else 1.0, call_us],
                        dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_ms, gather_ms, with_gather_ms, max_err, max_lse, bad, call_us = vals.tolist()
    parity = {"requests": len(picks) * n, "requests_per_rank": len(picks), "max_abs_err": max_err,
              "max_lse_err": max_lse, "atol_rtol": tol, "lse_tol": LSE_TOL, "ok": bad == 0.0,
              "checked": "output and LSE of one more graph replay after the timed steps, against dense fp32 "
                         "attention on the host over the K/V values read back from the GPU"}

    if rank != 0:
        leave_group(n, 0 if parity["ok"] else 3)
        return

    peak, peak_kind = measured_peak()
    elt = 2
    kv_bytes = lambda tokens: 2 * tokens * hk * D * elt
    dominant = max((k for k in k_ms if k != "merge_kernel"), key=lambda k_: k_ms[k_], default="merge_kernel")
    if dominant == "stream_kernel":
        alg = kv_bytes(hdr.stream_unique_tokens)
    elif dominant == "dense_tc_kernel":
        alg = kv_bytes(hdr.dense_unique_tokens)
    else:
        alg = hdr.num_entries * w.group * (D + 1) * 4 + B * hq * D * elt
    achieved = alg / (k_ms[dominant] * 1e-3) / 1e9
    # DRAM traffic per launch: dram__bytes_read + dram__bytes_write of an ncu capture of this kernel
    # on a scaled-down case of this workload, as a ratio to the algorithmic bytes of that launch,
    # scaled to this launch (the traffic grows in proportion to the tokens read).  The ratios and the
    # captures they come from are kept in a tracked file, not here.
    rec = traffic_record(args.config, args.scale_down, dominant)
    traffic = int(alg * rec["traffic_over_algorithmic"]) if rec else None
    step_gbs = bytes_rank / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": ms * 1e3, "unit": UNIT, "n_gpus": n, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic", "config": config,
        "clocks": dict(sampler.summary(wall0, wall2),
                       window="timed steps, per-kernel and end-to-end loops, then 0.6 s of the same steps untimed"),
        "e2e": {"value": e2e_ms * 1e3, "unit": UNIT,
                "h2d_bytes_per_step": int(q_host.numel() * elt + blob_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * elt),
                "python_call_us": call_us},
        "gpu_launches": launches,
        "parity_check": parity,
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": traffic,
                     "traffic_source": (f"{TRAFFIC_FILE}: {rec['capture']}" if rec else
                                        f"no capture of {dominant} on this workload in {TRAFFIC_FILE}"),
                     "algorithmic_bytes_per_launch": alg, "kernel_ms": k_ms[dominant]},
        "step_roofline": {"dedup_bytes_per_gpu": bytes_rank, "dedup_bytes_total": bytes_total,
                          "achieved_gbs_per_gpu": step_gbs, "frac_of_measured_copy": step_gbs / peak,
                          "frac_of_8tbs": step_gbs / 8000.0},
        "kernels_ms": k_ms,
        "work": {"stream_items": hdr.num_stream_items, "dense_items": hdr.num_dense_items, "dense_ctas": hdr.num_dense_ctas,
                 "entries": hdr.num_entries, "segments": hdr.num_segments,
                 "stream_tokens_read": hdr.stream_tokens, "dense_tokens_read": hdr.dense_tokens},
        "plan_build_ms": plan_ms,
        **({"all_gather_outputs": {"us": gather_ms * 1e3, "bytes_per_rank": int(out.numel() * elt),
                                   "note": "optional NCCL all-gather of the output heads + reorder kernel, direct launches; "
                                           "not part of value"},
            "value_with_gather": with_gather_ms * 1e3} if n > 1 else {}),
        "append_kv": {"us": append_ms * 1e3, "tokens": B, "bytes": int(2 * 2 * B * hk * D * elt),
                      "note": "KV-cache append of one token per request (separate launch, not part of value)"},
    }

    if n == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        attend, kind = host_attention()

        def rows(b):
            L = w.seq_lens[b]
            idx = torch.as_tensor(w.block_tables[b][:-(-L // page)], device=dev, dtype=torch.long)
            kk = k_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
            vv = v_cache[idx].reshape(-1, hk, D)[:L].float().cpu()
            return kk, vv

        sample, tok = pick_sample(w, args.cpu_seconds, attend, q_cpu, rows)
        s = time_sample(sample, attend, q_cpu)
        est = s * w.total_tokens / tok
        line["cpu_baseline"] = {"value": est * 1e6, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                                "extrapolated": tok < w.total_tokens,
                                "sample": f"{len(sample)} of {B} requests ({tok} of {w.total_tokens} context tokens, the "
                                          f"GPU's own K/V values), {s:.1f} s of dense fp32 attention, scaled by token count"}
        ref_ms = reference_scheduler_ms(w, w.group, hk, 9)
        if ref_ms is not None:
            own_tree, own_packed = own_scheduler_ms(w, w.group, hk, 9)
            line["plan_build_ms"]["back_to_back"] = {
                "reference_cpp_scheduler_tree_and_pack": ref_ms, "tree_only": own_tree, "tree_and_pack": own_packed,
                "note": "the reference's scheduler and this one on the same arrays in the same tight loop (warm cache); "
                        "the figures above are taken with an upload and a synchronise between repeats"}
    print(json.dumps(line), flush=True)
    leave_group(n, 0 if parity["ok"] else 3)


if __name__ == "__main__":
    main()
