"""The op and the native scheduler objects, bound over the C ABI.

Python-facing equivalent of the reference's compiled module
``prefix_attn._prefix_attn`` (``csrc/bindings.cpp:74-158``, stub
``prefix_attn/_prefix_attn.pyi``): the two forms of
``prefix_attn_with_kvcache``, ``PrefixTreeCPP`` and its ``KernelInfo``.  All
device work goes through ``libpat_b200.so``; nothing here computes attention.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from . import _native as N
from . import _plan_cache

__all__ = ["prefix_attn_with_kvcache", "PrefixTreeCPP", "KernelInfo", "WorkConfig", "DeviceWork",
           "status_word", "check_status"]


# --------------------------------------------------------------------------- options
class WorkConfig:
    """Tuning knobs of the work-list builder (0 = library default)."""

    __slots__ = ("num_sms", "dense_min_rows", "chunk_tokens_min", "chunk_tokens_max",
                 "dense_piece_tokens_min", "items_per_sm", "disable_dense", "dense_tile_ns", "grow_slack_pages")

    def __init__(self, **kw):
        for name in self.__slots__:
            setattr(self, name, int(kw.pop(name, 0)))
        if kw:
            raise TypeError(f"unknown work options: {sorted(kw)}")

    def key(self):
        return tuple(getattr(self, n) for n in self.__slots__)

    def as_struct(self) -> N.WorkOptions:
        s = N.WorkOptions()
        for name in self.__slots__:
            setattr(s, name, getattr(self, name))
        return s


def _env_config() -> WorkConfig:
    """Defaults, overridable through ``PAT_B200_<OPTION>`` environment variables."""
    kw = {}
    for name in WorkConfig.__slots__:
        v = os.environ.get("PAT_B200_" + name.upper())
        if v:
            kw[name] = int(v)
    return WorkConfig(**kw)


_default_config: Optional[WorkConfig] = None


def default_config() -> WorkConfig:
    global _default_config
    if _default_config is None:
        _default_config = _env_config()
    return _default_config


def set_default_config(cfg: Optional[WorkConfig]) -> None:
    global _default_config
    _default_config = cfg


_WS_HEAD = 256      # bytes of control words at the head of a workspace (include/pat_b200.h)


def _sm_count(device: torch.device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


# --------------------------------------------------------------------------- device work list
class DeviceWork:
    """A work list on one device: the int32 blob plus the host header."""

    def __init__(self, handle: int, device: torch.device, keep_native: bool = False):
        lib = N.load()
        self.header = N.WorkHeader()
        lib.pat_work_get_header(handle, C.byref(self.header))
        words = C.c_size_t()
        ptr = lib.pat_work_blob(handle, C.byref(words))
        # one copy: native blob -> (pinned) host tensor
        host = torch.empty(words.value, dtype=torch.int32, pin_memory=device.type == "cuda")
        if words.value:
            C.memmove(host.data_ptr(), ptr, words.value * 4)
        self._host = host                       # kept alive: the copy below is asynchronous
        self.blob = host.to(device, non_blocking=True)
        self.device = device
        self._handle = handle if keep_native else None     # native list, kept to be advanced in place
        self._host_alt = None                   # second pinned buffer, used alternately by refresh()
        self._host_busy = {}                    # id(host buffer) -> event of its last upload
        # The copy runs on the stream that is current in THIS thread (a plan-building worker thread
        # uses the default stream); the kernels may be launched on another one.  The event lets the
        # first launch on a different stream wait for the upload.
        self._uploaded = None
        self._upload_stream = None
        if device.type == "cuda":
            st = torch.cuda.current_stream(device)
            self._uploaded = torch.cuda.Event()
            self._uploaded.record(st)
            self._upload_stream = st.cuda_stream
        self._ordered = set()                   # streams already ordered after the upload
        self._scratch = {}                      # stream -> workspace tensor
        self._args = None                       # (key, DecodeArgs) of the last call
        # One workspace is allocated with the work list (sized for head_dim 128, the larger of the
        # two supported), so that the first call - which may sit inside a stream capture - does not
        # have to allocate and clear one.
        self._spare = None
        if device.type == "cuda":
            self._spare = self._new_workspace(lib.pat_b200_workspace_bytes(C.byref(self.header), 1, 128), device)
        if not keep_native:
            lib.pat_work_destroy(handle)

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            try:
                N.load().pat_work_destroy(h)
            except Exception:
                pass
            self._handle = None

    def refresh(self) -> None:
        """After the native list was advanced in place: copy it to the device again, into the SAME
        device buffer and on the current stream, so that launches on that stream before and after
        see the old and the new list respectively.  The blob's address and the item counts do not
        change, so a CUDA graph captured around the op stays valid."""
        lib = N.load()
        lib.pat_work_get_header(self._handle, C.byref(self.header))
        words = C.c_size_t()
        ptr = lib.pat_work_blob(self._handle, C.byref(words))
        # two pinned buffers take turns: the previous upload may still be reading the other one
        if self._host_alt is None:
            self._host_alt = torch.empty_like(self._host, pin_memory=self.device.type == "cuda")
        self._host, self._host_alt = self._host_alt, self._host
        busy = self._host_busy.get(id(self._host))
        if busy is not None:
            busy.synchronize()
        C.memmove(self._host.data_ptr(), ptr, words.value * 4)
        self.blob.copy_(self._host, non_blocking=True)
        if self.device.type == "cuda":
            st = torch.cuda.current_stream(self.device)
            ev = self._host_busy.get(id(self._host))
            if ev is None:
                ev = torch.cuda.Event()
                self._host_busy[id(self._host)] = ev
            ev.record(st)
            self._uploaded, self._upload_stream = ev, st.cuda_stream
            self._ordered = set()
        if self._args is not None:              # same pointers, new header
            self._args[1].work = self.header

    def order_after_upload(self, stream) -> None:
        """Makes ``stream`` wait for the upload of the blob (once per stream)."""
        h = stream.cuda_stream
        if self._uploaded is None or h == self._upload_stream or h in self._ordered:
            return
        if torch.cuda.is_current_stream_capturing():
            # Nothing is launched during a capture, and neither a wait for an event recorded outside
            # it nor a host-side synchronisation may be issued here.  Replays come after the capture
            # has ended; whoever captures a step has run it (or synchronised) before, as a capture
            # needs anyway.
            return
        stream.wait_event(self._uploaded)
        self._ordered.add(h)

    @staticmethod
    def _new_workspace(nbytes: int, device) -> torch.Tensor:
        ws = torch.empty(max(int(nbytes), _WS_HEAD), dtype=torch.uint8, device=device)
        ws[:_WS_HEAD].zero_()                   # the control words start at zero
        return ws

    def workspace(self, nbytes: int, stream, device) -> torch.Tensor:
        """Scratch for the partial results, reused by every call with this work list on ``stream``
        (calls on one stream run one after the other, so they can share it; calls on different
        streams get different ones)."""
        key = stream.cuda_stream
        ws = self._scratch.get(key)
        if ws is None or ws.numel() < nbytes:
            if self._spare is not None and self._spare.numel() >= nbytes:
                ws, self._spare = self._spare, None
            else:
                ws = self._new_workspace(nbytes, device)
            self._scratch[key] = ws
        return ws

    @classmethod
    def from_host_plan(cls, plan: "_plan_cache.HostPlan", hratio: int, kv_heads: int, page_size: int,
                       device: torch.device, cfg: WorkConfig) -> "DeviceWork":
        lib = N.load()
        n = len(plan.q_tables)
        buckets = (N.PlanBucket * max(n, 1))()
        for i in range(n):
            q, b = plan.q_tables[i], plan.block_tables[i]
            buckets[i].ctas = int(plan.num_seqs[i].shape[0])
            buckets[i].q_stride = int(q.shape[1])
            buckets[i].block_stride = int(b.shape[1])
            buckets[i].q_table = q.ctypes.data
            buckets[i].block_table = b.ctypes.data
            buckets[i].num_seqs = plan.num_seqs[i].ctypes.data
            buckets[i].kv_in_cta = plan.kv_lens[i].ctypes.data
        opts = cfg.as_struct()
        if opts.num_sms == 0 and device.type == "cuda":
            opts.num_sms = _sm_count(device)
        status = C.c_int(0)
        handle = lib.pat_work_create(buckets, n, plan.batch, hratio, kv_heads, page_size, 0,
                                     C.byref(opts), C.byref(status))
        if not handle:
            raise RuntimeError(f"invalid plan: {N.strerror(status.value)}")
        return cls(handle, device)

    @classmethod
    def from_tree(cls, tree_handle: int, hratio: int, kv_heads: int, device: torch.device,
                  cfg: WorkConfig, q_per_req: int = 1) -> "DeviceWork":
        lib = N.load()
        opts = cfg.as_struct()
        if opts.num_sms == 0 and device.type == "cuda":
            opts.num_sms = _sm_count(device)
        status = C.c_int(0)
        handle = lib.pat_work_from_tree_multi(tree_handle, hratio, kv_heads, int(q_per_req), 0, C.byref(opts),
                                              C.byref(status))
        if not handle:
            raise RuntimeError(f"invalid plan: {N.strerror(status.value)}")
        return cls(handle, device, keep_native=True)


# --------------------------------------------------------------------------- native scheduler
def _view_i32(ptr, shape) -> torch.Tensor:
    """A CPU int32 tensor holding a copy of native memory."""
    n = int(np.prod(shape)) if len(shape) else 1
    if n == 0:
        return torch.zeros(shape, dtype=torch.int32)
    return torch.from_numpy(np.ctypeslib.as_array(ptr, shape=(n,)).reshape(shape).copy())


class KernelInfo:
    """Plan produced by ``PrefixTreeCPP.pack_schedule`` (reference
    ``csrc/prefix_tree.h:7-39``): per-bucket int32 CPU tensors until
    ``to_gpu(device)`` moves them - and builds and uploads the device work
    list the kernels consume.

    The plan lives in the native tree; the tensors are only made (and moved) when one of the
    fields is read.  The kernels here never read them - they run from the work list - so a decode
    loop that just builds, packs, calls ``to_gpu`` and passes the tree to the op pays for none
    of the per-bucket tensors and their host-to-device copies."""

    _FIELDS = ("q_tables", "block_tables", "num_seqs_per_CTAs", "CTA_ranks", "kv_in_CTAs", "MNWs",
               "num_split_per_seq", "max_split_per_seq", "max_seqs_in_CTA", "max_blocks_in_CTA")

    def __init__(self, box: "_TreeBox"):
        self._box = box             # the native tree and its pack state (not the PrefixTreeCPP: no cycle)
        self._vals = None           # field values, once read
        self._device = None         # where to_gpu sent the plan
        self._work = {}

    def _invalidate(self):
        """The native plan changed (a pack, or an in-place advance of the tree)."""
        self._vals = None
        self._work = {}

    def __getattr__(self, name):
        if name in KernelInfo._FIELDS:
            if self._vals is None:
                self._vals = self._read()
            return self._vals[name]
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name in KernelInfo._FIELDS:
            if self._vals is None:
                self._vals = self._read()
            self._vals[name] = value
        else:
            object.__setattr__(self, name, value)

    def _read(self):
        lib = N.load()
        o = self._box
        o.ensure_packed()
        h = o.handle
        v = dict(q_tables=[], block_tables=[], num_seqs_per_CTAs=[], CTA_ranks=[], kv_in_CTAs=[], MNWs=[])
        view = N.BucketView()
        for i in range(lib.pat_tree_num_buckets(h)):
            lib.pat_tree_bucket(h, i, C.byref(view))
            v["MNWs"].append([view.mnw[0], view.mnw[1], view.mnw[2]])
            v["q_tables"].append(_view_i32(view.q_table, (view.ctas, view.max_seqs)))
            v["block_tables"].append(_view_i32(view.block_table, (view.ctas, view.max_blocks)))
            v["num_seqs_per_CTAs"].append(_view_i32(view.num_seqs, (view.ctas,)))
            v["CTA_ranks"].append(_view_i32(view.cta_ranks, (view.ctas,)))
            v["kv_in_CTAs"].append(_view_i32(view.kv_in_cta, (view.ctas,)))
        n = C.c_int(0)
        ptr = lib.pat_tree_split_per_seq(h, C.byref(n))
        v["num_split_per_seq"] = _view_i32(ptr, (n.value,)) if o.packed_once else torch.zeros(0, dtype=torch.int32)
        mx = (C.c_int32 * 3)()
        lib.pat_tree_maxima(h, mx)
        v["max_split_per_seq"], v["max_seqs_in_CTA"], v["max_blocks_in_CTA"] = mx[0], mx[1], mx[2]
        if self._device is not None:
            self._move(v, self._device)
        return v

    @staticmethod
    def _move(v, device):
        move = lambda t: t.to(device, non_blocking=True)
        for name in ("q_tables", "block_tables", "num_seqs_per_CTAs", "CTA_ranks", "kv_in_CTAs"):
            v[name] = [move(t) for t in v[name]]
        v["num_split_per_seq"] = move(v["num_split_per_seq"])

    def to_gpu(self, device: Union[torch.device, str]) -> None:
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self._device = device
        if self._vals is not None:
            self._move(self._vals, device)
        if device.type == "cuda":
            self.device_work(device)
            check_status(device, synchronize=False)     # a failed wait of an earlier step surfaces here

    def device_work(self, device: torch.device, cfg: Optional[WorkConfig] = None, q_per_req: int = 1) -> DeviceWork:
        """The work list on ``device`` (built and uploaded on first use).  ``q_per_req`` > 1: the list
        for that many query tokens per request (the last tokens of each request's context)."""
        cfg = cfg or default_config()
        key = (str(device), cfg.key()) if q_per_req == 1 else (str(device), cfg.key(), int(q_per_req))
        work = self._work.get(key)
        if work is None:
            o = self._box
            work = DeviceWork.from_tree(o.handle, o.hratio, o.kv_heads, device, cfg, q_per_req)
            self._work[key] = work
        return work


class _TreeBox:
    """The native tree and the state of its pack, shared by a ``PrefixTreeCPP`` and its
    ``KernelInfo``.  Neither of the two refers to the other through it, so dropping the last
    reference frees the native tree at once (a cycle would leave that to the garbage collector, and
    a decode loop that builds a tree per step would then run every build on fresh memory)."""

    __slots__ = ("handle", "hratio", "kv_heads", "pack_args", "deferred", "built", "packed", "packed_once")

    def __init__(self, handle):
        self.handle = handle
        self.hratio = 1
        self.kv_heads = 8
        self.pack_args = None           # arguments of the last pack_schedule
        self.deferred = None            # arguments of a pack that was put off
        self.built = False
        self.packed = False             # the native tree holds a plan for its current state
        self.packed_once = False

    def __del__(self):
        h = getattr(self, "handle", None)
        if h:
            try:
                N.load().pat_tree_destroy(h)
            except Exception:
                pass
            self.handle = None

    def run_pack(self, args) -> None:
        arr, hratio, kv_heads, ucm = args
        ptr, n = (arr.ctypes.data, arr.shape[0]) if arr is not None else (None, 0)
        rc = N.load().pat_tree_pack(self.handle, ptr, n, hratio, kv_heads, ucm)
        if rc != 0:
            raise RuntimeError(f"pack_schedule failed: {N.strerror(rc)}")
        self.packed = True

    def ensure_packed_before_repack(self) -> None:
        """A pack that was put off must have happened before the next one accumulates onto it."""
        if self.packed_once and not self.packed and self.deferred is not None:
            args, self.deferred = self.deferred, None
            self.run_pack(args)

    def ensure_packed(self) -> None:
        """Runs a pack that was put off, or packs again after an in-place advance dropped the plan
        (same arguments as last time)."""
        if self.packed or self.pack_args is None:
            return
        self.deferred = None
        self.run_pack(self.pack_args)


def _boxed(name):
    return property(lambda self: getattr(self._box, name), lambda self, v: setattr(self._box, name, v))


class PrefixTreeCPP:
    """Native radix tree + packer (reference ``csrc/bindings.cpp:100-146``).

    ``semantics="cpp"`` (default) follows ``csrc/prefix_tree.h``;
    ``semantics="py"`` follows ``prefix_attn/prefix_tree.py`` bit for bit (the
    two reference schedulers differ in thresholds and visiting order).
    """

    def __init__(self, block_size: int, semantics: str = "cpp"):
        if semantics not in ("cpp", "py"):
            raise ValueError("semantics must be 'cpp' or 'py'")
        lib = N.load()
        self.block_size = int(block_size)
        self.semantics = semantics
        handle = lib.pat_tree_create(self.block_size, 1 if semantics == "cpp" else 0)
        if not handle:
            raise RuntimeError("block_size must be positive")
        self._box = _TreeBox(handle)
        self._kernel_info = KernelInfo(self._box)

    _handle = _boxed("handle")
    _hratio = _boxed("hratio")
    _kv_heads = _boxed("kv_heads")
    _pack_args = _boxed("pack_args")
    _deferred = _boxed("deferred")
    _built = _boxed("built")
    _packed = _boxed("packed")
    _packed_once = _boxed("packed_once")

    @property
    def kernel_info(self) -> KernelInfo:
        return self._kernel_info

    def build_radix_tree(self, seq_lens, block_table) -> None:
        """``seq_lens``: list of ints or a CPU int32 tensor; ``block_table``: a
        CPU int32 tensor ``[num_seqs, max_blocks]`` (rows are cut to
        ``ceil(len / block_size)`` pages) or, as the Python scheduler takes
        it, a list of unpadded lists."""
        lib = N.load()
        if isinstance(seq_lens, torch.Tensor):
            if seq_lens.dtype != torch.int32 or seq_lens.device.type != "cpu":
                raise RuntimeError("seq_lens must be a List[int] or a CPU Int32 Tensor")
            lens = np.ascontiguousarray(seq_lens.numpy())
        elif isinstance(seq_lens, (list, tuple)):
            lens = np.asarray(seq_lens, dtype=np.int32)
        else:
            raise RuntimeError("seq_lens must be a List[int] or a CPU Int32 Tensor")
        if isinstance(block_table, torch.Tensor):
            if block_table.dtype != torch.int32 or block_table.device.type != "cpu" or block_table.dim() != 2:
                raise RuntimeError("block_table must be a 2-D CPU Int32 Tensor")
            table = np.ascontiguousarray(block_table.numpy())
            if lens.shape[0] != table.shape[0]:
                raise RuntimeError("Seq lens list mismatch")
            rc = lib.pat_tree_build(self._handle, lens.ctypes.data, table.ctypes.data,
                                    table.shape[0], table.shape[1])
        else:
            rows = [np.asarray(r, dtype=np.int32) for r in block_table]
            if lens.shape[0] != len(rows):
                raise RuntimeError("Seq lens list mismatch")
            offsets = np.zeros(len(rows) + 1, dtype=np.int64)
            np.cumsum([len(r) for r in rows], out=offsets[1:])
            flat = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int32)
            flat = np.ascontiguousarray(flat, dtype=np.int32)
            rc = lib.pat_tree_build_ragged(self._handle, lens.ctypes.data, flat.ctypes.data,
                                           offsets.ctypes.data, len(rows))
        if rc != 0:
            raise RuntimeError(f"build_radix_tree failed: {N.strerror(rc)}")
        self._built = True

    def pack_schedule(self, MNWs: Optional[List[List[int]]] = None, HRatio: int = 1, kvHead: int = 8,
                      use_compute_model: bool = False) -> None:
        lib = N.load()
        if MNWs:
            arr = np.asarray(MNWs, dtype=np.int32).reshape(-1, 3)
            ptr, n = arr.ctypes.data, arr.shape[0]
        else:
            arr, ptr, n = None, None, 0
        self._pack_args = (arr, int(HRatio), int(kvHead), int(bool(use_compute_model)))
        if self.semantics == "cpp" and int(HRatio) > 0 and self._built and not self._packed_once:
            # The C++ scheduler's pack cannot fail on a built tree, and the kernels here run from
            # the work list, not from the plan: the first pack is put off until somebody reads
            # ``kernel_info``.  (A second pack on the same tree accumulates, like the reference's,
            # so it runs at once, after the first.)
            self._hratio, self._kv_heads = int(HRatio), int(kvHead)
            self._packed = False
            self._packed_once = True
            self._deferred = self._pack_args
            self._kernel_info._invalidate()
            return
        self._ensure_packed_before_repack()
        rc = lib.pat_tree_pack(self._handle, ptr, n, int(HRatio), int(kvHead), int(bool(use_compute_model)))
        if rc == -2:
            raise IndexError(N.strerror(rc))
        if rc == -3:
            raise ValueError(N.strerror(rc))
        if rc == -4:
            raise KeyError(N.strerror(rc))
        if rc != 0:
            raise RuntimeError(f"pack_schedule failed: {N.strerror(rc)}")
        self._hratio, self._kv_heads = int(HRatio), int(kvHead)
        self._packed = self._packed_once = True
        self._kernel_info._invalidate()

    def _ensure_packed_before_repack(self) -> None:
        self._box.ensure_packed_before_repack()

    def _ensure_packed(self) -> None:
        self._box.ensure_packed()

    def advance(self, seq_lens, block_table: torch.Tensor, device=None) -> bool:
        """One decode step later: the same requests, each at least as long as before, each table row
        extended by the pages its new tokens need.  Returns ``True`` when tree and device work list
        were updated in place - the tree is then the tree a fresh ``build_radix_tree`` of the new
        tables would give, ``kernel_info`` is re-packed when (and only if) it is read, and the work
        list is re-uploaded into the same device buffer on the current stream.  Returns ``False``,
        with nothing changed, when the batch has to be rebuilt: other requests, a row whose old part
        changed, a request that shares its last segment, or no room left for new pages.

        The reference builds tree, plan and tables from scratch in every step
        (``prefix_attn/async_tree.py:23-30``) and leaves them stale during multi-step decode
        (``plugin/vllm/attention/backends/prefix_attn.py:430-438``)."""
        lib = N.load()
        if isinstance(seq_lens, torch.Tensor):
            lens = np.ascontiguousarray(seq_lens.numpy(), dtype=np.int32)
        else:
            lens = np.asarray(seq_lens, dtype=np.int32)
        if not isinstance(block_table, torch.Tensor) or block_table.dtype != torch.int32 or \
                block_table.device.type != "cpu" or block_table.dim() != 2:
            raise RuntimeError("block_table must be a 2-D CPU Int32 Tensor")
        table = np.ascontiguousarray(block_table.numpy())
        if lens.shape[0] != table.shape[0]:
            return False
        info = self._kernel_info
        works = list(info._work.values())
        if len(works) > 1:
            return False                        # several devices / option sets: rebuild
        if works:
            if works[0]._handle is None:
                return False
            rc = lib.pat_work_advance(works[0]._handle, self._handle, lens.ctypes.data, table.ctypes.data,
                                      table.shape[0], table.shape[1])
        else:
            rc = lib.pat_tree_advance(self._handle, lens.ctypes.data, table.ctypes.data,
                                      table.shape[0], table.shape[1])
        if rc < 0:
            raise RuntimeError(f"advance failed: {N.strerror(rc)}")
        if rc == 0:
            return False
        self._packed = False
        info._vals = None                       # the plan is stale; the work list was advanced with the tree
        if works:
            works[0].refresh()
        return True

    def _max_split(self) -> int:
        mx = (C.c_int32 * 3)()
        N.load().pat_tree_maxima(self._handle, mx)
        return mx[0]

    def _batch(self) -> int:
        n = C.c_int(0)
        N.load().pat_tree_split_per_seq(self._handle, C.byref(n))
        return n.value

    # ---- inspection helpers (not in the reference binding) -----------------
    def nodes(self):
        """``[(parent, s_value, length, seq_indices, pages, children)]`` per node."""
        lib = N.load()
        out = []
        info = (C.c_int32 * 4)()
        ptr, cnt = N.i32p(), C.c_int(0)
        for i in range(lib.pat_tree_num_nodes(self._handle)):
            lib.pat_tree_node(self._handle, i, info)
            lib.pat_tree_node_seqs(self._handle, i, C.byref(ptr), C.byref(cnt))
            seqs = [ptr[j] for j in range(cnt.value)]
            lib.pat_tree_node_pages(self._handle, i, C.byref(ptr), C.byref(cnt))
            pages = [ptr[j] for j in range(cnt.value)]
            nkids = lib.pat_tree_node_children(self._handle, i, None, 0)
            buf = (C.c_int32 * max(nkids, 1))()
            lib.pat_tree_node_children(self._handle, i, buf, nkids)
            out.append((info[0], info[1], info[2], seqs, pages, [buf[j] for j in range(nkids)]))
        return out


# --------------------------------------------------------------------------- the op
_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def _check(cond: bool, msg: str):
    if not cond:
        raise RuntimeError(msg)


def _check_index(t: torch.Tensor, name: str, shape=None):
    _check(t.is_cuda, f"{name} must be on CUDA")
    _check(t.dtype == torch.int32, f"{name} must have dtype torch.int32")
    _check(t.stride(-1) == 1 or t.shape[-1] <= 1, f"{name} must have contiguous last dimension")
    if shape is not None:
        _check(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The per-device int32[4] the kernels report a failed bounded wait in (zero = fine)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status_words.get(device)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status_words[device] = t
    return t


def check_status(device=None, synchronize: bool = True) -> None:
    """Raises if a kernel of an earlier call on ``device`` gave up on a bounded wait (its output is
    then not valid).  With ``synchronize=False`` the word is read on a side stream without waiting
    for queued work, which is how a plan build checks it in passing."""
    devices = [torch.device(device)] if device is not None else list(_status_words)
    for dev in devices:
        t = _status_words.get(dev if dev.index is not None else torch.device("cuda", torch.cuda.current_device()))
        if t is None:
            continue
        if synchronize:
            code = int(t[0].item())
        else:
            side = _side_stream(t.device)
            with torch.cuda.stream(side):
                code = int(t[0].item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"a decode-attention kernel gave up on a bounded wait (code {code}); "
                               "outputs since the last check are not valid")


_side_streams = {}


def _side_stream(device):
    s = _side_streams.get(device)
    if s is None:
        s = torch.cuda.Stream(device)
        _side_streams[device] = s
    return s


def _run(q, k_cache, v_cache, work: DeviceWork, scale: float, out, lse_out=None, status=None, flags=0,
         wait_limit_us=0):
    lib = N.load()
    stream = torch.cuda.current_stream(q.device)
    work.order_after_upload(stream)
    if status is None:
        status = status_word(q.device)
    key = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
           lse_out.data_ptr() if lse_out is not None else 0, status.data_ptr(), stream.cuda_stream,
           q.shape, q.stride(), k_cache.shape, k_cache.stride(), v_cache.stride(), out.stride(),
           q.dtype, float(scale), int(flags), int(wait_limit_us))
    cached = work._args
    if cached is not None and cached[0] == key:
        a = cached[1]
    else:
        B, T, H, D = q.shape
        a = N.DecodeArgs()
        a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
        a.lse_out = lse_out.data_ptr() if lse_out is not None else None
        a.q_batch_stride, a.q_head_stride = q.stride(0), q.stride(2)
        a.k_page_stride, a.k_row_stride, a.k_head_stride = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
        a.v_page_stride, a.v_row_stride, a.v_head_stride = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
        a.out_batch_stride, a.out_head_stride = out.stride(0), out.stride(2)
        a.q_per_req, a.q_pos_stride, a.out_pos_stride = T, q.stride(1), out.stride(1)
        a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = B, H, k_cache.shape[2], D
        a.page_size = k_cache.shape[1]
        a.dtype = _DTYPES[q.dtype]
        a.num_pages = k_cache.shape[0]
        a.softmax_scale = float(scale)
        a.flags = int(flags)
        a.work_blob = work.blob.data_ptr()
        a.work = work.header
        need = lib.pat_b200_workspace_bytes(C.byref(work.header), H, D)
        # (a graph captured around this call refers to the work list's blob and scratch: keep the
        # tree alive as long as the graph, like the tensors)
        ws = work.workspace(need, stream, q.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        a.status_word = status.data_ptr()
        a.wait_limit_us = int(wait_limit_us)
        work._args = (key, a)
    rc = lib.pat_b200_decode(C.byref(a), C.c_void_p(stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"prefix_attn_with_kvcache failed: {N.strerror(rc)} ({rc})")


def prefix_attn_with_kvcache(*args, **kwargs) -> None:
    """Prefix-aware decode attention over a paged KV cache; writes ``out`` in place.

    Two call forms, as in the reference (``csrc/bindings.cpp:76-95`` and ``:148-157``):

    ``(q, k_cache_paged, v_cache_paged, num_split_per_seq, query_tables, block_tables,
    num_seqs_per_CTAs, CTA_ranks, kv_in_CTAs, MNW, max_split_per_seq, max_seqs_in_CTA,
    max_blocks_in_CTA, softmax_scale, out, timing_=None)``

    ``(q, k_cache_paged, v_cache_paged, tree, softmax_scale, out)`` with ``tree`` a
    ``PrefixTreeCPP`` whose ``kernel_info`` was moved to the GPU.

    ``q``/``out``: ``[batch, 1, heads, head_dim]``; caches: ``[pages, page_size, kv_heads,
    head_dim]``; fp16 or bf16.  The tree form also takes ``[batch, T, heads, head_dim]`` with
    ``T`` > 1 query tokens per request (speculative decoding, a short prefill chunk on a cached
    prefix): the tree is then built from the full lengths, the ``T`` new tokens included, and
    position ``t`` attends to the first ``len - T + 1 + t`` tokens of its request.  Extra keyword (not in the reference): ``lse_out``, a float32
    CUDA tensor ``[batch, heads]`` that receives the natural-log LSE of the scaled scores
    (the reference computes it, ``csrc/api.h:195``, but never returns it).
    """
    lse_out = kwargs.pop("lse_out", None)
    status = kwargs.pop("_status", None)
    flags = kwargs.pop("_flags", 0)
    wait_limit_us = kwargs.pop("_wait_limit_us", 0)
    names16 = ["q", "k_cache_paged", "v_cache_paged", "num_split_per_seq", "query_tables", "block_tables",
               "num_seqs_per_CTAs", "CTA_ranks", "kv_in_CTAs", "MNW", "max_split_per_seq", "max_seqs_in_CTA",
               "max_blocks_in_CTA", "softmax_scale", "out", "timing_"]
    names6 = ["q", "k_cache_paged", "v_cache_paged", "tree", "softmax_scale", "out", "timing_"]
    tree_form = ("tree" in kwargs) or (len(args) >= 4 and isinstance(args[3], PrefixTreeCPP))
    names = names6 if tree_form else names16
    if len(args) > len(names):
        raise TypeError("prefix_attn_with_kvcache(): incompatible function arguments")
    bound = dict(zip(names, args))
    for k, v in kwargs.items():
        if k not in names or k in bound:
            raise TypeError(f"prefix_attn_with_kvcache(): incompatible function arguments ({k})")
        bound[k] = v
    bound.setdefault("timing_", None)
    missing = [n for n in names if n not in bound]
    if missing:
        raise TypeError(f"prefix_attn_with_kvcache(): missing arguments {missing}")

    q, k_cache, v_cache, out = bound["q"], bound["k_cache_paged"], bound["v_cache_paged"], bound["out"]
    scale = bound["softmax_scale"]

    # ---- the reference's argument checks (csrc/api.h:131-181) ----------------
    _check(q.dtype in _DTYPES, "only support fp16 and bf16 data type")
    _check(k_cache.dtype == q.dtype, "query and key must have the same dtype")
    _check(v_cache.dtype == q.dtype, "query and value must have the same dtype")
    for t, n in ((q, "q"), (k_cache, "kcache"), (v_cache, "vcache")):
        _check(t.is_cuda, f"{n} must be on CUDA")
    for t in (q, k_cache, v_cache):
        _check(t.stride(-1) == 1, "Input tensor must have contiguous last dimension")
    _check(q.dim() == 4 and k_cache.dim() == 4 and v_cache.dim() == 4, "q, kcache, vcache must be 4-D")
    B, seqlen_q, H, D = q.shape
    if D not in (64, 128):
        raise RuntimeError("head_size_og must be 64 / 128 currently")
    num_pages, page, Hkv = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    _check(page % 16 == 0, "Paged KV cache block size must be divisible by 16")
    _check(H % Hkv == 0, "Number of heads in key/value must divide number of heads in query")
    ratio = H // Hkv
    _check(ratio in (1, 2, 4, 8), "only support QGA with hq/hkv = 1, 2, 4, 8 now.")
    _check(B > 0, "batch size must be positive")
    _check(seqlen_q >= 1, "q must have shape (batch_size, seqlen_q, n_heads, head_size)")
    _check(tuple(k_cache.shape) == (num_pages, page, Hkv, D), "kcache must have shape (num_blocks, page_block_size, n_heads_kv, head_size_og)")
    _check(tuple(v_cache.shape) == (num_pages, page, Hkv, D), "vcache must have shape (num_blocks, page_block_size, n_heads_kv, head_size_og)")
    _check(out.is_cuda and out.dtype == q.dtype and tuple(out.shape) == tuple(q.shape) and out.stride(-1) == 1,
           "out must be a CUDA tensor with the shape and dtype of q")
    if lse_out is not None:
        want = (B, H) if seqlen_q == 1 else (B, seqlen_q, H)
        _check(lse_out.is_cuda and lse_out.dtype == torch.float32 and lse_out.is_contiguous()
               and tuple(lse_out.shape) == want,
               "lse_out must be a contiguous float32 CUDA tensor [batch, heads] ([batch, seqlen_q, heads])")
    if seqlen_q > 1:
        # Several query tokens per request (the reference sends these steps to another library,
        # plugin/vllm/attention/backends/prefix_attn.py:877-904): the requests' lengths in the tree
        # include the seqlen_q new tokens, which are already in the cache, and position t attends to
        # the first len - seqlen_q + 1 + t tokens.  Tree form only.
        _check(tree_form, "seqlen_q > 1 needs the tree form of the call")
        _check(seqlen_q <= 64, "seqlen_q must be at most 64")
        _check(q.stride(1) % 8 == 0 and out.stride(1) % 8 == 0, "q / out rows must be 16-byte aligned")

    if tree_form:
        tree = bound["tree"]
        inner = getattr(tree, "tree", None)         # an AsyncTree hands over its built tree
        if not isinstance(tree, PrefixTreeCPP) and isinstance(inner, PrefixTreeCPP):
            tree = inner
        _check(isinstance(tree, PrefixTreeCPP), "tree must be a PrefixTreeCPP")
        info = tree.kernel_info
        # the plan's own numbers, read from the native tree without making the plan tensors; a
        # tree advanced in place has no packed plan (and the reference's split limit is a limit
        # of its kernels, not of the work list used here)
        max_split = tree._max_split() if tree._packed else 1
        _check(info._device is not None and info._device.type == "cuda", "num_split_per_seq must be on CUDA")
        _check(tree._batch() == B, f"num_split_per_seq must have shape {(B,)}")
    else:
        max_split = int(bound["max_split_per_seq"])
        nsplit = bound["num_split_per_seq"]
        _check_index(nsplit, "num_split_per_seq", (B,))
    if max_split > 32:
        raise RuntimeError("Currently, only supports up to 32 splits per seq. Excessive splitting may reduce efficiency.")
    if max_split <= 0:
        raise RuntimeError("there is no case that a seq has no block")

    if tree_form:
        _check(tree._hratio == ratio, "the plan was packed for a different HRatio than q / k_cache imply")
        _check(tree.block_size == page, "the plan was built for a different page size than k_cache has")
        work = info.device_work(q.device, None, seqlen_q)
    else:
        qts, bts = list(bound["query_tables"]), list(bound["block_tables"])
        nss, rks, kvs = list(bound["num_seqs_per_CTAs"]), list(bound["CTA_ranks"]), list(bound["kv_in_CTAs"])
        mnw = bound["MNW"]
        _check(len(qts) == len(bts) == len(nss) == len(rks) == len(kvs) == len(mnw),
               "per-bucket plan lists must have one entry per MNW")
        for i in range(len(mnw)):
            ctas = qts[i].shape[0]
            _check_index(qts[i], "query_tables")
            _check_index(bts[i], "block_tables")
            _check(bts[i].shape[0] == ctas, "block_tables must have one row per CTA")
            _check_index(nss[i], "num_seqs_per_CTA", (ctas,))
            _check_index(rks[i], "CTA_rank", (ctas,))
            _check_index(kvs[i], "kv_in_CTA", (ctas,))
        tag = _plan_cache.find_tag(nsplit, qts, bts, nss, kvs)
        if tag is None:
            tag = _plan_cache.make_tag(nsplit, qts, bts, nss, kvs)
        cfg = default_config()
        key = (str(q.device), ratio, Hkv, page, cfg.key())
        work = tag.work.get(key)
        if work is None:
            work = DeviceWork.from_host_plan(tag.host_plan, ratio, Hkv, page, q.device, cfg)
            tag.work[key] = work

    with torch.cuda.device(q.device):
        _run(q, k_cache, v_cache, work, scale, out, lse_out, status, flags, wait_limit_us)


def last_launch_count() -> int:
    """Kernels launched by the last call on this thread."""
    return N.load().pat_b200_last_launch_count()
