"""Keeps the host copy of a plan next to the device tensors made from it.

The 16-argument form of ``prefix_attn_with_kvcache`` receives a plan only as
int32 device tensors.  The kernels here do not run the boxes as they are: a
work list is derived from them on the host (``csrc/pat_work.cpp``).  When the
plan came from ``KernelInfo.to_tensor`` the host lists are still at hand, so
they are remembered and attached to the ``num_split_per_seq`` tensor object;
the op then finds them without reading anything back from the GPU.  A plan
that arrives as bare tensors from elsewhere is copied back once (one
synchronising D2H per new plan) and the result is cached on the same tensor.

The cached host plan is matched by the identity and the version counter of the
plan tensors.  A plan must therefore be REPLACED, not rewritten: tensors that
are refilled through a raw pointer or a custom op (persistent metadata buffers
of a captured graph) keep both, and the old work list would be used.  Callers
that reuse buffers call ``invalidate(num_split_per_seq)`` after refilling them.
"""
from __future__ import annotations

import weakref
from typing import List, Optional

import numpy as np
import torch


class HostPlan:
    """A plan as zero-padded int32 numpy arrays, one set per bucket."""

    __slots__ = ("q_tables", "block_tables", "num_seqs", "kv_lens", "batch")

    def __init__(self, q_tables, block_tables, num_seqs, kv_lens, batch):
        self.q_tables: List[np.ndarray] = q_tables
        self.block_tables: List[np.ndarray] = block_tables
        self.num_seqs: List[np.ndarray] = num_seqs
        self.kv_lens: List[np.ndarray] = kv_lens
        self.batch: int = batch


def _pad2d(rows) -> np.ndarray:
    if len(rows) and not isinstance(rows[0], (list, tuple, np.ndarray)):
        rows = [[int(r)] for r in rows]          # flat legacy q_table: one query per box
    width = max((len(r) for r in rows), default=0)
    out = np.zeros((len(rows), max(width, 1)), dtype=np.int32)
    for i, r in enumerate(rows):
        out[i, :len(r)] = r
    return out


def host_plan_from_lists(q_tables, block_tables, num_seqs, kv_lens, batch) -> HostPlan:
    return HostPlan([_pad2d(t) for t in q_tables], [_pad2d(t) for t in block_tables],
                    [np.asarray(t, dtype=np.int32).reshape(-1) for t in num_seqs],
                    [np.asarray(t, dtype=np.int32).reshape(-1) for t in kv_lens], int(batch))


def host_plan_from_tensors(q_tables, block_tables, num_seqs, kv_lens, batch) -> HostPlan:
    """Synchronising copy of device (or CPU) plan tensors to the host."""
    def two_d(t):
        a = t.detach().to("cpu", torch.int32).numpy()
        return np.ascontiguousarray(a.reshape(a.shape[0], -1) if a.ndim != 2 else a)

    def one_d(t):
        return np.ascontiguousarray(t.detach().to("cpu", torch.int32).numpy().reshape(-1))

    return HostPlan([two_d(t) for t in q_tables], [two_d(t) for t in block_tables],
                    [one_d(t) for t in num_seqs], [one_d(t) for t in kv_lens], int(batch))


def remember_host_plan(ki) -> None:
    """Called by ``KernelInfo.to_tensor`` while the fields are still lists."""
    try:
        ki._host_plan = host_plan_from_lists(ki.q_tables, ki.block_tables, ki.num_seqs_per_CTAs,
                                             ki.kv_in_CTAs, len(ki.num_split_per_seq))
    except Exception:       # malformed lists: the op will read the tensors back instead
        ki._host_plan = None


class PlanTag:
    """What is attached to a ``num_split_per_seq`` tensor: the host plan, the
    tensor objects it belongs to (to detect a different plan passed with the
    same tensor) and the device work lists built from it so far."""

    def __init__(self, host_plan: HostPlan, tensors):
        self.host_plan = host_plan
        self.versions = tuple(t._version for t in tensors)
        # Weak references: the tag hangs on one of these tensors, so strong ones would form a
        # cycle that keeps the device tensors and work lists alive until the cycle collector
        # runs.  A dead reference (its id may have been reused) never matches.
        self.refs = tuple(weakref.ref(t) for t in tensors)
        self.work = {}                  # (device, hratio, kv_heads, page, options) -> DeviceWork

    def matches(self, tensors) -> bool:
        return (len(tensors) == len(self.refs)
                and all(r() is t for t, r in zip(tensors, self.refs))
                and all(t._version == v for t, v in zip(tensors, self.versions)))


def plan_tensors(num_split_per_seq, q_tables, block_tables, num_seqs, kv_lens):
    return [num_split_per_seq, *q_tables, *block_tables, *num_seqs, *kv_lens]


def attach_to_tensors(ki) -> None:
    plan = getattr(ki, "_host_plan", None)
    if plan is None or not isinstance(ki.num_split_per_seq, torch.Tensor):
        return
    tensors = plan_tensors(ki.num_split_per_seq, ki.q_tables, ki.block_tables,
                           ki.num_seqs_per_CTAs, ki.kv_in_CTAs)
    ki.num_split_per_seq._pat_plan_tag = PlanTag(plan, tensors)


def find_tag(num_split_per_seq, q_tables, block_tables, num_seqs, kv_lens) -> Optional[PlanTag]:
    tag = getattr(num_split_per_seq, "_pat_plan_tag", None)
    if tag is None:
        return None
    return tag if tag.matches(plan_tensors(num_split_per_seq, q_tables, block_tables, num_seqs, kv_lens)) else None


def make_tag(num_split_per_seq, q_tables, block_tables, num_seqs, kv_lens) -> PlanTag:
    plan = host_plan_from_tensors(q_tables, block_tables, num_seqs, kv_lens, num_split_per_seq.shape[0])
    tag = PlanTag(plan, plan_tensors(num_split_per_seq, q_tables, block_tables, num_seqs, kv_lens))
    num_split_per_seq._pat_plan_tag = tag
    return tag



def invalidate(num_split_per_seq) -> None:
    """Forgets the host plan and work lists cached on a plan's ``num_split_per_seq`` tensor (for
    callers that refill their plan tensors in place)."""
    if hasattr(num_split_per_seq, "_pat_plan_tag"):
        del num_split_per_seq._pat_plan_tag
