"""pat_b200 - prefix-aware decode attention for B200 (sm_100a).

Drop-in for the ``prefix_attn`` package of flashserve/PAT: the same exports
(reference ``prefix_attn/__init__.py:3-26``), with the device path implemented
by hand-written sm_100a kernels behind a C-ABI library (``libpat_b200.so``).
"""
from ._prefix_attn import prefix_attn_with_kvcache, PrefixTreeCPP
from .utils import generate_random_prefix_seqs, generate_random_kv_cache, generate_tree_seqs
from .data_class import PackedBox, Sequence, SeqGroup, KernelInfo
from .block_scheduler import pack_prefix_blocks, pack_without_prefix, schedule, schedule_naive
from .prefix_tree import PrefixTree
from .async_tree import AsyncTree
# not part of the reference's export list: carrying a plan across decode steps, and the report of
# a kernel whose bounded wait ran out
from ._prefix_attn import check_status, status_word
from .planner import DecodePlanner

__all__ = [
    "prefix_attn_with_kvcache",
    "PrefixTree",
    "PrefixTreeCPP",
    "AsyncTree",
    "generate_random_prefix_seqs",
    "generate_random_kv_cache",
    "generate_tree_seqs",
    "pack_prefix_blocks",
    "pack_without_prefix",
    "schedule",
    "schedule_naive",
    "PackedBox",
    "Sequence",
    "SeqGroup",
    "KernelInfo",
]
