"""Import alias: ``import prefix_attn`` resolves to :mod:`pat_b200`.

Code written against the reference package (``from prefix_attn import
prefix_attn_with_kvcache, AsyncTree, PrefixTreeCPP`` in the vLLM backend,
``from prefix_attn.prefix_tree import PrefixTree`` in the benchmarks) keeps
working unchanged; the submodules are the ``pat_b200`` ones.
"""
import importlib as _importlib
import sys as _sys

import pat_b200 as _impl
from pat_b200 import *  # noqa: F401,F403
from pat_b200 import __all__  # noqa: F401

for _name in ("_prefix_attn", "data_class", "prefix_tree", "block_scheduler", "utils", "async_tree", "cache_ops"):
    _mod = _importlib.import_module(f"pat_b200.{_name}")
    _sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
