"""TEST INFRASTRUCTURE ONLY - loads the upstream reference's pure-Python modules.

The reference package cannot be imported as shipped (its ``__init__`` needs the
compiled ``_prefix_attn`` extension), but ``data_class``, ``utils``,
``prefix_tree`` and ``block_scheduler`` are pure Python.  This loader registers
them under a private package name with a stub for the compiled module so that
they run unmodified, straight from the read-only reference checkout.  It is used
by ``tests/golden/make_golden.py`` to freeze golden plans and by tests that
cross-check live against the reference when the checkout is present.  Nothing
here is shipped or timed, and nothing outside ``tests/`` may import it.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

# The reference checkout: PAT_REFERENCE_ROOT, else a directory named "reference" beside this repository.
REFERENCE_ROOT = os.environ.get("PAT_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
_PKG = "_pat_reference_pkg"


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "prefix_attn", "prefix_tree.py"))


def load_reference_python():
    """Return ``{name: module}`` for the reference's pure-Python modules."""
    if not reference_available():
        raise FileNotFoundError(f"reference checkout not found under {REFERENCE_ROOT}")
    if _PKG in sys.modules and hasattr(sys.modules[_PKG], "_loaded"):
        return sys.modules[_PKG]._loaded
    src = os.path.join(REFERENCE_ROOT, "prefix_attn")
    pkg = types.ModuleType(_PKG)
    pkg.__path__ = [src]
    sys.modules[_PKG] = pkg

    stub = types.ModuleType(_PKG + "._prefix_attn")

    class _NoNative:  # the compiled classes are not needed by the Python scheduler
        def __init__(self, *a, **k):
            raise RuntimeError("compiled reference extension is not available")

    stub.PrefixTreeCPP = _NoNative
    stub.prefix_attn_with_kvcache = None
    sys.modules[_PKG + "._prefix_attn"] = stub
    pkg.PrefixTreeCPP = _NoNative

    loaded = {}
    for name in ("data_class", "utils", "prefix_tree", "block_scheduler"):
        full = f"{_PKG}.{name}"
        spec = importlib.util.spec_from_file_location(full, os.path.join(src, name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        spec.loader.exec_module(mod)
        setattr(pkg, name, mod)
        loaded[name] = mod
    pkg._loaded = loaded
    return loaded


def load_reference_attention():
    """The reference's dense fp32 PyTorch attention (``test/utils.py:7-58``)."""
    path = os.path.join(REFERENCE_ROOT, "test", "utils.py")
    spec = importlib.util.spec_from_file_location("_pat_reference_test_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.attention_ref
