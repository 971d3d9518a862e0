"""The serving backend that consumes this package (reference
``plugin/vllm/attention/backends/prefix_attn.py``) must load UNMODIFIED on top of it.

The file needs vLLM v0.9.0's V0 attention interfaces, which are not installed anywhere this
suite runs, so the handful of vLLM names it imports (``prefix_attn.py:13-34``) are replaced by
empty stand-ins.  What is checked is this package's side of the contract: the import block
``from prefix_attn import prefix_attn_with_kvcache, AsyncTree, PrefixTreeCPP`` resolves to the
objects defined here, and the two call sites (``:330-338`` and ``:908-915``) use only keyword
arguments that those objects accept.  The numerical behaviour of the same two calls is covered on
the GPU by ``test_gpu_attention.py::test_async_tree_and_strided_views_like_the_serving_backend``.
"""
import ast
import importlib.util
import inspect
import os
import sys
import types

import pytest

from oracle.ref_loader import REFERENCE_ROOT

PLUGIN = os.path.join(REFERENCE_ROOT, "plugin", "vllm", "attention", "backends", "prefix_attn.py")
pytestmark = pytest.mark.skipif(not os.path.isfile(PLUGIN), reason="reference checkout not present")


class _Generic:
    def __class_getitem__(cls, item):
        return cls


def _stub_modules():
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        return m

    anything = lambda *a, **k: None
    abstract = mod("vllm.attention.backends.abstract",
                   AttentionBackend=type("AttentionBackend", (), {}),
                   AttentionImpl=type("AttentionImpl", (_Generic,), {}),
                   AttentionLayer=type("AttentionLayer", (), {}),
                   AttentionMetadata=type("AttentionMetadata", (), {}),
                   AttentionMetadataBuilder=type("AttentionMetadataBuilder", (_Generic,), {}),
                   AttentionType=type("AttentionType", (), {"DECODER": "decoder", "ENCODER": "encoder",
                                                            "ENCODER_ONLY": "encoder_only",
                                                            "ENCODER_DECODER": "encoder_decoder"}),
                   is_quantized_kv_cache=anything)
    utils_names = ["PAD_SLOT_ID", "CommonAttentionState", "compute_slot_mapping", "compute_slot_mapping_start_idx",
                   "get_num_prefill_decode_query_kv_tokens", "get_seq_len_block_table_args",
                   "is_all_cross_attn_metadata_set", "is_all_encoder_attn_metadata_set", "is_block_tables_empty"]
    backends_utils = mod("vllm.attention.backends.utils", **{n: anything for n in utils_names})
    backends_utils.PAD_SLOT_ID = -1
    backends_utils.CommonAttentionState = type("CommonAttentionState", (), {})
    import logging
    mods = {
        "vllm": mod("vllm", _custom_ops=mod("vllm._custom_ops")),
        "vllm._custom_ops": mod("vllm._custom_ops"),
        "vllm.attention": mod("vllm.attention"),
        "vllm.attention.backends": mod("vllm.attention.backends"),
        "vllm.attention.backends.abstract": abstract,
        "vllm.attention.backends.utils": backends_utils,
        "vllm.logger": mod("vllm.logger", init_logger=logging.getLogger),
        "vllm.multimodal": mod("vllm.multimodal", MultiModalPlaceholderMap=type("MultiModalPlaceholderMap", (), {})),
        "vllm.utils": mod("vllm.utils", async_tensor_h2d=anything, make_tensor_with_pad=anything,
                          make_ndarray_with_pad=anything),
        "vllm.vllm_flash_attn": mod("vllm.vllm_flash_attn", flash_attn_varlen_func=anything,
                                    flash_attn_with_kvcache=anything),
    }
    return mods


@pytest.fixture()
def plugin(monkeypatch):
    for name, m in _stub_modules().items():
        monkeypatch.setitem(sys.modules, name, m)
    spec = importlib.util.spec_from_file_location("_reference_prefix_attn_backend", PLUGIN)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_backend_file_loads_on_this_package(plugin):
    import pat_b200
    assert plugin.prefix_attn_with_kvcache is pat_b200.prefix_attn_with_kvcache
    assert plugin.AsyncTree is pat_b200.AsyncTree
    assert plugin.PrefixTreeCPP is pat_b200.PrefixTreeCPP
    assert plugin.PrefixAttentionBackend.get_name() == "PREFIX_ATTN"
    assert plugin.PrefixAttentionBackend.get_kv_cache_shape(7, 16, 8, 128) == (2, 7, 16, 8, 128)


def _keyword_names(call):
    assert not call.args, "the backend calls with keywords only"
    return {k.arg for k in call.keywords}


def test_backend_call_sites_use_accepted_keywords():
    import pat_b200
    tree = ast.parse(open(PLUGIN).read())
    calls = {"AsyncTree": [], "prefix_attn_with_kvcache": []}
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in calls:
            calls[node.func.id].append(node)
    assert calls["AsyncTree"] and calls["prefix_attn_with_kvcache"]
    ctor = set(inspect.signature(pat_b200.AsyncTree.__init__).parameters) - {"self"}
    for c in calls["AsyncTree"]:
        assert _keyword_names(c) <= ctor
    # the op takes *args / **kwargs (two call forms); its keyword form is the five-tensor one
    accepted = {"q", "k_cache_paged", "v_cache_paged", "tree", "softmax_scale", "out"}
    for c in calls["prefix_attn_with_kvcache"]:
        assert _keyword_names(c) == accepted
