"""KV-cache append, the step right before decode attention in a serving loop.

``reshape_and_cache_flash`` has the signature of vLLM's op of the same name, which the
reference's serving backend calls through ``torch.ops._C_cache_ops``
(``plugin/vllm/attention/backends/prefix_attn.py:828-837``).  It runs this library's kernel on
PyTorch's current stream; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native as N

_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                            value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                            kv_cache_dtype: str = "auto", k_scale: Optional[torch.Tensor] = None,
                            v_scale: Optional[torch.Tensor] = None) -> None:
    """Writes ``key[i]`` / ``value[i]`` (``[num_tokens, kv_heads, head_dim]``) into the paged caches
    (``[pages, page_size, kv_heads, head_dim]``) at ``slot_mapping[i] = page * page_size + row``.
    Tokens with a negative slot are skipped.  ``kv_cache_dtype`` must be ``"auto"`` (caches in the
    dtype of the keys); the scales belong to vLLM's fp8 caches and are ignored."""
    if kv_cache_dtype != "auto":
        raise RuntimeError(f"kv_cache_dtype {kv_cache_dtype!r} is not supported (16-bit caches only)")
    for name, t in (("key", key), ("value", value), ("key_cache", key_cache), ("value_cache", value_cache),
                    ("slot_mapping", slot_mapping)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
    if key.dtype not in _DTYPES or value.dtype != key.dtype or key_cache.dtype != key.dtype or \
            value_cache.dtype != key.dtype:
        raise RuntimeError("key, value and both caches must share one dtype, fp16 or bf16")
    if key.dim() != 3 or value.shape != key.shape:
        raise RuntimeError("key and value must be [num_tokens, kv_heads, head_dim]")
    if key_cache.dim() != 4 or value_cache.shape != key_cache.shape:
        raise RuntimeError("caches must be [pages, page_size, kv_heads, head_dim]")
    tokens, heads, dim = key.shape
    if key_cache.shape[2] != heads or key_cache.shape[3] != dim:
        raise RuntimeError("caches and keys disagree on kv_heads / head_dim")
    for name, t in (("key", key), ("value", value), ("key_cache", key_cache), ("value_cache", value_cache)):
        if t.stride(-1) != 1:
            raise RuntimeError(f"{name} must have a contiguous last dimension")
    slots = slot_mapping.flatten()
    if slots.dtype != torch.int64:
        slots = slots.to(torch.int64)
    slots = slots.contiguous()
    if slots.numel() < tokens:
        raise RuntimeError("slot_mapping is shorter than the number of tokens")
    a = N.AppendArgs()
    a.key, a.value = key.data_ptr(), value.data_ptr()
    a.k_cache, a.v_cache = key_cache.data_ptr(), value_cache.data_ptr()
    a.slot_mapping = slots.data_ptr()
    a.key_token_stride, a.key_head_stride = key.stride(0), key.stride(1)
    a.value_token_stride, a.value_head_stride = value.stride(0), value.stride(1)
    a.k_page_stride, a.k_row_stride, a.k_head_stride = key_cache.stride(0), key_cache.stride(1), key_cache.stride(2)
    a.v_page_stride, a.v_row_stride, a.v_head_stride = (value_cache.stride(0), value_cache.stride(1),
                                                         value_cache.stride(2))
    a.num_pages = key_cache.shape[0]
    a.num_tokens, a.num_kv_heads, a.head_dim, a.page_size = tokens, heads, dim, key_cache.shape[1]
    a.dtype = _DTYPES[key.dtype]
    with torch.cuda.device(key.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = N.load().pat_b200_append_kv(C.byref(a), C.c_void_p(stream))
    if rc != 0:
        raise RuntimeError(f"reshape_and_cache_flash failed: {N.strerror(rc)} ({rc})")
