"""Attention backend for vLLM's V1 engine (the ``vllm.v1.attention.backend`` interface).

The reference ships a backend for vLLM v0.9.0's V0 engine
(``plugin/vllm/attention/backends/prefix_attn.py``: ``PrefixAttnBackend`` :76-95,
``PrefixAttnMetadata`` :137, ``PrefixAttnMetadataBuilder`` :451, ``PrefixAttnImpl`` :689).  Current
vLLM releases only have the V1 engine, whose backends are built from per-step
``CommonAttentionMetadata`` by an ``AttentionMetadataBuilder`` and called through
``AttentionImpl.forward(layer, query, key, value, kv_cache, attn_metadata, output)``.  This module
is the same backend for that interface:

* the builder keeps one ``DecodePlanner`` per uniform query length: a step whose requests all carry
  the same number of query tokens (1 = decode, a few = speculative decoding) gets its radix tree
  and device work list from the previous step's, grown in place, instead of a rebuild - the
  reference rebuilds every step on a worker thread (``:318-340``) and leaves the plan stale during
  multi-step decode (``:430-438``);
* ``forward`` runs such steps through ``prefix_attn_with_kvcache``; any other step (prefill,
  mixed batches) goes to vLLM's own flash-attention, as in the reference (``:877-898``);
* the KV-cache append before attention is this library's kernel (the reference calls vLLM's
  ``reshape_and_cache_flash``, ``:828-837``).

Register it with::

    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    register_backend(AttentionBackendEnum.CUSTOM, "pat_b200.vllm_v1.PrefixAttnBackend")

vLLM is imported when this module is; nothing else in the package needs it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Dict, Optional

import torch

from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadata,
                                       AttentionMetadataBuilder, AttentionType, CommonAttentionMetadata,
                                       MultipleOf)

from ._prefix_attn import PrefixTreeCPP, prefix_attn_with_kvcache
from .cache_ops import reshape_and_cache_flash
from .planner import DecodePlanner

MAX_UNIFORM_QUERY_LEN = 8       # steps with more query tokens per request count as prefill


class PrefixAttnBackend(AttentionBackend):
    accept_output_buffer: bool = True
    forward_includes_kv_cache_update: bool = False
    supported_dtypes: ClassVar[list] = [torch.float16, torch.bfloat16]
    supported_kv_cache_dtypes: ClassVar[list] = ["auto", "float16", "bfloat16"]

    @staticmethod
    def get_name() -> str:
        return "PREFIX_ATTN"

    @staticmethod
    def get_impl_cls():
        return PrefixAttnImpl

    @staticmethod
    def get_builder_cls():
        return PrefixAttnMetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes():
        return [MultipleOf(16)]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto"):
        if block_size % 16 != 0:
            raise ValueError("Block size must be a multiple of 16.")
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @classmethod
    def get_supported_head_sizes(cls):
        return [64, 128]

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return getattr(capability, "major", None) == 10        # sm_100 device code only

    @classmethod
    def supports_attn_type(cls, attn_type: str) -> bool:
        return attn_type == AttentionType.DECODER


@dataclass
class PrefixAttnMetadata(AttentionMetadata):
    num_actual_tokens: int
    num_reqs: int
    query_len: int                      # tokens per request when uniform and small, else 0
    tree: Optional[PrefixTreeCPP]       # plan of the step when query_len > 0
    max_query_len: int
    max_seq_len: int
    query_start_loc: torch.Tensor
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    causal: bool = True


class PrefixAttnMetadataBuilder(AttentionMetadataBuilder[PrefixAttnMetadata]):
    # The work list changes shape when the batch does, so full-graph capture of the attention is
    # not offered; an in-place step keeps blob address and item counts (see DeviceWork.refresh).
    _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.NEVER
    reorder_batch_threshold = None

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        model, parallel = vllm_config.model_config, vllm_config.parallel_config
        self.num_heads_q = model.get_num_attention_heads(parallel)
        self.num_heads_kv = model.get_num_kv_heads(parallel)
        self.block_size = kv_cache_spec.block_size
        self._planners: Dict[int, DecodePlanner] = {}

    def _planner(self, query_len: int) -> DecodePlanner:
        pl = self._planners.get(query_len)
        if pl is None:
            pl = DecodePlanner(self.block_size, self.num_heads_q // self.num_heads_kv, self.num_heads_kv, self.device)
            self._planners[query_len] = pl
        return pl

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> PrefixAttnMetadata:
        m = common_attn_metadata
        n = m.num_reqs
        qsl = m.query_start_loc_cpu[: n + 1]
        lens_q = qsl[1:] - qsl[:-1]
        first = int(lens_q[0]) if n > 0 else 0
        uniform = n > 0 and 1 <= first <= MAX_UNIFORM_QUERY_LEN and bool((lens_q == first).all()) and m.causal
        tree = None
        if uniform:
            seq_lens = getattr(m, "_seq_lens_cpu", None)
            if seq_lens is None:
                seq_lens = m.seq_lens[:n].cpu()
            seq_lens = seq_lens[:n].to(torch.int32)
            width = -(-int(seq_lens.max()) // self.block_size)
            table = m.block_table_tensor[:n, :width].to("cpu", torch.int32).contiguous()
            tree = self._planner(first).step(seq_lens, table)
        return PrefixAttnMetadata(num_actual_tokens=m.num_actual_tokens, num_reqs=n,
                                  query_len=first if uniform else 0, tree=tree,
                                  max_query_len=m.max_query_len, max_seq_len=m.max_seq_len,
                                  query_start_loc=m.query_start_loc, seq_lens=m.seq_lens,
                                  block_table=m.block_table_tensor, slot_mapping=m.slot_mapping, causal=m.causal)


class PrefixAttnImpl(AttentionImpl[PrefixAttnMetadata]):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes=None, sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None,
                 attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name=None, **_ignored) -> None:
        if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
            raise NotImplementedError("PREFIX_ATTN supports neither ALiBi, sliding windows nor logit soft caps")
        if kv_cache_dtype not in ("auto", "float16", "bfloat16"):
            raise NotImplementedError("PREFIX_ATTN needs a 16-bit KV cache")
        if attn_type != AttentionType.DECODER:
            raise NotImplementedError("PREFIX_ATTN implements decoder self-attention only")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.kv_cache_dtype = kv_cache_dtype
        self.attn_type = attn_type
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name

    def do_kv_cache_update(self, layer, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                           slot_mapping: torch.Tensor) -> None:
        key_cache, value_cache = kv_cache.unbind(0)
        n = slot_mapping.shape[0]       # key / value may be padded beyond the real tokens
        reshape_and_cache_flash(key[:n], value[:n], key_cache, value_cache, slot_mapping)

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                attn_metadata: Optional[PrefixAttnMetadata], output: torch.Tensor, output_scale=None,
                output_block_scale=None) -> torch.Tensor:
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not supported by PREFIX_ATTN")
        if attn_metadata is None:       # profiling run
            return output.fill_(0)
        md = attn_metadata
        n = md.num_actual_tokens
        key_cache, value_cache = kv_cache.unbind(0)
        q = query[:n].view(-1, self.num_heads, self.head_size)
        out = output[:n].view(-1, self.num_heads, self.head_size)
        if md.tree is not None:
            t = md.query_len
            prefix_attn_with_kvcache(q.view(md.num_reqs, t, self.num_heads, self.head_size), key_cache, value_cache,
                                     md.tree, self.scale, out.view(md.num_reqs, t, self.num_heads, self.head_size))
            return output
        # prefill and mixed steps: vLLM's flash-attention over the same paged cache
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func
        flash_attn_varlen_func(q=q, k=key_cache, v=value_cache, out=out, cu_seqlens_q=md.query_start_loc,
                               max_seqlen_q=md.max_query_len, seqused_k=md.seq_lens, max_seqlen_k=md.max_seq_len,
                               softmax_scale=self.scale, causal=md.causal, block_table=md.block_table)
        return output
