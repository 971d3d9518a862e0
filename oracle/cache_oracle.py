"""CPU restatement of the KV-cache append.  TEST INFRASTRUCTURE ONLY: nothing in the product
imports this file.

The reference's serving backend appends through vLLM's ``reshape_and_cache_flash``
(``plugin/vllm/attention/backends/prefix_attn.py:828-837``); the op itself lives in vLLM
(v0.9.0, ``csrc/cache_kernels.cu``), a dependency that is not part of the reference checkout.  Its
published behaviour for 16-bit caches, restated here: for every token ``i`` with
``slot = slot_mapping[i] >= 0``, ``key_cache[slot // block_size, slot % block_size] = key[i]``
and the same for the values; tokens with a negative slot are padding and are skipped.

Pinning: ``tests/test_gpu_cache_append.py`` compares this restatement with vLLM's own op on the
GPU wherever ``vllm._custom_ops`` loads (the image ships vLLM); where it does not, parity of the
append is unpinned beyond the restated definition.
"""
import torch


def reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping):
    """In place, on CPU tensors of any dtype."""
    page_size = key_cache.shape[1]
    for i, slot in enumerate(slot_mapping.flatten().tolist()):
        if i >= key.shape[0]:
            break
        if slot < 0:
            continue
        page, row = divmod(int(slot), page_size)
        key_cache[page, row] = key[i]
        value_cache[page, row] = value[i]
