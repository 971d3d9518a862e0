// KV-cache append: the step right before decode attention in a serving loop.
//
// Writes the new tokens' K and V rows into the paged caches at the slots the engine assigned
// (slot = page * page_size + row; a negative slot is a padding token and is skipped).  In the
// reference this is vLLM's op reshape_and_cache_flash, called from
// plugin/vllm/attention/backends/prefix_attn.py:828-837.  16-bit caches only (kv_cache_dtype
// "auto"): rows are copied bit for bit, 16 bytes per thread and access.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/pat_b200.h"

namespace {

struct AppendParams {
    const uint4* key;
    const uint4* value;
    uint4* k_cache;
    uint4* v_cache;
    const int64_t* slots;
    // strides in 16-byte units
    int64_t key_token, key_head, value_token, value_head;
    int64_t k_page, k_row, k_head, v_page, v_row, v_head;
    int64_t num_slots;       // num_pages * page_size
    int num_tokens, heads, vec_per_head, page_size;
};

// One CTA per token; thread i copies 16-byte piece i, i + blockDim.x, ... of the token's
// 2 * heads * vec_per_head pieces (K first, then V).
__global__ void __launch_bounds__(128) append_kv_kernel(const AppendParams p) {
    const int token = blockIdx.x;
    const int64_t slot = __ldg(p.slots + token);
    if (slot < 0 || slot >= p.num_slots) return;        // padding token (or a slot outside the cache)
    const int64_t page = slot / p.page_size, row = slot - page * p.page_size;
    const int per_tensor = p.heads * p.vec_per_head;
    for (int i = threadIdx.x; i < 2 * per_tensor; i += blockDim.x) {
        const bool is_v = i >= per_tensor;
        const int j = is_v ? i - per_tensor : i;
        const int h = j / p.vec_per_head, c = j - h * p.vec_per_head;
        if (!is_v)
            p.k_cache[page * p.k_page + row * p.k_row + h * p.k_head + c] =
                __ldg(p.key + token * p.key_token + h * p.key_head + c);
        else
            p.v_cache[page * p.v_page + row * p.v_row + h * p.v_head + c] =
                __ldg(p.value + token * p.value_token + h * p.value_head + c);
    }
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

}  // namespace

extern "C" int pat_b200_append_kv(const pat_append_args* args, void* stream_handle) {
    if (!args) return PAT_ERR_BAD_ARGUMENT;
    const pat_append_args& a = *args;
    if (a.num_tokens < 0 || a.num_kv_heads <= 0 || a.num_pages <= 0) return PAT_ERR_BAD_ARGUMENT;
    if (a.num_tokens == 0) return PAT_OK;
    if (!a.key || !a.value || !a.k_cache || !a.v_cache || !a.slot_mapping) return PAT_ERR_BAD_ARGUMENT;
    if (a.dtype != PAT_DTYPE_FP16 && a.dtype != PAT_DTYPE_BF16) return PAT_ERR_UNSUPPORTED;
    if (a.head_dim <= 0 || a.head_dim % 8 != 0 || a.page_size <= 0) return PAT_ERR_UNSUPPORTED;
    if (!aligned16(a.key) || !aligned16(a.value) || !aligned16(a.k_cache) || !aligned16(a.v_cache))
        return PAT_ERR_UNSUPPORTED;
    const int64_t strides[] = {a.key_token_stride, a.key_head_stride, a.value_token_stride, a.value_head_stride,
                               a.k_page_stride, a.k_row_stride, a.k_head_stride,
                               a.v_page_stride, a.v_row_stride, a.v_head_stride};
    for (int64_t s : strides)
        if (s <= 0 || s % 8 != 0) return PAT_ERR_UNSUPPORTED;     // 16-byte pieces
    AppendParams p{};
    p.key = static_cast<const uint4*>(a.key);
    p.value = static_cast<const uint4*>(a.value);
    p.k_cache = static_cast<uint4*>(a.k_cache);
    p.v_cache = static_cast<uint4*>(a.v_cache);
    p.slots = a.slot_mapping;
    p.key_token = a.key_token_stride / 8;
    p.key_head = a.key_head_stride / 8;
    p.value_token = a.value_token_stride / 8;
    p.value_head = a.value_head_stride / 8;
    p.k_page = a.k_page_stride / 8;
    p.k_row = a.k_row_stride / 8;
    p.k_head = a.k_head_stride / 8;
    p.v_page = a.v_page_stride / 8;
    p.v_row = a.v_row_stride / 8;
    p.v_head = a.v_head_stride / 8;
    p.num_slots = a.num_pages * static_cast<int64_t>(a.page_size);
    p.num_tokens = a.num_tokens;
    p.heads = a.num_kv_heads;
    p.vec_per_head = a.head_dim / 8;
    p.page_size = a.page_size;
    append_kv_kernel<<<static_cast<unsigned>(a.num_tokens), 128, 0, static_cast<cudaStream_t>(stream_handle)>>>(p);
    return cudaGetLastError() == cudaSuccess ? PAT_OK : PAT_ERR_CUDA;
}
