// Head reorder after the optional all-gather of a KV-head-sharded decode step.
//
// An all-gather hands every rank the other ranks' outputs rank by rank: [world][batch][H/world][D].
// Callers want [batch][1][H][D] with the heads in rank order.  This is that permutation, 16 bytes
// per thread and access.  (The reference has no multi-GPU path of its own; a tensor-parallel
// vLLM gives its backend per-rank head counts, plugin/vllm/attention/backends/prefix_attn.py:617-618,
// and never gathers.)
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/pat_b200.h"

namespace {

__global__ void __launch_bounds__(256)
reorder_heads_kernel(const uint4* __restrict__ staged, uint4* __restrict__ full, int world, int batch,
                     int vec_per_rank_row /* (H/world) * D * elt / 16 */, int64_t total) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // i indexes the destination: [batch][world][vec_per_rank_row]
        const int c = static_cast<int>(i % vec_per_rank_row);
        const int64_t br = i / vec_per_rank_row;
        const int r = static_cast<int>(br % world);
        const int64_t b = br / world;
        full[i] = __ldg(staged + (static_cast<int64_t>(r) * batch + b) * vec_per_rank_row + c);
    }
}

}  // namespace

extern "C" int pat_b200_reorder_heads(const void* staged, void* full, int world, int batch, int heads_per_rank,
                                      int head_dim, void* stream_handle) {
    if (!staged || !full || world <= 0 || batch <= 0 || heads_per_rank <= 0 || head_dim <= 0)
        return PAT_ERR_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(staged) & 15) || (reinterpret_cast<uintptr_t>(full) & 15) || head_dim % 8 != 0)
        return PAT_ERR_UNSUPPORTED;
    const int vec = heads_per_rank * head_dim / 8;       // 16-bit elements, 8 per 16 bytes
    const int64_t total = static_cast<int64_t>(batch) * world * vec;
    const int64_t want = (total + 255) / 256;
    const unsigned grid = static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8);
    reorder_heads_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_handle)>>>(
        static_cast<const uint4*>(staged), static_cast<uint4*>(full), world, batch, vec, total);
    return cudaGetLastError() == cudaSuccess ? PAT_OK : PAT_ERR_CUDA;
}
