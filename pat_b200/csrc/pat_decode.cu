// Host launcher of the decode-attention kernels (C ABI: pat_b200_decode).
//
// Replaces pat::pat_mha_fwd_kvcache (csrc/api.h:110-295: argument checks,
// scratch set-up, one parameter block per tile bucket) and
// pat_run_mha_fwd_splitkv_dispatch (csrc/pat_fwd_launch_template.h:52-98: one
// stream per bucket, gather on the legacy stream).  Here everything runs on the
// caller's stream: streaming items, dense items, then the merge.
#include "../../include/pat_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>

#include "pat_dense_tc.cuh"
#include "pat_kernels.cuh"

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeFn>(sym);
    }();
    return fn;
}

// View of a paged cache [pages, page_size, kv_heads, D] as a 4-D tensor
// (D, kv_heads, page_size, pages) with a [64, 1, 16, 1] box and 128-byte swizzle.
// A decode loop calls with the same two caches step after step, so the last few encoded maps are
// kept per host thread (a map depends only on the values in its key).
struct MapKey {
    const void* base;
    int dt, head_dim, kv_heads, page_size;
    int64_t pages, head_stride, row_stride, page_stride;
    bool operator==(const MapKey& o) const {
        return base == o.base && dt == o.dt && head_dim == o.head_dim && kv_heads == o.kv_heads &&
               page_size == o.page_size && pages == o.pages && head_stride == o.head_stride &&
               row_stride == o.row_stride && page_stride == o.page_stride;
    }
};
constexpr int kMapCache = 4;
struct MapCacheEntry { MapKey key; CUtensorMap map; bool valid; };
thread_local MapCacheEntry g_map_cache[kMapCache];
thread_local int g_map_next = 0;

int make_cache_map(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int head_dim, int kv_heads,
                   int page_size, int64_t pages, int64_t head_stride, int64_t row_stride, int64_t page_stride) {
    const MapKey key{base, static_cast<int>(dt), head_dim, kv_heads, page_size, pages, head_stride, row_stride, page_stride};
    for (const MapCacheEntry& e : g_map_cache)
        if (e.valid && e.key == key) { *map = e.map; return PAT_OK; }
    EncodeFn enc = get_encode_fn();
    if (!enc) return PAT_ERR_CUDA;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(kv_heads),
                                static_cast<cuuint64_t>(page_size), static_cast<cuuint64_t>(pages)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_stride) * 2, static_cast<cuuint64_t>(row_stride) * 2,
                                   static_cast<cuuint64_t>(page_stride) * 2};
    const cuuint32_t box[4] = {64u, 1, 16, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult rc = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return PAT_ERR_CUDA;
    MapCacheEntry& slot = g_map_cache[g_map_next];
    g_map_next = (g_map_next + 1) % kMapCache;
    slot.key = key;
    slot.map = *map;
    slot.valid = true;
    return PAT_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

thread_local int g_last_launches = 0;
constexpr int kMaxDevices = 64;

template <typename T, int D>
int launch_all(const pat_decode_args& a, cudaStream_t stream, int dev) {
    using namespace pat;
    CUtensorMap kmap, vmap;
    int rc = make_cache_map(&kmap, a.k_cache, Elt<T>::kTma, D, a.num_kv_heads, a.page_size, a.num_pages,
                            a.k_head_stride, a.k_row_stride, a.k_page_stride);
    if (rc != PAT_OK) return rc;
    rc = make_cache_map(&vmap, a.v_cache, Elt<T>::kTma, D, a.num_kv_heads, a.page_size, a.num_pages,
                        a.v_head_stride, a.v_row_stride, a.v_page_stride);
    if (rc != PAT_OK) return rc;

    // workspace: control words, then the partial outputs, then the partial LSEs
    const size_t rows = static_cast<size_t>(a.work.num_entries) * a.work.hratio;   // hratio rows per entry
    int32_t* sync_words = static_cast<int32_t*>(a.workspace);
    float* part_o = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + kWorkspaceHeadBytes);
    float* part_lse = part_o + rows * D;

    AttnParams p{};
    p.q = a.q;
    p.part_o = part_o;
    p.part_lse = part_lse;
    p.queries = a.work_blob + a.work.queries_off;
    p.pages = a.work_blob + a.work.pages_off;
    const int q_per_req = a.q_per_req > 1 ? a.q_per_req : 1;
    const bool limits = a.work.limits_off >= 0;
    p.limits = limits ? a.work_blob + a.work.limits_off : nullptr;
    p.q_per_req = q_per_req;
    p.q_batch_stride = a.q_batch_stride;
    p.q_head_stride = a.q_head_stride;
    p.q_pos_stride = q_per_req > 1 ? a.q_pos_stride : 0;
    p.kv_heads = a.num_kv_heads;
    p.hratio = a.work.hratio;
    p.num_q_heads = a.num_q_heads;
    p.page_size = a.page_size;
    p.scale = a.softmax_scale;
    p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
    p.status = a.status_word;
    p.wait_ns = a.wait_limit_us > 0 ? static_cast<uint64_t>(a.wait_limit_us) * 1000ull : kDefaultWaitNs;

    int launches = 0;
    const bool streaming = a.work.num_stream_items > 0 && !(a.flags & PAT_SKIP_STREAM);
    const bool dense = a.work.num_dense_items > 0 && !(a.flags & PAT_SKIP_DENSE);

    // The streaming kernel is bound by HBM, the dense kernel by the tensor and special-function
    // units of the SMs it holds, and it needs few of them when the work list sized it so
    // (num_dense_ctas below the SM count).  So the dense kernel is launched first and the
    // streaming kernel as its programmatic dependent: it may start as soon as every dense CTA is
    // running (each signals that at its top; the streaming kernel never waits for the dense
    // kernel's results), fills the SMs the dense kernel leaves and takes the others over as the
    // dense CTAs retire.  The merge kernel is an ordinary launch: stream order makes it wait for the
    // streaming kernel, and for the dense kernel it waits on a word in the workspace that the last
    // dense CTA sets (every dense CTA is running or done before the streaming kernel may start, so
    // that wait cannot outlast the dense kernel).
    const bool overlap = streaming && dense && !(a.flags & PAT_NO_OVERLAP);
    const bool merge = !(a.flags & PAT_SKIP_MERGE);
    int32_t* sync = (overlap && merge) ? sync_words : nullptr;
    if (dense) {
        // shared segments on tcgen05 / TMEM: persistent CTAs, one per share of the dense work
        static std::atomic<bool> configured[kMaxDevices][2];    // zero-initialised; set once per device
        auto kern = limits ? dense_tc_kernel<T, D, true> : dense_tc_kernel<T, D, false>;
        constexpr int smem = TcSmem<D>::kRequest;
        if (!configured[dev][limits].load(std::memory_order_acquire)) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                return PAT_ERR_CUDA;
            configured[dev][limits].store(true, std::memory_order_release);
        }
        AttnParams pd = p;
        pd.items = a.work_blob + a.work.items_off + static_cast<size_t>(a.work.num_stream_items) * 8;
        pd.num_items = a.work.num_dense_items;
        DenseTcParams dp{};
        dp.a = pd;
        dp.cta_begin = a.work_blob + a.work.dense_cta_off;
        dp.dense_q = a.work_blob + a.work.dense_q_off;
        dp.dense_q_width = a.work.dense_q_width;
        dp.sync = sync;
        kern<<<static_cast<unsigned>(a.work.num_dense_ctas), kTcThreads, smem, stream>>>(dp, kmap, vmap);
        ++launches;
    }
    if (streaming) {
        static std::atomic<bool> configured[kMaxDevices][2];    // zero-initialised; set once per device
        auto kern = limits ? stream_kernel<T, D, true> : stream_kernel<T, D, false>;
        constexpr int smem = stream_smem_bytes<D>();
        if (!configured[dev][limits].load(std::memory_order_acquire)) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                return PAT_ERR_CUDA;
            configured[dev][limits].store(true, std::memory_order_release);
        }
        p.items = a.work_blob + a.work.items_off;
        p.num_items = a.work.num_stream_items;
        const long long grid = static_cast<long long>(p.num_items) * a.num_kv_heads;
        if (grid > 0x7fffffffLL) return PAT_ERR_TOO_LARGE;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(grid));
        cfg.blockDim = dim3(kStreamWarps * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = overlap ? 1 : 0;
        if (cudaLaunchKernelEx(&cfg, kern, p, kmap, vmap) != cudaSuccess) return PAT_ERR_CUDA;
        ++launches;
    }
    if (merge) {
        MergeParams mp{};
        mp.sync = sync;
        mp.status = a.status_word;
        mp.wait_ns = p.wait_ns;
        mp.part_o = part_o;
        mp.part_lse = part_lse;
        mp.indptr = a.work_blob + a.work.merge_indptr_off;
        mp.entries = a.work_blob + a.work.merge_entries_off;
        mp.out = a.out;
        mp.lse_out = a.lse_out;
        mp.out_batch_stride = a.out_batch_stride;
        mp.out_head_stride = a.out_head_stride;
        mp.out_pos_stride = q_per_req > 1 ? a.out_pos_stride : 0;
        mp.q_per_req = q_per_req;
        mp.batch = a.batch * q_per_req;
        mp.num_q_heads = a.num_q_heads;
        mp.kv_heads = a.num_kv_heads;
        mp.hratio = a.work.hratio;
        const int total = a.batch * q_per_req * a.num_q_heads;
        const int warps_per_cta = 8;
        merge_kernel<T, D><<<(total + warps_per_cta - 1) / warps_per_cta, warps_per_cta * 32, 0, stream>>>(mp);
        ++launches;
    }
    if (cudaGetLastError() != cudaSuccess) return PAT_ERR_CUDA;
    g_last_launches = launches;
    return PAT_OK;
}

}  // namespace

extern "C" {

size_t pat_b200_workspace_bytes(const pat_work_header* work, int num_q_heads, int head_dim) {
    if (!work || num_q_heads <= 0 || head_dim <= 0) return 0;
    (void)num_q_heads;
    // one entry = hratio rows (the query heads of one KV head): partial outputs + partial LSEs
    const size_t rows = static_cast<size_t>(work->num_entries) * static_cast<size_t>(work->hratio);
    const size_t bytes = rows * (static_cast<size_t>(head_dim) + 1) * sizeof(float);
    return pat::kWorkspaceHeadBytes + (bytes + 255) / 256 * 256;
}

int pat_b200_last_launch_count(void) { return g_last_launches; }

int pat_b200_decode(const pat_decode_args* args, void* stream_handle) {
    if (!args) return PAT_ERR_BAD_ARGUMENT;
    const pat_decode_args& a = *args;
    if (!a.q || !a.k_cache || !a.v_cache || !a.out || !a.work_blob) return PAT_ERR_BAD_ARGUMENT;
    if (a.batch <= 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0 || a.num_pages <= 0) return PAT_ERR_BAD_ARGUMENT;
    if (a.num_q_heads % a.num_kv_heads != 0) return PAT_ERR_BAD_ARGUMENT;
    const int positions = a.q_per_req > 1 ? a.q_per_req : 1;
    if (a.work.q_per_req != positions || static_cast<int64_t>(a.work.batch) != static_cast<int64_t>(a.batch) * positions)
        return PAT_ERR_BAD_PLAN;
    if (positions > 1 && (a.q_pos_stride <= 0 || a.q_pos_stride % 8 != 0 || a.out_pos_stride <= 0 || a.out_pos_stride % 8 != 0))
        return PAT_ERR_UNSUPPORTED;
    if (a.work.hratio != a.num_q_heads / a.num_kv_heads ||
        a.work.page_size != a.page_size || a.work.kv_heads != a.num_kv_heads)
        return PAT_ERR_BAD_PLAN;
    if (a.work.max_page_id >= a.num_pages) return PAT_ERR_BAD_PLAN;
    if (a.head_dim != 64 && a.head_dim != 128) return PAT_ERR_UNSUPPORTED;
    if (a.dtype != PAT_DTYPE_FP16 && a.dtype != PAT_DTYPE_BF16) return PAT_ERR_UNSUPPORTED;
    if (a.page_size < 16 || a.page_size % 16 != 0 || a.page_size > 256) return PAT_ERR_UNSUPPORTED;
    if (a.work.hratio < 1 || a.work.hratio > 16) return PAT_ERR_UNSUPPORTED;
    if (!(a.softmax_scale > 0.f) || !std::isfinite(a.softmax_scale)) return PAT_ERR_BAD_ARGUMENT;
    // TMA: 16-byte aligned bases and strides; Q/O rows are read and written with vector accesses
    if (!aligned16(a.k_cache) || !aligned16(a.v_cache) || !aligned16(a.q) || !aligned16(a.out))
        return PAT_ERR_UNSUPPORTED;
    const int64_t strides[] = {a.k_page_stride, a.k_row_stride, a.k_head_stride, a.v_page_stride, a.v_row_stride,
                               a.v_head_stride, a.q_batch_stride, a.q_head_stride, a.out_batch_stride,
                               a.out_head_stride};
    for (int64_t s : strides)
        if (s <= 0 || s % 8 != 0) return PAT_ERR_UNSUPPORTED;
    if (!aligned16(a.work_blob)) return PAT_ERR_BAD_ARGUMENT;
    const size_t need = pat_b200_workspace_bytes(&a.work, a.num_q_heads, a.head_dim);
    // the dense kernel writes its partial rows with 32-byte stores
    if (!a.workspace || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 31) != 0)
        return PAT_ERR_WORKSPACE;

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PAT_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return PAT_ERR_UNSUPPORTED;
    static thread_local int checked_dev = -1;
    if (checked_dev != dev) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return PAT_ERR_CUDA;
        if (major != 10) return PAT_ERR_NO_DEVICE_CODE;
        checked_dev = dev;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    const bool bf16 = a.dtype == PAT_DTYPE_BF16;
    if (a.head_dim == 128)
        return bf16 ? launch_all<__nv_bfloat16, 128>(a, stream, dev) : launch_all<__half, 128>(a, stream, dev);
    return bf16 ? launch_all<__nv_bfloat16, 64>(a, stream, dev) : launch_all<__half, 64>(a, stream, dev);
}

}  // extern "C"

// ------------------------------------------------------------------------------
// Decode without any allocation: the partial results live in a fixed device array.
// ------------------------------------------------------------------------------
// Scratch for pat_b200_decode_static_scratch.  It is part of the module image, so every GPU
// that loads this library holds PAT_B200_STATIC_SCRATCH_BYTES of it until the process exits.
static __device__ __align__(256) unsigned char g_pat_static_scratch[PAT_B200_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_pat_static_scratch per device.  In host code the array's name is only a
// handle for the runtime, never a device pointer: the address has to be asked for, once per
// device, while that device is current.
std::atomic<void*> g_static_scratch_ptr[kMaxDevices];
}  // namespace

extern "C" int pat_b200_decode_static_scratch(const pat_decode_args* args, void* stream_handle) {
    if (!args) return PAT_ERR_BAD_ARGUMENT;
    if (args->num_q_heads <= 0 || args->head_dim <= 0 || args->work.num_entries < 0) return PAT_ERR_BAD_ARGUMENT;
    const size_t need = pat_b200_workspace_bytes(&args->work, args->num_q_heads, args->head_dim);
    if (need > static_cast<size_t>(PAT_B200_STATIC_SCRATCH_BYTES)) return PAT_ERR_TOO_LARGE;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PAT_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return PAT_ERR_UNSUPPORTED;
    void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        // first call on this device (which is current): resolve the symbol's device address
        if (cudaGetSymbolAddress(&ptr, g_pat_static_scratch) != cudaSuccess || !ptr) return PAT_ERR_CUDA;
        g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    pat_decode_args local = *args;
    local.workspace = ptr;
    local.workspace_bytes = PAT_B200_STATIC_SCRATCH_BYTES;
    return pat_b200_decode(&local, stream_handle);
}

// ------------------------------------------------------------------------------
// Self-test of the bounded wait
// ------------------------------------------------------------------------------
namespace {
// One thread waits on an mbarrier that nobody ever arrives on, with nothing asynchronous in
// flight: the wait must run out after `limit_ns`, report through the status word and return.
__global__ void selftest_wait_kernel(int32_t* status, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        pat::mbar_init(pat::smem_u32(&bar), 1);
        pat::mbar_fence_init();
        const uint64_t t0 = pat::global_timer_ns();
        const bool ok = pat::mbar_wait(pat::smem_u32(&bar), 0, limit_ns);
        const uint64_t waited = pat::global_timer_ns() - t0;
        status[0] = ok ? 0 : 99;
        status[1] = static_cast<int32_t>(waited > 0x7fffffffull ? 0x7fffffffull : waited);
    }
}
}  // namespace

extern "C" int pat_b200_selftest_wait(int32_t limit_us, int32_t* status_word, void* stream_handle) {
    if (!status_word || limit_us <= 0 || limit_us > 1000000) return PAT_ERR_BAD_ARGUMENT;
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_handle)>>>(
        status_word, static_cast<uint64_t>(limit_us) * 1000ull);
    return cudaGetLastError() == cudaSuccess ? PAT_OK : PAT_ERR_CUDA;
}
