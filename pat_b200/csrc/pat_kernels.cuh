// Attention kernels of the decode path (sm_100a): streaming tiles, dense tiles
// and the log-sum-exp merge.
//
// Work items are produced on the host (pat_work.h).  One CTA = one item x one
// KV head; blockIdx.x = item * kv_heads + kv_head, so the KV heads of an item
// (which touch the same pages, 256 B apart) run next to each other.
//
//   stream_kernel : <= 16 query rows (the GQA group of 1-2 requests).  HBM-bound.
//                   Every warp owns a private multi-stage TMA pipeline over its
//                   share of the item's 16-token sub-tiles - no CTA-wide barrier
//                   in the main loop - and the warps' partial softmax states are
//                   combined through shared memory at the end.
//   (segments that many queries share run in dense_tc_kernel, pat_dense_tc.cuh)
//   merge_kernel  : one warp per (request, head): out = sum_i e^(lse_i-lse) O_i.
//
// All kernels replace csrc/pat_fwd_kernel.h (pat_kernel :25-299, gather_kernel
// :314-467) of the reference.
#pragma once

#include "pat_device.cuh"
#include "pat_work.h"

namespace pat {

struct AttnParams {
    const void* q;
    float* part_o;        // [entries, H, D]
    float* part_lse;      // [entries, H]
    const int32_t* items;     // WorkItem[...]
    const int32_t* queries;
    const int32_t* pages;
    // Several query tokens per request: a query id is request * q_per_req + position, and
    // `limits` (parallel to `queries`, or null) holds how many tokens of its segment each query sees.
    const int32_t* limits;
    int64_t q_batch_stride, q_head_stride, q_pos_stride;
    int q_per_req;
    int num_items;
    int kv_heads;
    int hratio;
    int num_q_heads;
    int page_size;
    float scale;          // softmax scale
    float scale_log2;     // scale * log2(e)
    int32_t* status;      // optional
    uint64_t wait_ns;     // limit of every mbarrier wait
};

// 3 warps x 2 stages of 8 KB (D = 128): 49 KB per CTA, four CTAs and 192 KB of loads in flight per
// SM, twelve warps (the register file allows no more).  Measured against 3 x 3 (three CTAs per SM),
// 4 x 2, 2 x 2, 2 x 3, 5 x 2 and 6 x 2: this shape gave the shortest decode step on every workload.
constexpr int kStreamWarps = 3;
constexpr int kStreamStages = 2;
constexpr int kScratchPad = 8;          // floats of padding per scratch row

template <int D> constexpr int stream_smem_bytes() {
    return kStreamWarps * kStreamStages * TileGeom<D>::kSubBytes + 1024;
}

// Address of the Q row of query id `vq` (request * q_per_req + position) and query head `head`.
template <typename T>
__device__ __forceinline__ const T* q_row_ptr(const AttnParams& p, int vq, int head) {
    const int req = p.q_per_req == 1 ? vq : vq / p.q_per_req;
    const int pos = vq - req * p.q_per_req;
    return static_cast<const T*>(p.q) + static_cast<int64_t>(req) * p.q_batch_stride +
           static_cast<int64_t>(pos) * p.q_pos_stride + static_cast<int64_t>(head) * p.q_head_stride;
}

// Tokens of an item (first token tok_lo of its segment, kv_len tokens) that query slot `slot`
// of the query section may see.
__device__ __forceinline__ int visible_tokens(const AttnParams& p, int slot, int tok_lo, int kv_len) {
    return max(0, min(kv_len, __ldg(p.limits + slot) - tok_lo));
}

// Q rows of one 16-row tile straight into mma A fragments.
template <typename T, int D>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[D / 16][4], const AttnParams& p, const int32_t* qids,
                                             int row_base, int rows_valid, int kvh, int lane) {
    const int r0 = row_base + (lane >> 2), r1 = r0 + 8;
    const T* p0 = nullptr;
    const T* p1 = nullptr;
    if (r0 < rows_valid) {
        const int qi = r0 / p.hratio, g = r0 - qi * p.hratio;
        p0 = q_row_ptr<T>(p, __ldg(qids + qi), kvh * p.hratio + g);
    }
    if (r1 < rows_valid) {
        const int qi = r1 / p.hratio, g = r1 - qi * p.hratio;
        p1 = q_row_ptr<T>(p, __ldg(qids + qi), kvh * p.hratio + g);
    }
    const int col = (lane & 3) << 1;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = p0 ? __ldg(reinterpret_cast<const uint32_t*>(p0 + ks * 16 + col)) : 0u;
        qf[ks][1] = p1 ? __ldg(reinterpret_cast<const uint32_t*>(p1 + ks * 16 + col)) : 0u;
        qf[ks][2] = p0 ? __ldg(reinterpret_cast<const uint32_t*>(p0 + ks * 16 + 8 + col)) : 0u;
        qf[ks][3] = p1 ? __ldg(reinterpret_cast<const uint32_t*>(p1 + ks * 16 + 8 + col)) : 0u;
    }
}

// ------------------------------------------------------------------------------
// Streaming kernel
// ------------------------------------------------------------------------------
template <typename T, int D, bool kLimits>
__global__ void __launch_bounds__(kStreamWarps * 32)
stream_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using G = TileGeom<D>;
    constexpr int W = kStreamWarps, S = kStreamStages;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t bars[W * S];
    __shared__ float sm_m[W][16], sm_l[W][16];
    __shared__ int sm_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item_idx = blockIdx.x / p.kv_heads;
    const int kvh = blockIdx.x - item_idx * p.kv_heads;
    const int32_t* it = p.items + static_cast<size_t>(item_idx) * 8;
    const int q_off = __ldg(it + 0), nq = __ldg(it + 1), page_off = __ldg(it + 2), kv_len = __ldg(it + 3),
              entry_base = __ldg(it + 4);
    const int rows_valid = nq * p.hratio;
    // tokens of this item the thread's two rows (lane / 4 and lane / 4 + 8) may see
    int lim0 = kv_len, lim1 = kv_len;
    if constexpr (kLimits) {
        const int tok_lo = __ldg(it + 7);
        const int r0 = lane >> 2, r1 = r0 + 8;
        lim0 = r0 < rows_valid ? visible_tokens(p, q_off + r0 / p.hratio, tok_lo, kv_len) : 0;
        lim1 = r1 < rows_valid ? visible_tokens(p, q_off + r1 / p.hratio, tok_lo, kv_len) : 0;
    }

    if (tid == 0) {
        sm_abort = 0;
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        for (int i = 0; i < W * S; ++i) mbar_init(smem_u32(&bars[i]), 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int n_tiles = (kv_len + 15) >> 4;
    const int my_n = warp < n_tiles ? (n_tiles - warp + W - 1) / W : 0;
    const int tiles_per_page = p.page_size >> 4;
    unsigned char* my_stage = smem + static_cast<size_t>(warp) * S * G::kSubBytes;
    const uint32_t my_stage_addr = smem_u32(my_stage);
    const uint32_t my_bar = smem_u32(&bars[warp * S]);
    const int32_t* item_pages = p.pages + page_off;

    // page ids of my next 32 tiles, one per lane
    auto fetch_ids = [&](int jbase) -> int {
        const int j = jbase + lane;
        if (j >= my_n) return 0;
        const int t = warp + j * W;
        return __ldg(item_pages + t / tiles_per_page);
    };
    int ids_cur = fetch_ids(0);
    int ids_next = fetch_ids(32);

    auto issue = [&](int j, int page) {   // lane 0 only
        const int t = warp + j * W;
        const int row0 = (t % tiles_per_page) << 4;
        const int s = j % S;
        const uint32_t bar = my_bar + s * 8;
        const uint32_t dst = my_stage_addr + s * G::kSubBytes;
        mbar_expect_tx(bar, G::kSubBytes);
#pragma unroll
        for (int b = 0; b < G::kBoxes; ++b) {
            tma_load_4d(dst + b * 2048, &kmap, bar, b * 64, kvh, row0, page);
            tma_load_4d(dst + G::kOperandBytes + b * 2048, &vmap, bar, b * 64, kvh, row0, page);
        }
    };

#pragma unroll
    for (int j = 0; j < S; ++j) {
        const int page = __shfl_sync(kFullMask, ids_cur, j);
        if (j < my_n && lane == 0) issue(j, page);
    }

    uint32_t qf[D / 16][4];
    load_q_frags<T, D>(qf, p, p.queries + q_off, 0, rows_valid, kvh, lane);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    bool ok = true;

    for (int j = 0; j < my_n; ++j) {
        const int s = j % S;
        if (!mbar_wait(my_bar + s * 8, (j / S) & 1, p.wait_ns)) {
            // Give up: no further load is issued.  Tiles j .. j + S - 1 may still be on their way
            // into this warp's stages; give each a short second wait so that none lands after
            // the CTA has gone.
            ok = false;
            for (int jj = j; jj < min(j + S, my_n); ++jj) mbar_wait(my_bar + (jj % S) * 8, (jj / S) & 1, kDrainWaitNs);
            break;
        }
        const int t = warp + j * W;
        const int valid = min(16, kv_len - (t << 4));
        if (valid < 16) {
            zero_v_tail<D>(my_stage + s * G::kSubBytes, 0, valid, lane);
            __syncwarp();
        }
        warp_attend_tile<T, D, 1, kLimits>(qf, o, m, l, my_stage_addr + s * G::kSubBytes,
                                            kLimits ? min(valid, lim0 - (t << 4)) : valid,
                                            kLimits ? min(valid, lim1 - (t << 4)) : valid, p.scale_log2, lane);
        __syncwarp();
        const int jn = j + S;
        if ((jn & 31) == 0) { ids_cur = ids_next; ids_next = fetch_ids(jn + 32); }
        const int page = __shfl_sync(kFullMask, ids_cur, jn & 31);
        if (jn < my_n && lane == 0) issue(jn, page);
    }
    if (!ok) {
        if (lane == 0) { sm_abort = 1; if (p.status) atomicExch(p.status, 1); }
    }

    // ---- combine the warps' partial states --------------------------------------
    l[0] += __shfl_xor_sync(kFullMask, l[0], 1);
    l[0] += __shfl_xor_sync(kFullMask, l[0], 2);
    l[1] += __shfl_xor_sync(kFullMask, l[1], 1);
    l[1] += __shfl_xor_sync(kFullMask, l[1], 2);
    if ((lane & 3) == 0) {
        sm_m[warp][lane >> 2] = m[0];
        sm_m[warp][(lane >> 2) + 8] = m[1];
        sm_l[warp][lane >> 2] = l[0];
        sm_l[warp][(lane >> 2) + 8] = l[1];
    }
    __syncthreads();   // every warp is done with its pipeline memory
    if (!sm_abort) {
        constexpr int kRowStride = D + kScratchPad;
        float* scratch = reinterpret_cast<float*>(smem);     // [W][16][D + pad]
        {
            const int r0 = lane >> 2, r1 = r0 + 8;
            float g0 = -INFINITY, g1 = -INFINITY;
#pragma unroll
            for (int w = 0; w < W; ++w) { g0 = fmaxf(g0, sm_m[w][r0]); g1 = fmaxf(g1, sm_m[w][r1]); }
            const float f0 = (m[0] == -INFINITY) ? 0.f : fast_exp2((m[0] - g0) * p.scale_log2);
            const float f1 = (m[1] == -INFINITY) ? 0.f : fast_exp2((m[1] - g1) * p.scale_log2);
            float* base = scratch + static_cast<size_t>(warp) * 16 * kRowStride;
            const int col = (lane & 3) << 1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                *reinterpret_cast<float2*>(base + r0 * kRowStride + i * 8 + col) = make_float2(o[i][0] * f0, o[i][1] * f0);
                *reinterpret_cast<float2*>(base + r1 * kRowStride + i * 8 + col) = make_float2(o[i][2] * f1, o[i][3] * f1);
            }
        }
        __syncthreads();

        constexpr int kVec = D / 4;   // float4 per row
        for (int idx = tid; idx < rows_valid * kVec; idx += W * 32) {
            const int row = idx / kVec, v4 = idx - row * kVec;
            float g = -INFINITY;
#pragma unroll
            for (int w = 0; w < W; ++w) g = fmaxf(g, sm_m[w][row]);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const float mw = sm_m[w][row];
                const float f = (mw == -INFINITY) ? 0.f : fast_exp2((mw - g) * p.scale_log2);
                L += sm_l[w][row] * f;
                const float4 x = *reinterpret_cast<const float4*>(scratch + (static_cast<size_t>(w) * 16 + row) * kRowStride + v4 * 4);
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
            }
            const float inv = (!kLimits || L > 0.f) ? 1.f / L : 0.f;    // a row that sees none of the item's tokens
            const int qi = row / p.hratio, gg = row - qi * p.hratio;
            // entry of (query qi, KV head kvh) = entry_base + qi * kv_heads + kvh; hratio rows per entry
            const size_t slot = (static_cast<size_t>(entry_base) + static_cast<size_t>(qi) * p.kv_heads + kvh) * p.hratio + gg;
            *reinterpret_cast<float4*>(p.part_o + slot * D + v4 * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
            if (v4 == 0) p.part_lse[slot] = (!kLimits || L > 0.f) ? g * p.scale + logf(L) : -INFINITY;
        }
    }
}

// ------------------------------------------------------------------------------
// Merge kernel: one warp per (request, query head)
// ------------------------------------------------------------------------------
struct MergeParams {
    const float* part_o;
    const float* part_lse;
    const int32_t* indptr;    // [batch + 1]
    const int32_t* entries;
    void* out;
    float* lse_out;           // optional [batch, H]
    int64_t out_batch_stride, out_head_stride, out_pos_stride;
    int batch, num_q_heads, kv_heads, hratio;      // batch counts queries: requests x q_per_req
    int q_per_req;
    // Control words at the head of the workspace, or null.  Set when the dense kernel ran beside
    // the streaming kernel: this kernel is then ordered after the streaming kernel only, and waits
    // here for the word the last dense CTA sets (see dense_tc_kernel).
    int32_t* sync;
    int32_t* status;          // optional
    uint64_t wait_ns;
};

// Control words (int32) at the head of the workspace.
constexpr int kSyncDenseCount = 0;   // dense CTAs that have finished; wraps to 0 with the last one
constexpr int kSyncDenseDone = 1;    // 1 from the last dense CTA's exit until the last merge CTA's exit
constexpr int kSyncMergeCount = 2;   // merge CTAs that have passed the wait; wraps to 0 with the last one
constexpr int kWorkspaceHeadBytes = 256;

__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T, int D>
__global__ void __launch_bounds__(256) merge_kernel(const MergeParams p) {
    constexpr int kPer = D / 32;   // floats per lane
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const bool have_row = row < p.batch * p.num_q_heads;
    // The merge lists come from the host (read-only for this kernel): they are fetched before the
    // wait for the dense kernel.  The partial results are only read after it, with ordinary loads.
    int b = 0, h = 0, g = 0, n = 0;
    const int32_t* ent = p.entries;
    unsigned my_slot = 0;       // row of the partial buffers: entry * hratio + head in group (< 2^31 rows)
    if (have_row) {
        b = row / p.num_q_heads;
        h = row - b * p.num_q_heads;
        const int kvh = h / p.hratio;
        g = h - kvh * p.hratio;
        const int list = b * p.kv_heads + kvh;             // one list of entries per (request, KV head)
        const int lo = __ldg(p.indptr + list);
        n = __ldg(p.indptr + list + 1) - lo;
        ent = p.entries + lo;
        if (lane < n) my_slot = static_cast<unsigned>(__ldg(ent + lane)) * p.hratio + g;
    }
    if (p.sync) {
        if (threadIdx.x == 0) {
            // bounded: every dense CTA was running or done before the streaming kernel, which this
            // launch is ordered after, could start
            const uint64_t start = global_timer_ns();
            bool ok = true;
            for (uint32_t i = 1; ld_acquire_gpu(p.sync + kSyncDenseDone) == 0; ++i) {
                if ((i & 63u) == 0 && global_timer_ns() - start > p.wait_ns) { ok = false; break; }
            }
            if (!ok && p.status) atomicExch(p.status, 20);
        }
        __syncthreads();
    }
    float acc[kPer];
#pragma unroll
    for (int k = 0; k < kPer; ++k) acc[k] = 0.f;
    float wsum = 0.f, gmax = -INFINITY;
    if (have_row) {
        // Lane i owns entry i (and i + 32, ...).  The partial rows are read four at a time, the row
        // index and the weight of each coming from the owning lane by shuffle.  The addresses of
        // the rows do not depend on the weights, so the first four rows are requested together
        // with the LSEs: one dependent round trip to memory less per list.
        auto load_row = [&](unsigned slot) {
            const float* src = p.part_o + static_cast<size_t>(slot) * D + lane * kPer;
            if constexpr (kPer == 4) {
                return *reinterpret_cast<const float4*>(src);
            } else {
                const float2 y = *reinterpret_cast<const float2*>(src);
                return make_float4(y.x, y.y, 0.f, 0.f);
            }
        };
        float4 x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) x[k] = load_row(__shfl_sync(kFullMask, my_slot, k));   // lanes past the list: row 0, weight 0
        float my_lse = lane < n ? p.part_lse[my_slot] : -INFINITY;
        gmax = my_lse;
        for (int i = lane + 32; i < n; i += 32)
            gmax = fmaxf(gmax, p.part_lse[static_cast<size_t>(__ldg(ent + i)) * p.hratio + g]);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(kFullMask, gmax, d));

        for (int base = 0; base < n; base += 32) {
            if (base > 0) {
                my_slot = 0;
                my_lse = -INFINITY;
                if (base + lane < n) {
                    my_slot = static_cast<unsigned>(__ldg(ent + base + lane)) * p.hratio + g;
                    my_lse = p.part_lse[my_slot];
                }
            }
            const float my_w = (my_lse == -INFINITY) ? 0.f : __expf(my_lse - gmax);    // 0 for lanes past the list
            const int cnt = min(32, n - base);
            for (int i = 0; i < cnt; i += 4) {
                float w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int src_lane = min(i + k, 31);
                    if (base > 0 || i > 0) x[k] = load_row(__shfl_sync(kFullMask, my_slot, src_lane));
                    w[k] = (i + k < cnt) ? __shfl_sync(kFullMask, my_w, src_lane) : 0.f;
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (w[k] != 0.f) {      // a skipped row may hold anything (never written slots are not read: w = 0)
                        wsum += w[k];
                        acc[0] += w[k] * x[k].x;
                        acc[1] += w[k] * x[k].y;
                        if constexpr (kPer == 4) { acc[2] += w[k] * x[k].z; acc[3] += w[k] * x[k].w; }
                    }
                }
            }
        }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    const int req = p.q_per_req == 1 ? b : b / p.q_per_req;
    T* dst = static_cast<T*>(p.out) + static_cast<int64_t>(req) * p.out_batch_stride +
             static_cast<int64_t>(b - req * p.q_per_req) * p.out_pos_stride +
             static_cast<int64_t>(h) * p.out_head_stride + lane * kPer;
    if constexpr (kPer == 4) {
        uint2 v;
        v.x = Elt<T>::pack(acc[0] * inv, acc[1] * inv);
        v.y = Elt<T>::pack(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(dst) = v;
    } else {
        *reinterpret_cast<uint32_t*>(dst) = Elt<T>::pack(acc[0] * inv, acc[1] * inv);
    }
    if (p.lse_out && lane == 0) p.lse_out[row] = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
    }
    if (p.sync) {
        // the last CTA past the wait clears the word for the next call
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned old = atomicInc(reinterpret_cast<unsigned*>(p.sync + kSyncMergeCount), gridDim.x - 1);
            if (old == gridDim.x - 1) atomicExch(p.sync + kSyncDenseDone, 0);
        }
    }
}

}  // namespace pat
