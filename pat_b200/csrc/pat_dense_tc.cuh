// Dense-tile attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Persistent kernel, one CTA per SM.  A CTA walks its share of dense work items (each item:
// up to 256 query rows - two 128-row tiles - of one KV head over a range of tokens of a
// shared segment); the shares are cut on the host so that every CTA streams the same number
// of tokens.  Replaces the reference's M=64 mma.sync tile (csrc/pat_fwd_kernel.h:25-299,
// csrc/kernel_traits.h:45-123) for segments that many queries share.
//
//   warps 0-3 / 4-7: softmax groups 0 / 1.  Thread r of group w owns query row 128 w + r
//            (= TMEM lane r).  Per 64-token tile it reads its row of S = Q K^T from TMEM
//            (tcgen05.ld), does the online softmax without any cross-thread traffic and writes
//            P (bf16/fp16 pairs) back into TMEM over the S columns it has just consumed
//            (tcgen05.st); at the end of an item it reads O from TMEM and stores the
//            normalised fp32 partial and its LSE.
//   warp 8:  TMA producer: 5 stages of 64 tokens (K and V boxes of 16 tokens x 64 elements,
//            128-byte swizzle - the layout the UMMA shared-memory descriptors describe).
//   warp 9:  one thread issues every MMA: S_w(j) = Q_w K_j^T (M128 N64 K16 x D/16, operands
//            from shared memory) two tiles ahead of the softmax, and O_w += P_w(j) V_j (M128
//            N=D K16 x 4, A = P from TMEM, B = V from shared memory); completion is signalled
//            with tcgen05.commit on mbarriers.
//
// Both row tiles share the staged K/V tile, so a shared page is read from HBM (and from L2)
// once per 256 query rows.  TMEM (512 columns): S double-buffered per group (4 x 64) + O per
// group (2 x D).  The running maximum is only raised when a tile exceeds it by more than 2^8
// (the offset cancels in O / l), so the O accumulator in TMEM is rescaled rarely.
// Every mbarrier wait is bounded; a wait that gives up records a code in the status word,
// later waits are skipped and the CTA still frees its TMEM before it returns.
#pragma once

#include "pat_kernels.cuh"

namespace pat {

constexpr int kTcTile = 64;                 // tokens per tile
constexpr int kTcStages = 5;
constexpr int kTcThreads = 320;
constexpr int kTcTmemCols = 512;
constexpr float kTcLazyLog2 = 8.0f;

template <int D> struct TcSmem {
    static constexpr int kBoxes = D / 64;
    static constexpr int kQBytes = kBoxes * 128 * 128;          // per row tile: [box][128 rows][128 B]
    static constexpr int kKBytes = kBoxes * kTcTile * 128;      // [box][64 tokens][128 B]
    static constexpr int kStageBytes = 2 * kKBytes;             // K then V
    static constexpr int kQOff = 0;
    static constexpr int kStageOff = kQOff + 2 * kQBytes;
    static constexpr int kBarOff = kStageOff + kTcStages * kStageBytes;
    static constexpr int kRequest = kBarOff + 256;              // 17 mbarriers + tmem base word + flag
};

// ---- tcgen05 wrappers ------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 64 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st64(uint32_t taddr, const float (&v)[64]) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x64.b32 [%64], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]), "r"(r[37]), "r"(r[38]), "r"(r[39]),
          "r"(r[40]), "r"(r[41]), "r"(r[42]), "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]),
          "r"(r[48]), "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]), "r"(r[55]),
          "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]), "r"(r[61]), "r"(r[62]), "r"(r[63]),
          "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- UMMA descriptors -------------------------------------------------------------
// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4),
// descriptor version 1, 128-byte swizzle (layout type 2).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu) |
           (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32) |
           (1ull << 46) | (2ull << 61);
}
// K-major operand (rows of 128 B = 64 elements, groups of 8 rows 1024 B apart): the leading
// offset is unused by the swizzled K-major layouts and set to 16 B.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr) { return umma_desc(smem_addr, 16, 1024); }
// MN-major operand: 64 elements along MN per 128-B row, next 64 along MN `mn_stride` bytes on,
// groups of 8 K-rows 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t smem_addr, uint32_t mn_stride) {
    return umma_desc(smem_addr, mn_stride, 1024);
}
// Instruction descriptor of kind::f16: fp32 accumulate, A/B format (0 = f16, 1 = bf16),
// A K-major, B K-major or MN-major, N >> 3 at bit 17, M >> 4 at bit 24.
template <typename T> __device__ __forceinline__ uint32_t umma_idesc(int m, int n, bool b_mn_major) {
    const uint32_t fmt = sizeof(T) == 2 && Elt<T>::kTma == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct DenseTcParams {
    AttnParams a;
    const int32_t* cta_begin;   // [num_ctas + 1] first dense item of each CTA
};

// ------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 1)
dense_tc_kernel(const DenseTcParams dp, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using L = TcSmem<D>;
    const AttnParams& p = dp.a;
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    const uint32_t base = smem_u32(tc_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((base & 1023u) != 0) {          // the swizzled layouts need a 1024-byte aligned window
        if (tid == 0 && p.status) atomicExch(p.status, 10);
        return;
    }
    const uint32_t sQ = base + L::kQOff, sStage = base + L::kStageOff;
    const uint32_t bars = base + L::kBarOff;
    // barrier map (8 bytes each): full[5] empty[5] s_full[w][b] (4) p_ready[2] o_done[2] q_ready
    const uint32_t bar_full = bars, bar_empty = bars + 40, bar_s = bars + 80, bar_p = bars + 112, bar_o = bars + 128,
                   bar_q = bars + 144;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tc_smem + L::kBarOff + 160);
    volatile int* poisoned = reinterpret_cast<volatile int*>(tc_smem + L::kBarOff + 168);

    // If an earlier CTA of this call already gave up on a wait, do not start (uniform decision).
    if (tid == 0) *poisoned = (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1 : 0;
    __syncthreads();
    if (*poisoned) return;

    const int item_lo = __ldg(dp.cta_begin + blockIdx.x), item_hi = __ldg(dp.cta_begin + blockIdx.x + 1);

    if (tid == 0) {
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        for (int i = 0; i < 2 * kTcStages; ++i) mbar_init(bar_full + 8 * i, 1);   // full[], empty[]
        for (int i = 0; i < 4; ++i) mbar_init(bar_s + 8 * i, 1);       // s_full
        for (int i = 0; i < 2; ++i) mbar_init(bar_p + 8 * i, 128);     // p_ready: every thread of a group
        for (int i = 0; i < 2; ++i) mbar_init(bar_o + 8 * i, 1);       // o_done
        mbar_init(bar_q, 256);                                         // q_ready: both groups
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), kTcTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int tiles_per_page = p.page_size >> 4;

    if (warp == 8) {
        // ---- TMA producer ----------------------------------------------------------------
        bool ok = true;
        int g = 0;
        for (int item = item_lo; item < item_hi && ok; ++item) {
            const int32_t* it = p.items + static_cast<size_t>(item) * 8;
            const int page_off = __ldg(it + 2), kv_len = __ldg(it + 3), kvh = __ldg(it + 5);
            const int n_sub = (kv_len + 15) >> 4;
            const int n_tiles = (kv_len + kTcTile - 1) / kTcTile;
            const int32_t* item_pages = p.pages + page_off;
            for (int j = 0; j < n_tiles; ++j, ++g) {
                const int s = g % kTcStages;
                if (g >= kTcStages) ok = mbar_wait(bar_empty + 8 * s, ((g / kTcStages) - 1) & 1);
                if (!ok) break;
                const int subs = min(4, n_sub - j * 4);
                if (lane == 0) mbar_expect_tx(bar_full + 8 * s, subs * (2 * L::kBoxes * 2048));
                __syncwarp();
                if (lane < subs) {
                    const int t = j * 4 + lane;
                    const int page = __ldg(item_pages + t / tiles_per_page);
                    const int row0 = (t % tiles_per_page) << 4;
                    const uint32_t dst = sStage + s * L::kStageBytes + lane * 2048;
#pragma unroll
                    for (int b = 0; b < L::kBoxes; ++b) {
                        tma_load_4d(dst + b * (kTcTile * 128), &kmap, bar_full + 8 * s, b * 64, kvh, row0, page);
                        tma_load_4d(dst + L::kKBytes + b * (kTcTile * 128), &vmap, bar_full + 8 * s, b * 64, kvh, row0, page);
                    }
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 11);
        return;
    }

    if (warp == 9) {
        // ---- MMA issuer (one thread) ---------------------------------------------------------
        if (lane != 0) return;
        const uint32_t idesc_qk = umma_idesc<T>(128, kTcTile, false);
        const uint32_t idesc_pv = umma_idesc<T>(128, D, true);
        bool ok = true;
        int g = 0, g1 = 0, n_item = 0;
        for (int item = item_lo; item < item_hi; ++item, ++n_item) {
            const int32_t* it = p.items + static_cast<size_t>(item) * 8;
            const int nq = __ldg(it + 1), kv_len = __ldg(it + 3);
            const bool two = nq * p.hratio > 128;
            const int n_tiles = (kv_len + kTcTile - 1) / kTcTile;
            if (ok) ok = mbar_wait(bar_q, n_item & 1);                 // this item's Q rows are in place
            tc_fence_after();

            const int nw = two ? 2 : 1;
            auto wait_stage = [&](int j) {
                const int s = (g + j) % kTcStages;
                if (ok) ok = mbar_wait(bar_full + 8 * s, ((g + j) / kTcStages) & 1);
                tc_fence_after();
            };
            auto issue_qk = [&](int w, int j) {                        // S_w = Q_w K_j^T into buffer (t & 1)
                const int t = (w == 0 ? g : g1) + j;                   // this group's running tile index
                const uint32_t k_addr = sStage + ((g + j) % kTcStages) * L::kStageBytes;
                const uint32_t d_tmem = tmem_base + w * 128 + (t & 1) * kTcTile;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t a = umma_desc_kmajor(sQ + w * L::kQBytes + (ks >> 2) * (128 * 128) + (ks & 3) * 32);
                    const uint64_t b = umma_desc_kmajor(k_addr + (ks >> 2) * (kTcTile * 128) + (ks & 3) * 32);
                    tc_mma(d_tmem, a, b, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s + 8 * (2 * w + (t & 1)));
            };

            wait_stage(0);
            for (int w = 0; w < nw; ++w) issue_qk(w, 0);
            if (n_tiles > 1) {
                wait_stage(1);
                for (int w = 0; w < nw; ++w) issue_qk(w, 1);
            }
            for (int j = 0; j < n_tiles; ++j) {
                const int s = (g + j) % kTcStages;
                const uint32_t v_addr = sStage + s * L::kStageBytes + L::kKBytes;
                for (int w = 0; w < nw; ++w) {
                    const int t = (w == 0 ? g : g1) + j;
                    if (ok) ok = mbar_wait(bar_p + 8 * w, t & 1);      // P_w(j) is in TMEM (over S_w(j))
                    tc_fence_after();
                    const uint32_t p_tmem = tmem_base + w * 128 + (t & 1) * kTcTile;
#pragma unroll
                    for (int ks = 0; ks < kTcTile / 16; ++ks) {
                        const uint64_t b = umma_desc_mnmajor(v_addr + ks * 2048, kTcTile * 128);
                        tc_mma_ts(tmem_base + 256 + w * 128, p_tmem + ks * 8, b, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_o + 8 * w);
                    // the S/P buffer of tile j is free again once the product above has read it
                    // (MMAs execute in issue order): compute S two tiles ahead into it
                    if (j + 2 < n_tiles) {
                        if (w == 0) wait_stage(j + 2);
                        issue_qk(w, j + 2);
                    }
                }
                tc_commit(bar_empty + 8 * s);                           // K/V stage free when everything above is done
            }
            g += n_tiles;
            if (two) g1 += n_tiles;
        }
        if (!ok && p.status) atomicExch(p.status, 13);
        return;
    }

    // ---- softmax groups -----------------------------------------------------------------------
    const int w = warp >> 2;                    // group 0 / 1
    const int r = tid & 127;                    // row within the 128-row tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t tmem_s = lane_addr + w * 128, tmem_o = lane_addr + 256 + w * 128;
    const float c = p.scale_log2;
    bool ok = true;
    int t = 0;                                  // this group's running tile index
    int g = 0;                                  // running tile index of the stage ring
    int n_item = 0;
    for (int item = item_lo; item < item_hi; ++item) {
        const int32_t* it = p.items + static_cast<size_t>(item) * 8;
        const int q_off = __ldg(it + 0), nq = __ldg(it + 1), kv_len = __ldg(it + 3), entry_base = __ldg(it + 4),
                  kvh = __ldg(it + 5);
        const int rows_valid = nq * p.hratio;
        const bool active = (w == 0) || rows_valid > 128;
        const int n_tiles = (kv_len + kTcTile - 1) / kTcTile;
        const int row = w * 128 + r;

        // Q rows of this item into the swizzled K-major layout (every MMA of the previous item has
        // completed: its last o_done was awaited in the epilogue below)
        if (active) {
            const uint4* src = nullptr;
            if (row < rows_valid) {
                const int qi = row / p.hratio, gg = row - qi * p.hratio;
                const T* q = static_cast<const T*>(p.q) + static_cast<int64_t>(__ldg(p.queries + q_off + qi)) * p.q_batch_stride +
                             static_cast<int64_t>(kvh * p.hratio + gg) * p.q_head_stride;
                src = reinterpret_cast<const uint4*>(q);
            }
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch) {
                const uint4 v = src ? __ldg(src + ch) : make_uint4(0, 0, 0, 0);
                const uint32_t dst = sQ + w * L::kQBytes + (ch >> 3) * (128 * 128) + swz128(r, ch & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
            fence_async_smem();
        }
        tc_fence_before();
        mbar_arrive(bar_q);
        if (!active) {
            // an idle group must not run ahead: its next arrival may only count for the next phase
            if (ok) ok = mbar_wait(bar_q, n_item & 1);
            g += n_tiles;
            ++n_item;
            continue;
        }
        ++n_item;

        float m_used = -INFINITY, l = 0.f;
        for (int j = 0; j < n_tiles; ++j, ++t) {
            if (ok) ok = mbar_wait(bar_s + 8 * (2 * w + (t & 1)), (t >> 1) & 1);
            tc_fence_after();
            float sc[64];
            tmem_ld64(tmem_s + (t & 1) * kTcTile, sc);
            const int valid = min(kTcTile, kv_len - j * kTcTile);
            if (valid < kTcTile) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (i >= valid) sc[i] = -INFINITY;
            }
            float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]);
#pragma unroll
            for (int i = 4; i < 64; i += 4) {
                mx0 = fmaxf(mx0, fmaxf(sc[i], sc[i + 1]));
                mx1 = fmaxf(mx1, fmaxf(sc[i + 2], sc[i + 3]));
            }
            const float mx = fmaxf(mx0, mx1);

            bool o_waited = false;
            const bool raise = (j == 0) || (mx * c > m_used * c + kTcLazyLog2);
            if (j > 0 && __any_sync(kFullMask, raise)) {
                // O may only be touched once every earlier P V of this group has completed
                if (ok) ok = mbar_wait(bar_o + 8 * w, (t - 1) & 1);
                tc_fence_after();
                o_waited = true;
                const float alpha = raise ? fast_exp2((m_used - mx) * c) : 1.f;
                l *= alpha;
#pragma unroll 1
                for (int h = 0; h < D / 64; ++h) {
                    float ov[64];
                    tmem_ld64(tmem_o + h * 64, ov);
#pragma unroll
                    for (int i = 0; i < 64; ++i) ov[i] *= alpha;
                    tmem_st64(tmem_o + h * 64, ov);
                }
            }
            if (raise) m_used = mx;
            const float off = m_used * c;
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = fast_exp2(fmaf(sc[2 * i], c, -off));
                const float p1 = fast_exp2(fmaf(sc[2 * i + 1], c, -off));
                sum0 += p0;
                sum1 += p1;
                packed[i] = Elt<T>::pack(p0, p1);
            }
            l += sum0 + sum1;
            // P over the first 32 columns of the S buffer this thread has just read (its own lane)
            tmem_st32(tmem_s + (t & 1) * kTcTile, packed);
            if (valid < kTcTile && w == 0) {
                // V rows past the valid tokens may hold anything (stale tiles, never written pages):
                // zero them so that P = 0 times garbage cannot make a NaN.  The stage has landed
                // (its S was computed from it) and both groups' P V products are issued after
                // group 0 has arrived below.
                const int s = (g + j) % kTcStages;
                const int rows = kTcTile - valid;
                const int chunks = rows * 8 * L::kBoxes;
                for (int i = r; i < chunks; i += 128) {
                    const int b = i / (rows * 8);
                    const int rem = i - b * rows * 8;
                    const int vrow = valid + (rem >> 3);
                    const uint32_t dst = sStage + s * L::kStageBytes + L::kKBytes + b * (kTcTile * 128) + vrow * 128 + ((rem & 7) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
                }
                fence_async_smem();
            }
            // consume the o_done phase of the previous tile (issued a whole tile ago, so this does
            // not stall); every phase is waited for exactly once, which keeps the parities in step
            if (j > 0 && !o_waited && ok) ok = mbar_wait(bar_o + 8 * w, (t - 1) & 1);
            tc_fence_before();
            mbar_arrive(bar_p + 8 * w);
        }
        g += n_tiles;

        // ---- item epilogue: O / l -> fp32 partial, LSE ---------------------------------------------
        if (ok) ok = mbar_wait(bar_o + 8 * w, (t - 1) & 1);
        tc_fence_after();
        {
            const bool store = ok && row < rows_valid;
            size_t slot = 0;
            if (row < rows_valid) {
                const int qi = row / p.hratio, gg = row - qi * p.hratio;
                slot = static_cast<size_t>(entry_base + qi) * p.hratio + gg;
            }
            const float inv = 1.f / l;
#pragma unroll 1
            for (int h = 0; h < D / 64; ++h) {
                float ov[64];
                tmem_ld64(tmem_o + h * 64, ov);
                if (store) {
                    float4* dst = reinterpret_cast<float4*>(p.part_o + slot * D + h * 64);
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        dst[i] = make_float4(ov[4 * i] * inv, ov[4 * i + 1] * inv, ov[4 * i + 2] * inv, ov[4 * i + 3] * inv);
                }
            }
            if (store) p.part_lse[slot] = m_used * p.scale + logf(l);
        }
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 12);
    tc_fence_before();
    named_bar_sync(1, 256);
    if (warp == 0) tmem_dealloc(tmem_base, kTcTmemCols);
}

}  // namespace pat
