// Dense-tile attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Persistent kernel, one CTA per SM.  A CTA walks its list of dense work items (each item: up
// to 128 query rows of one KV head over a range of tokens of a shared segment); the lists are
// cut on the host so that every CTA streams the same number of tokens, and the CTAs that work
// on the same tokens (other KV heads, the other 128-row half) run side by side.  Replaces the
// reference's M=64 mma.sync tile (csrc/pat_fwd_kernel.h:25-299, csrc/kernel_traits.h:45-123)
// for segments that many queries share.
//
//   warps 0-7: softmax.  Thread (half, quad, lane) owns query row r = 32 quad + lane (= TMEM lane
//            r) and one half of the 128 token columns of every tile.  It reads its part of
//            S = Q K^T from TMEM (tcgen05.ld), does the online softmax (the two threads of a row
//            exchange their maxima through shared memory) and writes P (bf16/fp16 pairs) back
//            into TMEM over the S columns the row has consumed (tcgen05.st); at the end of an
//            item it reads its half of O from TMEM and stores the normalised fp32 partial.
//   warp 8 / warp 10: TMA producers for K and for V, rings of 3 tiles of 128 tokens each (boxes
//            of 16 tokens x 64 elements, 128-byte swizzle - the layout the UMMA shared-memory
//            descriptors describe).  A K tile is released as soon as its S = Q K^T has
//            completed, a V tile when its P V has.
//   warp 9:  issues every MMA (the whole warp runs the loop, one elected lane issues):
//            S(g + 2) = Q K^T (M128 N128 K16 x D/16, both operands from shared memory) two tiles
//            ahead of the softmax, interleaved with O += P(g) V(g) (M128 N=D K16 x 8, A = P from
//            TMEM, B = V from shared memory); completion is signalled with tcgen05.commit on
//            mbarriers.  The items of a CTA form one stream of tiles: the Q rows of the next item
//            are written into shared memory during the last tile of the current one, so its
//            first S tiles are requested before the current item has finished, and an "O free"
//            barrier keeps its first P V from overwriting an accumulator that is still being read.
//
// Two measured facts shape the pipeline.  A tcgen05.commit needs of the order of a microsecond
// to reach its mbarrier, so S lives in a ring of three 128-column TMEM buffers (3 x 128 + D
// columns of O = 512) and no thread waits for a product it has just requested.  And one thread
// issues an MMA only about every 80 clocks whatever its size, so the products are made as large
// as TMEM allows (N = 128 tokens for Q K^T).
// The running maximum is only raised when a tile exceeds it by more than 2^8 (the offset
// cancels in O / l), so the O accumulator in TMEM is rescaled rarely.
// Every mbarrier wait is bounded.  A wait that gives up records a code in the status word; the
// role that gave up issues nothing more (no TMA request, no MMA), waits briefly for what it had
// in flight, the other roles' waits then run out too, and all eleven warps meet at one barrier
// before the CTA frees its TMEM and returns.
#pragma once

#include "pat_kernels.cuh"

namespace pat {

constexpr int kTcTile = 128;                // tokens per tile
constexpr int kTcRing = 3;                  // depth of the K, V and S rings
constexpr int kTcSoftmaxWarps = 8;
constexpr int kTcThreads = (kTcSoftmaxWarps + 3) * 32;
constexpr int kTcTmemCols = 512;
constexpr float kTcLazyLog2 = 8.0f;

template <int D> struct TcSmem {
    static constexpr int kBoxes = D / 64;
    static constexpr int kQBytes = kBoxes * 128 * 128;          // [box][128 rows][128 B]
    static constexpr int kKBytes = kBoxes * kTcTile * 128;      // [box][128 tokens][128 B]
    static constexpr int kQOff = 0;
    static constexpr int kKOff = kQOff + kQBytes;               // K ring
    static constexpr int kVOff = kKOff + kTcRing * kKBytes;     // V ring
    static constexpr int kBarOff = kVOff + kTcRing * kKBytes;   // 43 mbarriers + tmem base word + flag
    static constexpr int kXchOff = kBarOff + 512;               // float[2][2][128]: row maxima / sums of the two column halves
    static constexpr int kRequest = kXchOff + 2048;
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
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
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

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// N consecutive fp32 columns (N = 32 or 64)
template <int N> __device__ __forceinline__ void tmem_ld_f(uint32_t taddr, float (&v)[N]) {
    if constexpr (N == 64) tmem_ld64(taddr, v); else tmem_ld32(taddr, v);
}
template <int N> __device__ __forceinline__ void tmem_st_f(uint32_t taddr, const float (&v)[N]) {
    if constexpr (N == 64) tmem_st64(taddr, v);
    else tmem_st32(taddr, reinterpret_cast<const uint32_t (&)[32]>(v));
}

struct DenseTcParams {
    AttnParams a;
    const int32_t* cta_begin;   // [num_ctas + 1] first dense item of each CTA
    const int32_t* dense_q;     // [num_items][dense_q_width] query ids of every item, -1 past its queries
    int dense_q_width;
    // Control words at the head of the workspace, or null.  Set when the streaming kernel runs
    // beside this one: the merge kernel is then ordered after the streaming kernel only, so every
    // CTA of this kernel counts itself out when its partial results are written and the last one
    // sets the word the merge kernel waits for.
    int32_t* sync;
};

// ------------------------------------------------------------------------------------
// kLimits: several query positions per request; a row may then see only the first part of an
// item's tokens (AttnParams::limits), down to none of them.
template <typename T, int D, bool kLimits>
__global__ void __launch_bounds__(kTcThreads, 1)
dense_tc_kernel(const DenseTcParams dp, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    // This CTA is running: a kernel launched as this one's programmatic dependent (the streaming
    // kernel, which does not use this kernel's results) may start once every CTA has said so.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    using L = TcSmem<D>;
    constexpr int R = kTcRing;
    constexpr int kSW = kTcSoftmaxWarps;        // warps 0..7 softmax, 8 = K producer, 9 = MMA, 10 = V producer
    const AttnParams& p = dp.a;
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    const uint32_t base = smem_u32(tc_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Called by thread 0 on every way out of the kernel, after a CTA-wide barrier that follows the
    // CTA's last global store.
    auto count_out = [&]() {
        if (!dp.sync) return;
        __threadfence();
        const unsigned old = atomicInc(reinterpret_cast<unsigned*>(dp.sync + kSyncDenseCount), gridDim.x - 1);
        if (old == gridDim.x - 1) {
            __threadfence();
            atomicExch(dp.sync + kSyncDenseDone, 1);
        }
    };
    if ((base & 1023u) != 0) {          // the swizzled layouts need a 1024-byte aligned window
        if (tid == 0) {
            if (p.status) atomicExch(p.status, 10);
            count_out();
        }
        return;
    }
    const uint32_t sQ = base + L::kQOff, sK = base + L::kKOff, sV = base + L::kVOff;
    const uint32_t bars = base + L::kBarOff;
    // barrier map (8 bytes each): full_k[R] empty_k[R] full_v[R] empty_v[R] s_full[R] p_ready[R]
    // o_done[R] q_ready o_free drain
    const uint32_t bar_full_k = bars, bar_empty_k = bars + 8 * R, bar_full_v = bars + 16 * R, bar_empty_v = bars + 24 * R,
                   bar_s = bars + 32 * R, bar_p = bars + 40 * R, bar_o = bars + 48 * R, bar_q = bars + 56 * R,
                   bar_ofree = bars + 56 * R + 8, bar_drain = bars + 56 * R + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tc_smem + L::kBarOff + 56 * R + 24);
    volatile int* poisoned = reinterpret_cast<volatile int*>(tc_smem + L::kBarOff + 56 * R + 32);
    float* xch = reinterpret_cast<float*>(tc_smem + L::kXchOff);      // [2][2][128]

    // If an earlier CTA of this call already gave up on a wait, do not start (uniform decision).
    if (tid == 0) *poisoned = (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1 : 0;
    __syncthreads();
    const int item_lo = __ldg(dp.cta_begin + blockIdx.x), item_hi = __ldg(dp.cta_begin + blockIdx.x + 1);
    if (*poisoned || item_lo >= item_hi) {      // an earlier failure, or a CTA without work (uniform)
        if (tid == 0) count_out();
        return;
    }

    if (tid == 0) {
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        for (int i = 0; i < 5 * R; ++i) mbar_init(bar_full_k + 8 * i, 1);       // full/empty k/v, s_full
        for (int i = 0; i < R; ++i) mbar_init(bar_p + 8 * i, kSW * 32);         // p_ready: every softmax thread
        for (int i = 0; i < R; ++i) mbar_init(bar_o + 8 * i, 1);                // o_done
        mbar_init(bar_q, kSW * 32);                                             // q_ready
        mbar_init(bar_ofree, kSW * 32);                                         // o_free
        mbar_init(bar_drain, 1);                                                // only used when a wait gave up
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), kTcTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o_col = R * kTcTile;    // O behind the S ring
    const int tiles_per_page = p.page_size >> 4;

    if (warp == kSW || warp == kSW + 2) {
        // ---- TMA producers: one warp streams K, one streams V ---------------------------------
        const bool is_k = warp == kSW;
        const CUtensorMap* map = is_k ? &kmap : &vmap;
        const uint32_t ring = is_k ? sK : sV;
        const uint32_t full = is_k ? bar_full_k : bar_full_v;
        const uint32_t empty = is_k ? bar_empty_k : bar_empty_v;
        bool ok = true;
        int t = 0, s = 0;
        uint32_t ph = 1;                        // parity of the release that precedes the current use of slot s
        for (int item = item_lo; item < item_hi && ok; ++item) {
            const int32_t* it = p.items + static_cast<size_t>(item) * 8;
            const int page_off = __ldg(it + 2), kv_len = __ldg(it + 3), kvh = __ldg(it + 5);
            const int n_sub = (kv_len + 15) >> 4;
            const int n_tiles = (kv_len + kTcTile - 1) / kTcTile;
            const int32_t* item_pages = p.pages + page_off;
            // The producers run up to R tiles ahead of the softmax warps.  The lanes of the K warp
            // that issue no TMA use that lead to pull the Q rows of the NEXT item (scattered by
            // query id) into L2, and with them the item record and the query ids into L1: the
            // softmax warps, which fetch those rows between two tiles, then find them close by.
            if (is_k && lane >= 8 && item + 1 < item_hi) {
                // (the same record words and id-table row the softmax warps will read: they end up in
                // this SM's L1 as well)
                const int4* nx = reinterpret_cast<const int4*>(p.items + static_cast<size_t>(item + 1) * 8);
                const int n_rows = __ldg(nx).y * p.hratio, n_kvh = __ldg(nx + 1).y;
                const int32_t* ids = dp.dense_q + static_cast<size_t>(item + 1) * dp.dense_q_width;
                for (int row = lane - 8; row < n_rows; row += 24) {
                    const int qi = row / p.hratio, gg = row - qi * p.hratio;
                    const T* q = q_row_ptr<T>(p, __ldg(ids + qi), n_kvh * p.hratio + gg);
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
                    if constexpr (D * sizeof(T) > 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(q + 64));
                }
            }
            __syncwarp();
            for (int j = 0; j < n_tiles; ++j, ++t) {
                if (t >= R) ok = mbar_wait(empty + 8 * s, ph, p.wait_ns);
                if (!ok) break;
                constexpr int kSub = kTcTile / 16;
                const int subs = min(kSub, n_sub - j * kSub);
                if (lane == 0) mbar_expect_tx(full + 8 * s, subs * (L::kBoxes * 2048));
                __syncwarp();
                if (lane < subs) {
                    const int st = j * kSub + lane;
                    const int page = __ldg(item_pages + st / tiles_per_page);
                    const int row0 = (st % tiles_per_page) << 4;
#pragma unroll
                    for (int b = 0; b < L::kBoxes; ++b)
                        tma_load_4d(ring + s * L::kKBytes + b * (kTcTile * 128) + lane * 2048, map, full + 8 * s,
                                    b * 64, kvh, row0, page);
                }
                __syncwarp();
                if (++s == R) { s = 0; ph ^= 1; }
            }
        }
        if (!ok) {
            // Gave up: nothing more is requested.  The last R tiles requested may still be on their
            // way into the ring; give each a short second wait so that none lands after the CTA
            // has handed its shared memory back.
            if (lane == 0 && p.status) atomicExch(p.status, 11);
            for (int tt = max(0, t - R); tt < t; ++tt) mbar_wait(full + 8 * (tt % R), (tt / R) & 1, kDrainWaitNs);
        }
    } else if (warp == kSW + 1) {
        // ---- MMA issuer (one thread) -------------------------------------------------------------
        // The issuing thread is the narrowest resource of the CTA, so every descriptor is reduced
        // to "base word + slot * stride + constant": the high words are constants, the low words
        // are one integer add per MMA.  Per tile it interleaves S(t + 2) with O += P(t) V(t).
        // The whole warp runs the loop (warp-uniform control flow and operands, which the compiler can
        // keep in uniform registers); one elected lane issues the tcgen05 instructions.
        const uint32_t idesc_qk = umma_idesc<T>(128, kTcTile, false);
        const uint32_t idesc_pv = umma_idesc<T>(128, D, true);
        constexpr int kSteps = D / 16;          // k-steps of a QK product
        static_assert(kTcTile == 128, "the k-step arithmetic below assumes K tiles of 128 rows, like Q");
        // Shared-memory matrix descriptor (64 bits): start address >> 4 in bits 0-13, leading byte
        // offset >> 4 in 16-29, stride byte offset >> 4 in 32-45, descriptor version 1 in 46-47,
        // layout type 2 (128-byte swizzle) in 61-63.  K-major operands (Q, K): rows of 128 B = 64
        // elements, groups of 8 rows 1024 B apart (stride offset), leading offset unused.  MN-major
        // operand (V): 64 elements along N per 128-B row, the next 64 one tile column on (leading
        // offset), groups of 8 K-rows 1024 B apart.
        constexpr uint32_t kHi = (1024u >> 4) | (1u << 14) | (2u << 29);     // SBO 1024 B, version 1, 128-B swizzle
        constexpr uint32_t kSlotStep = static_cast<uint32_t>(L::kKBytes) >> 4;
        const uint32_t q_lo = ((sQ >> 4) & 0x3fffu) | (1u << 16);            // K-major: leading offset unused (16 B)
        const uint32_t k_lo0 = ((sK >> 4) & 0x3fffu) | (1u << 16);
        const uint32_t v_lo0 = ((sV >> 4) & 0x3fffu) | (static_cast<uint32_t>((kTcTile * 128) >> 4) << 16);   // MN-major: next 64 elements
        auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(kHi) << 32) | lo; };

        // The CTA's items form one stream of tiles g = 0, 1, ...: S(g + 2) is requested while tile g
        // is multiplied into O, across item boundaries too, so that a new item costs no pipeline
        // fill.  Two cursors walk the item list: one for the Q K^T products, two tiles ahead of the
        // one for the P V products.
        bool ok = true;
        auto tiles_of = [&](int item) {
            return item < item_hi ? (__ldg(p.items + static_cast<size_t>(item) * 8 + 3) + kTcTile - 1) / kTcTile : 0;
        };
        int total_tiles = 0;
        for (int item = item_lo; item < item_hi; ++item) total_tiles += tiles_of(item);
        int qk_item = item_lo, qk_j = 0, qk_n = tiles_of(item_lo), qk_items = 0;     // cursor of the next Q K^T
        int qk_tile = 0;                                                             // its index in the tile stream
        int pv_j = 0, pv_n = qk_n, pv_item = item_lo, pv_items = 0;                  // cursor of the next P V
        // S products are issued strictly in tile order, up to two tiles ahead of the P V products
        // (ring slot of tile g + 2 = slot of tile g - 1, whose P V was issued an iteration ago; MMAs
        // execute in issue order).  The first S of an item needs the item's Q rows, which the
        // softmax warps write once they have handed the previous item's last P over - so it is
        // issued only after that item's last P V: nothing the epilogue waits for queues behind it.
        auto issue_qk_upto = [&](int pv_done) {     // pv_done: last tile whose P V has been issued (-1: none)
            while (ok && qk_tile < total_tiles && qk_tile <= pv_done + 2) {
                const bool opens = qk_j == 0;
                if (opens && qk_tile > pv_done + 1) break;
                const int slot = qk_tile % R;
                const uint32_t phase = static_cast<uint32_t>(qk_tile / R) & 1u;
                if (opens) {
                    ok = mbar_wait(bar_q, qk_items & 1, p.wait_ns);
                    ++qk_items;
                    fence_async_smem();     // the Q rows were written through the generic proxy
                }
                if (ok) ok = mbar_wait(bar_full_k + 8 * slot, phase, p.wait_ns);
                ok = __all_sync(kFullMask, ok);
                if (!ok) return;            // gave up: nothing more is issued
                tc_fence_after();
                uint32_t q_w = q_lo, k_w = k_lo0 + slot * kSlotStep, acc = 0;
#pragma unroll
                for (int ks = 0; ks < kSteps; ++ks) {
                    if (elect_one()) tc_mma(tmem_base + slot * kTcTile, desc(q_w), desc(k_w), idesc_qk, acc);
                    // k-step ks + 1 of a K-major operand of 128 rows: 32 B on, or into the next 64-element box
                    const uint32_t step = (ks & 3) == 3 ? ((128 * 128 - 96) >> 4) : (32 >> 4);
                    q_w += step;
                    k_w += step;
                    acc = 1;
                }
                if (elect_one()) tc_commit(bar_s + 8 * slot);
                if (elect_one()) tc_commit(bar_empty_k + 8 * slot);    // the K tile is free once this product has completed
                if (++qk_j == qk_n) { ++qk_item; qk_j = 0; qk_n = tiles_of(qk_item); }
                ++qk_tile;
            }
        };
        int s = 0;                              // ring slot and phase of tile g
        uint32_t ph = 0;
        issue_qk_upto(-1);
        for (int g = 0; g < total_tiles && ok; ++g) {
            // O += P(g) V(g)
            ok = mbar_wait(bar_full_v + 8 * s, ph, p.wait_ns);
            if (ok) ok = mbar_wait(bar_p + 8 * s, ph, p.wait_ns);  // P(g) is in TMEM (over S(g))
            if (pv_j == 0 && pv_items > 0 && ok)
                ok = mbar_wait(bar_ofree, (pv_items - 1) & 1, p.wait_ns);   // the softmax warps have read the previous item's O
            ok = __all_sync(kFullMask, ok);     // keep the warp converged on a timeout
            if (!ok) break;                     // gave up: nothing more is issued
            tc_fence_after();
            {
                uint32_t v_w = v_lo0 + s * kSlotStep;
                uint32_t p_col = tmem_base + s * kTcTile;
                const uint32_t o_col = tmem_base + tmem_o_col;
                uint32_t acc_o = pv_j > 0 ? 1u : 0u;
#pragma unroll
                for (int i = 0; i < kTcTile / 16; ++i) {
                    if (elect_one()) tc_mma_ts(o_col, p_col, desc(v_w), idesc_pv, acc_o);
                    v_w += 2048 >> 4;       // the next 16 tokens of V
                    p_col += 8;             // 16 tokens of P = 8 packed columns
                    acc_o = 1;
                }
            }
            if (elect_one()) tc_commit(bar_o + 8 * s);
            if (elect_one()) tc_commit(bar_empty_v + 8 * s);
            if (++pv_j == pv_n) { ++pv_item; ++pv_items; pv_j = 0; pv_n = tiles_of(pv_item); }
            issue_qk_upto(g);
            if (++s == R) { s = 0; ph ^= 1; }
        }
        if (!ok) {
            // Products issued before the wait that gave up may still be running: one last commit
            // arrives on the drain barrier when all of them have completed, and the warp waits for
            // that (bounded) before the CTA frees its tensor memory.
            if (lane == 0 && p.status) atomicExch(p.status, 13);
            if (elect_one()) tc_commit(bar_drain);
            mbar_wait(bar_drain, 0, p.wait_ns);
        }
    } else {
    // ---- softmax warps ---------------------------------------------------------------------------
    // Thread (half, quad, lane) owns row r = 32 quad + lane (TMEM lane r) and the token columns
    // [32 half, 32 half + 32) of every tile; the two threads of a row exchange their maxima through
    // shared memory and keep identical copies of the running maximum.
    constexpr int OC = D / 2;                   // O columns per thread
    const int half = warp >> 2, quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t tmem_o = lane_addr + tmem_o_col + half * OC;
    const float c = p.scale_log2;
    bool ok = true;
    int t = 0;                                  // running tile index (all rings)
    int s = 0;                                  // t % R and the phase bit (t / R) & 1, kept incrementally
    uint32_t ph = 0;
    int o_seen = 0, o_slot = 0;                 // tiles whose P V is known to have completed
    uint32_t o_ph = 0;
    auto ensure_o = [&](int upto) {             // every o_done phase is consumed exactly once, in order
        while (o_seen < upto) {
            if (ok) ok = mbar_wait(bar_o + 8 * o_slot, o_ph, p.wait_ns);
            ++o_seen;
            if (++o_slot == R) { o_slot = 0; o_ph ^= 1; }
        }
        tc_fence_after();
    };
    auto pair_sync = [&]() { named_bar_sync(2 + quad, 64); };   // the two warps that share TMEM lanes
    // Q rows of an item, half a row per thread.  A load from global memory takes a thousand
    // clocks or more here (the producers keep the memory system busy), so nothing on the way to a
    // row's address waits for anything else: the query id of this thread's row comes from a table
    // indexed by the item number alone, and item records (two 16-byte words) are loaded an item
    // ahead; both are requested at the top of the item before.
    const int my_q = r / p.hratio, my_g = r - my_q * p.hratio;
    auto q_id = [&](int item) { return my_q < dp.dense_q_width ? __ldg(dp.dense_q + static_cast<size_t>(item) * dp.dense_q_width + my_q) : -1; };
    auto q_addr = [&](int qid, int kvh) -> const uint4* {
        if (qid < 0) return nullptr;
        return reinterpret_cast<const uint4*>(q_row_ptr<T>(p, qid, kvh * p.hratio + my_g)) + half * (D / 16);
    };
    auto q_fetch = [&](const uint4* src, uint4 (&qv)[D / 16]) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) qv[i] = src ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
    };
    auto q_store = [&](const uint4 (&qv)[D / 16]) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            const int ch = half * (D / 16) + i;
            const uint32_t dst = sQ + (ch >> 3) * (128 * 128) + swz128(r, ch & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(qv[i].x), "r"(qv[i].y), "r"(qv[i].z), "r"(qv[i].w) : "memory");
        }
        fence_async_smem();
    };
    // record of an item: {q_off, nq, page_off, kv_len}, {entry_base, kv_head, cost, tok_lo}
    auto load_record = [&](int item, int4& a, int4& b) {
        const int4* rec = reinterpret_cast<const int4*>(p.items + static_cast<size_t>(item) * 8);
        a = __ldg(rec);
        b = __ldg(rec + 1);
    };
    int4 rec_a, rec_b;
    load_record(item_lo, rec_a, rec_b);
    for (int item = item_lo; item < item_hi; ++item) {
        const int q_off = rec_a.x, nq = rec_a.y, kv_len = rec_a.w, entry_base = rec_b.x;
        const int rows_valid = nq * p.hratio;
        const int n_tiles = (kv_len + kTcTile - 1) / kTcTile;
        int row_limit = kv_len;             // tokens of this item that row r may see
        if constexpr (kLimits)
            row_limit = r < rows_valid ? visible_tokens(p, q_off + r / p.hratio, rec_b.w, kv_len) : 0;
        int4 next_a = make_int4(0, 0, 0, 0), next_b = make_int4(0, 0, 0, 0);
        int next_qid = -1;
        if (item + 1 < item_hi) {           // in flight during this item's tiles
            load_record(item + 1, next_a, next_b);
            next_qid = q_id(item + 1);
        }

        // the first item's Q rows; those of every later item are written during the last tile of the
        // item before it (below)
        if (item == item_lo) {
            uint4 qv[D / 16];
            q_fetch(q_addr(q_id(item), rec_b.y), qv);
            q_store(qv);
            tc_fence_before();
            mbar_arrive(bar_q);
        }

        float m_used = -INFINITY, l = 0.f;
        for (int j = 0; j < n_tiles; ++j, ++t) {
            if (ok) ok = mbar_wait(bar_s + 8 * s, ph, p.wait_ns);
            tc_fence_after();
            if (j == n_tiles - 1 && item + 1 < item_hi) {
                // Last tile of the item.  Its S has completed, and with it every Q K^T of the item:
                // the Q rows of the next item can take their place.  They are copied from global
                // memory (from L2: the K producer warp has prefetched them) straight into the swizzled
                // layout by asynchronous 16-byte copies that take no registers and nobody waits for:
                // each thread's copies arrive on q_ready by themselves when they have landed, which
                // is during this tile's softmax, and the MMA warp - which issues a proxy fence after
                // that wait - can request the next item's first S right after this item's last P V.
                const uint4* src = q_addr(next_qid, next_b.y);
#pragma unroll
                for (int i = 0; i < D / 16; ++i) {
                    const int ch = half * (D / 16) + i;
                    const uint32_t dst = sQ + (ch >> 3) * (128 * 128) + swz128(r, ch & 7);
                    if (src) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + i) : "memory");
                    else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
                }
                if (src) {
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_q) : "memory");
                } else {            // a row beyond the item's queries: zeros, written synchronously
                    fence_async_smem();
                    mbar_arrive(bar_q);
                }
            }
            constexpr int CH = kTcTile / 2;     // token columns per thread
            float sc[CH];
            tmem_ld_f<CH>(lane_addr + s * kTcTile + half * CH, sc);
            const int valid = min(kTcTile, kv_len - j * kTcTile);
            const int row_valid = kLimits ? min(valid, row_limit - j * kTcTile) : valid;
            if (row_valid < kTcTile) {
#pragma unroll
                for (int i = 0; i < CH; ++i)
                    if (half * CH + i >= row_valid) sc[i] = -INFINITY;
            }
            float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]);
#pragma unroll
            for (int i = 4; i < CH; i += 4) {
                mx0 = fmaxf(mx0, fmaxf(sc[i], sc[i + 1]));
                mx1 = fmaxf(mx1, fmaxf(sc[i + 2], sc[i + 3]));
            }
            float* xbuf = xch + (t & 1) * 256;
            xbuf[half * 128 + r] = fmaxf(mx0, mx1);
            pair_sync();
            float mx = fmaxf(fmaxf(mx0, mx1), xbuf[(half ^ 1) * 128 + r]);
            // A row that sees nothing of this tile has mx = -inf; a large finite floor keeps the
            // offsets finite (exp2(-inf - finite) = 0) and gives way to the first real score.
            if constexpr (kLimits) mx = fmaxf(mx, -1e30f);
            const bool raise = (j == 0) || (mx * c > m_used * c + kTcLazyLog2);
            if (j > 0 && __any_sync(kFullMask, raise)) {
                ensure_o(t);            // O may only be touched once every earlier P V has completed
                const float alpha = raise ? fast_exp2((m_used - mx) * c) : 1.f;
                l *= alpha;
                float ov[OC];
                tmem_ld_f<OC>(tmem_o, ov);
#pragma unroll
                for (int i = 0; i < OC; ++i) ov[i] *= alpha;
                tmem_st_f<OC>(tmem_o, ov);
            }
            if (raise) m_used = mx;
            const float off = m_used * c;
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t packed[CH / 2];
            // One exponential per score on the special-function unit (16 per clock and SM) and about
            // as many cycles of FMA-pipe work (scale, sum, 16-bit packing) per tile: moving a share of
            // the exponentials to the FMA pipe as a polynomial made the tile slower, not faster.
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) {
                const float p0 = fast_exp2(fmaf(sc[2 * i], c, -off));
                const float p1 = fast_exp2(fmaf(sc[2 * i + 1], c, -off));
                sum0 += p0;
                sum1 += p1;
                packed[i] = Elt<T>::pack(p0, p1);
            }
            l += sum0 + sum1;
            // P over the S columns this row has consumed: CH / 2 packed columns per half
            tmem_st32(lane_addr + s * kTcTile + half * (CH / 2), packed);
            if (valid < kTcTile) {
                // V rows past the valid tokens may hold anything (stale tiles, never written pages):
                // zero them (once the tile's V has landed) so that P = 0 times garbage cannot make a NaN
                if (ok) ok = mbar_wait(bar_full_v + 8 * s, ph, p.wait_ns);
                const int rows = kTcTile - valid;
                const int chunks = rows * 8 * L::kBoxes;
                for (int i = tid; i < chunks; i += kSW * 32) {
                    const int b = i / (rows * 8);
                    const int rem = i - b * rows * 8;
                    const int vrow = valid + (rem >> 3);
                    const uint32_t dst = sV + s * L::kKBytes + b * (kTcTile * 128) + vrow * 128 + ((rem & 7) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
                }
                fence_async_smem();
            }
            // keep the o_done parities in step: the product of tile t - R was requested R - 1 tiles
            // ago, so this does not stall
            ensure_o(t - R + 1);
            tc_fence_before();
            mbar_arrive(bar_p + 8 * s);
            if (++s == R) { s = 0; ph ^= 1; }
        }

        // ---- item epilogue: O / l -> fp32 partial, LSE ---------------------------------------------
        {
            // row sum = the two halves' sums (same buffer discipline as the maxima: parity of t);
            // exchanged while the last P V is still on its way
            float* xbuf = xch + (t & 1) * 256;
            pair_sync();                        // partner has read the last tile's maximum
            xbuf[half * 128 + r] = l;
            pair_sync();
            const float l_row = l + xbuf[(half ^ 1) * 128 + r];
            pair_sync();                        // both have read before the buffer is reused
            ensure_o(t);
            const bool store = ok && r < rows_valid;
            size_t slot = 0;
            if (r < rows_valid) {
                const int qi = r / p.hratio, gg = r - qi * p.hratio;
                slot = static_cast<size_t>(entry_base + qi) * p.hratio + gg;
            }
            const float inv = (!kLimits || l_row > 0.f) ? 1.f / l_row : 0.f;    // a row that saw nothing
            float ov[OC];
            tmem_ld_f<OC>(tmem_o, ov);
            tc_fence_before();
            mbar_arrive(bar_ofree);             // O may be overwritten by the next item's first P V
            if (store) {
                // 32 bytes per store: the rows of a warp lie D floats apart, so every store instruction
                // touches 32 lines whatever its width, and the wide form halves their number
                float* dst = p.part_o + slot * D + half * OC;
#pragma unroll
                for (int i = 0; i < OC / 8; ++i)
                    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                 ::"l"(dst + 8 * i), "f"(ov[8 * i] * inv), "f"(ov[8 * i + 1] * inv), "f"(ov[8 * i + 2] * inv),
                                   "f"(ov[8 * i + 3] * inv), "f"(ov[8 * i + 4] * inv), "f"(ov[8 * i + 5] * inv),
                                   "f"(ov[8 * i + 6] * inv), "f"(ov[8 * i + 7] * inv)
                                 : "memory");
                if (half == 0)
                    p.part_lse[slot] = (!kLimits || l_row > 0.f) ? m_used * p.scale + logf(l_row) : -INFINITY;
            }
        }
        rec_a = next_a;
        rec_b = next_b;
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 12);
    }
    // Every warp of the CTA ends here, also after a wait that gave up (the producers and the MMA
    // warp have then waited for what they had in flight), so tensor memory and shared memory are
    // only handed back once nothing can still write to them.
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTcTmemCols);
    if (tid == 0) count_out();
}

}  // namespace pat
