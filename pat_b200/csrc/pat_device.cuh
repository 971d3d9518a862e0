// Device-side building blocks shared by the attention kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pat {

constexpr uint32_t kFullMask = 0xffffffffu;
// Upper bound on mbarrier polls before a wait gives up (each poll blocks for a
// hardware-defined slice, so this is seconds, far above any legitimate wait).
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
#ifndef PAT_MBAR_WAIT_OP
#define PAT_MBAR_WAIT_OP "mbarrier.try_wait.parity.shared::cta.b64"
#endif
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        PAT_MBAR_WAIT_OP " p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false if the phase did not complete within about `limit_ns` (or kMaxPolls
// polls, whichever comes first).  The clock is only read every 64 polls.  Kernels take the limit
// as a parameter (kDefaultWaitNs unless the caller asks otherwise).
constexpr uint64_t kDefaultWaitNs = 1000ull * 1000ull * 1000ull;
// The polling loop is kept out of line: a kernel waits in many places, and warps that run a
// little code per tile (TMA producers, the MMA issuer) are bound by instruction fetch.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t start = global_timer_ns();
    for (uint32_t i = 1; i < kMaxPolls; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0 && global_timer_ns() - start > limit_ns) return false;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, limit_ns);
}
// After a wait has given up: a short second chance (about 20 us) for copies or products that
// are still on their way, so that nothing lands in memory the CTA has already handed back.
constexpr uint64_t kDrainWaitNs = 20ull * 1000ull;

// ---- TMA: 4-D tiled load of one [16 tokens x 64 elements] box -----------------
// coordinates: (element within head, kv head, row within page, page)
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- ldmatrix / mma.sync ------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T> struct Elt;
template <> struct Elt<__nv_bfloat16> {
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    // low half = lo, high half = hi
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
template <> struct Elt<__half> {
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    __device__ static __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a
// [rows x 128 B] box written by TMA with the 128-byte swizzle (box base 1024-B aligned).
__device__ __forceinline__ uint32_t swz128(int row, int chunk) {
    return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// ---- one warp, 16 query rows, NSUB sub-tiles of 16 tokens ----------------------
// Shared-memory layout of a sub-tile (one 16-token slice of one page, one KV head):
//   K: D/64 boxes of [16 x 64] elements (2 KB each), then V: the same.
// Register layouts are those of mma.m16n8k16: a thread owns rows lane/4 and
// lane/4 + 8.  `m` is the running row maximum of the raw scores, `l` the
// thread-partial running sum of exp2((s - m) * c); `o` the unnormalised output.
template <int D> struct TileGeom {
    static constexpr int kBoxes = D / 64;              // 64-element boxes per row
    static constexpr int kOperandBytes = kBoxes * 2048;
    static constexpr int kSubBytes = 2 * kOperandBytes; // K + V of one 16-token sub-tile
    static constexpr int kKSteps = D / 16;
    static constexpr int kNTilesO = D / 8;
};

// valid0 / valid1: tokens of the tile the thread's first / second row may attend to (the same
// number unless kLimits: several query positions per request see different ends of the context;
// a row may then see nothing of a tile, or of all tiles so far, which the -inf handling covers).
template <typename T, int D, int NSUB, bool kLimits = false>
__device__ __forceinline__ void warp_attend_tile(const uint32_t (&qf)[D / 16][4], float (&o)[D / 8][4],
                                                 float (&m)[2], float (&l)[2], uint32_t stage_addr,
                                                 int valid0, int valid1, float c, int lane) {
    using G = TileGeom<D>;
    float s[2 * NSUB][4];
#pragma unroll
    for (int i = 0; i < 2 * NSUB; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;

    // S = Q K^T.  ldmatrix.x4: matrices (tokens 0-7 | 8-15) x (chunk c0 | c0+1)
    const int mi = lane >> 3;
    {
        const int row = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
        for (int u = 0; u < NSUB; ++u) {
            const uint32_t kbase = stage_addr + u * G::kSubBytes;
#pragma unroll
            for (int ks = 0; ks < G::kKSteps; ++ks) {
                const int box = ks >> 2;
                const int chunk = ((ks & 3) << 1) + (mi & 1);
                uint32_t r0, r1, r2, r3;
                ldsm_x4(kbase + box * 2048 + swz128(row, chunk), r0, r1, r2, r3);
                Elt<T>::mma(s[2 * u], qf[ks], r0, r1);
                Elt<T>::mma(s[2 * u + 1], qf[ks], r2, r3);
            }
        }
    }

    // mask the tail of the last tile (and, with limits, what a row must not see)
    if (valid0 < 16 * NSUB || (kLimits && valid1 < 16 * NSUB)) {
        const int col0 = (lane & 3) << 1;
#pragma unroll
        for (int i = 0; i < 2 * NSUB; ++i) {
            const int col = i * 8 + col0;
            if (col >= valid0) s[i][0] = -INFINITY;
            if (col + 1 >= valid0) s[i][1] = -INFINITY;
            if (col >= valid1) s[i][2] = -INFINITY;
            if (col + 1 >= valid1) s[i][3] = -INFINITY;
        }
    }

    // online softmax (base 2, scores scaled by c = scale * log2 e)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2 * NSUB; ++i) {
        mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
        mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const bool changed = (mn0 != m[0]) || (mn1 != m[1]);
    if (__any_sync(kFullMask, changed)) {
        // (a row that has seen nothing yet has m = -inf: its l and o are 0 and stay 0)
        const float a0 = (kLimits && m[0] == -INFINITY) ? 0.f : fast_exp2((m[0] - mn0) * c);
        const float a1 = (kLimits && m[1] == -INFINITY) ? 0.f : fast_exp2((m[1] - mn1) * c);
        l[0] *= a0;
        l[1] *= a1;
#pragma unroll
        for (int i = 0; i < G::kNTilesO; ++i) {
            o[i][0] *= a0; o[i][1] *= a0;
            o[i][2] *= a1; o[i][3] *= a1;
        }
    }
    m[0] = mn0;
    m[1] = mn1;
    // a row whose maximum is still -inf has only masked scores: any finite offset gives exp2(-inf) = 0
    const float b0 = (kLimits && mn0 == -INFINITY) ? 0.f : mn0 * c;
    const float b1 = (kLimits && mn1 == -INFINITY) ? 0.f : mn1 * c;
    uint32_t pa[NSUB][4];
#pragma unroll
    for (int u = 0; u < NSUB; ++u) {
        float p[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            p[h][0] = fast_exp2(fmaf(s[2 * u + h][0], c, -b0));
            p[h][1] = fast_exp2(fmaf(s[2 * u + h][1], c, -b0));
            p[h][2] = fast_exp2(fmaf(s[2 * u + h][2], c, -b1));
            p[h][3] = fast_exp2(fmaf(s[2 * u + h][3], c, -b1));
            l[0] += p[h][0] + p[h][1];
            l[1] += p[h][2] + p[h][3];
        }
        pa[u][0] = Elt<T>::pack(p[0][0], p[0][1]);
        pa[u][1] = Elt<T>::pack(p[0][2], p[0][3]);
        pa[u][2] = Elt<T>::pack(p[1][0], p[1][1]);
        pa[u][3] = Elt<T>::pack(p[1][2], p[1][3]);
    }

    // O += P V.  ldmatrix.x4.trans: matrices (chunk c0 | c0+1) x (tokens 0-7 | 8-15)
    {
        const int row = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int u = 0; u < NSUB; ++u) {
            const uint32_t vbase = stage_addr + u * G::kSubBytes + G::kOperandBytes;
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                const int box = dn >> 2;
                const int chunk = ((dn & 3) << 1) + (mi >> 1);
                uint32_t r0, r1, r2, r3;
                ldsm_x4_t(vbase + box * 2048 + swz128(row, chunk), r0, r1, r2, r3);
                Elt<T>::mma(o[2 * dn], pa[u], r0, r1);
                Elt<T>::mma(o[2 * dn + 1], pa[u], r2, r3);
            }
        }
    }
}

// Zero the V rows >= valid of the sub-tile that holds the tail (so that 0 * garbage
// can never produce NaN).  All lanes of the warp call this.
template <int D>
__device__ __forceinline__ void zero_v_tail(unsigned char* stage_ptr, int sub, int valid_in_sub, int lane) {
    using G = TileGeom<D>;
    unsigned char* v = stage_ptr + sub * G::kSubBytes + G::kOperandBytes;
    const int rows = 16 - valid_in_sub;
    const int chunks_per_row = 8 * G::kBoxes;
    for (int i = lane; i < rows * chunks_per_row; i += 32) {
        const int row = valid_in_sub + i / chunks_per_row;
        const int cc = i % chunks_per_row;
        *reinterpret_cast<uint4*>(v + (cc >> 3) * 2048 + row * 128 + ((cc & 7) << 4)) = make_uint4(0, 0, 0, 0);
    }
}

}  // namespace pat
