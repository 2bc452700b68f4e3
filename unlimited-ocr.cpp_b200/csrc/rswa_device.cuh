// Device-side building blocks of the R-SWA kernels (sm_100a): mbarrier + bulk-async-copy wrappers,
// bf16 conversion on raw bits, and the per-geometry lane mapping used by the attention kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace uocr_b200 {

constexpr int kBlockTokens = 16;  // tokens per paged block and per attention unit

// Device status bits recorded in the workspace status word (never trapped on).
enum : int {
    kStatusBadBlock = 1,     // block id outside [0, num_blocks)
    kStatusWaitTimeout = 2,  // an mbarrier wait ran out of iterations
    kStatusBadSlot = 4,      // logical position outside the table row
};

// ---------------------------------------------------------------------------------------------
// shared-memory barrier + bulk copy (TMA engine, untiled form)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    // make the initialised barriers visible to the async proxy before the first copy targets them
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after `limit` polls (each poll already blocks for a hardware-defined slice),
// records the fact and lets the caller leave its loop instead of spinning forever.  kWaitLimit is the
// limit every kernel uses unless the workspace was told otherwise (a limit of 0 makes every wait give
// up at once, which is how the give-up paths are exercised without hanging anything).
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status,
                                                  uint32_t limit = kWaitLimit) {
    for (uint32_t it = 0; it < limit; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicOr(status, kStatusWaitTimeout);
    return false;
}

// global -> shared bulk copy; completion is signalled on `bar` as `bytes` of transaction count.
// Source, destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst),
        "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
        : "memory");
}

// The same copy with an L2 eviction policy for the lines it brings in (createpolicy word in `policy`).
__device__ __forceinline__ void bulk_copy_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                                   uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(dst),
        "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---------------------------------------------------------------------------------------------
// bf16 on raw bits (round-to-nearest-even exactly as the reference's host helper does:
// add 0x7fff + lsb, shift; NaN is not special-cased -- include/uocr/common.h:56-64)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    u += 0x7fffu + ((u >> 16) & 1u);
    return u >> 16;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}

// Widening a bf16 pair held in one 32-bit word: one byte permute per element (the low half needs its
// two bytes moved up, the high half its low bytes cleared; both are a single PRMT).
__device__ __forceinline__ float bf16_lo(uint32_t w) {
    uint32_t r;
    asm("prmt.b32 %0, %1, 0, 0x1044;" : "=r"(r) : "r"(w));
    return __uint_as_float(r);
}
__device__ __forceinline__ float bf16_hi(uint32_t w) {
    uint32_t r;
    asm("prmt.b32 %0, %1, 0, 0x3244;" : "=r"(r) : "r"(w));
    return __uint_as_float(r);
}

// ---------------------------------------------------------------------------------------------
// KV element traits: how a 16-byte chunk of a cache row turns into floats
// ---------------------------------------------------------------------------------------------
struct BF16 {
    using storage = uint16_t;
    static constexpr int kBytes = 2;
    static constexpr int kPerChunk = 8;
    __device__ static __forceinline__ void unpack(const uint4& w, float (&f)[8]) {
        f[0] = bf16_lo(w.x); f[1] = bf16_hi(w.x);
        f[2] = bf16_lo(w.y); f[3] = bf16_hi(w.y);
        f[4] = bf16_lo(w.z); f[5] = bf16_hi(w.z);
        f[6] = bf16_lo(w.w); f[7] = bf16_hi(w.w);
    }
};

struct F32 {
    using storage = float;
    static constexpr int kBytes = 4;
    static constexpr int kPerChunk = 4;
    __device__ static __forceinline__ void unpack(const uint4& w, float (&f)[4]) {
        f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y);
        f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w);
    }
};

// Lane mapping for one (16-token x head_dim) tile held in shared memory, one warp per tile.
// A cache row of one head is kRowBytes = kChunks x 16 bytes.  kLanesPerRow lanes share a row (each
// owning kChunksPerLane 16-byte chunks), so one warp-wide 16-byte load covers kRowsPerLoad rows and
// a tile takes kIters loads.
template <typename KV, int HD>
struct TileMap {
    static constexpr int kRowBytes = HD * KV::kBytes;
    static constexpr int kChunks = kRowBytes / 16;
    static_assert(kRowBytes % 16 == 0 && kChunks >= 1, "head row must be a multiple of 16 bytes");
    static_assert((kChunks & (kChunks - 1)) == 0, "head_dim must be a power of two");
    static constexpr int kLanesPerRow = kChunks >= 32 ? 32 : kChunks;
    static constexpr int kChunksPerLane = kChunks > 32 ? kChunks / 32 : 1;
    static constexpr int kRowsPerLoad = 32 / kLanesPerRow;
    static constexpr int kIters = kRowsPerLoad >= kBlockTokens ? 1 : kBlockTokens / kRowsPerLoad;
    static constexpr int kElemsPerLane = KV::kPerChunk * kChunksPerLane;
    static constexpr int kTileBytes = kBlockTokens * kRowBytes;
};

}  // namespace uocr_b200
