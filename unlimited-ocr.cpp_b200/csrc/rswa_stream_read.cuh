// Read-only streaming-rate measurement of the copy path the attention kernels use.
//
// One persistent CTA per SM, every warp pulling 4 KB tiles of its CTA's contiguous share through a ring
// of bulk async copies -- the way the decode kernel reads its tiles, without the arithmetic.  Each CTA
// reports its duration and SM id; the host times the launch with events and divides the bytes by it.
// The figure is the denominator for "how much of what this copy path can stream does the attention
// kernel reach", next to the copy (read + write) peak measured outside this library.
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

constexpr int kStreamTile = 4096;  // bytes per copy: the bf16 x 128 tile of one (block, head)
constexpr int kStreamRing = 3;

struct StreamReadParams {
    const uint8_t* buf;           // gridDim.x * tiles_per_cta * kStreamTile bytes
    int tiles_per_cta;
    int passes;                   // times each CTA walks its share
    unsigned long long* out;      // [gridDim.x][2] = duration in ns, SM id
    int* status;
};

__global__ void __launch_bounds__(512, 1) rswa_stream_read_kernel(const StreamReadParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bar_bytes = (warps * kStreamRing * 8 + 127) & ~127;
    const uint32_t bar0 = smem_addr(smem) + warp * (kStreamRing * 8);
    const uint32_t tile0 = smem_addr(smem + bar_bytes + (size_t)warp * (kStreamRing * kStreamTile));
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStreamRing; ++s) mbar_init(bar0 + 8 * s, 1);
        mbar_init_fence();
    }
    __syncthreads();
    unsigned long long t0 = 0;
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));

    const uint8_t* base = p.buf + (size_t)blockIdx.x * p.tiles_per_cta * kStreamTile;
    const int per_pass = (p.tiles_per_cta - warp + warps - 1) / warps;  // this warp's tiles: warp, warp + warps, ...
    const int n = per_pass * p.passes;
    if (lane == 0) {
        uint32_t phases = 0;
        bool ok = true;
        for (int i = 0; i < n + kStreamRing - 1 && ok; ++i) {
            if (i < n) {
                const int s = i % kStreamRing;
                mbar_arrive_expect_tx(bar0 + 8 * s, kStreamTile);
                bulk_copy_g2s(tile0 + s * kStreamTile, base + (size_t)(warp + (i % per_pass) * warps) * kStreamTile, kStreamTile, bar0 + 8 * s);
            }
            const int j = i - (kStreamRing - 1);  // oldest copy in flight
            if (j >= 0) {
                const int s = j % kStreamRing;
                ok = mbar_wait_bounded(bar0 + 8 * s, (phases >> s) & 1u, p.status);
                phases ^= 1u << s;
            }
        }
        // copies still in flight after a wait ran out: give them their (bounded) time before leaving
        if (!ok)
            for (int s = 0; s < kStreamRing; ++s) mbar_wait_bounded(bar0 + 8 * s, (phases >> s) & 1u, nullptr);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t1;
        unsigned smid;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.out[2 * blockIdx.x] = t1 - t0;
        p.out[2 * blockIdx.x + 1] = smid;
    }
}

}  // namespace uocr_b200
