// Per-SM streaming-rate calibration for the SM-weighted split of the attention kernels.
//
// The SMs of one B200 do not stream from HBM at the same rate: with equal shares, the SMs of some
// GPCs finish 10-20 % later than the rest, launch after launch.  This kernel measures it the way the
// attention kernel reads: one persistent CTA per SM, every warp pulling 4 KB tiles of its CTA's
// contiguous share through a ring of bulk async copies.  Each CTA reports its duration and SM id;
// the host turns the durations into cumulative shares (rate = 1 / duration).
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

constexpr int kCalTile = 4096;  // bytes per copy: the bf16 x 128 tile of one (block, head)
constexpr int kCalRing = 3;
constexpr int kMaxSmid = 256;   // SM ids the weighted split can map
constexpr int kMaxCtas = 160;   // logical CTAs (== SMs) the weighted split can hold

struct CalibrateParams {
    const uint8_t* buf;           // gridDim.x * tiles_per_cta * kCalTile bytes
    int tiles_per_cta;
    int passes;                   // times each CTA walks its share
    unsigned long long* out;      // [gridDim.x][2] = duration in ns, SM id
    int* status;
};

__global__ void __launch_bounds__(512, 1) rswa_calibrate_kernel(const CalibrateParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bar_bytes = (warps * kCalRing * 8 + 127) & ~127;
    const uint32_t bar0 = smem_addr(smem) + warp * (kCalRing * 8);
    const uint32_t tile0 = smem_addr(smem + bar_bytes + (size_t)warp * (kCalRing * kCalTile));
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kCalRing; ++s) mbar_init(bar0 + 8 * s, 1);
        mbar_init_fence();
    }
    __syncthreads();
    unsigned long long t0 = 0;
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));

    const uint8_t* base = p.buf + (size_t)blockIdx.x * p.tiles_per_cta * kCalTile;
    const int per_pass = (p.tiles_per_cta - warp + warps - 1) / warps;  // this warp's tiles: warp, warp + warps, ...
    const int n = per_pass * p.passes;
    if (lane == 0) {
        uint32_t phases = 0;
        bool ok = true;
        for (int i = 0; i < n + kCalRing - 1 && ok; ++i) {
            if (i < n) {
                const int s = i % kCalRing;
                mbar_arrive_expect_tx(bar0 + 8 * s, kCalTile);
                bulk_copy_g2s(tile0 + s * kCalTile, base + (size_t)(warp + (i % per_pass) * warps) * kCalTile, kCalTile, bar0 + 8 * s);
            }
            const int j = i - (kCalRing - 1);  // oldest copy in flight
            if (j >= 0) {
                const int s = j % kCalRing;
                ok = mbar_wait_bounded(bar0 + 8 * s, (phases >> s) & 1u, p.status);
                phases ^= 1u << s;
            }
        }
        // copies still in flight after a wait ran out: give them their (bounded) time before leaving
        if (!ok)
            for (int s = 0; s < kCalRing; ++s) mbar_wait_bounded(bar0 + 8 * s, (phases >> s) & 1u, nullptr);
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
