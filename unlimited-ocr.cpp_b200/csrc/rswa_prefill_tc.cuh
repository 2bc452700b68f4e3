// Ragged prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// One CTA (128 threads) owns one tile of up to 128 consecutive query rows of one request and one
// head, and walks the 128-key tiles those rows can see: first the fixed (prefix) region through the
// block table, then -- for text rows -- the sliding text window in the text pool.  Per key tile:
//
//   S = Q K^T      tcgen05.mma kind::f16, M=128 N=128, K and Q tiles in shared memory (K-major,
//                  128-byte swizzle), accumulator in TMEM (128 lanes x 128 fp32 columns)
//   softmax        thread r owns query row r == TMEM lane r: tcgen05.ld, mask, online max/sum in the
//                  exp2 domain, probabilities written back to shared memory as the A operand
//   O_tile = P V   tcgen05.mma again, V tile as the MN-major B operand; the result is read from TMEM
//                  and folded into a per-thread fp32 accumulator with the usual rescale
//
// The queries arrive in fp32 and the oracle computes in fp32, so Q and P are each fed to the tensor
// cores as a bf16 pair (hi + lo): two MMAs per operand keep ~16 mantissa bits, which holds the
// stated tolerance (rel-L2 1e-3) that a single bf16 rounding of Q would not.  K and V are the cache's
// own bf16 payload.  Semantics: RSWACache::attention (src/scheduler/kv_cache.cpp:84-130) for vision
// rows (causal over the fixed region) and, for text rows, the append-then-attend composition that
// defines "prefix + last W tokens".
//
// Every wait is bounded; a wait that runs out sets a status bit and the CTA still frees its TMEM.
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

struct PrefillTile {
    int row0;    // first packed row of the tile
    int rows;    // 1..128 query rows, consecutive positions of one request
    int slot;    // cache slot (block-table row, prefix length)
    int kind;    // 0: vision rows, causal over the fixed region; 1: text rows, prefix + window
    int pos0;    // position of the first row (prefix index for kind 0, text index for kind 1)
    int block0;  // kind 1: first block of the request's tokens in the text pool
};

struct PrefillParams {
    const float* q;
    float* out;
    const uint8_t* k_pool;
    const uint8_t* v_pool;
    const uint8_t* k_text;
    const uint8_t* v_text;
    const int32_t* table;
    const int* d_prefill_len;
    const PrefillTile* tiles;
    int table_stride, num_blocks, text_blocks;
    int heads, kv_heads, group, window;
    float scale_log2e;
    int* status;
};

constexpr int kTcTile = 128;             // queries per CTA, keys per step, head_dim
constexpr int kTcHalfBytes = 128 * 128;  // one 64-element-wide half of a 128x128 bf16 tile
constexpr int kTcTileBytes = 2 * kTcHalfBytes;

// Byte offset of 16-byte chunk `chunk` (0..15 across the 256-byte row) of row `row` inside a
// 128 x 128 bf16 tile stored as two K-major / MN-major SWIZZLE_128B halves: rows of 128 bytes,
// 8-row atoms of 1024 bytes, chunk index XORed with (row % 8).
__device__ __forceinline__ uint32_t tc_tile_offset(int row, int chunk) {
    const int half = chunk >> 3, c = chunk & 7;
    return (uint32_t)(half * kTcHalfBytes + (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4));
}

// Shared-memory matrix descriptor (SWIZZLE_128B, descriptor version 1).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_byte_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;  // version
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: D fp32, A and B bf16, M = N = 128; B K-major or MN-major.
__device__ __forceinline__ uint32_t tc_instr_desc(bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;              // D format: f32
    d |= 1u << 7;              // A format: bf16
    d |= 1u << 10;             // B format: bf16
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(128 >> 3) << 17;  // N
    d |= (uint32_t)(128 >> 4) << 24;  // M
    return d;
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// hi/lo bf16 split of eight floats into two 16-byte chunks
__device__ __forceinline__ void tc_split8(const float (&x)[8], uint4& hi, uint4& lo) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t a = f32_to_bf16_bits(x[2 * i]), b = f32_to_bf16_bits(x[2 * i + 1]);
        h[i] = a | (b << 16);
        const float ra = x[2 * i] - __uint_as_float(a << 16), rb = x[2 * i + 1] - __uint_as_float(b << 16);
        l[i] = f32_to_bf16_bits(ra) | (f32_to_bf16_bits(rb) << 16);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ float tc_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int kTcSmemBytes = 6 * kTcTileBytes + 64 + 1024;  // Qhi Qlo K V Phi Plo + barriers + alignment slack

__global__ void __launch_bounds__(128, 1) rswa_prefill_tc_kernel(const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQh = base;
    uint8_t* sQl = base + 1 * kTcTileBytes;
    uint8_t* sK = base + 2 * kTcTileBytes;
    uint8_t* sV = base + 3 * kTcTileBytes;
    uint8_t* sPh = base + 4 * kTcTileBytes;
    uint8_t* sPl = base + 5 * kTcTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + 6 * kTcTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
    const uint32_t bar_s = smem_addr(bars), bar_o = smem_addr(bars + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const PrefillTile t = p.tiles[blockIdx.x];
    const int head = blockIdx.y, kvh = head / p.group;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_init_fence();
    }
    if (warp == 0) {  // 256 TMEM columns: S in [0,128), O_tile in [128,256)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const uint32_t tS = tmem + lane_base, tO = tmem + 128 + lane_base;

    // ---- this thread's query row ------------------------------------------------------------------
    const int r = tid;
    const bool live = r < t.rows;
    const int i = t.pos0 + r;
    const int pfx = max(p.d_prefill_len[t.slot], 0);
    const int phi = !live ? 0 : (t.kind == 0 ? min(i + 1, pfx) : pfx);  // fixed-region tokens [0, phi)
    const int tlo = max(0, i - p.window + 1);
    const int thi = (live && t.kind == 1) ? i + 1 : 0;                   // text tokens [tlo, thi)
    {
        const float* qp = p.q + ((size_t)(t.row0 + r) * p.heads + head) * kTcTile;
#pragma unroll 4
        for (int c = 0; c < 16; ++c) {
            float x[8];
            if (live) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(qp + c * 8));
                const float4 b = __ldg(reinterpret_cast<const float4*>(qp + c * 8 + 4));
                x[0] = a.x * p.scale_log2e; x[1] = a.y * p.scale_log2e; x[2] = a.z * p.scale_log2e; x[3] = a.w * p.scale_log2e;
                x[4] = b.x * p.scale_log2e; x[5] = b.y * p.scale_log2e; x[6] = b.z * p.scale_log2e; x[7] = b.w * p.scale_log2e;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = 0.f;
            }
            uint4 hi, lo;
            tc_split8(x, hi, lo);
            const uint32_t off = tc_tile_offset(r, c);
            *reinterpret_cast<uint4*>(sQh + off) = hi;
            *reinterpret_cast<uint4*>(sQl + off) = lo;
        }
    }

    // ---- key tiles this query tile can see ----------------------------------------------------------
    const int plim = t.kind == 0 ? min(t.pos0 + t.rows, pfx) : pfx;
    const int n_prefix_tiles = (plim + kTcTile - 1) / kTcTile;
    int text_tile0 = 0, n_text_tiles = 0;
    if (t.kind == 1) {
        text_tile0 = max(0, t.pos0 - p.window + 1) / kTcTile;
        n_text_tiles = (t.pos0 + t.rows - 1) / kTcTile - text_tile0 + 1;
    }
    const int prefix_blocks = (pfx + kBlockTokens - 1) / kBlockTokens;
    const uint32_t idesc_s = tc_instr_desc(false), idesc_o = tc_instr_desc(true);

    float acc[kTcTile];
#pragma unroll
    for (int d = 0; d < kTcTile; ++d) acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int step = 0; step < n_prefix_tiles + n_text_tiles && ok; ++step) {
        const bool text = step >= n_prefix_tiles;
        const int t0 = text ? (text_tile0 + step - n_prefix_tiles) * kTcTile : step * kTcTile;
        const uint32_t parity = (uint32_t)step & 1u;

        // ---- stage K and V (128 keys x 256 B each) in the swizzled operand layout -------------------
        for (int c = tid; c < kTcTile * 16; c += 128) {
            const int key = c >> 4, ch = c & 15;
            const int tok = t0 + key;
            int blk = -1;
            const uint8_t* kb = p.k_pool;
            const uint8_t* vb = p.v_pool;
            if (text) {
                blk = t.block0 + tok / kBlockTokens;
                if (blk >= p.text_blocks) blk = -1;
                kb = p.k_text;
                vb = p.v_text;
            } else {
                const int idx = tok / kBlockTokens;
                if (idx < prefix_blocks && idx < p.table_stride) {
                    blk = __ldg(p.table + (size_t)t.slot * p.table_stride + idx);
                    if (blk < 0 || blk >= p.num_blocks) {
                        atomicOr(p.status, kStatusBadBlock);
                        blk = -1;
                    }
                }
            }
            uint4 kw = make_uint4(0, 0, 0, 0), vw = kw;
            if (blk >= 0) {
                const size_t src = ((((size_t)blk * p.kv_heads + kvh) * kBlockTokens + (tok & (kBlockTokens - 1))) * kTcTile) * 2 + ch * 16;
                kw = __ldg(reinterpret_cast<const uint4*>(kb + src));
                vw = __ldg(reinterpret_cast<const uint4*>(vb + src));
            }
            const uint32_t off = tc_tile_offset(key, ch);
            *reinterpret_cast<uint4*>(sK + off) = kw;
            *reinterpret_cast<uint4*>(sV + off) = vw;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
        __syncthreads();

        // ---- S = (Qhi + Qlo) K^T ------------------------------------------------------------------
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int hq = 0; hq < 2; ++hq) {
                const uint32_t a0 = smem_addr(hq ? sQl : sQh), b0 = smem_addr(sK);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t koff = (uint32_t)((j >> 2) * kTcHalfBytes + (j & 3) * 32);
                    tc_mma(tmem, tc_smem_desc(a0 + koff, 16, 1024), tc_smem_desc(b0 + koff, 16, 1024), idesc_s,
                           !(hq == 0 && j == 0));
                }
            }
            tc_commit(bar_s);
        }
        if (!mbar_wait_bounded(bar_s, parity, p.status)) { ok = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- softmax on this thread's row --------------------------------------------------------------
        float alpha = 1.f, m_safe = 0.f;
        if (ok) {
            float mx = -INFINITY;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                float v[32];
                tc_ld32(tS + cc * 32, v);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int tok = t0 + cc * 32 + j;
                    const bool valid = text ? (tok >= tlo && tok < thi) : (tok < phi);
                    if (valid) mx = fmaxf(mx, v[j]);
                }
            }
            const float m_new = fmaxf(m_run, mx);
            m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            alpha = tc_exp2(m_run - m_safe);
            float lsum = 0.f;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                float v[32];
                tc_ld32(tS + cc * 32, v);
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    float pr[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int tok = t0 + cc * 32 + g8 * 8 + e;
                        const bool valid = text ? (tok >= tlo && tok < thi) : (tok < phi);
                        pr[e] = valid ? tc_exp2(v[g8 * 8 + e] - m_safe) : 0.f;
                        lsum += pr[e];
                    }
                    uint4 hi, lo;
                    tc_split8(pr, hi, lo);
                    const uint32_t off = tc_tile_offset(r, cc * 4 + g8);
                    *reinterpret_cast<uint4*>(sPh + off) = hi;
                    *reinterpret_cast<uint4*>(sPl + off) = lo;
                }
            }
            l_run = l_run * alpha + lsum;
            m_run = m_new;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (!ok) break;  // `ok` can differ between threads only after a wait ran out: leave together below

        // ---- O_tile = (Phi + Plo) V ------------------------------------------------------------------
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int hp = 0; hp < 2; ++hp) {
                const uint32_t a0 = smem_addr(hp ? sPl : sPh), b0 = smem_addr(sV);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t koff = (uint32_t)((j >> 2) * kTcHalfBytes + (j & 3) * 32);
                    // V is [key][dim]: MN-major B operand; 64-dim halves are 16 KB apart (LBO), 8-key groups 1 KB (SBO)
                    tc_mma(tmem + 128, tc_smem_desc(a0 + koff, 16, 1024), tc_smem_desc(b0 + j * 2048, kTcHalfBytes, 1024),
                           idesc_o, !(hp == 0 && j == 0));
                }
            }
            tc_commit(bar_o);
        }
        if (!mbar_wait_bounded(bar_o, parity, p.status)) { ok = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                float v[32];
                tc_ld32(tO + cc * 32, v);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[cc * 32 + j] = fmaf(acc[cc * 32 + j], alpha, v[j]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // TMEM and the K/V/P tiles are free for the next step
    }

    // ---- write the row; rows that attended nothing give zeros ------------------------------------------
    if (live) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        float* op = p.out + ((size_t)(t.row0 + r) * p.heads + head) * kTcTile;
#pragma unroll
        for (int d = 0; d < kTcTile; d += 4)
            *reinterpret_cast<float4*>(op + d) = make_float4(acc[d] * inv, acc[d + 1] * inv, acc[d + 2] * inv, acc[d + 3] * inv);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

}  // namespace uocr_b200
