// Split-KV R-SWA attention for sm_100a: plan kernel, persistent partial-attention kernel fed by
// bulk async copies (TMA engine) through per-warp shared-memory rings, and merge kernel.
//
// Work model.  A query row r with H heads attends n_r "units" per head; a unit is one 16-token tile
// of one KV head (a paged block, or 16 consecutive rows of a contiguous cache).  All units of a
// launch are laid out on one line, ordered (row, head, unit), and cut into equal pieces, one per
// warp of a persistent grid.  A warp walks its piece with a private ring of shared-memory stages;
// one lane issues `cp.async.bulk` copies that signal an mbarrier per tile, and the whole warp
// consumes tiles with 16-byte shared loads, warp-shuffle reductions and an online softmax in the
// exp2 domain.  When a piece does not cover a whole (row, head) item the warp leaves an
// un-normalised partial (max, sum, accumulator) in scratch and the merge kernel combines the
// partials of that item; items covered by one warp are written straight to the output.
//
// Semantics follow RSWACache::attention (src/scheduler/kv_cache.cpp:84-130): scale 1/sqrt(d),
// softmax over the attended slots, 0 for an empty set; decode is order-independent in the slot
// index, so ring slots are visited in storage order.
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

struct RowInfo {
    int slot;      // cache slot of this query row
    int pe;        // attended tokens in the fixed (prefix) region
    int re;        // attended tokens in the ring region
    int ring_off;  // table index of the first ring block of the slot
};

enum PlanMode : int { kPlanBatch = 0, kPlanRagged = 1, kPlanSingle = 2 };

struct PlanParams {
    int mode, rows, heads, paged;
    const int* d_slots;
    const int* d_len;
    const int* d_pos;
    const int* d_prefill_len;
    int fixed_slot, kv_len, prefill_len, q_start, causal;
    int* rs;        // [rows + 1] exclusive prefix sum of heads * units(row)
    RowInfo* info;  // [rows]
};

struct AttnParams {
    const float* q;
    float* out;
    const uint8_t* k_base;
    const uint8_t* v_base;
    const int32_t* table;
    int table_stride, num_blocks;
    long long slot_stride_bytes;  // contiguous layout: bytes between two slots' caches
    int row_stride_bytes;         // contiguous layout: bytes between two tokens
    int rows, heads, kv_heads, group;
    float scale_log2e;
    const int* rs;
    const RowInfo* info;
    float* part_acc;  // [2 * total_warps][head_dim]
    float* part_ml;   // [2 * total_warps][2]  (max in log2 domain, sum)
    int* status;
    int total_warps;
};

// -------------------------------------------------------------------------------------------------
// plan: per-row attended ranges and the prefix sum of unit counts (one CTA; rows are few)
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) rswa_plan_kernel(PlanParams p) {
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < p.rows; base += blockDim.x) {
        const int r = base + tid;
        int units = 0;
        if (r < p.rows) {
            int slot, len, pfx;
            if (p.mode == kPlanBatch) {
                slot = p.d_slots[r];
                len = p.d_len[slot];
            } else if (p.mode == kPlanRagged) {
                slot = p.d_slots[r];
                len = p.d_pos[r] + 1;
            } else {
                slot = p.fixed_slot;
                len = p.d_len ? p.d_len[p.paged ? slot : 0] : p.kv_len;
                if (p.causal) len = min(len, p.q_start + r + 1);
            }
            len = max(len, 0);
            RowInfo ri;
            ri.slot = slot;
            if (p.paged) {
                pfx = p.d_prefill_len ? p.d_prefill_len[slot] : p.prefill_len;
                pfx = max(pfx, 0);
                ri.pe = min(len, pfx);
                ri.re = len - ri.pe;
                ri.ring_off = (pfx + kBlockTokens - 1) / kBlockTokens;
            } else {
                ri.pe = len;
                ri.re = 0;
                ri.ring_off = 0;
            }
            p.info[r] = ri;
            units = ((ri.pe + kBlockTokens - 1) / kBlockTokens + (ri.re + kBlockTokens - 1) / kBlockTokens) *
                    p.heads;
        }
        // block-wide exclusive scan of `units`
        int incl = units;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = (lane < (int)(blockDim.x >> 5)) ? warp_sums[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += t;
            }
            warp_sums[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int carry = carry_s;
        const int before = carry + (warp ? warp_sums[warp - 1] : 0) + incl - units;
        if (r < p.rows) p.rs[r] = before;
        __syncthreads();
        if (tid == blockDim.x - 1) carry_s = before + units;
        __syncthreads();
    }
    if (tid == 0) p.rs[p.rows] = carry_s;
}

// -------------------------------------------------------------------------------------------------
// position on the unit line
// -------------------------------------------------------------------------------------------------
struct UnitCursor {
    int r, h, j, n;  // row, head, unit within the item, units per item of this row
    RowInfo info;
};

__device__ __forceinline__ void cursor_seek(UnitCursor& c, const AttnParams& p, long long u) {
    int lo = 0, hi = p.rows;  // rs[lo] <= u < rs[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)__ldg(p.rs + mid) <= u) lo = mid; else hi = mid;
    }
    c.r = lo;
    const int base = __ldg(p.rs + lo);
    c.n = (__ldg(p.rs + lo + 1) - base) / p.heads;
    const int rem = (int)(u - base);
    c.h = rem / c.n;
    c.j = rem - c.h * c.n;
    c.info = p.info[lo];
}

__device__ __forceinline__ void cursor_next(UnitCursor& c, const AttnParams& p) {
    if (++c.j < c.n) return;
    c.j = 0;
    if (++c.h < p.heads) return;
    c.h = 0;
    for (;;) {
        if (++c.r >= p.rows) { c.n = 0; return; }
        c.n = (__ldg(p.rs + c.r + 1) - __ldg(p.rs + c.r)) / p.heads;
        if (c.n > 0) break;
    }
    c.info = p.info[c.r];
}

__device__ __forceinline__ long long piece_start(long long w, long long total, int warps) {
    return (w * total) / warps;
}
// the warp whose piece holds unit u: the largest w with piece_start(w) <= u
__device__ __forceinline__ int piece_of(long long u, long long total, int warps) {
    return (int)(((u + 1) * warps - 1) / total);
}

// -------------------------------------------------------------------------------------------------
// reduce-scatter of N per-lane partial sums across the D*2 lanes that share a cache row:
// afterwards every lane holds one complete sum in v[0]
// -------------------------------------------------------------------------------------------------
template <int N, int D>
struct RowReduce {
    template <int ITER>
    __device__ static __forceinline__ void run(float (&v)[ITER], int lane) {
        if constexpr (D >= 1) {
            if constexpr (N > 1) {
                const bool upper = (lane & D) != 0;
#pragma unroll
                for (int k = 0; k < N / 2; ++k) {
                    const float send = upper ? v[k] : v[k + N / 2];
                    const float keep = upper ? v[k + N / 2] : v[k];
                    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, D);
                }
                RowReduce<N / 2, D / 2>::run(v, lane);
            } else {
                v[0] += __shfl_xor_sync(0xffffffffu, v[0], D);
                RowReduce<1, D / 2>::run(v, lane);
            }
        }
    }
};

// -------------------------------------------------------------------------------------------------
// partial attention
// -------------------------------------------------------------------------------------------------
template <typename KV, int HD, bool PAGED, int STAGES>
__global__ void __launch_bounds__(512, 1) rswa_attn_partial_kernel(const AttnParams p) {
    using M = TileMap<KV, HD>;
    constexpr int LPR = M::kLanesPerRow, CPL = M::kChunksPerLane, RPW = M::kRowsPerLoad;
    constexpr int ITER = M::kIters, EPC = KV::kPerChunk, EPL = M::kElemsPerLane;
    constexpr int ROWB = M::kRowBytes, TILE = M::kTileBytes;
    constexpr unsigned FULL = 0xffffffffu;

    extern __shared__ __align__(128) uint8_t smem[];
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * warps + warp;

    const int bar_bytes = (warps * STAGES * 2 * 8 + 127) & ~127;
    uint8_t* my_tiles = smem + bar_bytes + (size_t)warp * (STAGES * 2 * TILE);
    const uint32_t bar0 = smem_addr(smem) + warp * (STAGES * 2 * 8);
    const uint32_t tile0 = smem_addr(my_tiles);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES * 2; ++s) mbar_init(bar0 + 8 * s, 1);
        mbar_init_fence();
    }
    __syncwarp();

    const long long total = __ldg(p.rs + p.rows);
    if (total <= 0) return;
    const long long u0 = piece_start(gw, total, p.total_warps);
    const long long u1 = piece_start(gw + 1, total, p.total_warps);
    if (u0 >= u1) return;
    const int n_units = (int)(u1 - u0);

    const int g = lane % LPR;   // chunk position inside the row
    const int rg = lane / LPR;  // which of the RPW rows of a warp-wide load

    // ---- producer side: one stage = K tile + V tile of one unit ---------------------------------
    auto issue = [&](const UnitCursor& c, int stage) {
        const uint32_t kbar = bar0 + 16 * stage, vbar = kbar + 8;
        const uint32_t kdst = tile0 + stage * 2 * TILE, vdst = kdst + TILE;
        const int kvh = c.h / p.group;
        if constexpr (PAGED) {
            const int npb = (c.info.pe + kBlockTokens - 1) / kBlockTokens;
            const int idx = c.j < npb ? c.j : c.info.ring_off + (c.j - npb);
            int blk = 0;
            if (idx < p.table_stride) blk = __ldg(p.table + (size_t)c.info.slot * p.table_stride + idx);
            else if (lane == 0) atomicOr(p.status, kStatusBadSlot);
            if (blk < 0 || blk >= p.num_blocks) {
                if (lane == 0) atomicOr(p.status, kStatusBadBlock);
                blk = 0;
            }
            if (lane == 0) {
                const size_t off = ((size_t)blk * p.kv_heads + kvh) * (size_t)TILE;
                mbar_arrive_expect_tx(kbar, TILE);
                bulk_copy_g2s(kdst, p.k_base + off, TILE, kbar);
                mbar_arrive_expect_tx(vbar, TILE);
                bulk_copy_g2s(vdst, p.v_base + off, TILE, vbar);
            }
        } else {
            const int nvalid = min(kBlockTokens, c.info.pe - c.j * kBlockTokens);
            const size_t off = (size_t)c.info.slot * p.slot_stride_bytes +
                               (size_t)(c.j * kBlockTokens) * p.row_stride_bytes + (size_t)kvh * ROWB;
            if (lane == 0) {
                mbar_arrive_expect_tx(kbar, nvalid * ROWB);
                mbar_arrive_expect_tx(vbar, nvalid * ROWB);
            }
            const int t = lane & 15;
            if (t < nvalid) {
                const size_t roff = off + (size_t)t * p.row_stride_bytes;
                if (lane < 16) bulk_copy_g2s(kdst + t * ROWB, p.k_base + roff, ROWB, kbar);
                else bulk_copy_g2s(vdst + t * ROWB, p.v_base + roff, ROWB, vbar);
            }
        }
    };

    UnitCursor ic;  // issue cursor runs STAGES units ahead of the compute cursor
    cursor_seek(ic, p, u0);
    UnitCursor cc = ic;
    int issued = 0;
    for (; issued < STAGES && issued < n_units; ++issued) {
        issue(ic, issued);
        cursor_next(ic, p);
    }

    // ---- consumer state -------------------------------------------------------------------------
    float qreg[EPL], acc[EPL];
    float m_run = -INFINITY, l_run = 0.f;
    auto load_q = [&](const UnitCursor& c) {
        const float* qp = p.q + ((size_t)c.r * p.heads + c.h) * HD;
#pragma unroll
        for (int cp = 0; cp < CPL; ++cp) {
            const int d0 = (g + 32 * cp) * EPC;
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(qp + d0 + e));
                qreg[cp * EPC + e + 0] = t.x * p.scale_log2e;
                qreg[cp * EPC + e + 1] = t.y * p.scale_log2e;
                qreg[cp * EPC + e + 2] = t.z * p.scale_log2e;
                qreg[cp * EPC + e + 3] = t.w * p.scale_log2e;
            }
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
        m_run = -INFINITY;
        l_run = 0.f;
    };
    load_q(cc);
    bool first_segment = true;
    int seg_first_j = cc.j;

    for (int it = 0; it < n_units; ++it) {
        const int stage = it % STAGES;
        const uint32_t parity = (uint32_t)(it / STAGES) & 1u;
        const uint32_t kbar = bar0 + 16 * stage, vbar = kbar + 8;
        const uint8_t* ktile = my_tiles + stage * 2 * TILE;
        const uint8_t* vtile = ktile + TILE;

        int nvalid;
        {
            const int npb = (cc.info.pe + kBlockTokens - 1) / kBlockTokens;
            nvalid = cc.j < npb ? min(kBlockTokens, cc.info.pe - cc.j * kBlockTokens)
                                : min(kBlockTokens, cc.info.re - (cc.j - npb) * kBlockTokens);
        }

        // ---- scores: q . k for the 16 tokens of the tile ---------------------------------------
        if (!mbar_wait_bounded(kbar, parity, p.status)) return;
        float sc[ITER];
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int t = (i * RPW + rg) & (kBlockTokens - 1);
            float d = 0.f;
#pragma unroll
            for (int cp = 0; cp < CPL; ++cp) {
                const uint4 w = *reinterpret_cast<const uint4*>(ktile + t * ROWB + (g + 32 * cp) * 16);
                float f[EPC];
                KV::unpack(w, f);
#pragma unroll
                for (int e = 0; e < EPC; ++e) d = fmaf(qreg[cp * EPC + e], f[e], d);
            }
            sc[i] = d;
        }
        RowReduce<ITER, LPR / 2>::run(sc, lane);
        const int my_tok = (LPR >= 2 ? (g >> 1) * RPW : 0) + rg;
        const float s = (my_tok < nvalid) ? sc[0] : -INFINITY;

        // ---- online softmax, one running max per row group -------------------------------------
        float mt = s;
#pragma unroll
        for (int d = LPR / 2; d >= 2; d >>= 1) mt = fmaxf(mt, __shfl_xor_sync(FULL, mt, d));
        const float m_new = fmaxf(m_run, mt);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run - m_safe);
        const float pr = exp2f(s - m_safe);
        l_run = l_run * alpha + pr;
        m_run = m_new;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] *= alpha;

        // ---- acc += p . v ------------------------------------------------------------------------
        if (!mbar_wait_bounded(vbar, parity, p.status)) return;
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int t = i * RPW + rg;
            const float pi = (LPR >= 2) ? __shfl_sync(FULL, pr, rg * LPR + 2 * i) : pr;
            if (t < nvalid) {
#pragma unroll
                for (int cp = 0; cp < CPL; ++cp) {
                    const uint4 w = *reinterpret_cast<const uint4*>(vtile + t * ROWB + (g + 32 * cp) * 16);
                    float f[EPC];
                    KV::unpack(w, f);
#pragma unroll
                    for (int e = 0; e < EPC; ++e) acc[cp * EPC + e] = fmaf(pi, f[e], acc[cp * EPC + e]);
                }
            }
        }

        // ---- this stage is free again: refill it ------------------------------------------------
        __syncwarp();
        if (issued < n_units) {
            issue(ic, stage);
            cursor_next(ic, p);
            ++issued;
        }

        // ---- end of an item (or of the piece): emit ----------------------------------------------
        const bool item_done = (cc.j == cc.n - 1);
        const bool piece_done = (it == n_units - 1);
        if (item_done || piece_done) {
            float mx = m_run;
#pragma unroll
            for (int d = LPR; d < 32; d <<= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, d));
            const float mx_safe = (mx == -INFINITY) ? 0.f : mx;
            const float wgt = exp2f(m_run - mx_safe);
            float lsum = l_run * wgt;
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) lsum += __shfl_xor_sync(FULL, lsum, d);
            if (LPR >= 2) lsum *= 0.5f;  // the two lanes of a pair carry the same token
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                float a = acc[e] * wgt;
#pragma unroll
                for (int d = LPR; d < 32; d <<= 1) a += __shfl_xor_sync(FULL, a, d);
                acc[e] = a;
            }
            const bool whole = item_done && seg_first_j == 0;
            if (lane < LPR) {
                float* dst;
                float mul;
                if (whole) {
                    dst = p.out + ((size_t)cc.r * p.heads + cc.h) * HD;
                    mul = lsum > 0.f ? 1.f / lsum : 0.f;
                } else {
                    dst = p.part_acc + (size_t)(2 * gw + (first_segment ? 0 : 1)) * HD;
                    mul = 1.f;
                }
#pragma unroll
                for (int cp = 0; cp < CPL; ++cp) {
                    const int d0 = (g + 32 * cp) * EPC;
#pragma unroll
                    for (int e = 0; e < EPC; e += 4)
                        *reinterpret_cast<float4*>(dst + d0 + e) =
                            make_float4(acc[cp * EPC + e] * mul, acc[cp * EPC + e + 1] * mul,
                                        acc[cp * EPC + e + 2] * mul, acc[cp * EPC + e + 3] * mul);
                }
                if (!whole && lane == 0) {
                    float* ml = p.part_ml + (size_t)(2 * gw + (first_segment ? 0 : 1)) * 2;
                    ml[0] = mx;
                    ml[1] = lsum;
                }
            }
            first_segment = false;
            if (!piece_done) {
                cursor_next(cc, p);
                seg_first_j = 0;
                load_q(cc);
            }
        } else {
            cursor_next(cc, p);
        }
    }
}

// -------------------------------------------------------------------------------------------------
// merge: one warp per (row, head) item
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rswa_attn_merge_kernel(const AttnParams p, int head_dim) {
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= p.rows * p.heads) return;
    const int r = item / p.heads, h = item - r * p.heads;
    const int base = __ldg(p.rs + r);
    const int n = (__ldg(p.rs + r + 1) - base) / p.heads;
    float* out = p.out + (size_t)item * head_dim;
    if (n == 0) {
        for (int d = lane; d < head_dim; d += 32) out[d] = 0.f;
        return;
    }
    const long long total = __ldg(p.rs + p.rows);
    const long long s0 = (long long)base + (long long)h * n;
    const int wf = piece_of(s0, total, p.total_warps);
    const int wl = piece_of(s0 + n - 1, total, p.total_warps);
    if (wf == wl) return;  // written directly by the partial kernel

    float mx = -INFINITY;
    for (int w = wf; w <= wl; ++w) {
        const long long a = piece_start(w, total, p.total_warps);
        if (a >= piece_start(w + 1, total, p.total_warps)) continue;
        const int slot = 2 * w + ((w == wf && a < s0) ? 1 : 0);
        mx = fmaxf(mx, p.part_ml[2 * slot]);
    }
    const float mx_safe = (mx == -INFINITY) ? 0.f : mx;
    float lsum = 0.f;
    float accv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) accv[i] = 0.f;
    for (int w = wf; w <= wl; ++w) {
        const long long a = piece_start(w, total, p.total_warps);
        if (a >= piece_start(w + 1, total, p.total_warps)) continue;
        const int slot = 2 * w + ((w == wf && a < s0) ? 1 : 0);
        const float wgt = exp2f(p.part_ml[2 * slot] - mx_safe);
        lsum += p.part_ml[2 * slot + 1] * wgt;
        const float* pa = p.part_acc + (size_t)slot * head_dim;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) accv[i] = fmaf(pa[d], wgt, accv[i]);
        }
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) out[d] = accv[i] * inv;
    }
}

}  // namespace uocr_b200
