// Split-KV R-SWA attention for sm_100a: plan, then one persistent attention kernel fed by bulk
// async copies (TMA engine) through per-warp shared-memory rings; partial results of items that
// straddle two warps are combined in the same launch by whichever warp finishes the item last.
//
// Work model.  A query row r with H heads attends n_r "units" per head; a unit is one 16-token tile
// of one KV head (a paged block, or 16 consecutive rows of a contiguous cache).  All units of a
// launch are laid out on one line, ordered (row, head, unit), and cut into equal pieces, one per
// warp of a persistent grid.  A warp walks its piece with a private ring of shared-memory stages;
// one lane issues `cp.async.bulk` copies that signal an mbarrier per tile, and the whole warp
// consumes tiles with 16-byte shared loads, warp-shuffle reductions and an online softmax in the
// exp2 domain.  A piece that covers a whole (row, head) item writes the output directly; otherwise
// the warp leaves an un-normalised partial (max, sum, accumulator) in scratch, bumps the item's
// arrival counter, and the last arriver merges (no warp ever waits for another).
//
// The fused decode step (FUSED = true) additionally plans in shared memory from the pre-append
// cursors, patches the freshly appended token into the tile that holds its ring slot (and writes it
// to the pool), and lets the last CTA to finish publish the new cursors: one launch per layer.
//
// Semantics follow RSWACache::attention (src/scheduler/kv_cache.cpp:84-130): scale 1/sqrt(d),
// softmax over the attended slots, 0 for an empty set; decode is order-independent in the slot
// index, so ring slots are visited in storage order.  The append follows
// RSWACache::append_decode (src/scheduler/kv_cache.cpp:54-82).
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

struct RowInfo {
    int slot;  // cache slot of this query row
    int pe;    // attended tokens in the fixed (prefix) region; ring blocks start at table index ceil(pe/16)
    int re;    // attended tokens in the ring region (re > 0 implies pe == prefix length)
    int aux;   // fused step: (unit index << 4 | offset) of the token appended this step;
               // text prefill: (first block of the window in the text pool << 4 | tokens to skip in it);
               // else -1
};

// kPlanPrefillText: packed text rows of several requests during prefill.  Row t is text token
// d_pos[t] of slot d_slots[t]; it attends the slot's whole fixed region plus the text window
// (d_pos[t] - window, d_pos[t]] held in a separate text pool whose blocks for this request start
// at block d_text_block0[t].
enum PlanMode : int { kPlanBatch = 0, kPlanRagged = 1, kPlanSingle = 2, kPlanDecodeStep = 3, kPlanPrefillText = 4 };

struct PlanParams {
    int mode, rows, heads, paged;
    const int* d_slots;
    const int* d_len;
    const int* d_ring_pos;
    const int* d_pos;
    const int* d_prefill_len;
    const int* d_text_block0;
    int fixed_slot, kv_len, prefill_len, q_start, causal, window;
    int* rs;        // [rows + 1] exclusive prefix sum of heads * units(row)
    RowInfo* info;  // [rows]
    float* out;     // rows that attend nothing are zero-filled here
    int out_row_elems;
};

struct AttnParams {
    const float* q;
    float* out;
    const uint8_t* k_base;
    const uint8_t* v_base;
    const uint8_t* k_text;  // text prefill: second pool (same block layout) holding the window tokens
    const uint8_t* v_text;
    int text_blocks;
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
    int* counters;    // [total_warps] arrival counters, zero between launches
    int* status;
    int total_warps;
    // fused decode step only
    PlanParams plan;
    const float* k_new;
    const float* v_new;
    int* d_len;
    int* d_ring_pos;
    int* done_ctas;
};

// -------------------------------------------------------------------------------------------------
// plan: per-row attended ranges and the prefix sum of unit counts
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ int plan_row(const PlanParams& p, int r, RowInfo& ri) {
    int slot, len;
    ri.aux = -1;
    if (p.mode == kPlanBatch) {
        slot = p.d_slots[r];
        len = p.d_len[slot];
    } else if (p.mode == kPlanRagged) {
        slot = p.d_slots[r];
        len = p.d_pos[r] + 1;
    } else if (p.mode == kPlanSingle) {
        slot = p.fixed_slot;
        len = p.d_len ? p.d_len[p.paged ? slot : 0] : p.kv_len;
        if (p.causal) len = min(len, p.q_start + r + 1);
    } else if (p.mode == kPlanPrefillText) {
        slot = p.d_slots[r];
        const int i = p.d_pos[r];
        const int lo = max(0, i - p.window + 1);
        ri.slot = slot;
        ri.pe = max(p.d_prefill_len[slot], 0);
        ri.re = i - lo + 1;
        const int skip = lo & (kBlockTokens - 1);
        ri.aux = ((p.d_text_block0[r] + lo / kBlockTokens) << 4) | skip;
        return ((ri.pe + kBlockTokens - 1) / kBlockTokens + (skip + ri.re + kBlockTokens - 1) / kBlockTokens) * p.heads;
    } else {  // decode step: lengths as they will be after this step's append
        slot = p.d_slots[r];
        const int pfx = p.d_prefill_len[slot];
        const int cur = p.d_len[slot];
        int row;
        if (cur < pfx + p.window) {
            row = cur;
            len = cur + 1;
        } else {
            row = pfx + p.d_ring_pos[slot];
            len = cur;
        }
        const int rr = row - pfx;
        ri.aux = rr >= 0 ? ((((pfx + kBlockTokens - 1) / kBlockTokens + rr / kBlockTokens) << 4) | (rr & 15)) : -2;
    }
    len = max(len, 0);
    ri.slot = slot;
    if (p.paged) {
        int pfx = p.d_prefill_len ? p.d_prefill_len[slot] : p.prefill_len;
        pfx = max(pfx, 0);
        ri.pe = min(len, pfx);
        ri.re = len - ri.pe;
    } else {
        ri.pe = len;
        ri.re = 0;
    }
    return ((ri.pe + kBlockTokens - 1) / kBlockTokens + (ri.re + kBlockTokens - 1) / kBlockTokens) * p.heads;
}

// Block-wide: fills rs[0..rows] and info[0..rows) (global or shared memory).  `scratch` = 33 ints
// of shared memory.
__device__ __forceinline__ void plan_all_rows(const PlanParams& p, int* rs, RowInfo* info, int* scratch) {
    int* warp_sums = scratch;
    int* carry_s = scratch + 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = blockDim.x;
    if (tid == 0) *carry_s = 0;
    __syncthreads();
    for (int base = 0; base < p.rows; base += nthreads) {
        const int r = base + tid;
        int units = 0;
        if (r < p.rows) {
            RowInfo ri;
            units = plan_row(p, r, ri);
            info[r] = ri;
            if (units == 0 && p.out)
                for (int i = 0; i < p.out_row_elems; ++i) p.out[(size_t)r * p.out_row_elems + i] = 0.f;
        }
        int incl = units;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = (lane < (nthreads >> 5)) ? warp_sums[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += t;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int before = *carry_s + (warp ? warp_sums[warp - 1] : 0) + incl - units;
        if (r < p.rows) rs[r] = before;
        __syncthreads();
        if (tid == nthreads - 1) *carry_s = before + units;
        __syncthreads();
    }
    if (tid == 0) rs[p.rows] = *carry_s;
}

__global__ void __launch_bounds__(1024) rswa_plan_kernel(PlanParams p) {
    __shared__ int scratch[33];
    plan_all_rows(p, p.rs, p.info, scratch);
}

// -------------------------------------------------------------------------------------------------
// position on the unit line
// -------------------------------------------------------------------------------------------------
struct UnitCursor {
    int r, h, j, n;  // row, head, unit within the item, units per item of this row
    RowInfo info;
};

__device__ __forceinline__ void cursor_seek(UnitCursor& c, const int* rs, const RowInfo* info, int rows,
                                            int heads, long long u) {
    int lo = 0, hi = rows;  // rs[lo] <= u < rs[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)rs[mid] <= u) lo = mid; else hi = mid;
    }
    c.r = lo;
    const int base = rs[lo];
    c.n = (rs[lo + 1] - base) / heads;
    const int rem = (int)(u - base);
    c.h = rem / c.n;
    c.j = rem - c.h * c.n;
    c.info = info[lo];
}

__device__ __forceinline__ void cursor_next(UnitCursor& c, const int* rs, const RowInfo* info, int rows,
                                            int heads) {
    if (++c.j < c.n) return;
    c.j = 0;
    if (++c.h < heads) return;
    c.h = 0;
    for (;;) {
        if (++c.r >= rows) { c.n = 0; return; }
        c.n = (rs[c.r + 1] - rs[c.r]) / heads;
        if (c.n > 0) break;
    }
    c.info = info[c.r];
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

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// -------------------------------------------------------------------------------------------------
// attention
// -------------------------------------------------------------------------------------------------
template <typename KV, int HD, bool PAGED, bool FUSED, int STAGES>
__global__ void __launch_bounds__(512, 1) rswa_attn_kernel(const AttnParams p) {
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

    // ---- the plan: global (made by rswa_plan_kernel) or built here in shared memory ----------------
    const int* rs = p.rs;
    const RowInfo* info = p.info;
    if constexpr (FUSED) {
        uint8_t* plan_base = smem + bar_bytes + (size_t)warps * (STAGES * 2 * TILE);
        RowInfo* info_s = reinterpret_cast<RowInfo*>(plan_base);
        int* rs_s = reinterpret_cast<int*>(plan_base + sizeof(RowInfo) * p.rows);
        int* scratch = rs_s + p.rows + 1;
        plan_all_rows(p.plan, rs_s, info_s, scratch);
        __syncthreads();
        rs = rs_s;
        info = info_s;
    }

    const long long total = rs[p.rows];
    const int nw = (int)min((long long)p.total_warps, total);  // every piece is non-empty
    int n_units = 0;
    long long u0 = 0;
    if (gw < nw) {
        u0 = piece_start(gw, total, nw);
        n_units = (int)(piece_start(gw + 1, total, nw) - u0);
    }

    const int g = lane % LPR;   // chunk position inside the row
    const int rg = lane / LPR;  // which of the RPW rows of a warp-wide load

    // ---- producer side: one stage = K tile + V tile of one unit ---------------------------------
    auto issue = [&](const UnitCursor& c, int stage) {
        const uint32_t kbar = bar0 + 16 * stage, vbar = kbar + 8;
        const uint32_t kdst = tile0 + stage * 2 * TILE, vdst = kdst + TILE;
        const int kvh = c.h / p.group;
        if constexpr (PAGED) {
            // table row = prefix blocks, then ring blocks right after them (ceil(pe/16) prefix units
            // come first on the unit line too), so the unit index is the table index
            const int idx = c.j;
            int blk = 0;
            const uint8_t* kb = p.k_base;
            const uint8_t* vb = p.v_base;
            bool from_text = false;
            if constexpr (!FUSED) {
                // text prefill: units past the fixed region come from the text pool, consecutive blocks
                from_text = p.k_text != nullptr && idx >= (c.info.pe + kBlockTokens - 1) / kBlockTokens;
            }
            if (from_text) {
                blk = (c.info.aux >> 4) + (idx - (c.info.pe + kBlockTokens - 1) / kBlockTokens);
                kb = p.k_text;
                vb = p.v_text;
                if (blk < 0 || blk >= p.text_blocks) {
                    if (lane == 0) atomicOr(p.status, kStatusBadBlock);
                    blk = 0;
                }
            } else {
                if (idx < p.table_stride) blk = __ldg(p.table + (size_t)c.info.slot * p.table_stride + idx);
                else if (lane == 0) atomicOr(p.status, kStatusBadSlot);
                if (blk < 0 || blk >= p.num_blocks) {
                    if (lane == 0) atomicOr(p.status, kStatusBadBlock);
                    blk = 0;
                }
            }
            if (lane == 0) {
                const size_t off = ((size_t)blk * p.kv_heads + kvh) * (size_t)TILE;
                mbar_arrive_expect_tx(kbar, TILE);
                bulk_copy_g2s(kdst, kb + off, TILE, kbar);
                mbar_arrive_expect_tx(vbar, TILE);
                bulk_copy_g2s(vdst, vb + off, TILE, vbar);
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

    if (n_units > 0) {
        UnitCursor ic;  // issue cursor runs STAGES units ahead of the compute cursor
        cursor_seek(ic, rs, info, p.rows, p.heads, u0);
        UnitCursor cc = ic;
        int issued = 0;
        for (; issued < STAGES && issued < n_units; ++issued) {
            issue(ic, issued);
            cursor_next(ic, rs, info, p.rows, p.heads);
        }

        // ---- consumer state ---------------------------------------------------------------------
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
        int pend_r0 = 0, pend_h0 = 0, pend_r1 = 0, pend_h1 = 0, pend_n = 0;  // partial segments left in scratch
        bool gave_up = false;

        for (int it = 0; it < n_units; ++it) {
            const int stage = it % STAGES;
            const uint32_t parity = (uint32_t)(it / STAGES) & 1u;
            const uint32_t kbar = bar0 + 16 * stage, vbar = kbar + 8;
            uint8_t* ktile = my_tiles + stage * 2 * TILE;
            uint8_t* vtile = ktile + TILE;

            int nvalid, nskip = 0;  // tokens [nskip, nvalid) of this tile are attended
            {
                const int npb = (cc.info.pe + kBlockTokens - 1) / kBlockTokens;
                if (cc.j < npb) {
                    nvalid = min(kBlockTokens, cc.info.pe - cc.j * kBlockTokens);
                } else {
                    int lead = 0;  // text prefill: the window may start inside its first block
                    if constexpr (PAGED && !FUSED) lead = p.k_text != nullptr ? (cc.info.aux & 15) : 0;
                    const int jr = cc.j - npb;
                    nvalid = min(kBlockTokens, lead + cc.info.re - jr * kBlockTokens);
                    nskip = jr == 0 ? lead : 0;
                }
            }
            // fused step: does this tile hold the ring slot that receives the new token?
            bool patch = false;
            if constexpr (FUSED) patch = cc.info.aux >= 0 && (cc.info.aux >> 4) == cc.j;

            // ---- scores: q . k for the 16 tokens of the tile -----------------------------------
            if (!mbar_wait_bounded(kbar, parity, p.status)) { gave_up = true; break; }
            if constexpr (FUSED) {
                if (patch) {  // lanes 0..kChunks-1 convert one 16-byte chunk of the new K row each
                    const int kvh = cc.h / p.group, off = cc.info.aux & 15;
                    for (int ch = lane; ch < M::kChunks; ch += 32) {
                        const float* src = p.k_new + ((size_t)cc.r * p.kv_heads + kvh) * HD + ch * EPC;
                        uint4 w;
                        if constexpr (EPC == 8) {
                            const float4 a = __ldg(reinterpret_cast<const float4*>(src));
                            const float4 b = __ldg(reinterpret_cast<const float4*>(src + 4));
                            w = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                                           pack_bf16x2(b.z, b.w));
                        } else {
                            w = __ldg(reinterpret_cast<const uint4*>(src));
                        }
                        *reinterpret_cast<uint4*>(ktile + off * ROWB + ch * 16) = w;
                        if (cc.h % p.group == 0) {
                            const int blk = __ldg(p.table + (size_t)cc.info.slot * p.table_stride + cc.j);
                            if (blk >= 0 && blk < p.num_blocks)
                                *reinterpret_cast<uint4*>(const_cast<uint8_t*>(p.k_base) +
                                                          ((size_t)blk * p.kv_heads + kvh) * (size_t)TILE +
                                                          off * ROWB + ch * 16) = w;
                        }
                    }
                    __syncwarp();
                }
            }
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
            const float s = (my_tok >= nskip && my_tok < nvalid) ? sc[0] : -INFINITY;

            // ---- online softmax, one running max per row group ---------------------------------
            float mt = s;
#pragma unroll
            for (int d = LPR / 2; d >= 2; d >>= 1) mt = fmaxf(mt, __shfl_xor_sync(FULL, mt, d));
            const float m_new = fmaxf(m_run, mt);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = fast_exp2(m_run - m_safe);
            const float pr = fast_exp2(s - m_safe);
            l_run = l_run * alpha + pr;
            m_run = m_new;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] *= alpha;

            // ---- acc += p . v ----------------------------------------------------------------------
            if (!mbar_wait_bounded(vbar, parity, p.status)) { gave_up = true; break; }
            if constexpr (FUSED) {
                if (patch) {
                    const int kvh = cc.h / p.group, off = cc.info.aux & 15;
                    for (int ch = lane; ch < M::kChunks; ch += 32) {
                        const float* src = p.v_new + ((size_t)cc.r * p.kv_heads + kvh) * HD + ch * EPC;
                        uint4 w;
                        if constexpr (EPC == 8) {
                            const float4 a = __ldg(reinterpret_cast<const float4*>(src));
                            const float4 b = __ldg(reinterpret_cast<const float4*>(src + 4));
                            w = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                                           pack_bf16x2(b.z, b.w));
                        } else {
                            w = __ldg(reinterpret_cast<const uint4*>(src));
                        }
                        *reinterpret_cast<uint4*>(vtile + off * ROWB + ch * 16) = w;
                        if (cc.h % p.group == 0) {
                            const int blk = __ldg(p.table + (size_t)cc.info.slot * p.table_stride + cc.j);
                            if (blk >= 0 && blk < p.num_blocks)
                                *reinterpret_cast<uint4*>(const_cast<uint8_t*>(p.v_base) +
                                                          ((size_t)blk * p.kv_heads + kvh) * (size_t)TILE +
                                                          off * ROWB + ch * 16) = w;
                        }
                    }
                    __syncwarp();
                }
            }
            if (nvalid == kBlockTokens && nskip == 0) {
#pragma unroll
                for (int i = 0; i < ITER; ++i) {
                    const int t = (i * RPW + rg) & (kBlockTokens - 1);
                    float pi = (LPR >= 2) ? __shfl_sync(FULL, pr, rg * LPR + 2 * i) : pr;
                    if (RPW > kBlockTokens && rg >= kBlockTokens) pi = 0.f;
#pragma unroll
                    for (int cp = 0; cp < CPL; ++cp) {
                        const uint4 w = *reinterpret_cast<const uint4*>(vtile + t * ROWB + (g + 32 * cp) * 16);
                        float f[EPC];
                        KV::unpack(w, f);
#pragma unroll
                        for (int e = 0; e < EPC; ++e) acc[cp * EPC + e] = fmaf(pi, f[e], acc[cp * EPC + e]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < ITER; ++i) {
                    const int t = i * RPW + rg;
                    const float pi = (LPR >= 2) ? __shfl_sync(FULL, pr, rg * LPR + 2 * i) : pr;
                    if (t >= nskip && t < nvalid) {  // rows outside the valid range may hold anything
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
            }

            // ---- this stage is free again: refill it ------------------------------------------------
            __syncwarp();
            if constexpr (FUSED) {
                if (patch) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            if (issued < n_units) {
                issue(ic, stage);
                cursor_next(ic, rs, info, p.rows, p.heads);
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
                const float wgt = fast_exp2(m_run - mx_safe);
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
                float* out_item = p.out + ((size_t)cc.r * p.heads + cc.h) * HD;
                if (whole) {
                    if (lane < LPR) {
                        const float mul = lsum > 0.f ? 1.f / lsum : 0.f;
#pragma unroll
                        for (int cp = 0; cp < CPL; ++cp) {
                            const int d0 = (g + 32 * cp) * EPC;
#pragma unroll
                            for (int e = 0; e < EPC; e += 4)
                                *reinterpret_cast<float4*>(out_item + d0 + e) =
                                    make_float4(acc[cp * EPC + e] * mul, acc[cp * EPC + e + 1] * mul,
                                                acc[cp * EPC + e + 2] * mul, acc[cp * EPC + e + 3] * mul);
                        }
                    }
                } else {
                    // leave a partial, then see whether every other piece of this item has arrived
                    const int my_slot = 2 * gw + (first_segment ? 0 : 1);
                    if (lane < LPR) {
                        float* dst = p.part_acc + (size_t)my_slot * HD;
#pragma unroll
                        for (int cp = 0; cp < CPL; ++cp) {
                            const int d0 = (g + 32 * cp) * EPC;
#pragma unroll
                            for (int e = 0; e < EPC; e += 4)
                                __stcg(reinterpret_cast<float4*>(dst + d0 + e),
                                       make_float4(acc[cp * EPC + e], acc[cp * EPC + e + 1], acc[cp * EPC + e + 2],
                                                   acc[cp * EPC + e + 3]));
                        }
                        if (lane == 0) {
                            __stcg(p.part_ml + 2 * my_slot, mx);
                            __stcg(p.part_ml + 2 * my_slot + 1, lsum);
                        }
                    }
                    // the arrival (fence + counter) is deferred to the end of the piece so that one
                    // fence covers both partial segments and no copy is in flight when it executes
                    if (pend_n == 0) { pend_r0 = cc.r; pend_h0 = cc.h; } else { pend_r1 = cc.r; pend_h1 = cc.h; }
                    ++pend_n;
                }
                first_segment = false;
                if (!piece_done) {
                    cursor_next(cc, rs, info, p.rows, p.heads);
                    seg_first_j = 0;
                    load_q(cc);
                }
            } else {
                cursor_next(cc, rs, info, p.rows, p.heads);
            }
        }

        // ---- arrivals: whoever completes an item's set of partials merges them ------------------------
        if (pend_n > 0 && !gave_up) {
            __threadfence();  // this warp's partial stores are visible before its arrivals
            for (int k = 0; k < pend_n; ++k) {
                const int r = k ? pend_r1 : pend_r0, h = k ? pend_h1 : pend_h0;
                const int n = (rs[r + 1] - rs[r]) / p.heads;
                const long long s0 = (long long)rs[r] + (long long)h * n;
                const int wf = piece_of(s0, total, nw);
                const int wl = piece_of(s0 + n - 1, total, nw);
                int last = 0;
                if (lane == 0) {
                    const int old = atomicAdd(p.counters + wf, 1);
                    if (old == wl - wf) {
                        last = 1;
                        p.counters[wf] = 0;  // ready for the next launch
                    }
                }
                last = __shfl_sync(FULL, last, 0);
                if (!last) continue;
                __threadfence();  // the other arrivers' partials are visible after their arrivals
                float* out_item = p.out + ((size_t)r * p.heads + h) * HD;
                float mall = -INFINITY;
                for (int w = wf; w <= wl; ++w) {
                    const int slot = 2 * w + ((w == wf && piece_start(w, total, nw) < s0) ? 1 : 0);
                    mall = fmaxf(mall, __ldcg(p.part_ml + 2 * slot));
                }
                const float mall_safe = (mall == -INFINITY) ? 0.f : mall;
                float lall = 0.f;
                float o[(HD + 31) / 32];
#pragma unroll
                for (int i = 0; i < (HD + 31) / 32; ++i) o[i] = 0.f;
                for (int w = wf; w <= wl; ++w) {
                    const int slot = 2 * w + ((w == wf && piece_start(w, total, nw) < s0) ? 1 : 0);
                    const float wg = fast_exp2(__ldcg(p.part_ml + 2 * slot) - mall_safe);
                    lall += __ldcg(p.part_ml + 2 * slot + 1) * wg;
                    const float* pa = p.part_acc + (size_t)slot * HD;
#pragma unroll
                    for (int i = 0; i < (HD + 31) / 32; ++i) {
                        const int d = lane + 32 * i;
                        if (d < HD) o[i] = fmaf(__ldcg(pa + d), wg, o[i]);
                    }
                }
                const float inv = lall > 0.f ? 1.f / lall : 0.f;
#pragma unroll
                for (int i = 0; i < (HD + 31) / 32; ++i) {
                    const int d = lane + 32 * i;
                    if (d < HD) out_item[d] = o[i] * inv;
                }
            }
        }
    }

    // (arrivals of this warp's partial segments happen inside the block above)
    // ---- fused step: the last CTA to finish publishes the new cursors -------------------------------
    if constexpr (FUSED) {
        __shared__ int is_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const int old = atomicAdd(p.done_ctas, 1);
            is_last = (old == (int)gridDim.x - 1);
            if (is_last) *p.done_ctas = 0;
        }
        __syncthreads();
        if (is_last) {
            // every CTA has planned from the old cursors by now; nobody reads them again in this launch
            for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
                const int slot = p.plan.d_slots[r];
                const int pfx = p.plan.d_prefill_len[slot];
                const int cur = p.d_len[slot];
                if (cur < pfx + p.plan.window) {
                    p.d_len[slot] = cur + 1;
                    if (cur + 1 >= pfx + p.plan.window) p.d_ring_pos[slot] = 0;
                } else {
                    p.d_ring_pos[slot] = (p.d_ring_pos[slot] + 1) % p.plan.window;
                }
            }
        }
    }
}

}  // namespace uocr_b200
