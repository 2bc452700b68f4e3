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
// arrival counter, and the last arriver merges (no warp ever waits for another).  Every tile copy
// names an L2 eviction policy: ring tiles are read once per launch and leave L2 first, tiles of the
// fixed region are re-read by every sequence sharing the prefix and leave last.
//
// The fused decode step (FUSED = true) additionally plans in shared memory from the pre-append
// cursors, patches the freshly appended token into the tile that holds its ring slot (and writes it
// to the pool), and lets the last CTA to have planned store the new cursors: one launch per layer.
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
    int out_bf16;  // 1: `out` holds bf16 [rows][heads * head_dim] (round-to-nearest-even on the raw bits), else fp32
    const uint8_t* k_base;
    const uint8_t* v_base;
    const uint8_t* k_text;  // text prefill: second pool (same block layout) holding the window tokens
    const uint8_t* v_text;
    int text_blocks;
    const int32_t* table;
    int table_stride, num_blocks;
    int slot_rows;         // contiguous layout: cache rows per slot (batch_cap)
    int row_stride_bytes;  // contiguous layout: bytes between two tokens
    int rows, heads, kv_heads, group;
    float scale_log2e;
    const int* rs;
    const RowInfo* info;
    float* part_acc;  // [2 * pieces][head_dim]
    float* part_ml;   // [2 * pieces][2]  (max in log2 domain, sum)
    int* counters;    // [pieces] arrival counters, zero between launches
    int* status;
    uint32_t wait_limit;  // polls a tile wait may take before the warp gives up (kWaitLimit unless a test lowers it)
    int total_warps;
    // fused decode step with rotary embedding: q and the new k row are rotated on the fly
    // (uocr::cuda::rope, src/kernels/cuda/rope_fused.cu:12-40; src/kernels/cpu_ops.cpp:157-180)
    const int* rope_pos;    // [rows] position of each batch row
    float rope_freq[128];   // theta^(-2i/head_dim), i < head_dim/2, computed on the host in fp32
    // fused decode step only
    PlanParams plan;
    const float* k_new;
    const float* v_new;
    int* d_len;
    int* d_ring_pos;
    int late_cta;       // overlapped launches, even split: sixteenths of a share the last CTA's warps give up (0: none)
    int* planned_ctas;  // ticket counter: CTAs that have built their plan from the pre-append cursors; wraps to zero
                        // with the last ticket of a launch (atomicInc), so nothing has to reset it
};

// -------------------------------------------------------------------------------------------------
// plan: per-row attended ranges and the prefix sum of unit counts
// -------------------------------------------------------------------------------------------------
// `next_len` / `next_ring` (decode step only, may be null): the cursor values the step leaves behind for
// this row's slot, -1 where the reference's append leaves the cursor as it is.
__device__ __forceinline__ int plan_row(const PlanParams& p, int r, RowInfo& ri, int* next_len = nullptr,
                                        int* next_ring = nullptr) {
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
        int row, nl = -1, nr = -1;
        if (cur < pfx + p.window) {
            row = cur;
            len = cur + 1;
            nl = cur + 1;
            if (cur + 1 >= pfx + p.window) nr = 0;
        } else {
            const int ring = p.d_ring_pos[slot];
            row = pfx + ring;
            len = cur;
            nr = (ring + 1) % p.window;
        }
        if (next_len) {
            *next_len = nl;
            *next_ring = nr;
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
__device__ __forceinline__ void plan_all_rows(const PlanParams& p, int* rs, RowInfo* info, int* scratch,
                                              int* next_len = nullptr, int* next_ring = nullptr) {
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
            units = next_len ? plan_row(p, r, ri, next_len + r, next_ring + r) : plan_row(p, r, ri);
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

// How the unit line [0, total) is cut into pieces: one piece per warp of the persistent grid, consecutive
// and non-empty, so an item spans pieces of(first unit) .. of(last unit).
struct PieceMap {
    long long total;
    int ns;           // number of pieces: min(total warps, total units)
    int wpc;          // warps per CTA
    // Even split under launch overlap: the warps of the last CTA carry (16 - late) / 16 of a share.  CTAs of
    // an overlapped launch move in as their predecessor's CTAs leave, in block order, so the last block starts
    // several microseconds after the others (it cannot hide its prologue) and would finish last by as much.
    int late;
    long long wtot;   // sum of the piece weights (16 each, 16 - late for the last CTA's)
    __device__ __forceinline__ long long weight_before(int k) const {
        const int n1 = ns - wpc;
        return k <= n1 ? 16LL * k : 16LL * n1 + (long long)(16 - late) * (k - n1);
    }
    __device__ __forceinline__ long long start(int k) const {
        return late ? (total * weight_before(k)) / wtot : ((long long)k * total) / ns;
    }
    __device__ __forceinline__ long long end(int k) const { return k + 1 < ns ? start(k + 1) : total; }
    __device__ __forceinline__ int of(long long u) const {
        if (!late) return (int)(((u + 1) * ns - 1) / total);
        // the last piece whose weight prefix w satisfies floor(total * w / wtot) <= u
        const long long a = ((u + 1) * wtot - 1) / total;
        const int n1 = ns - wpc;
        if (a < 16LL * n1) return (int)(a / 16);
        const int k = n1 + (int)((a - 16LL * n1) / (16 - late));
        return k < ns ? k : ns - 1;
    }
};

constexpr int kPendMax = 4;  // per-warp list of partial segments awaiting their arrival (a piece leaves at most two)

// Whether the uneven (late-CTA) split applies to a launch: enough units that no piece can be empty and few
// enough that the bounds fit the arithmetic.
__device__ __forceinline__ bool uneven_split_ok(long long total, int total_warps) {
    return total >= 8LL * total_warps && total < (1LL << 26);
}

__device__ __forceinline__ PieceMap make_piece_map(long long total, int total_warps, int wpc, int late = 0) {
    PieceMap m;
    m.total = total;
    m.wpc = wpc;
    m.late = 0;
    m.wtot = 0;
    m.ns = (int)min((long long)total_warps, total);
    if (late > 0 && m.ns == total_warps && m.ns > wpc && uneven_split_ok(total, total_warps)) {
        m.late = min(late, 12);
        m.wtot = 16LL * m.ns - (long long)m.late * wpc;
    }
    return m;
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
// Tile slots per warp, and how many of them are kept in flight once the loop runs.  Two in flight (the K
// and the V tile of one unit, or V(u) and K(u+1)) measured faster than three at every size tried (16 to 512
// sequences, W = 1024 and 4096: 2-5 % per step): sixteen warps per SM already hold several times the bytes
// in flight that the memory latency asks for, and more only lengthens the queues in front of the memory.
// One is slower at small sizes.  UOCR_RING slots are filled before the loop starts -- under launch overlap
// that is while the previous launch drains and the memory has room -- and UOCR_STEADY are refilled.
#ifndef UOCR_RING
#define UOCR_RING 2
#endif
#ifndef UOCR_ATTN_THREADS
#define UOCR_ATTN_THREADS 512  // threads per CTA the attention kernel is compiled for (16 warps: 124 registers each)
#endif
#ifndef UOCR_STEADY
#define UOCR_STEADY 2
#endif
constexpr int kSteady = UOCR_STEADY < UOCR_RING ? UOCR_STEADY : UOCR_RING;
constexpr int kRing = UOCR_RING;  // shared-memory tile slots per warp; tiles K(0) V(0) K(1) V(1) ... rotate through them

// packed fp32x2 arithmetic: one instruction per two lanes of the dot products and accumulators
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }

// Unit descriptor bits (one 32-bit word per unit, built 32 units at a time, one per lane).
constexpr uint32_t kMetaValidMask = 0x1f;       // bits 0-4   tokens [skip, valid) of the tile are attended
constexpr int kMetaSkipShift = 5;               // bits 5-8
constexpr uint32_t kMetaLast = 1u << 9;         // last unit of its (row, head) item
constexpr uint32_t kMetaFirst = 1u << 10;       // first unit of its item
constexpr uint32_t kMetaText = 1u << 11;        // tile comes from the text pool
constexpr uint32_t kMetaPatch = 1u << 12;       // fused step: the new token lands in this tile
constexpr int kMetaPatchOffShift = 13;          // bits 13-16
constexpr int kMetaHeadShift = 17;              // bits 17-31 kv head (row-mode addressing)
constexpr uint32_t kMetaFixed = 1u << 17;       // paged addressing: tile of the fixed (possibly shared) region

template <typename KV>
__device__ __forceinline__ void unpack2(const uint4& w, float2 (&f)[KV::kPerChunk / 2]) {
    if constexpr (KV::kBytes == 2) {
        f[0] = make_float2(bf16_lo(w.x), bf16_hi(w.x));
        f[1] = make_float2(bf16_lo(w.y), bf16_hi(w.y));
        f[2] = make_float2(bf16_lo(w.z), bf16_hi(w.z));
        f[3] = make_float2(bf16_lo(w.w), bf16_hi(w.w));
    } else {
        f[0] = make_float2(__uint_as_float(w.x), __uint_as_float(w.y));
        f[1] = make_float2(__uint_as_float(w.z), __uint_as_float(w.w));
    }
}

// Rotation of one 16-byte chunk's worth of elements (EPC of them, first dim d0) of a head row.  `own`
// are the elements themselves, `other` the elements HD/2 away (the chunk lies in one half of the row):
// v[i] = x0 c - x1 s, v[i + HD/2] = x0 s + x1 c with x0 the lower-half and x1 the upper-half element.
template <int HD, int EPC>
__device__ __forceinline__ void rope_chunk(const float* freq, float pos, int d0, const float (&own)[EPC],
                                           const float (&other)[EPC], float (&out)[EPC]) {
    const bool lower = d0 < HD / 2;
#pragma unroll
    for (int e = 0; e < EPC; ++e) {
        float sn, cs;
        sincosf(pos * freq[(d0 + e) & (HD / 2 - 1)], &sn, &cs);
        out[e] = lower ? own[e] * cs - other[e] * sn : other[e] * sn + own[e] * cs;
    }
}

template <typename KV, int HD, bool PAGED, bool FUSED, bool ROPE = false>
__global__ void __launch_bounds__(UOCR_ATTN_THREADS, 1) rswa_attn_kernel(const __grid_constant__ AttnParams p) {
    static_assert(!ROPE || (FUSED && HD >= 2 * KV::kPerChunk), "rotary embedding: fused step only, a chunk must lie in one half of the head");
    using M = TileMap<KV, HD>;
    constexpr int LPR = M::kLanesPerRow, CPL = M::kChunksPerLane, RPW = M::kRowsPerLoad;
    constexpr int ITER = M::kIters, EPC = KV::kPerChunk, EPL = M::kElemsPerLane;
    constexpr int PPC = EPC / 2, PPL = EPL / 2;  // float2 pairs per chunk / per lane
    constexpr int ROWB = M::kRowBytes, TILE = M::kTileBytes;
    constexpr unsigned FULL = 0xffffffffu;

    extern __shared__ __align__(128) uint8_t smem[];
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- this warp's tile slots and their barriers ----------------------------------------------------
    const int bar_bytes = (warps * kRing * 8 + 127) & ~127;
    uint8_t* my_tiles = smem + bar_bytes + (size_t)warp * (kRing * TILE);
    const uint32_t bar0 = smem_addr(smem) + warp * (kRing * 8);
    const uint32_t tile0 = smem_addr(my_tiles);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kRing; ++s) mbar_init(bar0 + 8 * s, 1);
        mbar_init_fence();
    }
    __syncwarp();

    // ---- the plan: global (made by rswa_plan_kernel) or built here in shared memory ----------------
    const int* rs = p.rs;
    const RowInfo* info = p.info;
    int planner_ticket = -1;  // fused step, thread 0: how many CTAs had planned before this one
    const int* next_len = nullptr;
    const int* next_ring = nullptr;
    if constexpr (FUSED) {
        uint8_t* plan_base = smem + bar_bytes + (size_t)warps * (kRing * TILE) + (size_t)warps * kPendMax * sizeof(int);
        RowInfo* info_s = reinterpret_cast<RowInfo*>(plan_base);
        int* rs_s = reinterpret_cast<int*>(plan_base + sizeof(RowInfo) * p.rows);
        int* scratch = rs_s + p.rows + 1;
        int* next_len_s = scratch + 33;
        int* next_ring_s = next_len_s + p.rows;
        plan_all_rows(p.plan, rs_s, info_s, scratch, next_len_s, next_ring_s);
        __syncthreads();
        // The cursors move as soon as every CTA has planned from their old values.  Thread 0 announces
        // this CTA's plan; the answer is looked at once the first tiles are on their way, and the warp
        // that learns it was the last planner stores the new cursors (nobody reads them again in this
        // launch), which keeps the publication off the tail of the launch.
        // The counter wraps to zero with the launch's last ticket, so it needs no reset; a CTA of the next
        // (overlapped) launch cannot draw before every ticket of this one is taken, because a CTA releases
        // its dependents only after warp 0 has looked at its own ticket (see dependency_sync below).
        if (threadIdx.x == 0) {
            __threadfence();
            planner_ticket = (int)atomicInc(reinterpret_cast<unsigned*>(p.planned_ctas), gridDim.x - 1);
        }
        rs = rs_s;
        info = info_s;
        next_len = next_len_s;
        next_ring = next_ring_s;
    }

    const long long total = rs[p.rows];
    const int gw = (int)blockIdx.x * warps + warp;
    const PieceMap pm = make_piece_map(total, p.total_warps, warps, p.late_cta);
    // When there are fewer pieces than warps they are spread over the SMs (warp-major numbering) instead of
    // filling the first CTAs; otherwise CTA c owns pieces c * warps .. (the late-CTA shares rely on that).
    const int gw_spread = warp * (int)gridDim.x + (int)blockIdx.x;
    const int piece = pm.ns == p.total_warps ? gw : (gw_spread < pm.ns ? gw_spread : -1);
    int n_units = 0;
    long long u0 = 0;
    int* pend = reinterpret_cast<int*>(smem + bar_bytes + (size_t)warps * (kRing * TILE)) + warp * kPendMax;
    int pend_n = 0;
    bool gave_up = false, dep_synced = false;
    int issue_slot = 0, issue_seq = 0;  // issue_seq: position in the piece's tile sequence (unit = seq / 2, V if odd)
    int consumed = 0;                   // tiles of that sequence whose arrival has been waited for
    int use_slot = 0;                   // slot holding the next tile to consume
    uint32_t phases = 0;                // one phase bit per slot

    const int g = lane % LPR;   // chunk position inside the row
    const int rg = lane / LPR;  // which of the RPW rows of a warp-wide load

    {
        // ---- unit descriptors: lane l describes unit (desc_base + l) of this piece -------------------
        uint32_t d_tile = 0, d_meta = 0, d_item = 0;
        int desc_base = 0;
        auto build_desc = [&](int base) {
            desc_base = base;
            d_tile = d_meta = d_item = 0;
            if (base + lane < n_units) {
                UnitCursor c;
                cursor_seek(c, rs, info, p.rows, p.heads, u0 + base + lane);
                const int kvh = c.h / p.group;
                const int npb = (c.info.pe + kBlockTokens - 1) / kBlockTokens;
                int valid, skip = 0;
                uint32_t m = 0;
                if (c.j < npb) {
                    valid = min(kBlockTokens, c.info.pe - c.j * kBlockTokens);
                    if constexpr (PAGED) m |= kMetaFixed;
                } else {
                    int lead = 0;
                    if constexpr (PAGED && !FUSED) lead = p.k_text != nullptr ? (c.info.aux & 15) : 0;
                    const int jr = c.j - npb;
                    valid = min(kBlockTokens, lead + c.info.re - jr * kBlockTokens);
                    skip = jr == 0 ? lead : 0;
                }
                if constexpr (PAGED) {
                    int blk;
                    bool from_text = false;
                    if constexpr (!FUSED) from_text = p.k_text != nullptr && c.j >= npb;
                    if (from_text) {
                        blk = (c.info.aux >> 4) + (c.j - npb);
                        m |= kMetaText;
                        if (blk < 0 || blk >= p.text_blocks) { atomicOr(p.status, kStatusBadBlock); blk = 0; }
                    } else {
                        // table row = prefix blocks, then ring blocks right after them: unit index == table index
                        blk = -1;
                        if (c.j < p.table_stride) blk = __ldg(p.table + (size_t)c.info.slot * p.table_stride + c.j);
                        else atomicOr(p.status, kStatusBadSlot);
                        if (blk < 0 || blk >= p.num_blocks) { atomicOr(p.status, kStatusBadBlock); blk = 0; }
                    }
                    d_tile = (uint32_t)blk * p.kv_heads + kvh;
                } else {
                    d_tile = (uint32_t)(c.info.slot * p.slot_rows + c.j * kBlockTokens);  // first cache row of the tile
                    m |= (uint32_t)kvh << kMetaHeadShift;
                }
                if constexpr (FUSED) {
                    if (c.info.aux >= 0 && (c.info.aux >> 4) == c.j)
                        m |= kMetaPatch | ((uint32_t)(c.info.aux & 15) << kMetaPatchOffShift);
                }
                if (c.j == c.n - 1) m |= kMetaLast;
                if (c.j == 0) m |= kMetaFirst;
                d_meta = m | (uint32_t)valid | ((uint32_t)skip << kMetaSkipShift);
                d_item = (uint32_t)(c.r * p.heads + c.h);
            }
        };

        const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
        // ---- producer side: tiles K(0) V(0) K(1) V(1) ... rotate through the kRing slots -------------
        auto issue_tile = [&](int unit, bool is_v) {
            const uint32_t tile = __shfl_sync(FULL, d_tile, unit - desc_base);
            const uint32_t meta = __shfl_sync(FULL, d_meta, unit - desc_base);
            const uint32_t bar = bar0 + 8 * issue_slot;
            const uint32_t dst = tile0 + issue_slot * TILE;
            if constexpr (PAGED) {
                if (lane == 0) {
                    const uint8_t* base = (meta & kMetaText) ? (is_v ? p.v_text : p.k_text) : (is_v ? p.v_base : p.k_base);
                    mbar_arrive_expect_tx(bar, TILE);
                    // ring tiles are read once per launch: first out of L2; tiles of the fixed region are
                    // re-read by every sequence that shares the prefix: last out
                    bulk_copy_g2s_hint(dst, base + (size_t)tile * TILE, TILE, bar, (meta & kMetaFixed) ? pol_keep : pol_stream);
                }
            } else {
                const int nvalid = (int)(meta & kMetaValidMask);
                if (lane == 0) mbar_arrive_expect_tx(bar, nvalid * ROWB);
                if (lane < nvalid) {
                    const uint8_t* base = is_v ? p.v_base : p.k_base;
                    const size_t off = ((size_t)tile + lane) * p.row_stride_bytes + (size_t)(meta >> kMetaHeadShift) * ROWB;
                    bulk_copy_g2s(dst + lane * ROWB, base + off, ROWB, bar);
                }
            }
            issue_slot = issue_slot == kRing - 1 ? 0 : issue_slot + 1;
        };

        auto issue_next = [&]() {
            if (issue_seq < 2 * n_units) {
                issue_tile(issue_seq >> 1, (issue_seq & 1) != 0);
                ++issue_seq;
            }
        };
        // after `consumed` tiles of the piece have been used: refill while fewer than kSteady are in flight
        auto refill = [&](int used) {
            if (issue_seq - used < kSteady) issue_next();
        };
        // ---- consumer state ---------------------------------------------------------------------
        float2 q2[PPL], acc2[PPL];
        float m_run = -INFINITY, l_run = 0.f;
        auto load_q = [&](uint32_t item) {
            const float* qp = p.q + (size_t)item * HD;
#pragma unroll
            for (int cp = 0; cp < CPL; ++cp) {
                const int d0 = (g + 32 * cp) * EPC;
                if constexpr (ROPE) {
                    float own[EPC], other[EPC], rot[EPC];
#pragma unroll
                    for (int e = 0; e < EPC; e += 4) {
                        const float4 a = __ldg(reinterpret_cast<const float4*>(qp + d0 + e));
                        const float4 b = __ldg(reinterpret_cast<const float4*>(qp + (d0 ^ (HD / 2)) + e));
                        own[e] = a.x; own[e + 1] = a.y; own[e + 2] = a.z; own[e + 3] = a.w;
                        other[e] = b.x; other[e + 1] = b.y; other[e + 2] = b.z; other[e + 3] = b.w;
                    }
                    rope_chunk<HD, EPC>(p.rope_freq, (float)__ldg(p.rope_pos + item / p.heads), d0, own, other, rot);
#pragma unroll
                    for (int e = 0; e < EPC; e += 2)
                        q2[(cp * EPC + e) / 2] = make_float2(rot[e] * p.scale_log2e, rot[e + 1] * p.scale_log2e);
                } else {
#pragma unroll
                    for (int e = 0; e < EPC; e += 4) {
                        const float4 t = __ldg(reinterpret_cast<const float4*>(qp + d0 + e));
                        q2[(cp * EPC + e) / 2] = make_float2(t.x * p.scale_log2e, t.y * p.scale_log2e);
                        q2[(cp * EPC + e) / 2 + 1] = make_float2(t.z * p.scale_log2e, t.w * p.scale_log2e);
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < PPL; ++e) acc2[e] = make_float2(0.f, 0.f);
            m_run = -INFINITY;
            l_run = 0.f;
        };
        // Before the first read of q / k_new / v_new and before any access to the shared scratch, a
        // launch that was allowed to overlap its predecessor in the stream waits for it, then lets the
        // next launch begin its own prologue.  Both instructions are no-ops for an ordinary launch.
        // Only warp 0 releases the dependents, and only after publish_cursors() has consumed the ticket
        // its thread 0 drew: when the next launch's first CTA starts, every ticket of this launch has
        // been drawn, so the two launches never mix their tickets in the shared counter.
        auto dependency_sync = [&]() {
            if constexpr (FUSED) {
                if (!dep_synced) {
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                    if (warp == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
                }
            }
            dep_synced = true;
        };

        // Fused step, warp 0: if this CTA was the last to plan, store the cursors the step leaves behind.
        bool publish_checked = false;
        auto publish_cursors = [&]() {
            if constexpr (FUSED) {
                if (warp != 0 || publish_checked) return;
                publish_checked = true;
                if (!__shfl_sync(FULL, planner_ticket == (int)gridDim.x - 1, 0)) return;
                __threadfence();  // every other CTA's cursor reads precede its announcement
                for (int r = lane; r < p.rows; r += 32) {
                    const int slot = info[r].slot;
                    if (next_len[r] >= 0) p.d_len[slot] = next_len[r];
                    if (next_ring[r] >= 0) p.d_ring_pos[slot] = next_ring[r];
                }
            }
        };

        // ---- arrivals: whoever completes an item's set of partials merges them ------------------------
        auto flush_arrivals = [&]() {
            if (pend_n == 0) return;
            __syncwarp();  // orders the partial stores of every lane before the arriving lanes' releases
            // every lane arrives for one pending segment (the atomics overlap), then the warp merges the
            // items for which one of its arrivals was the last
            int my_item = -1, my_wf = 0, my_wl = 0;
            long long my_s0 = 0;
            bool my_last = false;
            if (lane < pend_n) {
                my_item = pend[lane];
                const int r = my_item / p.heads, h = my_item - r * p.heads;
                const int n = (rs[r + 1] - rs[r]) / p.heads;
                my_s0 = (long long)rs[r] + (long long)h * n;
                my_wf = pm.of(my_s0);
                my_wl = pm.of(my_s0 + n - 1);
                int old;  // release: the warp's partial stores (ordered before this by the barrier above); acquire: the other arrivers' partials
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + my_wf) : "memory");
                my_last = (old == my_wl - my_wf);
            }
            const unsigned all_todo = __ballot_sync(FULL, my_last);
            unsigned todo = all_todo;
            __syncwarp();  // the arriving lane's acquire covers the loads the whole warp issues next
            while (todo) {
                const int src = __ffs(todo) - 1;
                todo &= todo - 1;
                const int item = __shfl_sync(FULL, my_item, src);
                const int wf = __shfl_sync(FULL, my_wf, src);
                const int wl = __shfl_sync(FULL, my_wl, src);
                const long long s0 = __shfl_sync(FULL, my_s0, src);
                float* out_item = p.out + (size_t)item * HD;
                const bool wf_second = pm.start(wf) < s0;  // the item is piece wf's second segment
                constexpr int NK = (HD + 31) / 32;
                float o[NK];
#pragma unroll
                for (int i = 0; i < NK; ++i) o[i] = 0.f;
                float lall = 0.f;
                const int n_part = wl - wf + 1;
                if (n_part <= 32) {
                    // The usual case.  Lane i holds (max, sum) of partial i; the accumulators come in batches
                    // of kBatch partials whose loads are all issued before any of them is used, the first
                    // batch together with the (max, sum) loads: a merge costs about one round trip to L2 per
                    // batch instead of one per partial (the last arriver's merge ends the launch).
                    constexpr int kBatch = NK > 4 ? 4 : 8;
                    const int slot_l = 2 * (wf + lane) + ((lane == 0 && wf_second) ? 1 : 0);
                    float mi = -INFINITY, li = 0.f;
                    if (lane < n_part) {
                        mi = __ldcg(p.part_ml + 2 * slot_l);
                        li = __ldcg(p.part_ml + 2 * slot_l + 1);
                    }
                    float tmp[kBatch][NK];
                    auto load_batch = [&](int b0) {
#pragma unroll
                        for (int i = 0; i < kBatch; ++i) {
                            const int w = wf + b0 + i;
                            const int si = 2 * w + ((b0 + i == 0 && wf_second) ? 1 : 0);
                            const float* pa = p.part_acc + (size_t)si * HD;
#pragma unroll
                            for (int kk = 0; kk < NK; ++kk) {
                                const int d = lane + 32 * kk;
                                tmp[i][kk] = (b0 + i < n_part && d < HD) ? __ldcg(pa + d) : 0.f;
                            }
                        }
                    };
                    load_batch(0);
                    float mall = mi;
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) mall = fmaxf(mall, __shfl_xor_sync(FULL, mall, d));
                    const float mall_safe = (mall == -INFINITY) ? 0.f : mall;
                    const float wg = lane < n_part ? fast_exp2(mi - mall_safe) : 0.f;
                    lall = li * wg;
                    for (int b0 = 0;;) {
#pragma unroll
                        for (int i = 0; i < kBatch; ++i) {
                            const float wi = __shfl_sync(FULL, wg, (b0 + i) & 31);
#pragma unroll
                            for (int kk = 0; kk < NK; ++kk) o[kk] = fmaf(tmp[i][kk], wi, o[kk]);
                        }
                        b0 += kBatch;
                        if (b0 >= n_part) break;
                        load_batch(b0);
                    }
                } else {
                    // an item cut into more than 32 pieces (few rows on many warps): (max, sum) first, then the
                    // accumulators one partial at a time
                    float mall = -INFINITY;
                    for (int w0 = wf; w0 <= wl; w0 += 32) {
                        const int w = w0 + lane;
                        const float mi = w <= wl ? __ldcg(p.part_ml + 2 * (2 * w + (w == wf && wf_second ? 1 : 0))) : -INFINITY;
                        mall = fmaxf(mall, mi);
                    }
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) mall = fmaxf(mall, __shfl_xor_sync(FULL, mall, d));
                    const float mall_safe = (mall == -INFINITY) ? 0.f : mall;
                    for (int w0 = wf; w0 <= wl; w0 += 32) {
                        const int w = w0 + lane;
                        const int slot_w = 2 * w + (w == wf && wf_second ? 1 : 0);
                        float wg = 0.f;
                        if (w <= wl) {
                            wg = fast_exp2(__ldcg(p.part_ml + 2 * slot_w) - mall_safe);
                            lall += __ldcg(p.part_ml + 2 * slot_w + 1) * wg;
                        }
                        const int cnt = min(32, wl - w0 + 1);
                        for (int i = 0; i < cnt; ++i) {
                            const float wi = __shfl_sync(FULL, wg, i);
                            const int si = __shfl_sync(FULL, slot_w, i);
                            const float* pa = p.part_acc + (size_t)si * HD;
#pragma unroll
                            for (int kk = 0; kk < NK; ++kk) {
                                const int d = lane + 32 * kk;
                                if (d < HD) o[kk] = fmaf(__ldcg(pa + d), wi, o[kk]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) lall += __shfl_xor_sync(FULL, lall, d);
                const float inv = lall > 0.f ? 1.f / lall : 0.f;
#pragma unroll
                for (int i = 0; i < NK; ++i) {
                    const int d = lane + 32 * i;
                    if (d < HD) {
                        if (p.out_bf16)
                            reinterpret_cast<uint16_t*>(p.out)[(size_t)item * HD + d] = (uint16_t)f32_to_bf16_bits(o[i] * inv);
                        else
                            out_item[d] = o[i] * inv;
                    }
                }
            }
            // the counters of the merged items go back to zero for the next launch (after the merges: a store
            // ahead of the fence above would make that fence wait for it)
            if (my_last) p.counters[my_wf] = 0;
            pend_n = 0;
            __syncwarp();
        };

        // ---- this warp's piece of the unit line -----------------------------------------------------------
        if (piece >= 0) {
            u0 = pm.start(piece);
            n_units = (int)(pm.end(piece) - u0);
            issue_seq = 0;
            build_desc(0);
#pragma unroll
            for (int s = 0; s < kRing; ++s) issue_next();
            publish_cursors();
            // everything up to here read only this layer's own cursors, table and pool
            dependency_sync();
            uint32_t cur_item = __shfl_sync(FULL, d_item, 0);
            load_q(cur_item);
            bool first_segment = true;
            bool seg_from_start = (__shfl_sync(FULL, d_meta, 0) & kMetaFirst) != 0;

        for (int it = 0; it < n_units; ++it) {
            if (it - desc_base >= 32 - 2) {  // the producer looks two units ahead: keep those described
                build_desc(it);
            }
            const uint32_t meta = __shfl_sync(FULL, d_meta, it - desc_base);
            const int nvalid = (int)(meta & kMetaValidMask);
            const int nskip = (int)((meta >> kMetaSkipShift) & 15);

            // ---- scores: q . k for the 16 tokens of the tile -----------------------------------
            uint8_t* ktile = my_tiles + use_slot * TILE;
            if (!mbar_wait_bounded(bar0 + 8 * use_slot, (phases >> use_slot) & 1u, p.status, p.wait_limit)) { gave_up = true; break; }
            phases ^= 1u << use_slot;
            use_slot = use_slot == kRing - 1 ? 0 : use_slot + 1;
            ++consumed;
            if constexpr (FUSED) {
                if (meta & kMetaPatch) {  // the new K row replaces whatever the ring slot held
                    const int off = (int)((meta >> kMetaPatchOffShift) & 15);
                    const int r = (int)(cur_item / p.heads), h = (int)(cur_item - r * p.heads);
                    const int kvh = h / p.group;
                    const uint32_t tile = __shfl_sync(FULL, d_tile, it - desc_base);
                    for (int ch = lane; ch < M::kChunks; ch += 32) {
                        const float* src = p.k_new + ((size_t)r * p.kv_heads + kvh) * HD + ch * EPC;
                        uint4 w;
                        if constexpr (ROPE) {
                            const float* oth = p.k_new + ((size_t)r * p.kv_heads + kvh) * HD + ((ch * EPC) ^ (HD / 2));
                            float own[EPC], other[EPC], rot[EPC];
#pragma unroll
                            for (int e = 0; e < EPC; e += 4) {
                                const float4 a = __ldg(reinterpret_cast<const float4*>(src + e));
                                const float4 b = __ldg(reinterpret_cast<const float4*>(oth + e));
                                own[e] = a.x; own[e + 1] = a.y; own[e + 2] = a.z; own[e + 3] = a.w;
                                other[e] = b.x; other[e + 1] = b.y; other[e + 2] = b.z; other[e + 3] = b.w;
                            }
                            rope_chunk<HD, EPC>(p.rope_freq, (float)__ldg(p.rope_pos + r), ch * EPC, own, other, rot);
                            if constexpr (EPC == 8)
                                w = make_uint4(pack_bf16x2(rot[0], rot[1]), pack_bf16x2(rot[2], rot[3]),
                                               pack_bf16x2(rot[4], rot[5]), pack_bf16x2(rot[6], rot[7]));
                            else
                                w = make_uint4(__float_as_uint(rot[0]), __float_as_uint(rot[1]), __float_as_uint(rot[2]),
                                               __float_as_uint(rot[3]));
                        } else if constexpr (EPC == 8) {
                            const float4 a = __ldg(reinterpret_cast<const float4*>(src));
                            const float4 b = __ldg(reinterpret_cast<const float4*>(src + 4));
                            w = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                                           pack_bf16x2(b.z, b.w));
                        } else {
                            w = __ldg(reinterpret_cast<const uint4*>(src));
                        }
                        *reinterpret_cast<uint4*>(ktile + off * ROWB + ch * 16) = w;
                        if (h % p.group == 0)
                            *reinterpret_cast<uint4*>(const_cast<uint8_t*>(p.k_base) + (size_t)tile * TILE + off * ROWB +
                                                      ch * 16) = w;
                    }
                    __syncwarp();
                }
            }
            float sc[ITER];
#pragma unroll
            for (int i = 0; i < ITER; ++i) {
                const int t = (i * RPW + rg) & (kBlockTokens - 1);
                float2 d2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int cp = 0; cp < CPL; ++cp) {
                    const uint4 w = *reinterpret_cast<const uint4*>(ktile + t * ROWB + (g + 32 * cp) * 16);
                    float2 f[PPC];
                    unpack2<KV>(w, f);
#pragma unroll
                    for (int e = 0; e < PPC; ++e) d2 = fma2(q2[cp * PPC + e], f[e], d2);
                }
                sc[i] = d2.x + d2.y;
            }
            // the K slot is free: the tile kRing positions further down the sequence goes there
            __syncwarp();
            if constexpr (FUSED) {
                if (meta & kMetaPatch) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            refill(2 * it + 1);

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
            const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
            for (int e = 0; e < PPL; ++e) acc2[e] = mul2(acc2[e], alpha2);

            // ---- acc += p . v ----------------------------------------------------------------------
            uint8_t* vtile = my_tiles + use_slot * TILE;
            if (!mbar_wait_bounded(bar0 + 8 * use_slot, (phases >> use_slot) & 1u, p.status, p.wait_limit)) { gave_up = true; break; }
            phases ^= 1u << use_slot;
            use_slot = use_slot == kRing - 1 ? 0 : use_slot + 1;
            ++consumed;
            if constexpr (FUSED) {
                if (meta & kMetaPatch) {
                    const int off = (int)((meta >> kMetaPatchOffShift) & 15);
                    const int r = (int)(cur_item / p.heads), h = (int)(cur_item - r * p.heads);
                    const int kvh = h / p.group;
                    const uint32_t tile = __shfl_sync(FULL, d_tile, it - desc_base);
                    for (int ch = lane; ch < M::kChunks; ch += 32) {
                        const float* src = p.v_new + ((size_t)r * p.kv_heads + kvh) * HD + ch * EPC;
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
                        if (h % p.group == 0)
                            *reinterpret_cast<uint4*>(const_cast<uint8_t*>(p.v_base) + (size_t)tile * TILE + off * ROWB +
                                                      ch * 16) = w;
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
                    const float2 pi2 = make_float2(pi, pi);
#pragma unroll
                    for (int cp = 0; cp < CPL; ++cp) {
                        const uint4 w = *reinterpret_cast<const uint4*>(vtile + t * ROWB + (g + 32 * cp) * 16);
                        float2 f[PPC];
                        unpack2<KV>(w, f);
#pragma unroll
                        for (int e = 0; e < PPC; ++e) acc2[cp * PPC + e] = fma2(pi2, f[e], acc2[cp * PPC + e]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < ITER; ++i) {
                    const int t = i * RPW + rg;
                    const float pi = (LPR >= 2) ? __shfl_sync(FULL, pr, rg * LPR + 2 * i) : pr;
                    const float2 pi2 = make_float2(pi, pi);
                    if (t >= nskip && t < nvalid) {  // rows outside the valid range may hold anything
#pragma unroll
                        for (int cp = 0; cp < CPL; ++cp) {
                            const uint4 w = *reinterpret_cast<const uint4*>(vtile + t * ROWB + (g + 32 * cp) * 16);
                            float2 f[PPC];
                            unpack2<KV>(w, f);
#pragma unroll
                            for (int e = 0; e < PPC; ++e) acc2[cp * PPC + e] = fma2(pi2, f[e], acc2[cp * PPC + e]);
                        }
                    }
                }
            }

            // ---- the V slot is free as well -------------------------------------------------------------
            __syncwarp();
            if constexpr (FUSED) {
                if (meta & kMetaPatch) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            refill(2 * it + 2);

            // ---- end of an item (or of the piece): emit ----------------------------------------------
            const bool item_done = (meta & kMetaLast) != 0;
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
                float acc[EPL];
#pragma unroll
                for (int e = 0; e < PPL; ++e) {
                    acc[2 * e] = acc2[e].x * wgt;
                    acc[2 * e + 1] = acc2[e].y * wgt;
                }
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    float a = acc[e];
#pragma unroll
                    for (int d = LPR; d < 32; d <<= 1) a += __shfl_xor_sync(FULL, a, d);
                    acc[e] = a;
                }
                const bool whole = item_done && seg_from_start;
                if (whole) {
                    if (lane < LPR) {
                        float* out_item = p.out + (size_t)cur_item * HD;
                        const float mul = lsum > 0.f ? 1.f / lsum : 0.f;
#pragma unroll
                        for (int cp = 0; cp < CPL; ++cp) {
                            const int d0 = (g + 32 * cp) * EPC;
#pragma unroll
                            for (int e = 0; e < EPC; e += 4) {
                                if (p.out_bf16)
                                    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out) + (size_t)cur_item * HD + d0 + e) =
                                        make_uint2(pack_bf16x2(acc[cp * EPC + e] * mul, acc[cp * EPC + e + 1] * mul),
                                                   pack_bf16x2(acc[cp * EPC + e + 2] * mul, acc[cp * EPC + e + 3] * mul));
                                else
                                    *reinterpret_cast<float4*>(out_item + d0 + e) =
                                        make_float4(acc[cp * EPC + e] * mul, acc[cp * EPC + e + 1] * mul,
                                                    acc[cp * EPC + e + 2] * mul, acc[cp * EPC + e + 3] * mul);
                            }
                        }
                    }
                } else {
                    // leave a partial; the arrival (fence + counter) is deferred to the end of the piece so
                    // that one fence covers both partial segments and no copy is in flight when it executes
                    const int my_slot = 2 * piece + (first_segment ? 0 : 1);
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
                    if (lane == 0) pend[pend_n] = (int)cur_item;
                    if (++pend_n == kPendMax) flush_arrivals();
                }
                first_segment = false;
                if (!piece_done) {
                    cur_item = __shfl_sync(FULL, d_item, it + 1 - desc_base);
                    seg_from_start = true;
                    load_q(cur_item);
                }
            }
        }

        }
        publish_cursors();  // a warp without a piece gets here without having looked
        if (!gave_up) {
            flush_arrivals();
        } else {
            // A wait ran out (the status word says so and the launch's results are void).  Tiles issued and not
            // yet consumed may still be on their way into this warp's slots: see them land before the CTA exits
            // and its shared memory is handed to another CTA.  These waits keep the full limit.
            for (int t = consumed; t < issue_seq; ++t) {
                mbar_wait_bounded(bar0 + 8 * use_slot, (phases >> use_slot) & 1u, nullptr);
                phases ^= 1u << use_slot;
                use_slot = use_slot == kRing - 1 ? 0 : use_slot + 1;
            }
        }
    }

    if constexpr (FUSED) {
        if (!dep_synced) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (warp == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
    }
}

}  // namespace uocr_b200
